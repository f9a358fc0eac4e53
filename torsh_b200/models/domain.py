"""Domain models and multi-view diffusion parts (``crates/torsh-models/src/domain.rs``, ``crates/torsh-models/src/diffusion/``):
U-Net with attention gates and deep supervision, 3-D U-Net, physics-informed networks with physics / boundary / initial
losses and adaptive loss weights, Fourier neural operators; camera embeddings, classifier-free guidance helpers, IP-Adapter
image-token projection, latent upsampler, cross-view attention and a multi-view U-Net conditioned on time and camera."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.nn.functional as F
from torch import nn

_ACT = {"relu": nn.ReLU, "gelu": nn.GELU, "silu": nn.SiLU, "tanh": nn.Tanh, "leaky_relu": lambda: nn.LeakyReLU(0.01), "elu": nn.ELU, "sin": lambda: _Sine()}


class _Sine(nn.Module):
    def forward(self, x): return torch.sin(x)


# ================================================================================================ U-Net family
@dataclass
class UNetConfig:
    in_channels: int = 1
    out_channels: int = 2
    base_features: int = 64
    num_levels: int = 4
    batch_norm: bool = True
    dropout: float = 0.0
    attention: bool = False
    activation: str = "relu"
    deep_supervision: bool = False


class DoubleConv(nn.Module):
    def __init__(self, cin, cout, batch_norm=True, dropout=0.0, activation="relu", dims: int = 2):
        super().__init__()
        conv, bn, do = (nn.Conv2d, nn.BatchNorm2d, nn.Dropout2d) if dims == 2 else (nn.Conv3d, nn.BatchNorm3d, nn.Dropout3d)
        layers = []
        for a, b in ((cin, cout), (cout, cout)):
            layers += [conv(a, b, 3, padding=1, bias=not batch_norm)] + ([bn(b)] if batch_norm else []) + [_ACT[activation]()]
        if dropout:
            layers.append(do(dropout))
        self.block = nn.Sequential(*layers)
    def forward(self, x): return self.block(x)


class AttentionGate(nn.Module):
    """Additive attention over a skip connection: the coarser gating signal decides, per pixel, how much of the skip features
    pass (``alpha = sigmoid(psi(relu(W_g g + W_x x)))``)."""

    def __init__(self, gate_channels, skip_channels, inter_channels):
        super().__init__()
        self.wg, self.wx, self.psi = nn.Conv2d(gate_channels, inter_channels, 1), nn.Conv2d(skip_channels, inter_channels, 1), nn.Conv2d(inter_channels, 1, 1)
    def forward(self, gate, skip):
        g = F.interpolate(self.wg(gate), size=skip.shape[-2:], mode="bilinear", align_corners=False)
        self.last_alpha = torch.sigmoid(self.psi(F.relu(g + self.wx(skip))))
        return skip * self.last_alpha


class UNet(nn.Module):
    def __init__(self, cfg: UNetConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or UNetConfig(**kw)
        f = [cfg.base_features * 2 ** i for i in range(cfg.num_levels + 1)]
        dc = lambda a, b: DoubleConv(a, b, cfg.batch_norm, cfg.dropout, cfg.activation)
        self.down = nn.ModuleList([dc(cfg.in_channels if i == 0 else f[i - 1], f[i]) for i in range(cfg.num_levels)])
        self.bottleneck = dc(f[cfg.num_levels - 1], f[cfg.num_levels])
        self.up = nn.ModuleList([nn.ConvTranspose2d(f[i + 1], f[i], 2, stride=2) for i in reversed(range(cfg.num_levels))])
        self.dec = nn.ModuleList([dc(2 * f[i], f[i]) for i in reversed(range(cfg.num_levels))])
        self.gates = nn.ModuleList([AttentionGate(f[i + 1], f[i], max(f[i] // 2, 1)) for i in reversed(range(cfg.num_levels))]) if cfg.attention else None
        self.head = nn.Conv2d(f[0], cfg.out_channels, 1)
        self.aux_heads = nn.ModuleList([nn.Conv2d(f[i], cfg.out_channels, 1) for i in reversed(range(1, cfg.num_levels))]) if cfg.deep_supervision else None

    def forward(self, x):
        if x.shape[-1] % 2 ** self.cfg.num_levels or x.shape[-2] % 2 ** self.cfg.num_levels:
            raise ValueError(f"spatial size {tuple(x.shape[-2:])} must be a multiple of {2 ** self.cfg.num_levels}")
        skips = []
        for d in self.down:
            x = d(x); skips.append(x); x = F.max_pool2d(x, 2)
        x, aux = self.bottleneck(x), []
        for i, (up, dec) in enumerate(zip(self.up, self.dec)):
            skip = skips[-1 - i]
            if self.gates is not None:
                skip = self.gates[i](x, skip)
            x = dec(torch.cat([up(x), skip], 1))
            if self.aux_heads is not None and i < len(self.aux_heads):
                aux.append(F.interpolate(self.aux_heads[i](x), size=skips[0].shape[-2:], mode="bilinear", align_corners=False))
        out = self.head(x)
        return (out, aux) if self.aux_heads is not None and self.training else out

    @staticmethod
    def deep_supervision_loss(out, aux, target, loss_fn=F.cross_entropy, decay: float = 0.5):
        """Main loss plus the auxiliary heads' losses weighted ``decay^k`` from the finest auxiliary level down."""
        total, w = loss_fn(out, target), decay
        for a in reversed(aux):
            total, w = total + w * loss_fn(a, target), w * decay
        return total


@dataclass
class UNet3DConfig:
    in_channels: int = 1
    out_channels: int = 2
    base_features: int = 32
    num_levels: int = 3
    batch_norm: bool = True
    dropout: float = 0.0
    activation: str = "relu"


class UNet3D(nn.Module):
    def __init__(self, cfg: UNet3DConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or UNet3DConfig(**kw)
        f = [cfg.base_features * 2 ** i for i in range(cfg.num_levels + 1)]
        dc = lambda a, b: DoubleConv(a, b, cfg.batch_norm, cfg.dropout, cfg.activation, dims=3)
        self.down = nn.ModuleList([dc(cfg.in_channels if i == 0 else f[i - 1], f[i]) for i in range(cfg.num_levels)])
        self.bottleneck = dc(f[cfg.num_levels - 1], f[cfg.num_levels])
        self.up = nn.ModuleList([nn.ConvTranspose3d(f[i + 1], f[i], 2, stride=2) for i in reversed(range(cfg.num_levels))])
        self.dec = nn.ModuleList([dc(2 * f[i], f[i]) for i in reversed(range(cfg.num_levels))])
        self.head = nn.Conv3d(f[0], cfg.out_channels, 1)

    def forward(self, x):
        skips = []
        for d in self.down:
            x = d(x); skips.append(x); x = F.max_pool3d(x, 2)
        x = self.bottleneck(x)
        for i, (up, dec) in enumerate(zip(self.up, self.dec)):
            x = dec(torch.cat([up(x), skips[-1 - i]], 1))
        return self.head(x)


def dice_loss(logits: torch.Tensor, target: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Soft Dice over classes; ``target`` holds class indices."""
    p = logits.softmax(1)
    oh = F.one_hot(target, logits.shape[1]).movedim(-1, 1).to(p.dtype)
    dims = tuple(range(2, p.dim()))
    inter, denom = (p * oh).sum(dims), p.sum(dims) + oh.sum(dims)
    return 1 - ((2 * inter + eps) / (denom + eps)).mean()


# ================================================================================================ physics-informed networks
@dataclass
class PINNConfig:
    input_dim: int = 2
    output_dim: int = 1
    hidden_dims: Sequence[int] = (64, 64, 64)
    activation: str = "tanh"
    physics_weight: float = 1.0
    boundary_weight: float = 1.0
    initial_weight: float = 1.0
    adaptive_weights: bool = False


class PINN(nn.Module):
    """Fully connected network whose loss is the PDE residual at collocation points plus boundary and initial mismatches.  With
    ``adaptive_weights`` the three weights are learned log-variances (each term is ``exp(-s) L + s``), which balances terms
    of different magnitude without tuning."""

    def __init__(self, cfg: PINNConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or PINNConfig(**kw)
        dims = [cfg.input_dim, *cfg.hidden_dims]
        layers = []
        for a, b in zip(dims, dims[1:]):
            layers += [nn.Linear(a, b), _ACT[cfg.activation]()]
        self.net = nn.Sequential(*layers, nn.Linear(dims[-1], cfg.output_dim))
        for m in self.net:
            if isinstance(m, nn.Linear):
                nn.init.xavier_normal_(m.weight); nn.init.zeros_(m.bias)
        self.log_vars = nn.Parameter(torch.zeros(3)) if cfg.adaptive_weights else None

    def forward(self, x): return self.net(x)

    @staticmethod
    def derivative(u: torch.Tensor, x: torch.Tensor, dim: int, order: int = 1) -> torch.Tensor:
        """``d^order u / d x_dim^order`` by repeated reverse-mode differentiation (``x`` must require gradients)."""
        for _ in range(order):
            u = torch.autograd.grad(u.sum(), x, create_graph=True)[0][:, dim:dim + 1]
        return u

    def physics_loss(self, x: torch.Tensor, residual: Callable[["PINN", torch.Tensor], torch.Tensor]) -> torch.Tensor:
        x = x.detach().requires_grad_(True)
        return residual(self, x).pow(2).mean()

    def boundary_loss(self, x: torch.Tensor, value: torch.Tensor) -> torch.Tensor: return (self(x) - value).pow(2).mean()
    initial_loss = boundary_loss

    def compute_total_loss(self, physics: torch.Tensor, boundary: torch.Tensor | None = None, initial: torch.Tensor | None = None) -> tuple[torch.Tensor, dict]:
        terms = {"physics": (physics, self.cfg.physics_weight, 0), "boundary": (boundary, self.cfg.boundary_weight, 1), "initial": (initial, self.cfg.initial_weight, 2)}
        total, parts = 0.0, {}
        for name, (val, w, i) in terms.items():
            if val is None:
                continue
            parts[name] = float(val.detach())
            total = total + (torch.exp(-self.log_vars[i]) * val + self.log_vars[i] if self.log_vars is not None else w * val)
        return total, parts


# ================================================================================================ Fourier neural operator
class FourierLayer(nn.Module):
    """Spectral convolution: FFT, multiply the lowest ``modes`` frequencies by learned complex weights, inverse FFT; plus a
    point-wise linear path.  1-D and 2-D."""

    def __init__(self, width: int, modes: Sequence[int]):
        super().__init__()
        self.width, self.modes = width, tuple(modes)
        scale = 1 / (width * width)
        if len(self.modes) == 1:
            self.w = nn.Parameter(scale * torch.randn(width, width, self.modes[0], dtype=torch.cfloat))
            self.skip = nn.Conv1d(width, width, 1)
        else:
            self.w1 = nn.Parameter(scale * torch.randn(width, width, *self.modes, dtype=torch.cfloat))
            self.w2 = nn.Parameter(scale * torch.randn(width, width, *self.modes, dtype=torch.cfloat))
            self.skip = nn.Conv2d(width, width, 1)

    def forward(self, x):
        if len(self.modes) == 1:
            m = self.modes[0]
            xf = torch.fft.rfft(x, dim=-1)
            out = torch.zeros_like(xf)
            out[..., :m] = torch.einsum("bim,iom->bom", xf[..., :m], self.w)
            return torch.fft.irfft(out, n=x.shape[-1], dim=-1) + self.skip(x)
        m1, m2 = self.modes
        xf = torch.fft.rfft2(x)
        out = torch.zeros_like(xf)
        out[..., :m1, :m2] = torch.einsum("bixy,ioxy->boxy", xf[..., :m1, :m2], self.w1)
        out[..., -m1:, :m2] = torch.einsum("bixy,ioxy->boxy", xf[..., -m1:, :m2], self.w2)
        return torch.fft.irfft2(out, s=x.shape[-2:]) + self.skip(x)


@dataclass
class FNOConfig:
    input_dim: int = 1
    output_dim: int = 1
    num_layers: int = 4
    hidden_dim: int = 128
    modes: Sequence[int] = (16,)
    width: int = 32
    activation: str = "gelu"


class FNO(nn.Module):
    """Lift to ``width`` channels (with the grid coordinates appended), ``num_layers`` Fourier layers, project back.  Resolution
    independent: trained on one grid, evaluated on another."""

    def __init__(self, cfg: FNOConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or FNOConfig(**kw)
        nd = len(cfg.modes)
        self.lift = nn.Linear(cfg.input_dim + nd, cfg.width)
        self.layers = nn.ModuleList([FourierLayer(cfg.width, cfg.modes) for _ in range(cfg.num_layers)])
        self.act = _ACT[cfg.activation]()
        self.proj = nn.Sequential(nn.Linear(cfg.width, cfg.hidden_dim), _ACT[cfg.activation](), nn.Linear(cfg.hidden_dim, cfg.output_dim))

    def forward(self, x):
        """``x``: ``[batch, *grid, input_dim]`` -> ``[batch, *grid, output_dim]``."""
        grid = torch.stack(torch.meshgrid(*[torch.linspace(0, 1, s, device=x.device, dtype=x.dtype) for s in x.shape[1:-1]], indexing="ij"), -1)
        h = self.lift(torch.cat([x, grid.expand(x.shape[0], *grid.shape)], -1)).movedim(-1, 1)
        for i, l in enumerate(self.layers):
            h = l(h)
            if i < len(self.layers) - 1:
                h = self.act(h)
        return self.proj(h.movedim(1, -1))


# ================================================================================================ diffusion: guidance
def apply_classifier_free_guidance(cond_pred: torch.Tensor, uncond_pred: torch.Tensor, guidance_scale: float) -> torch.Tensor:
    if cond_pred.shape != uncond_pred.shape:
        raise ValueError(f"conditional and unconditional predictions must have the same shape: {tuple(cond_pred.shape)} vs {tuple(uncond_pred.shape)}")
    return torch.lerp(uncond_pred, cond_pred, guidance_scale)                    # uncond + s (cond - uncond), one fused pass


def prepare_cfg_batch(cond: torch.Tensor, uncond: torch.Tensor) -> torch.Tensor:
    if cond.shape != uncond.shape:
        raise ValueError("conditional and unconditional inputs must have the same shape")
    return torch.cat([uncond, cond], 0)


def split_cfg_batch(pred: torch.Tensor, batch_size: int) -> tuple[torch.Tensor, torch.Tensor]:
    if pred.shape[0] != 2 * batch_size:
        raise ValueError(f"expected a batch of {2 * batch_size}, got {pred.shape[0]}")
    return pred[:batch_size], pred[batch_size:]


def guidance_scale_with_warmup(timestep: int, num_steps: int, target_scale: float, warmup_steps: int | None = None) -> float:
    warm = num_steps // 10 if warmup_steps is None else warmup_steps
    return target_scale if timestep >= warm or warm == 0 else 1.0 + timestep / warm * (target_scale - 1.0)


def rescale_guidance(guided: torch.Tensor, cond_pred: torch.Tensor, phi: float = 0.7) -> torch.Tensor:
    """Pulls the per-sample standard deviation of a strongly guided prediction back toward the conditional one (fixes the
    over-exposure of large guidance scales)."""
    dims = tuple(range(1, guided.dim()))
    rescaled = guided * (cond_pred.std(dims, keepdim=True) / guided.std(dims, keepdim=True).clamp_min(1e-12))
    return phi * rescaled + (1 - phi) * guided


# ================================================================================================ diffusion: conditioning modules
class CameraEmbedding(nn.Module):
    """Camera intrinsics ``(fx, fy, cx, cy)`` and extrinsics (rotation 3x3 row-major, translation 3) — 16 numbers — to one
    embedding per view."""

    def __init__(self, embed_dim: int = 768, hidden_dims: Sequence[int] = (256, 512)):
        super().__init__()
        dims = [16, *hidden_dims]
        layers = []
        for a, b in zip(dims, dims[1:]):
            layers += [nn.Linear(a, b), nn.SiLU()]
        self.mlp = nn.Sequential(*layers, nn.Linear(dims[-1], embed_dim))

    def forward(self, camera_params):
        if camera_params.shape[-1] != 16:
            raise ValueError(f"camera parameters must have 16 entries (4 intrinsics, 9 rotation, 3 translation), got {camera_params.shape[-1]}")
        return self.mlp(camera_params)

    @staticmethod
    def pack(fx, fy, cx, cy, rotation: torch.Tensor, translation: torch.Tensor) -> torch.Tensor:
        return torch.cat([torch.stack([torch.as_tensor(v, dtype=rotation.dtype).expand(rotation.shape[:-2]) for v in (fx, fy, cx, cy)], -1), rotation.flatten(-2), translation], -1)


@dataclass
class IPAdapterProjectionConfig:
    num_tokens: int = 4
    cross_attn_dim: int = 768
    clip_feature_dim: int = 1024
    hidden_dim: int = 1024

    @classmethod
    def sd15_vit_l(cls): return cls(16, 768, 1024, 2048)
    @classmethod
    def sdxl_vit_g(cls): return cls(16, 2048, 1280, 4096)
    def validate(self):
        for k in ("num_tokens", "cross_attn_dim", "clip_feature_dim", "hidden_dim"):
            if getattr(self, k) <= 0:
                raise ValueError(f"{k} must be positive")


class IPAdapterProjection(nn.Module):
    """One pooled image feature to ``num_tokens`` context tokens for cross attention."""

    def __init__(self, cfg: IPAdapterProjectionConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or IPAdapterProjectionConfig(**kw)
        cfg.validate()
        self.net = nn.Sequential(nn.Linear(cfg.clip_feature_dim, cfg.hidden_dim), nn.GELU(), nn.Linear(cfg.hidden_dim, cfg.num_tokens * cfg.cross_attn_dim))
        self.norm = nn.LayerNorm(cfg.cross_attn_dim)
    def forward(self, clip_features): return self.norm(self.net(clip_features).unflatten(-1, (self.cfg.num_tokens, self.cfg.cross_attn_dim)))
    def num_parameters(self): return sum(p.numel() for p in self.parameters())


def _time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    a = t.float()[:, None] * freqs[None]
    return torch.cat([a.sin(), a.cos()], -1)


class _TimeResBlock(nn.Module):
    def __init__(self, cin, cout, tdim, groups=8, batch_norm=False):
        super().__init__()
        norm = (lambda c: nn.BatchNorm2d(c)) if batch_norm else (lambda c: nn.GroupNorm(min(groups, c), c))
        self.n1, self.c1, self.t, self.n2, self.c2 = norm(cin), nn.Conv2d(cin, cout, 3, padding=1), nn.Linear(tdim, cout), norm(cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else nn.Identity()
    def forward(self, x, temb):
        h = self.c1(F.silu(self.n1(x))) + self.t(F.silu(temb))[:, :, None, None]
        return self.c2(F.silu(self.n2(h))) + self.skip(x)


class LatentUpsampler(nn.Module):
    """Doubles the spatial size of a latent, conditioned on the diffusion time step: residual blocks, a learned 2x upsampling
    (nearest + convolution) and a residual connection from the bilinearly upsampled input, so that it starts as plain
    interpolation."""

    def __init__(self, channels: int = 4, timestep_dim: int = 128, base_dim: int = 64, use_batch_norm: bool = False):
        super().__init__()
        self.tdim = timestep_dim
        self.temb = nn.Sequential(nn.Linear(timestep_dim, timestep_dim * 2), nn.SiLU(), nn.Linear(timestep_dim * 2, timestep_dim))
        self.inp = nn.Conv2d(channels, base_dim, 3, padding=1)
        self.b1, self.b2 = _TimeResBlock(base_dim, base_dim, timestep_dim, batch_norm=use_batch_norm), _TimeResBlock(base_dim, base_dim, timestep_dim, batch_norm=use_batch_norm)
        self.up = nn.Conv2d(base_dim, base_dim, 3, padding=1)
        self.out = nn.Conv2d(base_dim, channels, 3, padding=1)
        nn.init.zeros_(self.out.weight); nn.init.zeros_(self.out.bias)

    def forward(self, latents, timestep):
        t = self.temb(_time_embedding(timestep, self.tdim))
        h = self.b1(self.inp(latents), t)
        h = self.b2(self.up(F.interpolate(h, scale_factor=2.0, mode="nearest")), t)
        return self.out(F.silu(h)) + F.interpolate(latents, scale_factor=2.0, mode="bilinear", align_corners=False)


class CrossViewAttention(nn.Module):
    """Attention across the views of one object: features ``[batch * views, C, H, W]`` are regrouped so that every spatial
    token attends to the tokens of all views of its sample.  The output projection starts at zero, so an untrained layer is
    the identity."""

    def __init__(self, num_heads: int = 8, channels: int = 320, dropout: float = 0.0):
        super().__init__()
        if channels % num_heads:
            raise ValueError("channels must be divisible by the number of heads")
        self.h, self.norm, self.qkv, self.proj, self.p = num_heads, nn.GroupNorm(min(32, channels), channels), nn.Linear(channels, 3 * channels), nn.Linear(channels, channels), dropout
        nn.init.zeros_(self.proj.weight); nn.init.zeros_(self.proj.bias)

    def forward(self, features, num_views: int):
        bv, c, hh, ww = features.shape
        if bv % num_views:
            raise ValueError(f"batch {bv} is not a multiple of the number of views {num_views}")
        b = bv // num_views
        tok = self.norm(features).flatten(2).transpose(1, 2).reshape(b, num_views * hh * ww, c)
        q, k, v = self.qkv(tok).reshape(b, -1, 3, self.h, c // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, dropout_p=self.p if self.training else 0.0)
        out = self.proj(a.transpose(1, 2).reshape(b, num_views * hh * ww, c))
        return features + out.reshape(bv, hh * ww, c).transpose(1, 2).reshape(bv, c, hh, ww)


@dataclass
class MultiviewUNetConfig:
    in_channels: int = 4
    num_heads: int = 4
    base_dim: int = 64
    timestep_dim: int = 128
    camera_embed_dim: int = 128
    use_cross_view_attention: bool = True


class MultiviewUNet(nn.Module):
    """Two-level denoiser for several views of one object: time and camera embeddings are added and drive every residual
    block; cross-view attention at the bottleneck and the lower decoder level ties the views together."""

    def __init__(self, cfg: MultiviewUNetConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or MultiviewUNetConfig(**kw)
        d, t = cfg.base_dim, cfg.timestep_dim
        self.temb = nn.Sequential(nn.Linear(t, t * 2), nn.SiLU(), nn.Linear(t * 2, t))
        self.cam, self.cam_proj = CameraEmbedding(cfg.camera_embed_dim, (64, 128)), nn.Linear(cfg.camera_embed_dim, t)
        self.inp = nn.Conv2d(cfg.in_channels, d, 3, padding=1)
        self.d1, self.d2 = _TimeResBlock(d, d, t), _TimeResBlock(d, 2 * d, t)
        self.mid = _TimeResBlock(2 * d, 2 * d, t)
        self.u2, self.u1 = _TimeResBlock(4 * d, d, t), _TimeResBlock(2 * d, d, t)
        self.attn_mid = CrossViewAttention(cfg.num_heads, 2 * d) if cfg.use_cross_view_attention else None
        self.attn_up = CrossViewAttention(cfg.num_heads, d) if cfg.use_cross_view_attention else None
        self.out = nn.Sequential(nn.GroupNorm(min(8, d), d), nn.SiLU(), nn.Conv2d(d, cfg.in_channels, 3, padding=1))

    def forward(self, x, timestep, camera_params, num_views: int):
        e = self.temb(_time_embedding(timestep, self.cfg.timestep_dim)) + self.cam_proj(self.cam(camera_params))
        h0 = self.inp(x)
        h1 = self.d1(h0, e)
        h2 = self.d2(F.avg_pool2d(h1, 2), e)
        m = self.mid(h2, e)
        if self.attn_mid is not None:
            m = self.attn_mid(m, num_views)
        u = self.u2(torch.cat([m, h2], 1), e)
        if self.attn_up is not None:
            u = self.attn_up(u, num_views)
        u = self.u1(torch.cat([F.interpolate(u, scale_factor=2.0, mode="nearest"), h1], 1), e)
        return self.out(u)
