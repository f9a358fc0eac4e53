"""Generative models: a convolutional VAE (reparameterisation, ELBO), a DCGAN-style generator / discriminator pair with
the standard and Wasserstein objectives, and a denoising-diffusion model (time-conditioned UNet, linear / cosine noise
schedules, training loss, ancestral and DDIM sampling). Reference: crates/torsh-models/src/generative.rs (VAE, GAN,
DiffusionUNet) and src/diffusion/.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn


# ---- VAE ---------------------------------------------------------------------------------------------------------
@dataclass
class VAEConfig:
    in_channels: int = 3
    image_size: int = 32
    latent_dim: int = 32
    widths: tuple = (32, 64)
    beta: float = 1.0


class VAEEncoder(nn.Module):
    def __init__(self, c: VAEConfig):
        super().__init__()
        layers, cin = [], c.in_channels
        for w in c.widths:
            layers += [nn.Conv2d(cin, w, 4, 2, 1), nn.ReLU(inplace=True)]
            cin = w
        self.conv = nn.Sequential(*layers)
        self.side = c.image_size // 2 ** len(c.widths)
        self.mu, self.logvar = nn.Linear(cin * self.side ** 2, c.latent_dim), nn.Linear(cin * self.side ** 2, c.latent_dim)

    def forward(self, x):
        h = self.conv(x).flatten(1)
        return self.mu(h), self.logvar(h)


class VAEDecoder(nn.Module):
    def __init__(self, c: VAEConfig):
        super().__init__()
        self.side, self.c0 = c.image_size // 2 ** len(c.widths), c.widths[-1]
        self.fc = nn.Linear(c.latent_dim, self.c0 * self.side ** 2)
        layers, cin = [], self.c0
        for w in list(c.widths[-2::-1]) + [c.in_channels]:
            layers += [nn.ConvTranspose2d(cin, w, 4, 2, 1), nn.ReLU(inplace=True)]
            cin = w
        self.deconv = nn.Sequential(*layers[:-1])

    def forward(self, z):
        return torch.sigmoid(self.deconv(self.fc(z).reshape(-1, self.c0, self.side, self.side)))


class VAE(nn.Module):
    def __init__(self, cfg: VAEConfig | None = None):
        super().__init__()
        self.cfg = cfg or VAEConfig()
        self.encoder, self.decoder = VAEEncoder(self.cfg), VAEDecoder(self.cfg)

    def reparameterize(self, mu, logvar):
        return mu + torch.randn_like(mu) * torch.exp(0.5 * logvar) if self.training else mu

    def forward(self, x):
        mu, logvar = self.encoder(x)
        return self.decoder(self.reparameterize(mu, logvar)), mu, logvar

    def loss(self, x) -> dict:
        recon, mu, logvar = self(x)
        rec = nn.functional.mse_loss(recon, x, reduction="sum") / x.shape[0]
        kl = -0.5 * torch.sum(1 + logvar - mu.pow(2) - logvar.exp()) / x.shape[0]
        return {"reconstruction": rec, "kl": kl, "total": rec + self.cfg.beta * kl}

    @torch.no_grad()
    def sample(self, n: int, device="cpu"):
        return self.decoder(torch.randn(n, self.cfg.latent_dim, device=device))


# ---- GAN ---------------------------------------------------------------------------------------------------------
@dataclass
class GANConfig:
    latent_dim: int = 64
    channels: int = 3
    image_size: int = 32
    width: int = 64


class GANGenerator(nn.Module):
    def __init__(self, c: GANConfig):
        super().__init__()
        ups = int(math.log2(c.image_size)) - 2
        w = c.width * 2 ** (ups - 1)
        layers = [nn.ConvTranspose2d(c.latent_dim, w, 4, 1, 0, bias=False), nn.BatchNorm2d(w), nn.ReLU(inplace=True)]
        for _ in range(ups - 1):
            layers += [nn.ConvTranspose2d(w, w // 2, 4, 2, 1, bias=False), nn.BatchNorm2d(w // 2), nn.ReLU(inplace=True)]
            w //= 2
        layers += [nn.ConvTranspose2d(w, c.channels, 4, 2, 1), nn.Tanh()]
        self.net = nn.Sequential(*layers)

    def forward(self, z):
        return self.net(z.reshape(z.shape[0], -1, 1, 1))


class GANDiscriminator(nn.Module):
    def __init__(self, c: GANConfig):
        super().__init__()
        downs = int(math.log2(c.image_size)) - 2
        layers, cin, w = [], c.channels, c.width
        for i in range(downs):
            layers += [nn.Conv2d(cin, w, 4, 2, 1, bias=False)] + ([nn.BatchNorm2d(w)] if i else []) + [nn.LeakyReLU(0.2, inplace=True)]
            cin, w = w, w * 2
        layers += [nn.Conv2d(cin, 1, 4, 1, 0)]
        self.net = nn.Sequential(*layers)

    def forward(self, x):
        return self.net(x).reshape(-1)


class GAN(nn.Module):
    def __init__(self, cfg: GANConfig | None = None):
        super().__init__()
        self.cfg = cfg or GANConfig()
        self.generator, self.discriminator = GANGenerator(self.cfg), GANDiscriminator(self.cfg)

    def generate(self, n: int, device="cpu"):
        return self.generator(torch.randn(n, self.cfg.latent_dim, device=device))

    def discriminator_loss(self, real, fake, wasserstein: bool = False):
        dr, df = self.discriminator(real), self.discriminator(fake.detach())
        if wasserstein:
            return df.mean() - dr.mean()
        bce = nn.functional.binary_cross_entropy_with_logits
        return bce(dr, torch.ones_like(dr)) + bce(df, torch.zeros_like(df))

    def generator_loss(self, fake, wasserstein: bool = False):
        df = self.discriminator(fake)
        return -df.mean() if wasserstein else nn.functional.binary_cross_entropy_with_logits(df, torch.ones_like(df))

    def gradient_penalty(self, real, fake, weight: float = 10.0):
        from ..nn.losses import gradient_penalty_loss
        eps = torch.rand(real.shape[0], 1, 1, 1, device=real.device)
        x = (eps * real + (1 - eps) * fake.detach()).requires_grad_(True)
        g, = torch.autograd.grad(self.discriminator(x).sum(), x, create_graph=True)
        return gradient_penalty_loss(g, weight)


# ---- diffusion ---------------------------------------------------------------------------------------------------
@dataclass
class DiffusionConfig:
    channels: int = 3
    image_size: int = 32
    width: int = 32
    timesteps: int = 1000
    schedule: str = "linear"          # or "cosine"
    beta_start: float = 1e-4
    beta_end: float = 0.02


def timestep_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.sin(args), torch.cos(args)], -1)


class _ResBlock(nn.Module):
    def __init__(self, cin, cout, tdim):
        super().__init__()
        self.n1, self.c1 = nn.GroupNorm(min(8, cin), cin), nn.Conv2d(cin, cout, 3, padding=1)
        self.t = nn.Linear(tdim, cout)
        self.n2, self.c2 = nn.GroupNorm(min(8, cout), cout), nn.Conv2d(cout, cout, 3, padding=1)
        self.skip = nn.Conv2d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x, temb):
        h = self.c1(nn.functional.silu(self.n1(x))) + self.t(nn.functional.silu(temb))[:, :, None, None]
        return self.c2(nn.functional.silu(self.n2(h))) + self.skip(x)


class DiffusionUNet(nn.Module):
    """Two-level UNet that predicts the noise added at step t."""

    def __init__(self, cfg: DiffusionConfig | None = None):
        super().__init__()
        self.cfg = cfg or DiffusionConfig()
        c, w = self.cfg, self.cfg.width
        self.tdim = w * 4
        self.temb = nn.Sequential(nn.Linear(w, self.tdim), nn.SiLU(), nn.Linear(self.tdim, self.tdim))
        self.inp = nn.Conv2d(c.channels, w, 3, padding=1)
        self.d1, self.down = _ResBlock(w, w, self.tdim), nn.Conv2d(w, w, 3, 2, 1)
        self.d2 = _ResBlock(w, 2 * w, self.tdim)
        self.mid = _ResBlock(2 * w, 2 * w, self.tdim)
        self.up = nn.ConvTranspose2d(2 * w, w, 4, 2, 1)
        self.u1 = _ResBlock(2 * w, w, self.tdim)
        self.out = nn.Sequential(nn.GroupNorm(min(8, w), w), nn.SiLU(), nn.Conv2d(w, c.channels, 3, padding=1))

    def forward(self, x, t):
        temb = self.temb(timestep_embedding(t, self.cfg.width))
        h1 = self.d1(self.inp(x), temb)
        h2 = self.mid(self.d2(self.down(h1), temb), temb)
        return self.out(self.u1(torch.cat([self.up(h2), h1], 1), temb))


class GaussianDiffusion:
    """Forward noising q(x_t | x_0), the epsilon-prediction training loss, and samplers."""

    def __init__(self, cfg: DiffusionConfig):
        T = cfg.timesteps
        if cfg.schedule == "cosine":
            s = 0.008
            f = torch.cos((torch.arange(T + 1) / T + s) / (1 + s) * math.pi / 2) ** 2
            betas = (1 - f[1:] / f[:-1]).clamp(max=0.999)
        else:
            betas = torch.linspace(cfg.beta_start, cfg.beta_end, T)
        self.betas, self.T = betas, T
        self.alphas_bar = torch.cumprod(1 - betas, 0)

    def q_sample(self, x0, t, noise):
        ab = self.alphas_bar.to(x0.device)[t][:, None, None, None]
        return ab.sqrt() * x0 + (1 - ab).sqrt() * noise

    def loss(self, model, x0, gen: torch.Generator | None = None):
        t = torch.randint(0, self.T, (x0.shape[0],), generator=gen).to(x0.device)
        noise = torch.randn(x0.shape, generator=gen).to(x0)
        return nn.functional.mse_loss(model(self.q_sample(x0, t, noise), t), noise)

    @torch.no_grad()
    def sample(self, model, shape, steps: int | None = None, eta: float = 1.0, device="cpu", gen: torch.Generator | None = None):
        """``steps`` None: ancestral sampling over all T steps; otherwise DDIM over ``steps`` evenly spaced steps
        (``eta`` = 0 deterministic)."""
        x = torch.randn(shape, generator=gen).to(device)
        ts = list(range(self.T - 1, -1, -1)) if steps is None else torch.linspace(self.T - 1, 0, steps).long().tolist()
        ab_all = self.alphas_bar.to(device)
        for i, t in enumerate(ts):
            tt = torch.full((shape[0],), t, device=device, dtype=torch.long)
            eps = model(x, tt)
            ab = ab_all[t]
            ab_prev = ab_all[ts[i + 1]] if i + 1 < len(ts) else torch.tensor(1.0, device=device)
            x0 = (x - (1 - ab).sqrt() * eps) / ab.sqrt()
            sigma = eta * ((1 - ab_prev) / (1 - ab) * (1 - ab / ab_prev)).clamp(min=0).sqrt()
            x = ab_prev.sqrt() * x0 + (1 - ab_prev - sigma ** 2).clamp(min=0).sqrt() * eps
            if i + 1 < len(ts):
                x = x + sigma * torch.randn(shape, generator=gen).to(device)
        return x
