"""Low-precision floating-point formats of the Blackwell tensor cores, as encode / decode routines with their scaling
schemes: FP8 (E4M3 / E5M2) with per-tensor or delayed (amax-history) scaling, the OCP microscaling formats MXFP8 / MXFP6 /
MXFP4 (blocks of 32 elements sharing a power-of-two E8M0 scale) and NVFP4 (blocks of 16 FP4 E2M1 values with an FP8 E4M3
block scale under one fp32 tensor scale), packed two FP4 codes per byte; 2:4 structured sparsity (prune, compress to values
+ 2-bit indices, expand) as the sparse tensor-core layout wants it; and error reports against the fp32 source.

These are the storage formats behind the 4.5 / 9 PFLOP/s FP8 / FP4 rates of a B200; the arithmetic here is exact emulation
in PyTorch (CPU or GPU), usable for calibration, checkpoint conversion and accuracy studies. Reference:
crates/torsh-quantization/src/ (fp8 / low-bit schemes, calibration), crates/torsh-sparse/src/ (structured sparsity).
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass

import torch

FP8_MAX = {"e4m3": 448.0, "e5m2": 57344.0}
_FP8_DTYPE = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
# the eight non-negative magnitudes of FP4 E2M1
FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
FP6_MAX = {"e2m3": 7.5, "e3m2": 28.0}


# ---- FP8 -------------------------------------------------------------------------------------------------------------
def fp8_quantize(x: torch.Tensor, fmt: str = "e4m3", scale: torch.Tensor | float | None = None):
    """Returns (fp8 tensor, scale) with ``x ≈ fp8.float() * scale``. Without ``scale`` the tensor's absolute maximum is
    mapped to the format's largest finite value; values are saturated, never turned into NaN / Inf."""
    mx = FP8_MAX[fmt]
    if scale is None:
        scale = x.detach().abs().amax().clamp(min=1e-12).float() / mx
    scale = torch.as_tensor(scale, dtype=torch.float32, device=x.device)
    y = (x.float() / scale).clamp(-mx, mx)
    return y.to(_FP8_DTYPE[fmt]), scale


def fp8_dequantize(q: torch.Tensor, scale, dtype=torch.float32) -> torch.Tensor:
    return (q.float() * scale).to(dtype)


class DelayedScaling:
    """Scale from the maximum of the last ``history`` absolute maxima (the recipe of FP8 training: the scale used at step t
    comes from steps < t, so no extra pass over the tensor is needed before the cast)."""

    def __init__(self, fmt: str = "e4m3", history: int = 16, margin: int = 0):
        self.fmt, self.hist, self.margin = fmt, deque(maxlen=history), margin
        self.scale = torch.tensor(1.0)

    def quantize(self, x: torch.Tensor):
        q, _ = fp8_quantize(x, self.fmt, self.scale.to(x.device))
        self.hist.append(float(x.detach().abs().amax()))
        amax = max(self.hist)
        self.scale = torch.tensor(max(amax, 1e-12) / FP8_MAX[self.fmt] * 2.0 ** self.margin)
        return q, self.scale if len(self.hist) > 1 else self.scale


# ---- element formats on a grid -----------------------------------------------------------------------------------------
def _round_to_grid(mag: torch.Tensor, grid: torch.Tensor) -> torch.Tensor:
    """Index of the nearest grid value (ties to the even index, as round-to-nearest-even on the code)."""
    d = (mag[..., None] - grid.to(mag)).abs()
    idx = d.argmin(-1)
    # argmin returns the lower index of a tie, so a tie is always between idx and idx + 1: take the even code of the two
    hi = (idx + 1).clamp(max=grid.numel() - 1)
    tie = (d.gather(-1, hi[..., None])[..., 0] == d.gather(-1, idx[..., None])[..., 0]) & (hi != idx)
    return torch.where(tie & (hi % 2 == 0), hi, idx)


def fp4_encode(x: torch.Tensor) -> torch.Tensor:
    """FP4 E2M1 codes (uint8 in 0..15: sign bit 3, magnitude index 0..7) of values already divided by their scale."""
    idx = _round_to_grid(x.abs().clamp(max=6.0), FP4_VALUES)
    return (idx + 8 * (x < 0)).to(torch.uint8)


def fp4_decode(codes: torch.Tensor) -> torch.Tensor:
    mag = FP4_VALUES.to(codes.device)[(codes & 7).long()]
    return torch.where((codes & 8) > 0, -mag, mag)


def pack_fp4(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte along the last dimension: element 2i in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    return torch.stack([packed & 0xF, packed >> 4], -1).flatten(-2)


def _fp6_grid(fmt: str) -> torch.Tensor:
    e, m = (2, 3) if fmt == "e2m3" else (3, 2)
    bias = 1 if fmt == "e2m3" else 3
    vals = []
    for ee in range(2 ** e):
        for mm in range(2 ** m):
            vals.append((mm / 2 ** m) * 2.0 ** (1 - bias) if ee == 0 else (1 + mm / 2 ** m) * 2.0 ** (ee - bias))
    return torch.tensor(sorted(set(vals)))


# ---- microscaling (MX) formats ---------------------------------------------------------------------------------------------
@dataclass
class MXTensor:
    fmt: str                  # "mxfp8_e4m3", "mxfp8_e5m2", "mxfp6_e2m3", "mxfp6_e3m2", "mxfp4"
    data: torch.Tensor        # fp8 tensor, fp6 values (float, on the grid) or packed fp4 bytes
    scale_exp: torch.Tensor   # int8 exponents of the E8M0 block scales: scale = 2 ** exp, one per block of 32
    shape: tuple


def _emax(fmt: str) -> int:
    return {"mxfp8_e4m3": 8, "mxfp8_e5m2": 15, "mxfp6_e2m3": 2, "mxfp6_e3m2": 4, "mxfp4": 2}[fmt]


def mx_quantize(x: torch.Tensor, fmt: str = "mxfp8_e4m3", block: int = 32) -> MXTensor:
    """Blocks of ``block`` consecutive elements of the last dimension share the scale 2 ** (floor(log2(amax)) - emax_elem)."""
    if x.shape[-1] % block:
        raise ValueError(f"last dimension ({x.shape[-1]}) must be a multiple of the block size {block}")
    xb = x.float().reshape(*x.shape[:-1], -1, block)
    amax = xb.abs().amax(-1, keepdim=True)
    exp = torch.floor(torch.log2(amax.clamp(min=2.0 ** -126))) - _emax(fmt)
    exp = exp.clamp(-127, 127)
    y = xb / torch.exp2(exp)
    if fmt.startswith("mxfp8"):
        f = fmt[-4:]
        data = y.clamp(-FP8_MAX[f], FP8_MAX[f]).to(_FP8_DTYPE[f]).reshape(x.shape)
    elif fmt.startswith("mxfp6"):
        f = fmt[-4:]
        grid = _fp6_grid(f)
        mag = grid.to(y.device)[_round_to_grid(y.abs().clamp(max=FP6_MAX[f]), grid)]
        data = torch.where(y < 0, -mag, mag).reshape(x.shape)
    else:
        data = pack_fp4(fp4_encode(y).reshape(x.shape))
    return MXTensor(fmt, data, exp.squeeze(-1).to(torch.int8), tuple(x.shape))


def mx_dequantize(t: MXTensor, dtype=torch.float32, block: int = 32) -> torch.Tensor:
    if t.fmt == "mxfp4":
        vals = fp4_decode(unpack_fp4(t.data))
    else:
        vals = t.data.float()
    vb = vals.reshape(*t.shape[:-1], -1, block)
    return (vb * torch.exp2(t.scale_exp.float())[..., None]).reshape(t.shape).to(dtype)


# ---- NVFP4 ---------------------------------------------------------------------------------------------------------------
@dataclass
class NVFP4Tensor:
    packed: torch.Tensor          # uint8, two E2M1 codes per byte
    block_scale: torch.Tensor     # float8_e4m3fn, one per 16 elements
    tensor_scale: torch.Tensor    # fp32 scalar
    shape: tuple


def nvfp4_quantize(x: torch.Tensor, block: int = 16) -> NVFP4Tensor:
    """Two-level scaling: tensor_scale maps the largest block scale into E4M3's range; each block's E4M3 scale maps its
    absolute maximum to 6 (the largest FP4 magnitude)."""
    if x.shape[-1] % block:
        raise ValueError(f"last dimension ({x.shape[-1]}) must be a multiple of the block size {block}")
    xb = x.float().reshape(*x.shape[:-1], -1, block)
    amax = xb.abs().amax(-1, keepdim=True)
    tscale = (amax.amax().clamp(min=1e-12) / (6.0 * FP8_MAX["e4m3"])).float()
    bs = (amax / 6.0 / tscale).clamp(max=FP8_MAX["e4m3"]).to(torch.float8_e4m3fn)
    eff = (bs.float() * tscale).clamp(min=1e-30)
    codes = fp4_encode(xb / eff)
    return NVFP4Tensor(pack_fp4(codes.reshape(x.shape)), bs.squeeze(-1), tscale, tuple(x.shape))


def nvfp4_dequantize(t: NVFP4Tensor, dtype=torch.float32, block: int = 16) -> torch.Tensor:
    vals = fp4_decode(unpack_fp4(t.packed)).reshape(*t.shape[:-1], -1, block)
    return (vals * (t.block_scale.float() * t.tensor_scale)[..., None]).reshape(t.shape).to(dtype)


def bits_per_element(fmt: str) -> float:
    """Storage cost including the scales."""
    return {"fp8": 8.0, "mxfp8_e4m3": 8 + 8 / 32, "mxfp8_e5m2": 8 + 8 / 32, "mxfp6_e2m3": 6 + 8 / 32, "mxfp6_e3m2": 6 + 8 / 32,
            "mxfp4": 4 + 8 / 32, "nvfp4": 4 + 8 / 16, "int4_g128": 4 + 32 / 128}[fmt]


# ---- 2:4 structured sparsity -------------------------------------------------------------------------------------------------
def prune_2_4(w: torch.Tensor) -> torch.Tensor:
    """Keeps the two largest magnitudes of every group of four consecutive elements of the last dimension."""
    if w.shape[-1] % 4:
        raise ValueError("the last dimension must be a multiple of 4")
    g = w.reshape(*w.shape[:-1], -1, 4)
    keep = g.abs().topk(2, dim=-1).indices
    mask = torch.zeros_like(g, dtype=torch.bool).scatter_(-1, keep, True)
    return (g * mask).reshape(w.shape)


def compress_2_4(w: torch.Tensor):
    """(values [..., K/2], metadata uint8 [..., K/4]) of a 2:4-sparse tensor: per group the two kept values in index order
    and their positions packed as ``pos0 | pos1 << 2``. Groups with fewer than two non-zeros are padded with zeros at the
    lowest free positions."""
    g = w.reshape(*w.shape[:-1], -1, 4)
    nz = g != 0
    if (nz.sum(-1) > 2).any():
        raise ValueError("tensor is not 2:4 sparse: prune it first")
    # rank positions: non-zeros first (in index order), then zeros (in index order)
    order = torch.argsort((~nz).to(torch.int8) * 4 + torch.arange(4, device=w.device), dim=-1)[..., :2]
    order = order.sort(-1).values
    vals = g.gather(-1, order)
    meta = (order[..., 0] | (order[..., 1] << 2)).to(torch.uint8)
    return vals.reshape(*w.shape[:-1], -1), meta


def expand_2_4(vals: torch.Tensor, meta: torch.Tensor) -> torch.Tensor:
    v = vals.reshape(*vals.shape[:-1], -1, 2)
    pos = torch.stack([meta & 3, (meta >> 2) & 3], -1).long()
    out = torch.zeros(*v.shape[:-1], 4, dtype=vals.dtype, device=vals.device)
    out.scatter_(-1, pos, v)
    return out.reshape(*vals.shape[:-1], -1)


# ---- reports -------------------------------------------------------------------------------------------------------------------
def quantization_error(x: torch.Tensor, x_hat: torch.Tensor) -> dict:
    x, x_hat = x.double(), x_hat.double()
    err = x - x_hat
    sig, noise = float((x ** 2).mean()), float((err ** 2).mean())
    return {"sqnr_db": 10 * math.log10(sig / noise) if noise > 0 else float("inf"), "max_abs": float(err.abs().max()),
            "rel_fro": float(err.norm() / x.norm().clamp(min=1e-30)), "cosine": float(torch.nn.functional.cosine_similarity(x.flatten(), x_hat.flatten(), dim=0))}


def compare_formats(x: torch.Tensor) -> dict:
    """SQNR and storage cost of every format on ``x`` (last dimension a multiple of 32)."""
    out = {}
    q, s = fp8_quantize(x, "e4m3")
    out["fp8"] = {**quantization_error(x, fp8_dequantize(q, s)), "bits": bits_per_element("fp8")}
    for fmt in ("mxfp8_e4m3", "mxfp6_e2m3", "mxfp6_e3m2", "mxfp4"):
        out[fmt] = {**quantization_error(x, mx_dequantize(mx_quantize(x, fmt))), "bits": bits_per_element(fmt)}
    out["nvfp4"] = {**quantization_error(x, nvfp4_dequantize(nvfp4_quantize(x))), "bits": bits_per_element("nvfp4")}
    return out
