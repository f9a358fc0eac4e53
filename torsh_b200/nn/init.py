"""Initialisers (``crates/torsh-nn/src/init.rs``): constant, xavier, kaiming, uniform, normal, lecun,
trunc_normal, orthogonal, sparse, dirac, siren, fixup, rezero, lsuv."""
from __future__ import annotations

import math

import torch
from torch.nn import init as _i

constant_, zeros_, ones_, uniform_, normal_ = _i.constant_, _i.zeros_, _i.ones_, _i.uniform_, _i.normal_
xavier_uniform_, xavier_normal_ = _i.xavier_uniform_, _i.xavier_normal_
kaiming_uniform_, kaiming_normal_ = _i.kaiming_uniform_, _i.kaiming_normal_
trunc_normal_, orthogonal_, sparse_, dirac_, eye_ = _i.trunc_normal_, _i.orthogonal_, _i.sparse_, _i.dirac_, _i.eye_
calculate_gain = _i.calculate_gain


def _fan_in(t: torch.Tensor) -> int:
    return _i._calculate_fan_in_and_fan_out(t)[0]


def lecun_normal_(t: torch.Tensor) -> torch.Tensor:
    return _i.normal_(t, 0.0, math.sqrt(1.0 / _fan_in(t)))


def lecun_uniform_(t: torch.Tensor) -> torch.Tensor:
    b = math.sqrt(3.0 / _fan_in(t))
    return _i.uniform_(t, -b, b)


def siren_(t: torch.Tensor, w0: float = 30.0, first_layer: bool = False) -> torch.Tensor:
    fan = _fan_in(t)
    b = 1.0 / fan if first_layer else math.sqrt(6.0 / fan) / w0
    return _i.uniform_(t, -b, b)


def fixup_(t: torch.Tensor, num_layers: int, depth_per_block: int = 2) -> torch.Tensor:
    _i.kaiming_normal_(t)
    with torch.no_grad():
        t.mul_(num_layers ** (-1.0 / (2 * depth_per_block - 2)) if depth_per_block > 1 else 1.0)
    return t


def rezero_(t: torch.Tensor) -> torch.Tensor:
    return _i.zeros_(t)


@torch.no_grad()
def lsuv_(module: torch.nn.Module, sample: torch.Tensor, tol: float = 0.1, max_iter: int = 10) -> None:
    """Layer-sequential unit-variance: orthogonal init then rescale each Linear/Conv so its output variance is 1."""
    layers = [m for m in module.modules() if hasattr(m, "weight") and getattr(m, "weight", None) is not None and m.weight.dim() >= 2]
    for m in layers:
        _i.orthogonal_(m.weight)
        for _ in range(max_iter):
            out = {}
            h = m.register_forward_hook(lambda mod, inp, o: out.__setitem__("o", o))
            module(sample)
            h.remove()
            var = out["o"].float().var().item()
            if abs(var - 1.0) < tol or var == 0.0:
                break
            m.weight.div_(math.sqrt(var))
