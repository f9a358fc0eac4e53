"""Model summary table (``crates/torsh-nn/src/summary``)."""
from __future__ import annotations

import torch


def summarize(model: torch.nn.Module, max_depth: int = 3) -> str:
    rows = []
    for name, m in model.named_modules():
        depth = name.count(".") + (1 if name else 0)
        if depth > max_depth:
            continue
        own = sum(p.numel() for p in m.parameters(recurse=False))
        total = sum(p.numel() for p in m.parameters())
        rows.append((name or "(root)", type(m).__name__, own, total))
    w = max(len(r[0]) for r in rows)
    lines = [f"{'module'.ljust(w)}  {'type':<28} {'own params':>12} {'total params':>14}", "-" * (w + 60)]
    lines += [f"{n.ljust(w)}  {t:<28} {o:>12,} {tt:>14,}" for n, t, o, tt in rows]
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    lines.append(f"trainable parameters: {trainable:,}")
    return "\n".join(lines)
