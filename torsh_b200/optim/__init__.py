"""Optimizers, LR schedulers and mixed-precision helpers."""
from .flat import FlatAdamW, FlatParameters
from .fused import LAMB, SGD, Adam, AdamW

__all__ = ["AdamW", "Adam", "SGD", "LAMB", "FlatParameters", "FlatAdamW"]
