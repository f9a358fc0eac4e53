"""``rstorch.optim`` (``crates/torsh-python/src/optim/mod.rs:29-36``)."""
import torch as _torch

from torsh_b200.optim import *  # noqa: F401,F403
from torsh_b200.optim import SGD, Adagrad, Adam, AdamW, RMSprop, lr_scheduler  # noqa: F401

Optimizer = _torch.optim.Optimizer
