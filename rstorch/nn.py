"""``rstorch.nn`` (``crates/torsh-python/src/nn/mod.rs:39-67``)."""
from torsh_b200.nn import *  # noqa: F401,F403
from torsh_b200.nn import (AdaptiveAvgPool2d, AdaptiveMaxPool2d, AlphaDropout, AvgPool2d, BatchNorm1d, BatchNorm2d,  # noqa: F401
                           BCELoss, Conv1d, Conv2d, CrossEntropyLoss, Dropout, Dropout2d, Dropout3d, LayerNorm, Linear,
                           MaxPool2d, Module, ModuleList, MSELoss, Parameter, ReLU, Sequential, Sigmoid, Tanh)
