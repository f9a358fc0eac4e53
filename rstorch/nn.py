"""``rstorch.nn`` (``crates/torsh-python/src/nn/mod.rs:39-67``)."""
from torsh_b200.nn import *  # noqa: F401,F403
from torsh_b200.nn import (AdaptiveAvgPool2d, AdaptiveMaxPool2d, AlphaDropout, AvgPool2d, BatchNorm1d, BatchNorm2d,  # noqa: F401
                           BCELoss, Conv1d, Conv2d, CrossEntropyLoss, Dropout, Dropout2d, Dropout3d, LayerNorm, Linear,
                           MaxPool2d, Module, ModuleList, MSELoss, Parameter, ReLU, Sequential, Sigmoid, Tanh)
from torsh_b200.nn.functional import cross_entropy, log_softmax, mse_loss, relu, sigmoid, softmax, tanh  # noqa: E402,F401  (re-exported by the reference's ``rstorch.nn``)


def parameter(data, requires_grad=True):
    """``rstorch.nn.parameter(data)``: convenience constructor of the reference (``python/rstorch/nn.py:40``)."""
    return Parameter(data, requires_grad)
