"""``rstorch.functional`` (``python/rstorch/functional.py:11-31``)."""
from torsh_b200.nn.functional import *  # noqa: F401,F403
from torsh_b200.nn.functional import (cross_entropy, gelu, layer_norm, linear, log_softmax, relu, sigmoid, silu, softmax,  # noqa: F401
                                      tanh)
