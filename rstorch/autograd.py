"""``rstorch.autograd``: no_grad, enable_grad, set_grad_enabled, Function, grad, backward, is_grad_enabled, detect_anomaly."""
from torsh_b200.autograd import *  # noqa: F401,F403
from torsh_b200.autograd import (Function, backward, detect_anomaly, enable_grad, grad, is_grad_enabled, no_grad,  # noqa: F401
                                 set_grad_enabled)
