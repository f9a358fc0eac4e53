"""Neural-network layers, containers, initialisers and the functional API."""
from . import functional, init, losses
from .layers import *  # noqa: F401,F403
from .layers import _ADOPTED
from .extra_layers import *  # noqa: F401,F403
from .blocks import *  # noqa: F401,F403
from .module import (DynamicGraph, FunctionModule, LazyModule, Module, ModuleDict, ModuleList, ModuleMixin, Parameter,
                     ParameterDict, ParameterList, Sequential)

F = functional
