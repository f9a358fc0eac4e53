"""``Module`` / ``Parameter`` / containers with ToRSh's API shape on top of ``torch.nn``.

The reference ``Module`` trait (``crates/torsh-nn/src/core/mod.rs:294-900``) exposes
``forward``, ``parameters()/named_parameters()`` as name→Parameter maps, ``train/eval/training``,
``to_device``, ``state_dict/load_state_dict(strict)`` (parameters only, strict lists missing and
unexpected keys, shape mismatch always errors: ``:414-478``), ``buffers``, ``children/modules``,
``zero_grad``, ``freeze/unfreeze``, hooks and ``num_parameters``. Here those live in a mixin over
``torch.nn.Module`` so every PyTorch facility (autograd, hooks, device moves) keeps working:
``parameters()`` stays PyTorch's iterator, the name→Parameter map is ``parameters_dict()``.
Parameter names are unique dotted paths (the reference's composite models collide on bare
``"weight"``/``"bias"`` keys: ``crates/torsh-models/src/nlp/gpt2.rs:447-452``).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, Iterable

import torch

from ..core.error import TorshError


class Parameter(torch.nn.Parameter):
    """Trainable tensor (``crates/torsh-nn/src/parameter/mod.rs:32-128``)."""

    def __new__(cls, data=None, requires_grad: bool = True):
        if data is None:
            data = torch.empty(0)
        return torch.Tensor._make_subclass(cls, data, requires_grad)

    def tensor(self) -> torch.Tensor:
        return self.data

    def numel_bytes(self) -> int:
        return self.numel() * self.element_size()


class ModuleMixin:
    """ToRSh-shaped conveniences shared by every layer."""

    # ---- parameter maps -------------------------------------------------
    def parameters_dict(self) -> "OrderedDict[str, torch.nn.Parameter]":
        return OrderedDict(self.named_parameters())

    def buffers_dict(self) -> "OrderedDict[str, torch.Tensor]":
        return OrderedDict(self.named_buffers())

    def num_parameters(self, trainable_only: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not trainable_only)

    # ---- modes / devices ------------------------------------------------
    def is_training(self) -> bool:
        return self.training

    def to_device(self, device):
        return self.to(torch.device(str(device)) if not isinstance(device, torch.device) else device)

    def freeze(self):
        for p in self.parameters():
            p.requires_grad_(False)
        return self

    def unfreeze(self):
        for p in self.parameters():
            p.requires_grad_(True)
        return self

    # ---- state dict with the reference's rules ---------------------------
    def torsh_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        """Parameters only, cloned (buffers such as BatchNorm running stats are not included)."""
        return OrderedDict((k, p.detach().clone()) for k, p in self.named_parameters())

    def load_torsh_state_dict(self, state: dict, strict: bool = True) -> None:
        own = self.parameters_dict()
        missing = [k for k in own if k not in state]
        unexpected = [k for k in state if k not in own]
        if strict and (missing or unexpected):
            raise TorshError.invalid_argument(
                f"load_state_dict(strict): missing keys {missing}, unexpected keys {unexpected}")
        with torch.no_grad():
            for k, p in own.items():
                if k in state:
                    src = state[k]
                    if tuple(src.shape) != tuple(p.shape):
                        raise TorshError.shape_mismatch(tuple(p.shape), tuple(src.shape), context=k)
                    p.copy_(src.to(device=p.device, dtype=p.dtype))

    # ---- hooks (PreForward / PostForward / PreBackward / PostBackward) ----
    def register_hook(self, kind: str, fn: Callable):
        """``kind`` ∈ pre_forward, post_forward, pre_backward, post_backward
        (``crates/torsh-nn/src/hooks/mod.rs:18-117``)."""
        if kind == "pre_forward":
            return self.register_forward_pre_hook(fn)
        if kind == "post_forward":
            return self.register_forward_hook(fn)
        if kind == "pre_backward":
            return self.register_full_backward_pre_hook(fn)
        if kind == "post_backward":
            return self.register_full_backward_hook(fn)
        raise TorshError.invalid_argument(f"unknown hook kind {kind!r}")

    def summary(self) -> str:
        from .summary import summarize
        return summarize(self)


class Module(ModuleMixin, torch.nn.Module):
    """Base class of every layer and model."""


class Sequential(ModuleMixin, torch.nn.Sequential):
    pass


class ModuleList(ModuleMixin, torch.nn.ModuleList):
    pass


class ModuleDict(ModuleMixin, torch.nn.ModuleDict):
    pass


class ParameterList(ModuleMixin, torch.nn.ParameterList):
    pass


class ParameterDict(ModuleMixin, torch.nn.ParameterDict):
    pass


class FunctionModule(Module):
    """Wraps a plain function as a layer (``crates/torsh-nn/src/container/basic.rs``)."""

    def __init__(self, fn: Callable, name: str = "function"):
        super().__init__()
        self.fn, self.name = fn, name

    def forward(self, *args, **kwargs):
        return self.fn(*args, **kwargs)

    def extra_repr(self) -> str:
        return self.name


class DynamicGraph(Module):
    """Named nodes with explicit edges, evaluated in topological order
    (``crates/torsh-nn/src/container/dynamic_graph.rs``)."""

    def __init__(self):
        super().__init__()
        self.nodes = ModuleDict()
        self.edges: dict[str, list[str]] = {}
        self.output: str | None = None

    def add_node(self, name: str, module: torch.nn.Module, inputs: Iterable[str] = ("input",)):
        self.nodes[name] = module
        self.edges[name] = list(inputs)
        self.output = name
        return self

    def forward(self, x):
        values = {"input": x}
        pending = dict(self.edges)
        while pending:
            ready = [n for n, ins in pending.items() if all(i in values for i in ins)]
            if not ready:
                raise TorshError.invalid_argument("DynamicGraph has a cycle or a missing input")
            for n in ready:
                values[n] = self.nodes[n](*[values[i] for i in pending.pop(n)])
        return values[self.output]


class LazyModule(Module):
    """Builds its inner module from the first input's shape (``crates/torsh-nn/src/container/lazy.rs``)."""

    def __init__(self, factory: Callable[[torch.Size], torch.nn.Module]):
        super().__init__()
        self.factory = factory
        self.inner: torch.nn.Module | None = None

    def forward(self, x):
        if self.inner is None:
            self.inner = self.factory(x.shape).to(x.device)
        return self.inner(x)
