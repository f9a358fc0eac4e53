"""``Shape`` with broadcasting rules (``crates/torsh-core/src/shape/core/mod.rs:20-27``)."""
from __future__ import annotations

import math
from typing import Iterable, Sequence

from .error import TorshError


class Shape:
    __slots__ = ("dims",)

    def __init__(self, dims: Iterable[int] = ()):
        self.dims = tuple(int(d) for d in dims)
        if any(d < 0 for d in self.dims):
            raise TorshError.invalid_argument(f"negative dimension in {self.dims}")

    def ndim(self) -> int:
        return len(self.dims)

    def numel(self) -> int:
        return math.prod(self.dims)

    def is_scalar(self) -> bool:
        return len(self.dims) == 0

    def strides(self) -> tuple[int, ...]:
        """Row-major contiguous strides in elements."""
        st, acc = [], 1
        for d in reversed(self.dims):
            st.append(acc)
            acc *= d
        return tuple(reversed(st))

    def size(self, dim: int) -> int:
        n = len(self.dims)
        if not -n <= dim < n:
            raise TorshError.index_out_of_bounds(dim, n)
        return self.dims[dim]

    def broadcast_with(self, other: "Shape | Sequence[int]") -> "Shape":
        o = other.dims if isinstance(other, Shape) else tuple(other)
        out = []
        for i in range(max(len(self.dims), len(o))):
            a = self.dims[-1 - i] if i < len(self.dims) else 1
            b = o[-1 - i] if i < len(o) else 1
            if a != b and a != 1 and b != 1:
                raise TorshError.shape_mismatch(self.dims, o, context="broadcast")
            out.append(max(a, b) if 0 not in (a, b) else 0)
        return Shape(reversed(out))

    def is_broadcastable_with(self, other) -> bool:
        try:
            self.broadcast_with(other)
            return True
        except TorshError:
            return False

    def __iter__(self):
        return iter(self.dims)

    def __len__(self):
        return len(self.dims)

    def __getitem__(self, i):
        return self.dims[i]

    def __eq__(self, other):
        return self.dims == (other.dims if isinstance(other, Shape) else tuple(other))

    def __hash__(self):
        return hash(self.dims)

    def __repr__(self):
        return f"Shape({list(self.dims)})"
