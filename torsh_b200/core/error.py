"""Error taxonomy.

``TorshError`` mirrors ``crates/torsh-core/src/error/general_errors.rs:9-118``;
``TorshDistributedError`` mirrors ``crates/torsh-distributed/src/lib.rs:24-97`` including
``is_retryable`` / ``recovery_suggestions`` (``:223-292``).
"""
from __future__ import annotations


class TorshError(RuntimeError):
    """Base error with a ``kind`` tag."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind, self.message = kind, message

    @classmethod
    def shape_mismatch(cls, expected, got, context: str = ""):
        where = f" ({context})" if context else ""
        return cls("ShapeMismatch", f"expected {tuple(expected)}, got {tuple(got)}{where}")

    @classmethod
    def invalid_argument(cls, msg):
        return cls("InvalidArgument", msg)

    @classmethod
    def unsupported(cls, msg):
        return cls("UnsupportedOperation", msg)

    @classmethod
    def device_error(cls, msg):
        return cls("DeviceError", msg)

    @classmethod
    def io_error(cls, msg):
        return cls("IoError", msg)

    @classmethod
    def serialization(cls, msg):
        return cls("SerializationError", msg)

    @classmethod
    def index_out_of_bounds(cls, index, size):
        return cls("IndexOutOfBounds", f"index {index} out of bounds for size {size}")

    @classmethod
    def not_implemented(cls, msg):
        return cls("NotImplemented", msg)


_RETRYABLE = {"CommunicationError", "OperationTimeout", "BackendError", "IoError"}
_SUGGESTIONS = {
    "BackendNotInitialized": ["call init_process_group() before using collectives"],
    "CommunicationError": ["check network connectivity between ranks", "retry the operation"],
    "OperationTimeout": ["increase the timeout", "check for a straggling or failed rank"],
    "ProcessFailure": ["restart the failed rank", "resume from the latest checkpoint"],
    "RankOutOfBounds": ["use a rank in [0, world_size)"],
    "TensorShapeMismatch": ["make tensor shapes identical on every rank"],
    "MemoryAllocationFailed": ["reduce the batch size", "enable sharding or CPU offload"],
    "CheckpointError": ["verify the checkpoint directory and free disk space"],
}


class TorshDistributedError(TorshError):
    KINDS = ("BackendNotInitialized", "InvalidArgument", "CommunicationError", "BackendError", "RankOutOfBounds",
             "FeatureNotAvailable", "ProcessGroupNotFound", "TensorShapeMismatch", "OperationTimeout", "ProcessFailure",
             "MemoryAllocationFailed", "SerializationError", "IoError", "InternalError", "ConfigurationError",
             "CheckpointError")

    def __init__(self, kind: str, message: str):
        if kind not in self.KINDS:
            raise ValueError(f"unknown distributed error kind {kind}")
        super().__init__(kind, message)

    def is_retryable(self) -> bool:
        return self.kind in _RETRYABLE

    def recovery_suggestions(self) -> list[str]:
        return list(_SUGGESTIONS.get(self.kind, ["inspect the logs of every rank"]))


def _mk(kind):
    def f(cls, msg):
        return cls(kind, msg)
    return classmethod(f)


for _k in TorshDistributedError.KINDS:
    _name = "".join("_" + c.lower() if c.isupper() else c for c in _k).lstrip("_")
    setattr(TorshDistributedError, _name, _mk(_k))
