"""Serialization: TRSH tensor files, model state, training checkpoints."""
from .trsh import crc32, decode_trsh, encode_trsh, load_tensor, save_tensor

__all__ = ["crc32", "encode_trsh", "decode_trsh", "save_tensor", "load_tensor"]
from . import checkpoint, model_state  # noqa: E402,F401
from .checkpoint import CheckpointManager, DistributedCheckpointManager  # noqa: E402,F401
