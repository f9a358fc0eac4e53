"""Arrow / Parquet, HDF5 and ONNX entry points of the tensor serializer
(``crates/torsh-tensor/src/serialize/{data_science,scientific,ml_formats}.rs``; feature-gated in the reference).
Arrow and Parquet use ``pyarrow``; HDF5 needs ``h5py`` and ONNX needs ``onnx`` — when a package is missing the function
raises ``FeatureNotAvailable`` with the package's name, as the reference does for a disabled feature."""
from __future__ import annotations

import json

import torch

from ..core.error import TorshError


def _need(mod: str):
    try:
        return __import__(mod)
    except ImportError as e:
        raise TorshError("FeatureNotAvailable", f"this format needs the '{mod}' package: {e}") from e


def _to_table(tensors: dict[str, torch.Tensor]):
    pa = _need("pyarrow")
    cols, meta = {}, {}
    for name, t in tensors.items():
        c = t.detach().cpu().contiguous()
        store = c.float() if c.dtype == torch.bfloat16 else c
        cols[name] = pa.array([store.reshape(-1).numpy()], type=pa.list_(pa.from_numpy_dtype(store.numpy().dtype)))
        meta[name] = {"shape": list(c.shape), "dtype": str(c.dtype).replace("torch.", "")}
    return pa.table(cols).replace_schema_metadata({"torsh": json.dumps(meta)})


def _from_table(table) -> dict[str, torch.Tensor]:
    meta = json.loads(table.schema.metadata[b"torsh"].decode())
    out = {}
    for name, m in meta.items():
        flat = torch.from_numpy(table.column(name)[0].values.to_numpy(zero_copy_only=False).copy())
        out[name] = flat.reshape(m["shape"]).to(getattr(torch, m["dtype"]))
    return out


def save_parquet(tensors: dict[str, torch.Tensor], path: str, compression: str = "zstd") -> None:
    """One row; one list column per tensor; shapes and dtypes in the schema metadata."""
    _need("pyarrow")
    import pyarrow.parquet as pq
    pq.write_table(_to_table(tensors), path, compression=compression)


def load_parquet(path: str) -> dict[str, torch.Tensor]:
    _need("pyarrow")
    import pyarrow.parquet as pq
    return _from_table(pq.read_table(path))


def save_arrow(tensors: dict[str, torch.Tensor], path: str) -> None:
    pa = _need("pyarrow")
    table = _to_table(tensors)
    with pa.OSFile(path, "wb") as f, pa.ipc.new_file(f, table.schema) as w:
        w.write_table(table)


def load_arrow(path: str) -> dict[str, torch.Tensor]:
    pa = _need("pyarrow")
    with pa.memory_map(path, "rb") as f:
        return _from_table(pa.ipc.open_file(f).read_all())


def save_hdf5(tensors: dict[str, torch.Tensor], path: str) -> None:
    h5 = _need("h5py")
    with h5.File(path, "w") as f:
        for name, t in tensors.items():
            c = t.detach().cpu()
            d = f.create_dataset(name, data=(c.float() if c.dtype == torch.bfloat16 else c).numpy())
            d.attrs["torsh_dtype"] = str(c.dtype).replace("torch.", "")


def load_hdf5(path: str) -> dict[str, torch.Tensor]:
    h5 = _need("h5py")
    with h5.File(path, "r") as f:
        return {k: torch.from_numpy(f[k][()]).to(getattr(torch, f[k].attrs.get("torsh_dtype", "float32"))) for k in f}


def export_onnx(module: torch.nn.Module, example_inputs, path: str, opset: int = 17) -> None:
    """ONNX export through ``torch.onnx`` (the reference's ONNX writer is a stub)."""
    _need("onnx")
    torch.onnx.export(module, example_inputs, path, opset_version=opset)
