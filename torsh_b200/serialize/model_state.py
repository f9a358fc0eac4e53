"""Model state containers with the reference's schemas.

``ModelState{parameters: {name: SerializableTensor{shape, dtype:"f32", data: [f32], requires_grad}}, config:
{name: bool|i64|f64|string|array}, metadata{architecture, version "1.0.0", created_at RFC3339, framework_version,
tags}}`` as JSON (pretty), bincode binary, or safetensors with ``__metadata__`` keys ``torsh_metadata`` /
``torsh_config`` (``crates/torsh-nn/src/serialization.rs:26-72,145-270``); the loader accepts F32 only (``:232-238``).
"""
from __future__ import annotations

import datetime
import json
import struct
from pathlib import Path

import numpy as np
import torch

from ..core.error import TorshError
from . import bincode

FRAMEWORK_VERSION = "0.1.3"


def _meta(architecture: str, tags=None) -> dict:
    return {"architecture": architecture, "version": "1.0.0",
            "created_at": datetime.datetime.now(datetime.timezone.utc).isoformat().replace("+00:00", "Z"),
            "framework_version": FRAMEWORK_VERSION, "tags": list(tags or [])}


def model_state(module: torch.nn.Module, config: dict | None = None, architecture: str | None = None, tags=None) -> dict:
    params = {}
    for name, p in module.named_parameters():
        t = p.detach().float().cpu()
        params[name] = {"shape": list(t.shape), "dtype": "f32", "data": t.reshape(-1).tolist(),
                        "requires_grad": bool(p.requires_grad)}
    return {"parameters": params, "config": dict(config or {}), "metadata": _meta(architecture or type(module).__name__, tags)}


def load_model_state(module: torch.nn.Module, state: dict, strict: bool = True) -> None:
    sd = {}
    for name, st in state["parameters"].items():
        if st.get("dtype", "f32") != "f32":
            raise TorshError.serialization(f"parameter {name}: only f32 model states are supported, got {st['dtype']}")
        sd[name] = torch.tensor(st["data"], dtype=torch.float32).reshape(st["shape"])
    if hasattr(module, "load_torsh_state_dict"):
        module.load_torsh_state_dict(sd, strict)
    else:
        module.load_state_dict(sd, strict=strict)


# ---- JSON ----------------------------------------------------------------------------------------------
def save_json(state: dict, path) -> None:
    Path(path).write_text(json.dumps(state, indent=2))


def load_json(path) -> dict:
    return json.loads(Path(path).read_text())


# ---- bincode binary ------------------------------------------------------------------------------------
def _w_value(w: bincode.Writer, v):
    """SerializableValue is an untagged enum in JSON; in bincode it carries a variant index:
    0 bool, 1 int (i64), 2 float (f64), 3 string, 4 array."""
    if isinstance(v, bool):
        w.varu(0); w.boolean(v)
    elif isinstance(v, int):
        w.varu(1); w.vari(v)
    elif isinstance(v, float):
        w.varu(2); w.f64(v)
    elif isinstance(v, str):
        w.varu(3); w.string(v)
    elif isinstance(v, (list, tuple)):
        w.varu(4); w.seq(list(v), lambda x: _w_value(w, x))
    else:
        raise TorshError.serialization(f"config value of type {type(v).__name__} is not serialisable")


def _r_value(r: bincode.Reader):
    tag = r.varu()
    if tag == 0: return r.boolean()
    if tag == 1: return r.vari()
    if tag == 2: return r.f64()
    if tag == 3: return r.string()
    if tag == 4: return r.seq(lambda: _r_value(r))
    raise TorshError.serialization(f"unknown config value tag {tag}")


def encode_binary(state: dict) -> bytes:
    w = bincode.Writer()

    def tensor(st):
        w.seq(st["shape"], w.varu)
        w.string(st["dtype"])
        data = np.asarray(st["data"], dtype="<f4")
        w.varu(data.size)
        w.raw(data.tobytes())
        w.boolean(st["requires_grad"])

    w.map(state["parameters"], w.string, tensor)
    w.map(state["config"], w.string, lambda v: _w_value(w, v))
    m = state["metadata"]
    w.string(m["architecture"]); w.string(m["version"]); w.string(m["created_at"]); w.string(m["framework_version"])
    w.seq(m["tags"], w.string)
    return w.bytes()


def decode_binary(buf: bytes) -> dict:
    r = bincode.Reader(buf)

    def tensor():
        shape = r.seq(r.varu)
        dtype = r.string()
        n = r.varu()
        data = np.frombuffer(r.raw(4 * n), dtype="<f4").tolist()
        return {"shape": shape, "dtype": dtype, "data": data, "requires_grad": r.boolean()}

    params = r.map(r.string, tensor)
    config = r.map(r.string, lambda: _r_value(r))
    meta = {"architecture": r.string(), "version": r.string(), "created_at": r.string(), "framework_version": r.string()}
    meta["tags"] = r.seq(r.string)
    return {"parameters": params, "config": config, "metadata": meta}


def save_binary(state: dict, path) -> None:
    Path(path).write_bytes(encode_binary(state))


def load_binary(path) -> dict:
    return decode_binary(Path(path).read_bytes())


# ---- safetensors (written and read without the safetensors package) -----------------------------------
def save_safetensors(state: dict, path) -> None:
    header, blobs, off = {}, [], 0
    for name in sorted(state["parameters"]):
        st = state["parameters"][name]
        raw = np.asarray(st["data"], dtype="<f4").tobytes()
        header[name] = {"dtype": "F32", "shape": st["shape"], "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    header["__metadata__"] = {"torsh_metadata": json.dumps(state["metadata"]), "torsh_config": json.dumps(state["config"])}
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_safetensors(path) -> dict:
    buf = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", buf[:8])
    header = json.loads(buf[8:8 + n])
    base = 8 + n
    md = header.pop("__metadata__", {})
    params = {}
    for name, h in header.items():
        if h["dtype"] != "F32":
            raise TorshError.serialization(f"tensor {name}: only F32 is supported, got {h['dtype']}")
        a, b = h["data_offsets"]
        params[name] = {"shape": h["shape"], "dtype": "f32", "requires_grad": True,
                        "data": np.frombuffer(buf[base + a:base + b], dtype="<f4").tolist()}
    return {"parameters": params, "config": json.loads(md.get("torsh_config", "{}")),
            "metadata": json.loads(md.get("torsh_metadata", "{}"))}
