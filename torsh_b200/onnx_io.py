"""ONNX export and import without the ``onnx`` package: the protobuf wire format is written and parsed directly.

``export_onnx(module, example_inputs, path)`` traces the module with ``torch.fx``, maps each node to ONNX operators
(opset 20) and writes a ``ModelProto`` with the parameters as initializers. ``load_onnx(path)`` parses such a file back
into an ``OnnxModel`` that evaluates the graph with PyTorch ops, which is both the importer for hub checkpoints in ONNX
form and the round-trip check of the exporter. Supported: Linear (Gemm), MatMul, Add / Sub / Mul / Div, ReLU, GELU, Tanh,
Sigmoid, SiLU, Softmax, LayerNorm, Conv2d, BatchNorm2d (inference), MaxPool2d, AvgPool2d, global average pooling,
Flatten, Reshape, Transpose, Embedding (Gather), Dropout (Identity), concatenation.
Reference: crates/torsh-fx/src/ (ONNX export, code generation), crates/torsh-hub/src/ (ONNX import).
"""
from __future__ import annotations

import operator
import struct

import torch
import torch.fx
from torch import nn

from .data.formats import _fields, _ld, _varint

FLOAT, INT64 = 1, 7


# ---- protobuf builders -----------------------------------------------------------------------------------------------
def _vi(field: int, value: int) -> bytes:
    return _varint(field << 3) + _varint(value & 0xFFFFFFFFFFFFFFFF)


def _s(field: int, text) -> bytes:
    return _ld(field, text.encode() if isinstance(text, str) else text)


def _tensor(name: str, t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.int64, torch.int32, torch.bool):
        dt, raw = INT64, t.to(torch.int64).numpy().tobytes()
    else:
        dt, raw = FLOAT, t.to(torch.float32).numpy().tobytes()
    return b"".join(_vi(1, d) for d in t.shape) + _vi(2, dt) + _s(8, name) + _ld(9, raw)


def _attr(name: str, value) -> bytes:
    out = _s(1, name)
    if isinstance(value, bool):
        value = int(value)
    if isinstance(value, int):
        return out + _vi(3, value) + _vi(20, 2)
    if isinstance(value, float):
        return out + _varint((2 << 3) | 5) + struct.pack("<f", value) + _vi(20, 1)
    if isinstance(value, str):
        return out + _s(4, value) + _vi(20, 3)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        return out + b"".join(_vi(8, v) for v in value) + _vi(20, 7)
    if isinstance(value, (list, tuple)):
        return out + b"".join(_varint((7 << 3) | 5) + struct.pack("<f", float(v)) for v in value) + _vi(20, 6)
    raise TypeError(f"unsupported attribute {name}={value!r}")


def _node(op: str, inputs, outputs, name: str = "", **attrs) -> bytes:
    return (b"".join(_s(1, i) for i in inputs) + b"".join(_s(2, o) for o in outputs) + _s(3, name) + _s(4, op)
            + b"".join(_ld(5, _attr(k, v)) for k, v in attrs.items()))


def _value_info(name: str, shape, elem=FLOAT) -> bytes:
    dims = b"".join(_ld(1, _vi(1, d) if isinstance(d, int) else _s(2, d)) for d in shape)
    return _s(1, name) + _ld(2, _ld(1, _vi(1, elem) + _ld(2, dims)))


# ---- export ----------------------------------------------------------------------------------------------------------
class _Exporter:
    def __init__(self, gm: torch.fx.GraphModule):
        self.gm, self.nodes, self.inits, self.names = gm, [], [], {}
        self._n = 0

    def tmp(self, hint="t") -> str:
        self._n += 1
        return f"{hint}_{self._n}"

    def const(self, t, hint="c") -> str:
        name = self.tmp(hint)
        self.inits.append(_tensor(name, torch.as_tensor(t)))
        return name

    def emit(self, op, inputs, n_out=1, **attrs):
        outs = [self.tmp(op.lower()) for _ in range(n_out)]
        self.nodes.append(_node(op, inputs, outs, outs[0], **attrs))
        return outs[0] if n_out == 1 else outs

    def arg(self, a) -> str:
        if isinstance(a, torch.fx.Node):
            return self.names[a]
        return self.const(torch.tensor(a, dtype=torch.float32 if isinstance(a, float) else torch.int64))

    def module(self, node, m):
        x = self.arg(node.args[0])
        if isinstance(m, nn.Linear):
            ins = [x, self.const(m.weight, "w")] + ([self.const(m.bias, "b")] if m.bias is not None else [])
            shape = node.meta.get("in_rank", 2)
            if shape == 2:
                return self.emit("Gemm", ins, transB=1)
            y = self.emit("MatMul", [x, self.const(m.weight.t().contiguous(), "wt")])
            return self.emit("Add", [y, ins[2]]) if m.bias is not None else y
        if isinstance(m, nn.ReLU): return self.emit("Relu", [x])
        if isinstance(m, nn.GELU): return self.emit("Gelu", [x], approximate="tanh" if m.approximate == "tanh" else "none")
        if isinstance(m, nn.Tanh): return self.emit("Tanh", [x])
        if isinstance(m, nn.Sigmoid): return self.emit("Sigmoid", [x])
        if isinstance(m, nn.SiLU): return self.emit("Mul", [x, self.emit("Sigmoid", [x])])
        if isinstance(m, nn.Softmax): return self.emit("Softmax", [x], axis=m.dim if m.dim is not None else -1)
        if isinstance(m, (nn.Dropout, nn.Identity)): return self.emit("Identity", [x])
        if isinstance(m, nn.Flatten): return self.emit("Flatten", [x], axis=m.start_dim)
        if isinstance(m, nn.LayerNorm):
            return self.emit("LayerNormalization", [x, self.const(m.weight, "g"), self.const(m.bias, "b")], axis=-len(m.normalized_shape), epsilon=float(m.eps))
        if isinstance(m, nn.Conv2d):
            ins = [x, self.const(m.weight, "w")] + ([self.const(m.bias, "b")] if m.bias is not None else [])
            p = list(m.padding) if not isinstance(m.padding, str) else [0, 0]
            return self.emit("Conv", ins, kernel_shape=list(m.kernel_size), strides=list(m.stride), pads=p + p, dilations=list(m.dilation), group=m.groups)
        if isinstance(m, nn.BatchNorm2d):
            return self.emit("BatchNormalization", [x, self.const(m.weight, "g"), self.const(m.bias, "b"), self.const(m.running_mean, "m"),
                                                    self.const(m.running_var, "v")], epsilon=float(m.eps))
        if isinstance(m, (nn.MaxPool2d, nn.AvgPool2d)):
            k = m.kernel_size if isinstance(m.kernel_size, (tuple, list)) else (m.kernel_size,) * 2
            s = m.stride if isinstance(m.stride, (tuple, list)) else (m.stride or k[0],) * 2
            p = m.padding if isinstance(m.padding, (tuple, list)) else (m.padding,) * 2
            return self.emit("MaxPool" if isinstance(m, nn.MaxPool2d) else "AveragePool", [x], kernel_shape=list(k), strides=list(s), pads=list(p) * 2)
        if isinstance(m, nn.AdaptiveAvgPool2d) and m.output_size in (1, (1, 1)):
            return self.emit("GlobalAveragePool", [x])
        if isinstance(m, nn.Embedding):
            return self.emit("Gather", [self.const(m.weight, "emb"), x], axis=0)
        raise NotImplementedError(f"ONNX export of {type(m).__name__}")

    def function(self, node):
        t, a = node.target, node.args
        binary = {operator.add: "Add", torch.add: "Add", operator.sub: "Sub", torch.sub: "Sub", operator.mul: "Mul", torch.mul: "Mul",
                  operator.truediv: "Div", torch.div: "Div", torch.matmul: "MatMul", operator.matmul: "MatMul"}
        if t in binary:
            return self.emit(binary[t], [self.arg(a[0]), self.arg(a[1])])
        unary = {torch.relu: "Relu", nn.functional.relu: "Relu", torch.tanh: "Tanh", torch.sigmoid: "Sigmoid"}
        if t in unary:
            return self.emit(unary[t], [self.arg(a[0])])
        if t in (nn.functional.gelu,):
            return self.emit("Gelu", [self.arg(a[0])], approximate=node.kwargs.get("approximate", "none"))
        if t in (torch.softmax, nn.functional.softmax):
            return self.emit("Softmax", [self.arg(a[0])], axis=node.kwargs.get("dim", a[1] if len(a) > 1 else -1))
        if t is torch.flatten:
            return self.emit("Flatten", [self.arg(a[0])], axis=a[1] if len(a) > 1 else node.kwargs.get("start_dim", 0))
        if t is torch.cat:
            return self.emit("Concat", [self.arg(x) for x in a[0]], axis=node.kwargs.get("dim", a[1] if len(a) > 1 else 0))
        raise NotImplementedError(f"ONNX export of function {t}")

    def method(self, node):
        name, a = node.target, node.args
        x = self.arg(a[0])
        if name in ("reshape", "view"):
            shape = a[1] if isinstance(a[1], (tuple, list)) else a[1:]
            return self.emit("Reshape", [x, self.const(torch.tensor(list(shape), dtype=torch.int64), "shape")])
        if name == "flatten":
            return self.emit("Flatten", [x], axis=a[1] if len(a) > 1 else 0)
        if name in ("transpose", "permute"):
            rank = node.meta["in_rank"]
            if name == "transpose":
                perm = list(range(rank))
                d0, d1 = a[1] % rank, a[2] % rank
                perm[d0], perm[d1] = perm[d1], perm[d0]
            else:
                perm = [d % rank for d in (a[1] if isinstance(a[1], (tuple, list)) else a[1:])]
            return self.emit("Transpose", [x], perm=perm)
        if name == "contiguous":
            return self.emit("Identity", [x])
        if name in ("relu", "tanh", "sigmoid"):
            return self.emit(name.capitalize(), [x])
        raise NotImplementedError(f"ONNX export of method {name}")


def export_onnx(module: nn.Module, example_inputs, path=None, input_names=None, dynamic_batch: bool = True, producer: str = "torsh_b200") -> bytes:
    """Returns (and optionally writes) the serialized ``ModelProto`` of ``module`` in inference mode."""
    module = module.eval()
    example_inputs = example_inputs if isinstance(example_inputs, (tuple, list)) else (example_inputs,)
    gm = torch.fx.symbolic_trace(module)
    # ranks of node inputs (for Linear on >2-D inputs and transposes) by running the graph once
    from torch.fx.passes.shape_prop import ShapeProp
    ShapeProp(gm).propagate(*example_inputs)
    for n in gm.graph.nodes:
        if n.args and isinstance(n.args[0], torch.fx.Node) and hasattr(n.args[0].meta.get("tensor_meta"), "shape"):
            n.meta["in_rank"] = len(n.args[0].meta["tensor_meta"].shape)
    ex = _Exporter(gm)
    inputs, outputs, k = [], [], 0
    mods = dict(gm.named_modules())
    for n in gm.graph.nodes:
        if n.op == "placeholder":
            name = (input_names[k] if input_names else n.name)
            t = example_inputs[k]
            shape = list(t.shape)
            if dynamic_batch and shape:
                shape[0] = "batch"
            inputs.append(_value_info(name, shape, INT64 if t.dtype in (torch.int64, torch.int32) else FLOAT))
            ex.names[n] = name
            k += 1
        elif n.op == "get_attr":
            obj = gm
            for part in n.target.split("."):
                obj = getattr(obj, part)
            ex.names[n] = ex.const(obj, "attr")
        elif n.op == "call_module":
            ex.names[n] = ex.module(n, mods[n.target])
        elif n.op == "call_function":
            ex.names[n] = ex.function(n)
        elif n.op == "call_method":
            ex.names[n] = ex.method(n)
        elif n.op == "output":
            outs = n.args[0] if isinstance(n.args[0], (tuple, list)) else [n.args[0]]
            for o in outs:
                shape = list(o.meta["tensor_meta"].shape)
                if dynamic_batch and shape:
                    shape[0] = "batch"
                outputs.append(_value_info(ex.names[o], shape))
    graph = (b"".join(_ld(1, nd) for nd in ex.nodes) + _s(2, type(module).__name__) + b"".join(_ld(5, t) for t in ex.inits)
             + b"".join(_ld(11, i) for i in inputs) + b"".join(_ld(12, o) for o in outputs))
    model = _vi(1, 9) + _s(2, producer) + _ld(7, graph) + _ld(8, _s(1, "") + _vi(2, 20))
    if path is not None:
        with open(path, "wb") as f:
            f.write(model)
    return model


# ---- import / evaluation ---------------------------------------------------------------------------------------------
def _parse_tensor(buf: bytes):
    dims, dt, name, raw = [], FLOAT, "", b""
    for f, wt, v in _fields(buf):
        if f == 1:
            dims.append(v)
        elif f == 2:
            dt = v
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
    import numpy as np
    arr = np.frombuffer(raw, dtype=np.float32 if dt == FLOAT else np.int64).reshape(dims).copy()
    return name, torch.from_numpy(arr)


def _parse_attr(buf: bytes):
    name, val, ints, floats, kind = "", None, [], [], None
    for f, wt, v in _fields(buf):
        if f == 1:
            name = v.decode()
        elif f == 2:
            val = struct.unpack("<f", v)[0]
        elif f == 3:
            val = v - (1 << 64) if v >> 63 else v
        elif f == 4:
            val = v.decode()
        elif f == 7:
            floats.append(struct.unpack("<f", v)[0])
        elif f == 8:
            ints.append(v - (1 << 64) if v >> 63 else v)
        elif f == 20:
            kind = v
    if kind == 7:
        val = ints
    elif kind == 6:
        val = floats
    return name, val


class OnnxModel(nn.Module):
    """A parsed ONNX graph evaluated with PyTorch ops; initializers are registered as buffers."""

    def __init__(self, data: bytes):
        super().__init__()
        self.nodes, self.input_names, self.output_names, self.opset, self.producer = [], [], [], None, ""
        init_names = set()
        for f, _, v in _fields(data):
            if f == 2:
                self.producer = v.decode()
            elif f == 8:
                for f2, _, v2 in _fields(v):
                    if f2 == 2:
                        self.opset = v2
            elif f == 7:
                for f2, _, v2 in _fields(v):
                    if f2 == 1:
                        ins, outs, op, attrs = [], [], "", {}
                        for f3, _, v3 in _fields(v2):
                            if f3 == 1: ins.append(v3.decode())
                            elif f3 == 2: outs.append(v3.decode())
                            elif f3 == 4: op = v3.decode()
                            elif f3 == 5:
                                k, a = _parse_attr(v3)
                                attrs[k] = a
                        self.nodes.append((op, ins, outs, attrs))
                    elif f2 == 5:
                        name, t = _parse_tensor(v2)
                        self.register_buffer("init_" + str(len(init_names)), t)
                        init_names.add(name)
                        self.__dict__.setdefault("_init_map", {})[name] = "init_" + str(len(init_names) - 1)
                    elif f2 in (11, 12):
                        nm = next(v3.decode() for f3, _, v3 in _fields(v2) if f3 == 1)
                        (self.input_names if f2 == 11 else self.output_names).append(nm)
        self.input_names = [n for n in self.input_names if n not in init_names]

    def forward(self, *inputs):
        env = {n: getattr(self, b) for n, b in self.__dict__.get("_init_map", {}).items()}
        env.update(zip(self.input_names, inputs))
        F = nn.functional
        for op, ins, outs, a in self.nodes:
            x = [env[i] for i in ins]
            if op == "Gemm":
                y = x[0] @ (x[1].t() if a.get("transB", 0) else x[1])
                y = y + x[2] if len(x) > 2 else y
            elif op == "MatMul": y = x[0] @ x[1]
            elif op == "Add": y = x[0] + x[1]
            elif op == "Sub": y = x[0] - x[1]
            elif op == "Mul": y = x[0] * x[1]
            elif op == "Div": y = x[0] / x[1]
            elif op == "Relu": y = torch.relu(x[0])
            elif op == "Tanh": y = torch.tanh(x[0])
            elif op == "Sigmoid": y = torch.sigmoid(x[0])
            elif op == "Gelu": y = F.gelu(x[0], approximate=a.get("approximate", "none"))
            elif op == "Softmax": y = torch.softmax(x[0], a.get("axis", -1))
            elif op == "Identity": y = x[0]
            elif op == "Flatten": y = x[0].flatten(a.get("axis", 1))
            elif op == "Reshape": y = x[0].reshape([int(v) for v in x[1]])
            elif op == "Transpose": y = x[0].permute(a["perm"])
            elif op == "Concat": y = torch.cat(x, a.get("axis", 0))
            elif op == "Gather": y = x[0][x[1]] if a.get("axis", 0) == 0 else torch.index_select(x[0], a["axis"], x[1])
            elif op == "LayerNormalization":
                nd = -a.get("axis", -1)
                y = F.layer_norm(x[0], x[0].shape[-nd:], x[1], x[2] if len(x) > 2 else None, a.get("epsilon", 1e-5))
            elif op == "Conv":
                p = a.get("pads", [0, 0, 0, 0])
                y = F.conv2d(x[0], x[1], x[2] if len(x) > 2 else None, a.get("strides", [1, 1]), p[:2], a.get("dilations", [1, 1]), a.get("group", 1))
            elif op == "BatchNormalization": y = F.batch_norm(x[0], x[3], x[4], x[1], x[2], False, 0.0, a.get("epsilon", 1e-5))
            elif op == "MaxPool": y = F.max_pool2d(x[0], a["kernel_shape"], a.get("strides"), a.get("pads", [0, 0])[:2])
            elif op == "AveragePool": y = F.avg_pool2d(x[0], a["kernel_shape"], a.get("strides"), a.get("pads", [0, 0])[:2])
            elif op == "GlobalAveragePool": y = x[0].mean((2, 3), keepdim=True)
            else:
                raise NotImplementedError(f"ONNX operator {op}")
            env[outs[0]] = y
        res = [env[o] for o in self.output_names]
        return res[0] if len(res) == 1 else tuple(res)

    def op_types(self) -> list[str]:
        return [n[0] for n in self.nodes]


def load_onnx(path_or_bytes) -> OnnxModel:
    data = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    return OnnxModel(bytes(data))
