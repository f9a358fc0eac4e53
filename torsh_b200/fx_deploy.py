"""Graph deployment targets and extension points (``crates/torsh-fx/src``): TorchScript export / import of traced graphs
(``torchscript_compat.rs``), registries for custom operations and custom value types checked along graph edges
(``custom_operations.rs``, ``custom_types.rs``), container / Kubernetes / serving manifests with capacity and cost planning
(``cloud_deployment.rs``), descriptors of unconventional accelerators with partitioning and noise-aware evaluation
(``emerging_hardware.rs``), conversion of rectifier networks to spiking networks with threshold balancing
(``neuromorphic_optimization.rs``) and a differentiable variational quantum layer simulated on state vectors
(``quantum_computing.rs``)."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch
import torch.fx
from torch import nn


# ================================================================================================ TorchScript
def to_torchscript(gm: torch.fx.GraphModule, example_inputs: Sequence[torch.Tensor] | None = None, check: bool = True) -> torch.jit.ScriptModule:
    """Scripts the generated ``forward`` (tracing as a fallback for code the scripter rejects) and, with ``check``, compares the
    outputs on the example inputs."""
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        try:
            sm = torch.jit.script(gm)
        except Exception:
            if example_inputs is None:
                raise
            sm = torch.jit.trace(gm, tuple(example_inputs))
    if check and example_inputs is not None:
        a, b = gm(*example_inputs), sm(*example_inputs)
        if not torch.allclose(a, b, atol=1e-6):
            raise RuntimeError("the scripted module does not reproduce the graph module")
    return sm


def describe_torchscript(sm: torch.jit.ScriptModule) -> dict:
    """Operator histogram, inputs and constants of a scripted module's inlined graph."""
    g = sm.inlined_graph
    kinds = [n.kind() for n in g.nodes()]
    from collections import Counter
    return {"inputs": [i.debugName() for i in list(g.inputs())[1:]], "operators": dict(Counter(k for k in kinds if k.startswith("aten::"))), "constants": sum(k == "prim::Constant" for k in kinds), "nodes": len(kinds)}


def from_torchscript(sm: torch.jit.ScriptModule, example_inputs: Sequence[torch.Tensor]) -> torch.fx.GraphModule:
    """Brings a scripted module back as a graph module: the module becomes one leaf call whose behaviour is preserved, wrapped
    so that graph passes can compose it with other nodes."""
    class _Wrapper(nn.Module):
        def __init__(self, inner): super().__init__(); self.inner = inner
        def forward(self, *args): return self.inner(*args)
    class _Tracer(torch.fx.Tracer):
        def is_leaf_module(self, m, name): return isinstance(m, torch.jit.ScriptModule) or super().is_leaf_module(m, name)
    w = _Wrapper(sm)
    graph = torch.fx.Graph()
    ins = [graph.placeholder(f"arg{i}") for i in range(len(example_inputs))]
    graph.output(graph.call_module("inner", tuple(ins)))
    return torch.fx.GraphModule(w, graph)


# ================================================================================================ custom operations and types
@dataclass
class CustomOp:
    name: str
    forward: Callable
    infer_shape: Callable[..., tuple] | None = None
    cost: Callable[..., float] | None = None
    backward: Callable | None = None
    doc: str = ""


class CustomOperationRegistry:
    """Named operations usable inside traced graphs: each becomes a graph leaf (not traced through), with optional shape
    inference, cost model and hand-written gradient."""

    def __init__(self): self.ops: dict[str, CustomOp] = {}

    def register(self, name: str, forward: Callable, infer_shape=None, cost=None, backward=None, doc: str = "") -> Callable:
        if name in self.ops:
            raise ValueError(f"operation {name!r} is already registered")
        op = CustomOp(name, forward, infer_shape, cost, backward, doc)
        if backward is not None:
            class _Fn(torch.autograd.Function):
                @staticmethod
                def forward(ctx, *args): ctx.save_for_backward(*[a for a in args if isinstance(a, torch.Tensor)]); return forward(*args)
                @staticmethod
                def backward(ctx, g): r = backward(g, *ctx.saved_tensors); return r if isinstance(r, tuple) else (r,)
            real = lambda *a: _Fn.apply(*a)
        else:
            real = lambda *a: forward(*a)
        real.__name__ = real.__qualname__ = name
        def call(*a):                                                               # under a tracer the operation is recorded as one node, not traced through
            for v in a:
                if isinstance(v, torch.fx.Proxy):
                    return v.tracer.create_proxy("call_function", real, a, {})
            return real(*a)
        call.__name__ = name
        op.callable = call
        self.ops[name] = op
        return call

    def get(self, name: str) -> Callable: return self.ops[name].callable
    def unregister(self, name: str): self.ops.pop(name)

    def nodes_in(self, gm: torch.fx.GraphModule) -> list[str]: return [n.name for n in gm.graph.nodes if n.op == "call_function" and getattr(n.target, "__name__", "") in self.ops]

    def infer_shapes(self, gm: torch.fx.GraphModule, input_shapes: Sequence[tuple]) -> dict[str, tuple]:
        """Shapes of the custom nodes from their own inference functions (others by running on ``meta`` tensors)."""
        env, it = {}, iter(input_shapes)
        for n in gm.graph.nodes:
            if n.op == "placeholder":
                env[n] = torch.empty(next(it), device="meta")
            elif n.op == "call_function" and getattr(n.target, "__name__", "") in self.ops and self.ops[n.target.__name__].infer_shape:
                shp = self.ops[n.target.__name__].infer_shape(*[tuple(env[a].shape) if isinstance(a, torch.fx.Node) else a for a in n.args])
                env[n] = torch.empty(shp, device="meta")
            elif n.op == "call_function":
                env[n] = n.target(*[env[a] if isinstance(a, torch.fx.Node) else a for a in n.args], **n.kwargs)
            elif n.op == "call_module":
                env[n] = gm.get_submodule(n.target).to("meta")(*[env[a] for a in n.args])
            elif n.op == "call_method":
                env[n] = getattr(env[n.args[0]], n.target)(*[env[a] if isinstance(a, torch.fx.Node) else a for a in n.args[1:]], **n.kwargs)
        return {n.name: tuple(v.shape) for n, v in env.items() if isinstance(v, torch.Tensor)}

    def total_cost(self, gm: torch.fx.GraphModule, input_shapes: Sequence[tuple]) -> float:
        shapes, total = self.infer_shapes(gm, input_shapes), 0.0
        for n in gm.graph.nodes:
            if n.op == "call_function" and getattr(n.target, "__name__", "") in self.ops and self.ops[n.target.__name__].cost:
                total += self.ops[n.target.__name__].cost(*[shapes[a.name] if isinstance(a, torch.fx.Node) else a for a in n.args])
        return total


@dataclass
class CustomType:
    name: str
    pack: Callable[[torch.Tensor], Any]
    unpack: Callable[[Any], torch.Tensor]
    bits: float
    validate: Callable[[Any], bool] = lambda v: True


class CustomTypeRegistry:
    """Value types beyond the built-in dtypes (fixed point, logarithmic, block floating point ...): conversion functions, storage
    cost, and a check that every edge of an annotated graph connects a producer and a consumer of the same type (or that a
    registered conversion exists)."""

    def __init__(self): self.types: dict[str, CustomType] = {}; self.conversions: dict[tuple[str, str], Callable] = {}
    def register(self, t: CustomType): self.types[t.name] = t; return t
    def register_conversion(self, src: str, dst: str, fn: Callable): self.conversions[(src, dst)] = fn

    def with_defaults(self):
        def fixed(total, frac):
            s, lim = 2.0 ** frac, 2 ** (total - 1)
            return CustomType(f"fixed<{total},{frac}>", lambda t: (t * s).round().clamp(-lim, lim - 1).to(torch.int32), lambda q: q.float() / s, total, lambda q: bool((q >= -lim).all() and (q < lim).all()))
        self.register(fixed(8, 4)); self.register(fixed(16, 8))
        self.register(CustomType("log8", lambda t: (torch.sign(t).to(torch.int8), (torch.log2(t.abs().clamp_min(2.0 ** -16)) * 8).round().clamp(-128, 127).to(torch.int8)), lambda p: p[0].float() * 2.0 ** (p[1].float() / 8), 9))
        def bfp_pack(t, block=16, mant=8):
            f = t.flatten(); pad = (-len(f)) % block
            b = nn.functional.pad(f, (0, pad)).view(-1, block)
            e = torch.ceil(torch.log2(b.abs().amax(1, keepdim=True).clamp_min(2.0 ** -126)))
            m = (b / 2.0 ** e * 2 ** (mant - 1)).round().clamp(-(2 ** (mant - 1)), 2 ** (mant - 1) - 1)
            return m.to(torch.int16), e.to(torch.int8), t.shape, pad
        def bfp_unpack(p, mant=8):
            m, e, shape, pad = p
            f = (m.float() / 2 ** (mant - 1) * 2.0 ** e.float()).flatten()
            return (f[:len(f) - pad] if pad else f).reshape(shape)
        self.register(CustomType("bfp16x8", bfp_pack, bfp_unpack, 8 + 8 / 16))
        return self

    def roundtrip_error(self, name: str, t: torch.Tensor) -> float:
        ty = self.types[name]
        return float((ty.unpack(ty.pack(t)) - t).norm() / t.norm().clamp_min(1e-30))

    def check_graph(self, gm: torch.fx.GraphModule, annotations: dict[str, tuple[str, str]]) -> list[dict]:
        """``annotations[node] = (input type, output type)``; returns the edges whose producer output type differs from the
        consumer input type and for which no conversion is registered."""
        issues = []
        for n in gm.graph.nodes:
            if n.name not in annotations:
                continue
            for src in n.all_input_nodes:
                if src.name in annotations:
                    a, b = annotations[src.name][1], annotations[n.name][0]
                    if a != b and (a, b) not in self.conversions:
                        issues.append({"edge": (src.name, n.name), "producer": a, "consumer": b})
        return issues


# ================================================================================================ cloud deployment
@dataclass
class ServingSpec:
    name: str
    image: str
    model_path: str
    gpus_per_replica: int = 1
    max_batch: int = 32
    batch_timeout_ms: float = 5.0
    port: int = 8080
    cpu: str = "8"
    memory: str = "64Gi"
    min_replicas: int = 1
    max_replicas: int = 8
    target_gpu_utilisation: int = 70


INSTANCE_TYPES = {"b200x8": {"gpus": 8, "hourly": 98.0, "gpu_memory_gb": 180}, "h100x8": {"gpus": 8, "hourly": 60.0, "gpu_memory_gb": 80}, "a100x8": {"gpus": 8, "hourly": 33.0, "gpu_memory_gb": 80}, "l4x1": {"gpus": 1, "hourly": 0.8, "gpu_memory_gb": 24}}


def dockerfile(spec: ServingSpec, base: str = "nvcr.io/nvidia/pytorch:25.01-py3", extra_packages: Sequence[str] = ()) -> str:
    pip = f"RUN pip install --no-cache-dir {' '.join(extra_packages)}\n" if extra_packages else ""
    return (f"FROM {base}\nWORKDIR /srv\nCOPY . /srv\n{pip}ENV MODEL_PATH={spec.model_path} MAX_BATCH={spec.max_batch} BATCH_TIMEOUT_MS={spec.batch_timeout_ms}\nEXPOSE {spec.port}\n"
            f"HEALTHCHECK --interval=30s --timeout=5s CMD curl -fs http://localhost:{spec.port}/healthz || exit 1\nCMD [\"python\", \"-m\", \"torsh_b200.cli\", \"model\", \"benchmark\", \"{spec.model_path}\"]\n")


def kubernetes_manifests(spec: ServingSpec) -> str:
    """Deployment, Service and HorizontalPodAutoscaler as one multi-document YAML string."""
    dep = f"""apiVersion: apps/v1
kind: Deployment
metadata:
  name: {spec.name}
  labels: {{app: {spec.name}}}
spec:
  replicas: {spec.min_replicas}
  selector:
    matchLabels: {{app: {spec.name}}}
  template:
    metadata:
      labels: {{app: {spec.name}}}
    spec:
      containers:
      - name: server
        image: {spec.image}
        ports:
        - containerPort: {spec.port}
        env:
        - {{name: MODEL_PATH, value: "{spec.model_path}"}}
        - {{name: MAX_BATCH, value: "{spec.max_batch}"}}
        resources:
          limits: {{nvidia.com/gpu: {spec.gpus_per_replica}, cpu: "{spec.cpu}", memory: {spec.memory}}}
        readinessProbe:
          httpGet: {{path: /healthz, port: {spec.port}}}
          periodSeconds: 10
"""
    svc = f"""apiVersion: v1
kind: Service
metadata:
  name: {spec.name}
spec:
  selector: {{app: {spec.name}}}
  ports:
  - {{port: 80, targetPort: {spec.port}}}
"""
    hpa = f"""apiVersion: autoscaling/v2
kind: HorizontalPodAutoscaler
metadata:
  name: {spec.name}
spec:
  scaleTargetRef: {{apiVersion: apps/v1, kind: Deployment, name: {spec.name}}}
  minReplicas: {spec.min_replicas}
  maxReplicas: {spec.max_replicas}
  metrics:
  - type: Pods
    pods:
      metric: {{name: gpu_utilisation}}
      target: {{type: AverageValue, averageValue: "{spec.target_gpu_utilisation}"}}
"""
    return "---\n".join([dep, svc, hpa])


def plan_capacity(qps: float, latency_ms_at_batch: dict[int, float], slo_ms: float, spec: ServingSpec, instance: str = "b200x8", headroom: float = 0.3) -> dict:
    """Largest batch whose latency (plus the batching delay) meets the objective, the throughput of one replica at that
    batch, the replicas and instances needed for the load with headroom, and the monthly cost."""
    ok = {b: l for b, l in latency_ms_at_batch.items() if b <= spec.max_batch and l + spec.batch_timeout_ms <= slo_ms}
    if not ok:
        return {"feasible": False, "reason": f"no batch size meets {slo_ms} ms"}
    batch = max(ok)
    per_replica = batch / (ok[batch] / 1e3)
    replicas = max(spec.min_replicas, math.ceil(qps * (1 + headroom) / per_replica))
    inst = INSTANCE_TYPES[instance]
    per_instance = inst["gpus"] // spec.gpus_per_replica
    instances = math.ceil(replicas / per_instance)
    return {"feasible": replicas <= spec.max_replicas, "batch": batch, "replica_qps": per_replica, "replicas": replicas, "instances": instances, "monthly_cost": instances * inst["hourly"] * 730, "cost_per_million_requests": instances * inst["hourly"] / (qps * 3600) * 1e6,
            "utilisation": qps / (replicas * per_replica)}


# ================================================================================================ unconventional accelerators
@dataclass
class AcceleratorModel:
    name: str
    supported: Sequence[str]                                                           # module class names / function names it can run
    weight_bits: int
    activation_bits: int
    weight_noise: float = 0.0                                                          # relative Gaussian noise on stored weights
    energy_per_mac_pj: float = 1.0
    host_energy_per_mac_pj: float = 20.0
    transfer_energy_per_byte_pj: float = 50.0


ACCELERATORS = {"analog_in_memory": AcceleratorModel("analog_in_memory", ("Linear", "Conv2d"), 6, 8, 0.03, 0.05), "photonic": AcceleratorModel("photonic", ("Linear",), 8, 8, 0.01, 0.01),
                "digital_npu": AcceleratorModel("digital_npu", ("Linear", "Conv2d", "ReLU", "add", "MaxPool2d", "BatchNorm2d"), 8, 8, 0.0, 0.3)}


def map_to_accelerator(gm: torch.fx.GraphModule, example: torch.Tensor, accel: AcceleratorModel) -> dict:
    """Splits the graph into nodes the accelerator runs and nodes left on the host, counts multiply-accumulates and the bytes
    that cross the boundary (each host/accelerator alternation moves an activation), and estimates energy both ways."""
    from .fx import ShapeProp
    ShapeProp(gm).run(example)
    mods = dict(gm.named_modules())
    on, off, macs_on, macs_off, crossings, prev_on, prev_numel = [], [], 0.0, 0.0, 0.0, None, 0
    for n in gm.graph.nodes:
        if n.op not in ("call_module", "call_function", "call_method"):
            continue
        kind = type(mods[n.target]).__name__ if n.op == "call_module" else getattr(n.target, "__name__", str(n.target))
        m = mods.get(n.target) if n.op == "call_module" else None
        numel = math.prod(n.meta.get("shape", (0,)))
        macs = numel * m.in_features if isinstance(m, nn.Linear) else numel * m.in_channels // m.groups * math.prod(m.kernel_size) if isinstance(m, nn.Conv2d) else 0
        here = kind in accel.supported
        (on if here else off).append(n.name)
        if here:
            macs_on += macs
        else:
            macs_off += macs
        if prev_on is not None and here != prev_on:
            crossings += prev_numel * accel.activation_bits / 8                      # the previous node's output moves to the other side
        prev_on, prev_numel = here, numel
    e_acc = macs_on * accel.energy_per_mac_pj + macs_off * accel.host_energy_per_mac_pj + crossings * accel.transfer_energy_per_byte_pj
    e_host = (macs_on + macs_off) * accel.host_energy_per_mac_pj
    return {"on_accelerator": on, "on_host": off, "macs_on": macs_on, "macs_off": macs_off, "boundary_bytes": crossings, "energy_pj": e_acc, "host_only_energy_pj": e_host, "energy_saving": 1 - e_acc / e_host if e_host else 0.0}


@torch.no_grad()
def evaluate_with_device_noise(model: nn.Module, x: torch.Tensor, accel: AcceleratorModel, trials: int = 8, generator: torch.Generator | None = None) -> dict:
    """Runs the model with its weights quantised to the device's width and perturbed by its write noise; reports the mean and
    worst relative deviation from the exact output and the agreement of the arg-max."""
    import copy
    ref = model(x)
    devs, agree = [], []
    for _ in range(trials):
        m = copy.deepcopy(model)
        for mod in m.modules():
            if type(mod).__name__ in accel.supported and hasattr(mod, "weight") and mod.weight is not None and mod.weight.dim() >= 2:
                w = mod.weight
                qmax = 2 ** (accel.weight_bits - 1) - 1
                s = w.abs().amax() / qmax
                wq = (w / s).round().clamp(-qmax - 1, qmax) * s
                mod.weight.copy_(wq + accel.weight_noise * w.abs().amax() * torch.randn(w.shape, generator=generator))
        out = m(x)
        devs.append(float((out - ref).norm() / ref.norm()))
        agree.append(float((out.argmax(-1) == ref.argmax(-1)).float().mean()))
    return {"mean_deviation": sum(devs) / trials, "worst_deviation": max(devs), "argmax_agreement": sum(agree) / trials}


# ================================================================================================ spiking conversion
class SpikingNetwork(nn.Module):
    """Rate-coded integrate-and-fire copy of a feed-forward rectifier network (``Linear`` / ``Conv2d`` / ``ReLU`` / pooling /
    ``Flatten`` in an ``nn.Sequential``): every rectifier becomes a layer of neurons with soft reset whose threshold is the
    ``percentile`` of that layer's activations on calibration data (weights are rescaled accordingly), the input is applied
    as a constant current and the output is the accumulated potential of the last layer divided by the number of steps."""

    def __init__(self, ann: nn.Sequential, calibration: torch.Tensor, percentile: float = 99.9):
        super().__init__()
        self.layers, self.scales = nn.ModuleList(list(ann)), []
        x = calibration
        with torch.no_grad():
            for m in ann:
                x = m(x)
                if isinstance(m, nn.ReLU):
                    self.scales.append(float(torch.quantile(x.flatten()[:1_000_000].float(), percentile / 100)) or 1.0)
        self.ann = ann

    def forward(self, x: torch.Tensor, steps: int = 64) -> tuple[torch.Tensor, dict]:
        """Returns the rate-decoded output and spike statistics."""
        mem, spikes_total, neurons, out_acc = {}, 0.0, 0, None
        for t in range(steps):
            h, k = x, 0
            for i, m in enumerate(self.layers):
                if isinstance(m, nn.ReLU):
                    lam = self.scales[k]
                    v = mem.get(i, torch.zeros_like(h)) + h
                    s = (v >= lam).to(h.dtype)
                    mem[i] = v - s * lam                                             # soft reset keeps the residual
                    h = s * lam                                                      # a spike carries the threshold's worth of activation
                    spikes_total += float(s.sum()); k += 1
                    if t == 0:
                        neurons += s[0].numel()
                else:
                    h = m(h)
            out_acc = h if out_acc is None else out_acc + h
        return out_acc / steps, {"spikes_per_neuron_per_step": spikes_total / max(neurons * steps * x.shape[0], 1), "total_spikes": spikes_total, "neurons": neurons}


def snn_energy_estimate(stats: dict, synaptic_ops_per_spike: float, energy_per_synop_pj: float = 0.9, ann_macs: float | None = None, energy_per_mac_pj: float = 4.6) -> dict:
    e = stats["total_spikes"] * synaptic_ops_per_spike * energy_per_synop_pj
    out = {"snn_energy_pj": e}
    if ann_macs is not None:
        out.update(ann_energy_pj=ann_macs * energy_per_mac_pj, ratio=e / (ann_macs * energy_per_mac_pj))
    return out


# ================================================================================================ variational quantum layer
class VariationalQuantumLayer(nn.Module):
    """``n`` qubits simulated as a state vector: inputs enter as ``RY`` angles (angle encoding), followed by ``depth`` blocks of
    trainable ``RY`` / ``RZ`` rotations and a ring of ``CNOT`` gates; the outputs are the ``Z`` expectation values.  Everything is
    ordinary tensor algebra, so gradients come from autograd (they equal the parameter-shift gradients)."""

    def __init__(self, n_qubits: int = 4, depth: int = 2):
        super().__init__()
        if n_qubits > 12:
            raise ValueError("state-vector simulation is limited to 12 qubits here")
        self.n, self.depth = n_qubits, depth
        self.theta = nn.Parameter(torch.randn(depth, n_qubits, 2) * 0.1)

    def _apply_1q(self, state, gate, q):
        """``state [batch, 2^n]``, ``gate [batch or 1, 2, 2]`` on qubit ``q`` (qubit 0 is the most significant)."""
        b = state.shape[0]
        s = state.reshape(b, 2 ** q, 2, 2 ** (self.n - q - 1))
        return torch.einsum("bij,bajc->baic", gate.expand(b, 2, 2), s).reshape(b, -1)

    def _cnot(self, state, c, t):
        idx = torch.arange(2 ** self.n, device=state.device)
        cbit = (idx >> (self.n - 1 - c)) & 1
        return state[:, torch.where(cbit == 1, idx ^ (1 << (self.n - 1 - t)), idx)]

    @staticmethod
    def _ry(a):
        c, s = torch.cos(a / 2), torch.sin(a / 2)
        return torch.stack([torch.stack([c, -s], -1), torch.stack([s, c], -1)], -2).to(torch.complex64)

    @staticmethod
    def _rz(a):
        e = torch.exp(-0.5j * a.to(torch.complex64))
        z = torch.zeros_like(e)
        return torch.stack([torch.stack([e, z], -1), torch.stack([z, e.conj()], -1)], -2)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b = x.shape[0]
        state = torch.zeros(b, 2 ** self.n, dtype=torch.complex64, device=x.device); state[:, 0] = 1
        for q in range(self.n):
            state = self._apply_1q(state, self._ry(x[:, q % x.shape[1]]), q)
        for d in range(self.depth):
            for q in range(self.n):
                state = self._apply_1q(state, self._ry(self.theta[d, q, 0])[None], q)
                state = self._apply_1q(state, self._rz(self.theta[d, q, 1])[None], q)
            for q in range(self.n):
                if self.n > 1:
                    state = self._cnot(state, q, (q + 1) % self.n)
        p = state.abs() ** 2
        idx = torch.arange(2 ** self.n, device=x.device)
        signs = torch.stack([1 - 2 * ((idx >> (self.n - 1 - q)) & 1).float() for q in range(self.n)], 1)
        return p @ signs

    def circuit_summary(self) -> dict: return {"qubits": self.n, "depth": self.depth, "parameters": self.theta.numel(), "two_qubit_gates": self.depth * (self.n if self.n > 1 else 0), "single_qubit_gates": self.n + 2 * self.depth * self.n}
