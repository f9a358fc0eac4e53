"""The example programs run end to end on the CPU (single process; the multi-rank ones degrade to world size 1,
and a two-rank gloo launch covers the pipeline and DDP examples)."""
import importlib.util
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_single_process_examples(tmp_path):
    losses = _load("gpt2").main(["--model", "gpt2-tiny", "--steps", "4", "--batch", "2", "--seq", "32"])
    assert len(losses) == 4 and all(l == l for l in losses) and losses[-1] < losses[0] - 0.05
    losses = _load("resnet").main(["--model", "resnet18", "--steps", "2", "--image", "32", "--batch", "4"])
    assert losses[1] < losses[0] * 1.5
    assert _load("checkpointing").main([str(tmp_path)]) is True
    assert _load("tensor_operations").main([]) >= 0
    assert _load("gradient_checkpointing").main([]) < 1e-6
    out, losses = _load("distributed_rpc").main([])
    assert out.tolist() == [3.0, 3.0, 3.0] and losses[-1] < 0.05 * losses[0]
    assert _load("mnist").main(["--epochs", "2", "--samples", "256"])[-1] > 0.5
    assert _load("stream_management").main([]) in ("cpu", "cuda")


def test_two_rank_examples_gloo():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for script, port in (("pipeline.py", "29571"), ("distributed.py", "29572"), ("model_parallelism.py", "29573"),
                         ("distributed_nccl.py", "29574")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", port, os.path.join(ROOT, "examples", script)]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        assert "loss" in r.stdout or "all_reduce" in r.stdout
