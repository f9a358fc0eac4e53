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
    assert len(losses) == 4 and all(l == l for l in losses)
    losses = _load("resnet").main(["--model", "resnet18", "--steps", "2", "--image", "32", "--batch", "4"])
    assert losses[1] < losses[0] * 1.5
    assert _load("checkpointing").main([str(tmp_path)]) is True
    assert _load("tensor_operations").main([]) >= 0
    assert _load("gradient_checkpointing").main([]) < 1e-6
    out, losses = _load("distributed_rpc").main([])
    assert out.tolist() == [3.0, 3.0, 3.0] and losses[-1] < 0.05 * losses[0]
    assert _load("mnist").main(["--epochs", "2", "--samples", "256"])[-1] > 0.5
    assert _load("stream_management").main([]) in ("cpu", "cuda")
    losses = _load("train_from_tokens").main(["--steps", "10"])
    assert len(losses) == 10 and losses[-1] < losses[0] - 1.0


def test_two_rank_examples_gloo():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for script, port in (("pipeline.py", "29571"), ("distributed.py", "29572"), ("model_parallelism.py", "29573"),
                         ("distributed_nccl.py", "29574")):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", port, os.path.join(ROOT, "examples", script)]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0, r.stderr[-2000:]
        assert "loss" in r.stdout or "all_reduce" in r.stdout


def test_trainer_learns_on_cpu_without_the_kernels():
    """The flat optimizer's CPU path picks up the gradients autograd left in ``p.grad``."""
    import torch
    import torsh_b200 as tb
    torch.manual_seed(0)
    model = tb.models.create_model("gpt2-tiny")
    trainer = tb.engine.CausalLMTrainer(model, lr=3e-4, batch_size=4, seq_len=64, use_graph=False)
    ids = torch.randint(0, model.config.vocab_size, (4, 65))
    losses = [trainer.step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous()) for _ in range(6)]
    assert losses[-1] < losses[0] - 0.5, losses
    assert all(p.grad is None for p in model.parameters())
