"""End-to-end: the GPT-2 training step through the sm_100a kernels tracks a plain PyTorch fp32 run."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_reference_losses(cfg, ids, steps, lr):
    """Independent fp32 implementation with stock PyTorch ops (the oracle)."""
    import torch.nn.functional as F
    from torsh_b200.models import GPTForCausalLM
    torch.manual_seed(0)
    m = GPTForCausalLM(cfg).float()  # CPU tensors: every op falls back to PyTorch maths
    opt = torch.optim.AdamW(m.parameters(), lr=lr, weight_decay=0.01)
    out = []
    for _ in range(steps):
        loss = m(ids[:, :-1], ids[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
        out.append(loss.item())
    return out


def test_gpt2_tiny_training_matches_fp32_oracle():
    from torsh_b200.engine import CausalLMTrainer
    from torsh_b200.models import GPT2Config, GPTForCausalLM
    cfg = GPT2Config.tiny()
    ids = torch.randint(0, cfg.vocab_size, (8, 129), generator=torch.Generator().manual_seed(0))
    ref = _torch_reference_losses(cfg, ids, 8, 3e-4)
    torch.manual_seed(0)
    model = GPTForCausalLM(cfg).to("cuda")
    tr = CausalLMTrainer(model, lr=3e-4, weight_decay=0.01, batch_size=8, seq_len=128, use_graph=True, warmup_eager=2)
    x, y = ids[:, :-1].contiguous().pin_memory(), ids[:, 1:].contiguous().pin_memory()
    got = [tr.step(x, y) for _ in range(8)]
    assert tr.graph is not None and tr.launches_per_step > 50
    for a, b in zip(got, ref):
        assert abs(a - b) < 0.05 * abs(b), (got, ref)
    assert got[-1] < got[0] - 1.0


def test_layernorm_params_receive_gradient_through_flat_buffers():
    from torsh_b200.models import GPT2Config, GPTForCausalLM
    from torsh_b200.optim import FlatParameters
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPTForCausalLM(cfg).to("cuda")
    flat = FlatParameters(model.parameters())
    ids = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda")
    model(ids[:, :-1], ids[:, 1:], loss_scale=1.0).backward()
    for name, p in model.named_parameters():
        assert p.grad is None, name
        assert p.main_grad.abs().sum().item() > 0, f"{name} got no gradient"
