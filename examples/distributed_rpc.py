"""Remote procedure calls and a parameter server over TCP (roles of ``examples/distributed_rpc.rs`` and
``crates/torsh-distributed/src/parameter_server.rs``). One process plays both sides: it registers functions, calls them
through its own RPC endpoint (a real TCP round trip), and serves a parameter server that a client trains against.
With several processes give every worker its own name and a shared TCP store instead of the in-memory one."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from torsh_b200.parallel import rpc
from torsh_b200.parallel.parameter_server import ParameterServer, ParameterServerClient, ParameterServerConfig
from torsh_b200.parallel.store import MemoryStore


def main(argv=None):
    rpc.init_rpc("worker0", MemoryStore(), rank=0, world_size=1)
    try:
        rpc.register_function("add", lambda a, b: a + b)
        rpc.register_function("make_weights", lambda n: torch.arange(float(n)))
        out = rpc.rpc_sync("worker0", "add", (torch.ones(3), torch.full((3,), 2.0)))
        fut = rpc.rpc_async("worker0", "add", (1, 2))
        ref = rpc.remote("worker0", "make_weights", (4,))
        print("rpc add:", out.tolist(), "| async:", fut.result(10), "| rref:", ref.to_here().tolist())
        rpc.delete_rref(ref)

        # a linear model trained through the parameter server: push gradients, pull fresh parameters
        server = ParameterServer(ParameterServerConfig(learning_rate=0.1))
        server.serve("ps")
        torch.manual_seed(0)
        model = torch.nn.Linear(4, 1)
        client = ParameterServerClient("worker0", "ps")
        client.register_module(model)
        x = torch.randn(64, 4)
        y = x @ torch.tensor([[1.0], [-2.0], [0.5], [3.0]])
        losses = []
        for _ in range(30):
            client.sync(model)
            model.zero_grad()
            loss = torch.nn.functional.mse_loss(model(x), y)
            loss.backward()
            client.push_gradients(model)
            losses.append(loss.item())
        print(f"parameter server: loss {losses[0]:.3f} -> {losses[-1]:.3f}, stats {server.stats}")
        return out, losses
    finally:
        rpc.shutdown()


if __name__ == "__main__":
    main()
