"""Streams, events, the caching memory pools and the CUDA-graph cache of the native runtime (roles of
``examples/advanced_stream_management.rs``, ``cuda_event_coordination.rs`` and ``unified_memory_demo.rs``). Needs a GPU;
without one it prints the host pool's behaviour only."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch

from torsh_b200.core import runtime as rt


def main(argv=None):
    pool = rt.HostPool()
    a = pool.alloc(1000)
    b = pool.alloc(3 << 20)
    print("host pool rounds 1000 B to", pool.size_of(a), "and 3 MiB to", pool.size_of(b), "| stats", pool.stats())
    pool.free(a); pool.free(b)
    a2 = pool.alloc(900)
    print("a freed small block is reused:", a2 == a)
    pool.free(a2); pool.close()
    if not torch.cuda.is_available():
        return "cpu"
    info = rt.device_info()
    print(f"device: {info.name}, {info.sm_count} SMs, {info.total_memory >> 30} GiB, TMEM columns {info.tmem_columns}")
    print("occupancy of a 512-thread, 64-register kernel:", rt.occupancy(512, 64, 0))
    streams = rt.StreamPool(size_per_class=2)
    hi, lo = streams.get(rt.HIGH), streams.get(rt.LOW)
    x = torch.randn(1 << 22, device="cuda")
    done, start = rt.Event(timing=True), rt.Event(timing=True)
    with torch.cuda.stream(lo):
        start.record(lo)
        y = x * 2
        done.record(lo)
    done.wait(hi)                                   # the high-priority stream consumes what the low one produced
    with torch.cuda.stream(hi):
        z = y + 1
    torch.cuda.synchronize()
    print(f"producer kernel took {start.elapsed_ms(done):.3f} ms; result ok: {bool((z == x * 2 + 1).all())}")
    buf = rt.DeviceMemoryPool.alloc(8 << 20)
    t = buf.tensor((1 << 20,), torch.float32)
    pin = rt.PinnedBuffer(4 << 20)
    pin.tensor((1 << 20,), torch.float32).fill_(3.0)
    pin.copy_to_device_async(t)
    torch.cuda.synchronize()
    print("pinned -> device copy:", float(t.sum()) == 3.0 * (1 << 20), "| device pool", rt.DeviceMemoryPool.stats())
    buf.free(); pin.free()
    return "cuda"


if __name__ == "__main__":
    main()
