"""The batched count exchange on a CUDA device (one-rank NCCL group in a child process): slots are written by
kernels on a side stream, as the pipelined loop does, the exchange runs in stream order, and the host is
never blocked inside the loop."""
import os
import socket
import sys

import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(port, steps, depth, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import time
    import torch
    import torch.distributed as dist
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        from sbnet_b200 import dist as sd
        ex = sd.CountExchange(dev, depth=depth, timeout_s=30.0)
        side = torch.cuda.Stream()
        values = torch.arange(1000, 1000 + steps, dtype=torch.int32, device=dev)
        busy = torch.empty(64 * 1024 * 1024, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize()
        longest = 0.0
        for i in range(steps):
            t = time.perf_counter()
            slot = ex.slot(i, side)
            longest = max(longest, time.perf_counter() - t)
            with torch.cuda.stream(side):
                slot[:1].copy_(values[i:i + 1])          # what reduce_mask would publish, on the side stream
            done = torch.cuda.Event()
            done.record(side)
            torch.cuda.current_stream().wait_event(done)  # the step's own kernels follow the mask
            busy.fill_(i & 1)
            ex.step_done(i, steps)
        table = ex.finish()
        q.put(("ok", {k: v for k, v in table.items() if k < steps}, longest))
    except Exception as e:   # noqa: BLE001 - reported to the parent
        q.put(("error", repr(e), 0.0))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("steps,depth", [(70, 8), (5, 8), (40, 32)])
def test_count_exchange_on_a_cuda_device(steps, depth):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_worker, args=(_free_port(), steps, depth, q))
    p.start()
    status, table, longest = q.get(timeout=300)
    p.join(timeout=60)
    assert status == "ok", table
    assert p.exitcode == 0
    assert sorted(table) == list(range(steps))
    for i in range(steps):
        assert table[i] == [1000 + i]
    assert longest < 0.25          # slot() never waits out a collective on the host
