"""World-size-2 gloo test (CPU) of the batch sharding: each rank reduces its slice of the masks with
the CPU checker standing in for the device op, the counts are all-gathered, and the union of the
per-rank block lists (shifted to global image indices) must equal the single-process result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_images, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        from sbnet_b200 import configs as cfg, dist as sd
        o = oracle.get("port")
        H, W = 64, 48
        g = cfg.halo_geom(H, W)
        mask = cfg.rect_union_mask(n_images, H, W, seed=9, occupancy=0.2, side=(4, 12))
        lo, hi = sd.shard_bounds(n_images, world, rank)
        if hi > lo:
            idx, cnt = o.reduce_mask(mask[lo:hi], *g.as_lists(), tol=0.5, op_fixup=False)
            n_local = int(cnt[0])
        else:
            idx, n_local = np.zeros((0, 3), np.int16), 0
        counts, _ = sd.all_gather_counts(torch.tensor([n_local], dtype=torch.int32))
        offs = sd.block_offsets(counts.tolist())
        glob = sd.to_global_indices(torch.from_numpy(np.ascontiguousarray(idx)), n_local, lo)
        q.put((rank, counts.tolist(), offs, glob.tolist()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_images", [5, 1])
def test_sharded_reduce_mask_counts_and_indices(n_images, oracle_port):
    from sbnet_b200 import configs as cfg
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_images, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g = cfg.halo_geom(64, 48)
    mask = cfg.rect_union_mask(n_images, 64, 48, seed=9, occupancy=0.2, side=(4, 12))
    idx, cnt = oracle_port.reduce_mask(mask, *g.as_lists(), tol=0.5, op_fixup=False)
    full = sorted(map(tuple, idx[: int(cnt[0])].tolist()))
    assert results[0][1] == results[1][1]                       # every rank sees the same counts
    assert sum(results[0][1]) == int(cnt[0])
    assert results[0][2] == [0, results[0][1][0]]
    merged = sorted(map(tuple, results[0][3] + results[1][3]))
    assert merged == full


def test_shard_bounds_cover_the_batch():
    from sbnet_b200.dist import shard_bounds
    for n in (0, 1, 7, 32):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _exchange_worker(rank, world, port, steps, depth, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sbnet_b200 import dist as sd
        ex = sd.CountExchange("cpu", depth=depth, timeout_s=60)
        for i in range(steps):
            slot = ex.slot(i)
            assert slot.numel() == 4 and int(slot[2]) == 0 and int(slot[3]) == 0
            slot[0] = 1000 * (rank + 1) + i          # what reduce_mask would publish
            ex.step_done(i, steps)
        q.put((rank, ex.finish()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("steps,depth", [(19, 4), (8, 8), (3, 8)])
def test_batched_count_exchange_delivers_every_step(steps, depth):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_worker, args=(r, world, port, steps, depth, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0] == results[1]
    for i in range(steps):
        assert results[0][i] == [1000 + i, 2000 + i]


def _absent_peer_worker(rank, world, port, q):
    """Rank 1 joins the process group and then never calls the exchange (it sits out, as a rank stuck
    in its own work would); rank 0 must get RankFailure after its timeout, not wait for ever."""
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sbnet_b200 import dist as sd
    if rank == 1:
        time.sleep(6.0)        # between steps, nothing in flight; then leaves without the collective
        q.put((1, "left", 0.0))
        q.close()
        q.join_thread()
        os._exit(0)
    t0 = time.time()
    try:
        sd.all_gather_counts(torch.tensor([7], dtype=torch.int32), timeout_s=1.5)
        q.put((0, "returned", time.time() - t0))
    except sd.RankFailure as e:
        q.put((0, "RankFailure: " + str(e)[:80], time.time() - t0))
    q.close()
    q.join_thread()
    os._exit(0)                # the group cannot be torn down collectively any more


def test_a_rank_that_never_joins_becomes_an_error_on_the_others():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict((r, (what, dt)) for r, what, dt in (q.get(timeout=120) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
    assert got[0][0].startswith("RankFailure"), got
    assert 1.0 <= got[0][1] < 5.5, got           # after its own timeout, well before the peer left
