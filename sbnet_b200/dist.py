"""Batch sharding of the block-op pipeline over the GPUs of one node.

Every op of the path is independent per image (a block never crosses images), so the path shards
over batch N with no data-path exchange: one process per GPU, rank r owns a contiguous slice of the
batch and runs reduce_mask -> gather -> ... -> scatter on it with rank-local image indices.  The only
exchange is an all-gather of one int32 per rank -- the per-rank block counts -- which gives the global
block count and each rank's offset in a notional global block list.  The reference has no
counterpart (it is single-GPU); this module is host-side plumbing over ``torch.distributed`` (NCCL
for device tensors, gloo for CPU tests).
"""
from __future__ import annotations

import datetime
import time
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class RankFailure(RuntimeError):
    """A peer did not take part in the count exchange within the time allowed (it never joined, died,
    or is stuck).  The reference has one process and no such case; its convention for any failure is to
    print and ``exit()`` (``sbnet_ops/op_utils.h:27-37``).  Here the survivors get an exception they can act on
    between steps, with nothing of theirs in flight on the GPU."""


def shard_bounds(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous ``[start, stop)`` slice of ``n_items`` for ``rank``; the first ``n_items % world``
    ranks get one extra item, empty slices are possible when ``world > n_items``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def wait_for(work, timeout_s: Optional[float] = None, what: str = "count exchange") -> None:
    """Waits for an asynchronous collective.  With ``timeout_s`` a peer that does not show up turns into
    :class:`RankFailure` after that many seconds instead of a wait without end (host-side collectives
    honour the timeout directly; NCCL work is additionally bounded by the process group's own timeout,
    given to ``init_process_group``)."""
    if work is None:
        return
    try:
        if timeout_s is None:
            work.wait()
        else:
            ok = work.wait(datetime.timedelta(seconds=float(timeout_s)))
            if ok is False:
                raise RankFailure(f"{what}: not complete after {timeout_s} s")
    except RankFailure:
        raise
    except RuntimeError as e:   # gloo / NCCL report a timeout or a lost peer as RuntimeError
        raise RankFailure(f"{what}: {e}") from e


def all_gather_counts(count: torch.Tensor, group=None, async_op: bool = False, timeout_s: Optional[float] = None):
    """All-gathers one int32 per rank.  ``count`` is a 1-element int32 tensor (device tensor for NCCL,
    e.g. the device count published by reduce_mask; CPU tensor for gloo).  Returns ``(counts, work)``:
    ``counts`` is an int32 tensor of ``world`` entries, valid once ``work`` (None if synchronous) is
    waited for (:func:`wait_for`).  A synchronous call with ``timeout_s`` raises :class:`RankFailure` when a
    peer does not join in time."""
    world = dist.get_world_size(group)
    out = torch.empty(world, dtype=torch.int32, device=count.device)
    work = dist.all_gather_into_tensor(out, count.reshape(1).to(torch.int32), group=group, async_op=True)
    if async_op:
        return out, work
    wait_for(work, timeout_s)
    return out, None


class CountExchange:
    """Exchange of the per-step block counts of a pipelined loop, batched so that no step waits for it.

    Every step's reduce_mask publishes its count into a scratch slot of its own (``slot(step)``, to be
    passed as the op's scratch); slots form rings of ``depth`` steps, and after the last step of a ring
    ONE all-gather moves the whole ring (``16 * depth`` bytes per rank).  Two rings alternate, so the
    wait for a ring's all-gather happens ``depth`` steps later, just before its slots are reused --
    by then it has long finished, and no rank ever waits for a slower peer inside a step.  On a CUDA
    device the collective is issued on a side stream behind an event recorded after the step's last
    launch, so its kernel does not run beside the step's own kernels, and nothing here ever blocks
    the HOST inside the loop: the stream that rewrites a ring's slots waits for the exchange in stream
    order (a host that waits for a collective with a timeout is put to sleep a millisecond at a time
    by the process-group library -- longer than the few queued steps of a short loop last, which
    would drain the GPU's queue every ring).  ``timeout_s`` is then enforced where the host may wait:
    in ``finish()``, and on an exchange still incomplete when its ring comes round a second time.
    Building one is collective on a CUDA device (it runs a first, empty exchange).
    """

    SLOT = 4   # int32 words of one reduce_mask scratch slot; word 0 is the count

    def __init__(self, device, depth: int = 8, group=None, timeout_s: Optional[float] = None):
        self.device, self.depth, self.group, self.timeout_s = torch.device(device), int(depth), group, timeout_s
        self.world = dist.get_world_size(group)
        n = self.depth * self.SLOT
        self.rings = [torch.zeros(n, dtype=torch.int32, device=self.device) for _ in range(2)]
        self.slots = [[r[k * self.SLOT:(k + 1) * self.SLOT] for k in range(self.depth)] for r in self.rings]
        self.gathered = [torch.zeros(self.world * n, dtype=torch.int32, device=self.device) for _ in range(2)]
        self.work = [None, None]          # CPU: the collective's work; CUDA: (done event, count table)
        self.pending = []                 # CUDA: (done event, time it was handed to a stream) not yet seen complete
        self.first_step = [None, None]
        self.history: List[torch.Tensor] = []    # [world, depth] count tables of finished rings
        self.side = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        if self.side is not None:
            # One exchange of each ring before any step (the constructor is therefore collective: every rank
            # builds its CountExchange at the same point).  The first collective on a new stream and the first
            # allocation under it take 0.6 ms and at times tens of ms of host time (measured), more than the few
            # queued steps of a short loop last; afterwards an exchange costs the host about 0.1 ms.
            with torch.cuda.stream(self.side):
                for b in range(2):
                    work = dist.all_gather_into_tensor(self.gathered[b], self.rings[b], group=self.group, async_op=True)
                    work.wait()
                    self.gathered[b].view(self.world, self.depth, self.SLOT)[:, :, 0].clone()
            self.side.synchronize()

    def slot(self, step: int, stream=None) -> torch.Tensor:
        """The 4-word scratch slot of ``step``.  The exchange that last read this slot's ring is waited
        for first: by the host on a CPU group, in stream order on a GPU -- ``stream`` is the torch stream
        the reduce_mask writing the slot will run on (default: the current stream)."""
        b, k = (step // self.depth) % 2, step % self.depth
        if k == 0:
            self._collect(b, stream)
        return self.slots[b][k]

    def step_done(self, step: int, steps_total: Optional[int] = None) -> None:
        """Call after the step's last launch.  Starts the ring's all-gather when the ring is full (or
        when ``step`` is the last of ``steps_total``)."""
        b, k = (step // self.depth) % 2, step % self.depth
        last = steps_total is not None and step == steps_total - 1
        if k != self.depth - 1 and not last:
            return
        self.first_step[b] = step - k
        if self.side is not None:
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(self.side):
                self.side.wait_event(ev)
                work = dist.all_gather_into_tensor(self.gathered[b], self.rings[b], group=self.group, async_op=True)
                work.wait()   # no timeout: the side STREAM waits for the collective, the host does not
                table = self.gathered[b].view(self.world, self.depth, self.SLOT)[:, :, 0].clone()
                done = torch.cuda.Event()
                done.record(self.side)
            self.work[b] = (done, table)
        else:
            self.work[b] = dist.all_gather_into_tensor(self.gathered[b], self.rings[b], group=self.group, async_op=True)

    def _host_wait(self, done, since: float) -> None:
        """Host-side wait for an exchange's event, bounded by ``timeout_s`` counted from ``since``."""
        while not done.query():
            if self.timeout_s is not None and time.time() - since > self.timeout_s:
                raise RankFailure(f"count exchange: not complete after {self.timeout_s} s")
            time.sleep(0.0005)

    def _collect(self, b: int, stream=None) -> None:
        if self.work[b] is None:
            return
        if self.side is None:
            wait_for(self.work[b], self.timeout_s)
            table = self.gathered[b].view(self.world, self.depth, self.SLOT)[:, :, 0].clone()
        else:
            done, table = self.work[b]
            # an exchange handed to a stream a whole round of both rings ago must be complete by now
            for ev, since in self.pending:
                self._host_wait(ev, since)
            self.pending = []
            if not done.query():
                (stream if stream is not None else torch.cuda.current_stream(self.device)).wait_event(done)
                self.pending.append((done, time.time()))
        self.work[b] = None
        self.history.append((self.first_step[b], table))

    def finish(self):
        """Waits for what is outstanding and returns ``{step: [count of rank 0, count of rank 1, ...]}``
        for every step exchanged so far (a partly filled last ring reports its unused slots as 0)."""
        for b in range(2):
            self._collect(b)
        for ev, since in self.pending:
            self._host_wait(ev, since)
        self.pending = []
        if self.side is not None:
            self.side.synchronize()
        out = {}
        for first, table in self.history:
            t = table.cpu().tolist()
            for k in range(self.depth):
                out[first + k] = [t[r][k] for r in range(self.world)]
        return out


def block_offsets(counts: Sequence[int]) -> List[int]:
    """Exclusive prefix sum: where each rank's blocks start in the global block list."""
    out, total = [], 0
    for c in counts:
        out.append(total)
        total += int(c)
    return out


def to_global_indices(local_indices: torch.Tensor, count: int, batch_start: int) -> torch.Tensor:
    """Rank-local ``(n, bh, bw)`` triples -> global ones (adds the rank's first image index)."""
    g = local_indices[:count].clone()
    g[:, 0] += batch_start
    return g
