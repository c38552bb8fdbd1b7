"""The reference's op interface on torch CUDA tensors, backed by the C ABI.

Names, argument order and meaning follow the registered TensorFlow ops
(``sbnet_ops/reduce_mask.cc:100-110``, ``sbnet_ops/sparse_gather.cc:48-57,242-268``) as the reference's
callers use them (``benchmark/sparse_conv_lib.py:452-459,547-587``): geometry is passed as length-2
``[H, W]`` host sequences, ``bin_counts`` is a length-1 int32 HOST tensor, ``active_block_indices`` is
a ``[N*bCntH*bCntW, 3]`` int16 device tensor.  torch is used for device memory and the current stream
only; every computation happens in ``libsbnet_b200.so``.
"""
from __future__ import annotations

import ctypes as C
import threading
from collections import namedtuple
from typing import Sequence

import torch

from . import lib as _lib

ReduceMaskResult = namedtuple("ReduceMask", ["active_block_indices", "bin_counts"])

_DTYPES = {torch.float32: _lib.SBNET_F32, torch.float16: _lib.SBNET_F16, torch.bfloat16: _lib.SBNET_BF16}
_scratch: dict = {}


class _on:
    """Makes a tensor's device current for the call; free when it already is (the usual case)."""

    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()

    def __enter__(self):
        self.prev = torch.cuda.current_device()
        if self.prev != self.idx:
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev != self.idx:
            torch.cuda.set_device(self.prev)


def _pair(v, name) -> tuple:
    if type(v) in (tuple, list) and len(v) == 2 and type(v[0]) is int and type(v[1]) is int:
        return v[0], v[1]
    if isinstance(v, torch.Tensor):
        v = v.detach().cpu().tolist()
    v = list(v)
    if len(v) != 2:  # reduce_mask.cc:132-138, sparse_gather.cc:170-175
        raise ValueError(f"{name} should be one-dimensional with shape[0] == 2.")
    return int(v[0]), int(v[1])


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device) -> int:
    """Handle of torch's current stream on ``device`` (the raw getter skips building a Stream object)."""
    if _raw_stream is not None:
        idx = device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path in this library)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _check_mask(mask: torch.Tensor):
    """Shape / dtype rules of the ReduceMask input (``sbnet_ops/reduce_mask.cc:140-143``); device-free,
    so they can be exercised without a GPU.  Returns (N, H, W)."""
    if mask.dtype != torch.float32:
        raise ValueError("mask must be float32")
    if mask.dim() not in (3, 4) or (mask.dim() == 4 and mask.shape[3] != 1):
        raise ValueError("mask must be [N,H,W,1]")
    if not mask.is_contiguous():
        raise ValueError("mask must be contiguous")
    return mask.shape[0], mask.shape[1], mask.shape[2]


def _check_indices(active_block_indices: torch.Tensor, rows: int) -> None:
    """``active_block_indices`` is int16 ``[>= rows, 3]``, contiguous: every kernel reads ``rows`` triples."""
    a = active_block_indices
    if a.dtype != torch.int16:
        raise ValueError("active_block_indices must be int16")
    if a.dim() != 2 or a.shape[1] != 3 or not a.is_contiguous():
        raise ValueError("active_block_indices must be a contiguous [numBlocks, 3] tensor")
    if a.shape[0] < rows:
        raise ValueError(f"active_block_indices holds {a.shape[0]} rows, the call reads {rows}")


def _check_image(t: torch.Tensor, name: str):
    if t.dim() != 4:  # sparse_gather.cc:164, :327
        raise ValueError(f"{name} must be rank 4")
    if t.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return tuple(t.shape)


def _check_stack(t: torch.Tensor, name: str, blocks: int, block_elems: int, like: torch.Tensor) -> None:
    """A block stack (gather output / scatter input): same dtype and device as the image, contiguous,
    room for ``blocks`` blocks of ``block_elems`` elements."""
    if t.dtype != like.dtype:
        raise ValueError(f"{name} and the image tensor must share a dtype, got {t.dtype} and {like.dtype}")
    if t.device != like.device:
        raise ValueError(f"{name} and the image tensor must live on one device")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if t.numel() < blocks * block_elems:
        raise ValueError(f"{name} holds {t.numel()} elements, the call needs {blocks * block_elems}")


def _check_count_dev(count_dev: torch.Tensor, like: torch.Tensor) -> None:
    if not isinstance(count_dev, torch.Tensor) or count_dev.dtype != torch.int32 or count_dev.numel() < 1:
        raise ValueError("count_dev must be an int32 tensor with at least one element")
    if count_dev.device != like.device:
        raise ValueError("count_dev must live on the device of the tensors")


def _count(bin_counts) -> int:
    if isinstance(bin_counts, torch.Tensor):
        if bin_counts.is_cuda:
            raise ValueError("bin_counts lives in host memory (use the *_dyn functions for a device count)")
        if bin_counts.numel() == 1:
            return int(bin_counts.item())       # the usual case, without building a view first
        return int(bin_counts.reshape(-1)[0])
    return int(list(bin_counts)[0]) if not isinstance(bin_counts, int) else int(bin_counts)


_pinned_slab: list = [None, 0]
_pinned_lock = threading.Lock()


def _pinned_count() -> torch.Tensor:
    """A fresh one-element pinned int32 tensor.  Pinned allocations are slow, so slots are handed out
    from a slab of 1,024; every slot is used once (the caller keeps the returned view), and a slab
    is released by reference counting when the last of its views is gone."""
    with _pinned_lock:
        slab, used = _pinned_slab
        if slab is None or used >= slab.numel():
            slab, used = torch.empty(1024, dtype=torch.int32, pin_memory=True), 0
        _pinned_slab[0], _pinned_slab[1] = slab, used + 1
    return slab[used:used + 1]


_SLOTS = 1024


def scratch_for(device, stream: int) -> tuple:
    """A fresh, zero-filled reduce_mask scratch slot (4 int32, 16-byte aligned) for ``(device, stream)``
    and the flag that says so.  Slots come from a slab of 1,024 that is zero-filled once on that stream;
    every slot is handed out once, so word 0 -- where the kernel publishes the count -- stays an
    independent device-side count for as long as the caller keeps the returned view (two results in
    flight on one stream never alias).  A slab is released when the last view of it is gone.  A slab
    that had to be created while the stream was being captured into a CUDA graph belongs to that graph
    (its zero fill is a node of the graph) and is not reused by later calls outside the capture."""
    key = (device.index if isinstance(device, torch.device) else torch.device(device).index, stream)
    capturing = torch.cuda.is_current_stream_capturing()
    hit = _scratch.get(key)
    if hit is None or hit[1] >= _SLOTS or (hit[2] and not capturing):
        hit = [torch.zeros(_SLOTS * _lib.SBNET_REDUCE_MASK_SCRATCH_INTS, dtype=torch.int32, device=device), 0, capturing]
        _scratch[key] = hit
    k = hit[1]
    hit[1] = k + 1
    n = _lib.SBNET_REDUCE_MASK_SCRATCH_INTS
    return hit[0][k * n:(k + 1) * n], _lib.SBNET_SCRATCH_CLEAN


def _reduce_mask_call(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol, avgpool,
                      counts, flags, scratch=None):
    _require_cuda(mask, "mask")
    N, H, W = _check_mask(mask)
    bch, bcw = _pair(dynamic_bcount, "dynamic_bcount")
    bsh, bsw = _pair(dynamic_bsize, "dynamic_bsize")
    bth, btw = _pair(dynamic_bstride, "dynamic_bstride")
    boh, bow = _pair(dynamic_boffset, "dynamic_boffset")
    with _on(mask.device):
        stream = _stream(mask.device)
        idx = torch.empty((max(N * bch * bcw, 0), 3), dtype=torch.int16, device=mask.device)
        if scratch is None:
            scratch, clean = scratch_for(mask.device, stream)
        else:   # a slot of the caller's (e.g. one of a ring that is exchanged between ranks): zero-filled once
            if scratch.dtype != torch.int32 or scratch.numel() < _lib.SBNET_REDUCE_MASK_SCRATCH_INTS or \
                    scratch.device != mask.device or not scratch.is_contiguous():
                raise ValueError("scratch must be a contiguous int32 device tensor of at least 4 elements")
            clean = _lib.SBNET_SCRATCH_CLEAN
        _lib.check(_lib.load().sbnet_reduce_mask(
            mask.data_ptr(), N, H, W, float(tol), int(bool(avgpool)), boh, bow, bsh, bsw, bth, btw,
            bch, bcw, idx.data_ptr(), scratch.data_ptr(), None if counts is None else counts.data_ptr(),
            flags | clean, stream))
    return idx, scratch[:1]


def reduce_mask(mask: torch.Tensor, dynamic_bcount: Sequence[int], dynamic_bsize: Sequence[int],
                dynamic_bstride: Sequence[int], dynamic_boffset: Sequence[int], tol: float,
                avgpool: bool = False, mask_stable: bool = False, yield_core: bool = False) -> ReduceMaskResult:
    """``ReduceMask``: pools ``mask`` ([N,H,W,1] or [N,H,W] fp32) per block and lists the active blocks.

    Returns ``(active_block_indices, bin_counts)``; ``bin_counts`` is a pinned host tensor whose value
    is final when the call returns (the op interface requires the count on the host).
    ``mask_stable=True`` promises that the mask is not written by the operation queued just before this
    call on the current stream, which lets the kernel read it while that operation drains
    (``SBNET_MASK_STABLE``); ``yield_core=True`` makes the wait for the count give its core away between
    looks (``SBNET_COUNT_YIELD``: one process per GPU on shared cores)."""
    _require_cuda(mask, "mask")   # before the pinned slot: a host mask must fail as an argument error
    counts = _pinned_count()
    flags = _lib.SBNET_COUNT_POLL | (_lib.SBNET_MASK_STABLE if mask_stable else 0) \
        | (_lib.SBNET_COUNT_YIELD if yield_core else 0)
    idx, _ = _reduce_mask_call(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                               avgpool, counts, flags)
    return ReduceMaskResult(idx, counts)


def reduce_mask_with_device_count(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                                  avgpool=False, mask_stable=False, yield_core=False, scratch=None):
    """:func:`reduce_mask` that also returns the count as a one-element device tensor (for a count
    exchange between ranks, or for the ``*_dyn`` calls): ``(active_block_indices, bin_counts, count_dev)``.
    ``scratch``: a 16-byte aligned, zero-filled int32 device tensor of 4 elements owned by the caller,
    whose word 0 then receives the count (words 2..3 are left at zero, so the slot can be used again by
    a later call on the same stream)."""
    _require_cuda(mask, "mask")   # before the pinned slot: a host mask must fail as an argument error
    counts = _pinned_count()
    flags = _lib.SBNET_COUNT_POLL | (_lib.SBNET_MASK_STABLE if mask_stable else 0) \
        | (_lib.SBNET_COUNT_YIELD if yield_core else 0)
    idx, count_dev = _reduce_mask_call(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                                       tol, avgpool, counts, flags, scratch)
    return idx, counts, count_dev


def reduce_mask_async(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                      avgpool=False, mask_stable=False):
    """Same as :func:`reduce_mask` but never touches the host: returns ``(active_block_indices,
    count_dev)`` where ``count_dev`` is a one-element device int32 tensor that holds the count in stream
    order, for the ``*_dyn`` gather / scatter calls.  Every call gets a count word of its own, so results
    of several calls may be outstanding at once."""
    return _reduce_mask_call(mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                             avgpool, None, _lib.SBNET_MASK_STABLE if mask_stable else 0)


def _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset):
    bsh, bsw = _pair(dynamic_bsize, "dynamic_bsize")
    bth, btw = _pair(dynamic_bstride, "dynamic_bstride")
    boh, bow = _pair(dynamic_boffset, "dynamic_boffset")
    return (boh, bow, bsh, bsw, bth, btw)


def sparse_gather(x: torch.Tensor, bin_counts, active_block_indices: torch.Tensor, dynamic_bsize,
                  dynamic_bstride, dynamic_boffset, transpose: bool = False, out=None) -> torch.Tensor:
    """``SparseGather``: ``[bin_counts[0], bSzH, bSzW, C]``, or ``[bin_counts[0], C, bSzH, bSzW]`` when
    ``transpose``; pixels outside ``x`` read as zero."""
    _require_cuda(x, "x")
    _require_cuda(active_block_indices, "active_block_indices")
    N, H, W, Cc = _check_image(x, "x")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    nb = _count(bin_counts)
    _check_indices(active_block_indices, nb)
    shape = (nb, Cc, g[2], g[3]) if transpose else (nb, g[2], g[3], Cc)
    if out is not None:
        _require_cuda(out, "out")
        _check_stack(out, "out", nb, g[2] * g[3] * Cc, x)
    with _on(x.device):
        y = out if out is not None else torch.empty(shape, dtype=x.dtype, device=x.device)
        _lib.check(_lib.load().sbnet_sparse_gather(
            x.data_ptr(), _DTYPES[x.dtype], N, H, W, Cc, y.data_ptr(), *g, nb,
            active_block_indices.data_ptr(), int(bool(transpose)), _stream(x.device)))
    return y


def sparse_scatter_var(x: torch.Tensor, bin_counts, active_block_indices: torch.Tensor,
                       ybase: torch.Tensor, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                       add: bool, atomic: bool = False, transpose: bool = False) -> torch.Tensor:
    """``SparseScatterVar``: writes (``add=False``) or accumulates (``add=True``) the block stack ``x``
    into ``ybase`` in place and returns it."""
    _require_cuda(x, "x")
    _require_cuda(ybase, "ybase")
    _require_cuda(active_block_indices, "active_block_indices")
    N, H, W, Cc = _check_image(ybase, "ybase")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    nb = _count(bin_counts)
    _check_indices(active_block_indices, nb)
    _check_stack(x, "x", nb, g[2] * g[3] * Cc, ybase)
    if x.numel() != nb * g[2] * g[3] * Cc:
        raise ValueError("x must hold bin_counts[0]*bsize[0]*bsize[1]*C elements")
    with _on(ybase.device):
        _lib.check(_lib.load().sbnet_sparse_scatter(
            x.data_ptr(), _DTYPES[ybase.dtype], N, H, W, Cc, ybase.data_ptr(), *g, nb,
            active_block_indices.data_ptr(), int(bool(add)), int(bool(transpose)),
            int(bool(atomic)), _stream(ybase.device)))
    return ybase


def copy_tensor(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    _require_cuda(dst, "dst")
    _require_cuda(src, "src")
    nbytes = src.numel() * src.element_size()
    if dst.numel() * dst.element_size() != nbytes:
        raise ValueError("size mismatch")
    with _on(dst.device):
        _lib.check(_lib.load().sbnet_copy_tensor(dst.data_ptr(), src.data_ptr(), nbytes,
                                                 _stream(dst.device)))
    return dst


def sparse_scatter(x, bin_counts, active_block_indices, ybase, dynamic_bsize, dynamic_bstride,
                   dynamic_boffset, add: bool, atomic: bool = False, transpose: bool = False):
    """``SparseScatter``: like :func:`sparse_scatter_var` on a fresh copy of ``ybase``
    (``sbnet_ops/sparse_gather.cc:338-347``)."""
    _require_cuda(ybase, "ybase")
    if ybase.dim() != 4:
        raise ValueError("ybase must be rank 4")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    if add and not atomic and not (g[4] >= g[2] and g[5] >= g[3]):  # reject before allocating
        raise ValueError("SparseScatter: Only non-overlapping blocks are supported with add=True, atomic=False")
    y = copy_tensor(torch.empty_like(ybase), ybase)
    return sparse_scatter_var(x, bin_counts, active_block_indices, y, dynamic_bsize, dynamic_bstride,
                              dynamic_boffset, add=add, atomic=atomic, transpose=transpose)


def sparse_gather_dyn(x, count_dev: torch.Tensor, max_blocks: int, active_block_indices, dynamic_bsize,
                      dynamic_bstride, dynamic_boffset, transpose=False, out=None):
    """Gather with the block count read on the device (no host synchronisation).  The result has
    room for ``max_blocks`` blocks; only the first ``count_dev[0]`` are written."""
    _require_cuda(x, "x")
    _require_cuda(active_block_indices, "active_block_indices")
    N, H, W, Cc = _check_image(x, "x")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    max_blocks = int(max_blocks)
    _check_count_dev(count_dev, x)
    _check_indices(active_block_indices, max_blocks)
    shape = (max_blocks, Cc, g[2], g[3]) if transpose else (max_blocks, g[2], g[3], Cc)
    if out is not None:
        _require_cuda(out, "out")
        _check_stack(out, "out", max_blocks, g[2] * g[3] * Cc, x)
    with _on(x.device):
        y = out if out is not None else torch.empty(shape, dtype=x.dtype, device=x.device)
        _lib.check(_lib.load().sbnet_sparse_gather_dyn(
            x.data_ptr(), _DTYPES[x.dtype], N, H, W, Cc, y.data_ptr(), *g, int(max_blocks),
            count_dev.data_ptr(), active_block_indices.data_ptr(), int(bool(transpose)),
            _stream(x.device)))
    return y


def sparse_scatter_var_dyn(x, count_dev: torch.Tensor, max_blocks: int, active_block_indices, ybase,
                           dynamic_bsize, dynamic_bstride, dynamic_boffset, add, atomic=False,
                           transpose=False):
    """Scatter with the block count read on the device; ``x`` has room for ``max_blocks`` blocks."""
    _require_cuda(ybase, "ybase")
    _require_cuda(x, "x")
    _require_cuda(active_block_indices, "active_block_indices")
    N, H, W, Cc = _check_image(ybase, "ybase")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    max_blocks = int(max_blocks)
    _check_count_dev(count_dev, ybase)
    _check_indices(active_block_indices, max_blocks)
    _check_stack(x, "x", max_blocks, g[2] * g[3] * Cc, ybase)
    with _on(ybase.device):
        _lib.check(_lib.load().sbnet_sparse_scatter_dyn(
            x.data_ptr(), _DTYPES[ybase.dtype], N, H, W, Cc, ybase.data_ptr(), *g, int(max_blocks),
            count_dev.data_ptr(), active_block_indices.data_ptr(), int(bool(add)),
            int(bool(transpose)), int(bool(atomic)), _stream(ybase.device)))
    return ybase


# ---- pre-validated calls for hot loops ---------------------------------------------------------------
# The wrappers above re-check every argument on every call (about 7 us of interpreter time each, beside
# the ~5 us of the foreign call itself).  A loop that calls the same op on the same buffers with the
# same geometry -- every layer of a network at inference time -- can bind those once: the returned
# function takes only what changes from call to call.  Same library entry points, same results.

def count_ready(bin_counts: torch.Tensor) -> bool:
    """True once the kernel of a ``wait=False`` reduce_mask call has stored its count."""
    return int(bin_counts[0]) != _lib.SBNET_COUNT_PENDING


def wait_count(bin_counts: torch.Tensor, timeout_s: float = 10.0) -> int:
    """Spins until the count of a ``wait=False`` reduce_mask call is on the host and returns it."""
    n = int(bin_counts[0])
    if n != _lib.SBNET_COUNT_PENDING:
        return n
    import time
    t0 = time.perf_counter()
    while True:
        n = int(bin_counts[0])
        if n != _lib.SBNET_COUNT_PENDING:
            return n
        if time.perf_counter() - t0 > timeout_s:
            raise RuntimeError(f"reduce_mask count not delivered within {timeout_s} s")


def bind_reduce_mask(mask_like: torch.Tensor, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                     avgpool=False, mask_stable=False, yield_core=False, stream: int = None, wait: bool = True):
    """Returns ``call(mask, scratch=None, out=None) -> (active_block_indices, bin_counts, count_dev)`` for
    masks of ``mask_like``'s shape, dtype and device.  ``stream``: raw handle of the stream to launch on
    (default: torch's current stream at call time).  Every call takes a fresh pinned count and (unless
    ``scratch`` is given) a fresh scratch slot, as :func:`reduce_mask` does, and allocates its index list
    unless ``out`` (int16 ``[N*bcount_h*bcount_w, 3]``, contiguous) is given: a caller that rotates a few
    such buffers keeps the caching allocator out of its steps, and orders their reuse itself.
    ``wait=False``: the call returns right after the launch (``SBNET_COUNT_NOWAIT``); ``bin_counts`` holds
    the count once :func:`count_ready` says so (:func:`wait_count` spins for it)."""
    _require_cuda(mask_like, "mask")
    N, H, W = _check_mask(mask_like)
    bch, bcw = _pair(dynamic_bcount, "dynamic_bcount")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    device, shape = mask_like.device, tuple(mask_like.shape)
    rows = max(N * bch * bcw, 0)
    flags = _lib.SBNET_SCRATCH_CLEAN | (_lib.SBNET_MASK_STABLE if mask_stable else 0) \
        | ((_lib.SBNET_COUNT_POLL | (_lib.SBNET_COUNT_YIELD if yield_core else 0)) if wait else _lib.SBNET_COUNT_NOWAIT)
    fn = _lib.load().sbnet_reduce_mask
    head = (N, H, W, float(tol), int(bool(avgpool)), *g, bch, bcw)
    n_scratch = _lib.SBNET_REDUCE_MASK_SCRATCH_INTS

    def call(mask, scratch=None, out=None):
        if tuple(mask.shape) != shape or mask.dtype != torch.float32 or mask.device != device or not mask.is_contiguous():
            raise ValueError("mask differs from the one this call was bound for")
        st = stream if stream is not None else _stream(device)
        if out is None:
            idx = torch.empty((rows, 3), dtype=torch.int16, device=device)
        elif out.dtype != torch.int16 or tuple(out.shape) != (rows, 3) or out.device != device or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous int16 [{rows}, 3] tensor on the mask's device")
        else:
            idx = out
        counts = _pinned_count()
        if scratch is None:
            scratch = scratch_for(device, st)[0]
        elif scratch.dtype != torch.int32 or scratch.numel() < n_scratch or scratch.device != device:
            raise ValueError("scratch must be an int32 device tensor of at least 4 elements")
        _lib.check(fn(mask.data_ptr(), *head, idx.data_ptr(), scratch.data_ptr(), counts.data_ptr(), flags, st))
        return idx, counts, scratch[:1]
    return call


def bind_sparse_gather(x: torch.Tensor, out: torch.Tensor, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                       transpose=False, stream: int = None):
    """Returns ``call(bin_counts, active_block_indices) -> out`` gathering from ``x`` into ``out`` (room for
    the largest count that will be passed; checked per call)."""
    _require_cuda(x, "x")
    _require_cuda(out, "out")
    N, H, W, Cc = _check_image(x, "x")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    block = g[2] * g[3] * Cc
    _check_stack(out, "out", 0, block, x)
    cap = out.numel() // block
    device = x.device
    fn = _lib.load().sbnet_sparse_gather
    head = (x.data_ptr(), _DTYPES[x.dtype], N, H, W, Cc, out.data_ptr(), *g)
    tr = int(bool(transpose))
    keep = (x, out)   # the bound buffers stay alive as long as the call does

    def call(bin_counts, active_block_indices):
        nb = _count(bin_counts)
        if nb > cap:
            raise ValueError(f"out holds {cap} blocks, the call needs {nb}")
        a = active_block_indices
        if a.dtype != torch.int16 or a.device != device or a.shape[0] < nb or not a.is_contiguous():
            raise ValueError("active_block_indices must be a contiguous int16 [>= count, 3] tensor on the image's device")
        _lib.check(fn(*head, nb, a.data_ptr(), tr, stream if stream is not None else _stream(device)))
        return keep[1]
    return call


def bind_sparse_scatter_var(x: torch.Tensor, ybase: torch.Tensor, dynamic_bsize, dynamic_bstride, dynamic_boffset,
                            add: bool, atomic=False, transpose=False, stream: int = None):
    """Returns ``call(bin_counts, active_block_indices) -> ybase`` scattering the first ``bin_counts[0]``
    blocks of the stack ``x`` into ``ybase`` in place."""
    _require_cuda(x, "x")
    _require_cuda(ybase, "ybase")
    N, H, W, Cc = _check_image(ybase, "ybase")
    g = _geom(dynamic_bsize, dynamic_bstride, dynamic_boffset)
    block = g[2] * g[3] * Cc
    _check_stack(x, "x", 0, block, ybase)
    cap = x.numel() // block
    device = ybase.device
    fn = _lib.load().sbnet_sparse_scatter
    head = (x.data_ptr(), _DTYPES[ybase.dtype], N, H, W, Cc, ybase.data_ptr(), *g)
    tail = (int(bool(add)), int(bool(transpose)), int(bool(atomic)))
    keep = (x, ybase)

    def call(bin_counts, active_block_indices):
        nb = _count(bin_counts)
        if nb > cap:
            raise ValueError(f"x holds {cap} blocks, the call needs {nb}")
        a = active_block_indices
        if a.dtype != torch.int16 or a.device != device or a.shape[0] < nb or not a.is_contiguous():
            raise ValueError("active_block_indices must be a contiguous int16 [>= count, 3] tensor on the image's device")
        _lib.check(fn(*head, nb, a.data_ptr(), *tail, stream if stream is not None else _stream(device)))
        return keep[1]
    return call


def cuda_timer_start() -> int:
    """``CudaTimerStart``: returns an event handle (``sbnet_ops/sparse_gather.cc:398-423``)."""
    h = C.c_int64(0)
    _lib.check(_lib.load().sbnet_cuda_timer_start(C.byref(h)))
    return h.value


def cuda_timer_end(handle: int) -> float:
    """``CudaTimerEnd``: milliseconds since the matching start (``sbnet_ops/sparse_gather.cc:425-461``)."""
    ms = C.c_float(0.0)
    _lib.check(_lib.load().sbnet_cuda_timer_end(C.c_int64(handle), C.byref(ms)))
    return ms.value
