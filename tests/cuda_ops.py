"""numpy-in / numpy-out adapter over the CUDA library's op interface, so the same case runners drive
either the CPU checker or the GPU.  Every call goes through the C ABI (sbnet_b200.ops -> ctypes)."""
from __future__ import annotations

import numpy as np
import torch

from sbnet_b200 import ops


def to_torch(a: np.ndarray) -> torch.Tensor:
    """numpy -> torch on the host; bfloat16 (``ml_dtypes``) crosses as its 16-bit pattern."""
    a = np.ascontiguousarray(a)
    if a.dtype.name == "bfloat16":
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(a)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.cpu()
    if t.dtype == torch.bfloat16:
        import ml_dtypes
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.numpy()


class CudaOps:
    kind = "cuda"

    def __init__(self, device="cuda:0", guard: bool = True):
        self.device = torch.device(device)
        self.guard = guard

    def _dev(self, a):
        return to_torch(a).to(self.device)

    def reduce_mask(self, mask, dynamic_bcount, dynamic_bsize, dynamic_bstride, dynamic_boffset, tol,
                    avgpool=False):
        idx, cnt = ops.reduce_mask(self._dev(np.asarray(mask, dtype=np.float32)), dynamic_bcount,
                                   dynamic_bsize, dynamic_bstride, dynamic_boffset, tol=tol,
                                   avgpool=avgpool)
        return idx.cpu().numpy(), cnt.numpy().copy()

    def sparse_gather(self, x, bin_counts, active_block_indices, dynamic_bsize, dynamic_bstride,
                      dynamic_boffset, transpose=False):
        y = ops.sparse_gather(self._dev(x), torch.from_numpy(np.asarray(bin_counts, dtype=np.int32)),
                              self._dev(np.asarray(active_block_indices, dtype=np.int16)),
                              dynamic_bsize, dynamic_bstride, dynamic_boffset, transpose=transpose)
        return to_numpy(y)

    def _scatter(self, fn, x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                 dynamic_bstride, dynamic_boffset, add, atomic, transpose):
        yb = np.ascontiguousarray(ybase)
        y = fn(self._dev(np.asarray(x, dtype=yb.dtype)),
               torch.from_numpy(np.asarray(bin_counts, dtype=np.int32)),
               self._dev(np.asarray(active_block_indices, dtype=np.int16)), self._dev(yb),
               dynamic_bsize, dynamic_bstride, dynamic_boffset, add=add, atomic=atomic,
               transpose=transpose)
        return to_numpy(y)

    def sparse_scatter(self, x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                       dynamic_bstride, dynamic_boffset, add, atomic=False, transpose=False):
        return self._scatter(ops.sparse_scatter, x, bin_counts, active_block_indices, ybase,
                             dynamic_bsize, dynamic_bstride, dynamic_boffset, add, atomic, transpose)

    def sparse_scatter_var(self, x, bin_counts, active_block_indices, ybase, dynamic_bsize,
                           dynamic_bstride, dynamic_boffset, add, atomic=False, transpose=False):
        out = self._scatter(ops.sparse_scatter_var, x, bin_counts, active_block_indices, ybase,
                            dynamic_bsize, dynamic_bstride, dynamic_boffset, add, atomic, transpose)
        if isinstance(ybase, np.ndarray) and ybase.flags["WRITEABLE"]:
            ybase[...] = out  # the Var op updates its argument
        return out
