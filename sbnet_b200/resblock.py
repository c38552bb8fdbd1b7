"""Sparse ResNet bottleneck block on the block ops: y = x + F(x) evaluated only on active blocks.

Mirrors the structure of the reference's ``sparse_res_block_bottleneck``
(``benchmark/sparse_conv_lib.py:677-824``): sparse_gather of 18x18 (in general ``bsize``) windows ->
BN-ReLU-1x1, BN-ReLU-3x3 VALID, BN-ReLU-1x1 on the block stack (the host framework's dense ops, here
torch / cuDNN in NCHW, i.e. ``transpose=True``) -> sparse_scatter(add=True) of the ``bsize_out``
interiors onto the residual.  The convolutions are NOT part of this library; the module exists so
the op pipeline can be exercised and timed in its real setting.
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import autograd as sb
from . import geometry, ops


class SparseBottleneck(nn.Module):
    def __init__(self, channels: int, mid: int, bsize: Sequence[int] = (18, 18), dtype=torch.float16,
                 device="cuda"):
        super().__init__()
        self.channels, self.mid, self.bsize = channels, mid, tuple(bsize)
        kw = dict(device=device, dtype=dtype)
        self.bn = nn.ModuleList([nn.BatchNorm2d(channels, **kw), nn.BatchNorm2d(mid, **kw), nn.BatchNorm2d(mid, **kw)])
        self.conv1 = nn.Conv2d(channels, mid, 1, bias=False, **kw)
        self.conv2 = nn.Conv2d(mid, mid, 3, bias=False, **kw)          # VALID: 18x18 -> 16x16
        self.conv3 = nn.Conv2d(mid, channels, 1, bias=False, **kw)
        for c in (self.conv1, self.conv2, self.conv3):
            nn.init.kaiming_normal_(c.weight, nonlinearity="relu")

    def block_params(self, x_shape) -> geometry.BlockParams:
        N, H, W, C = x_shape
        ks = [[1, 1, C, self.mid], [3, 3, self.mid, self.mid], [1, 1, self.mid, C]]
        return geometry.calc_block_params_res_block([N, H, W, C], [1, *self.bsize, 1], ks, [1, 1, 1, 1], "SAME")

    def residual(self, p: torch.Tensor) -> torch.Tensor:
        q = self.conv1(F.relu(self.bn[0](p)))
        q = self.conv2(F.relu(self.bn[1](q)))
        return self.conv3(F.relu(self.bn[2](q)))

    def forward(self, x: torch.Tensor, mask: torch.Tensor, tol: float = 0.5, avgpool: bool = False):
        """``x`` NHWC, ``mask`` [N,H,W,1] fp32.  Returns NHWC ``x + F(x)`` on active blocks, ``x`` elsewhere."""
        bp = self.block_params(x.shape)
        idx, cnt = ops.reduce_mask(mask, bp.bcount, bp.bsize, bp.bstrides, bp.boffset, tol=tol, avgpool=avgpool)
        p = sb.sparse_gather(x, cnt, idx, bp.bsize, bp.bstrides, bp.boffset, transpose=True)
        q = self.residual(p).contiguous()
        return sb.sparse_scatter(q, cnt, idx, x, bp.bsize_out, bp.bsize_out, [0, 0], add=True, transpose=True)
