"""The parameter sweep of the reference's op integration test, as data.

Each entry restates one ``runTestForOneSize`` call of
``sbnet_ops/tests/test_sparse_blocks.py:345-449`` (same layer size, block size ``RS``, stride ``UV``,
offset, sparsity percentile, add/atomic/avgpool flags, batch N, Var or non-Var scatter).  Inputs are
drawn exactly as that test draws them (``generateInputs``, ``:124-134``: ``np.random.seed(0)``,
``randn`` mask then ``randn`` x, ``tol = percentile(x, sparsity)``, base tensor of constant 10.0).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Tuple

import numpy as np


@dataclass(frozen=True)
class RefCase:
    name: str
    layer: Tuple[int, int, int]          # (H, W, C)
    RS: Tuple[int, int]                  # block size
    UV: Tuple[int, int]                  # block stride
    BOFFS: Tuple[int, int] = (-1, -2)    # the reference's default offset
    sparsity: float = 70
    do_add: bool = False
    N: int = 1
    test_var: bool = False
    avgpool: bool = False
    use_atomics: bool = False
    big: bool = False                    # too large for the quick CPU suite


def _count1d(size, bstride, boffset):
    return 1 + (size - boffset - 1) // bstride


def make_inputs(case: RefCase):
    np.random.seed(0)
    H, W, C = case.layer
    mask = np.random.randn(case.N, H, W, 1).astype(np.float32)
    x = np.random.randn(case.N, H, W, C).astype(np.float32)
    tol = np.float32(1e32) if case.sparsity == 100 else np.float32(np.percentile(x, case.sparsity))
    bcount = (_count1d(H, case.UV[0], case.BOFFS[0]), _count1d(W, case.UV[1], case.BOFFS[1]))
    return mask, x, float(tol), bcount


def _permutation_cases():
    out = []
    sizes = [(1, 1, 1), (1, 1, 2), (1, 2, 3), (2, 1, 3), (3, 2, 1), (1, 2, 1), (3, 2, 7)]
    for nn in (1, 7):
        for tv in (True, False):
            for avgpool in (True, False):
                for sp in (0, 10, 50, 99):
                    for sz in sizes:
                        out.append(RefCase(
                            f"perm_n{nn}_var{int(tv)}_avg{int(avgpool)}_sp{sp}_{sz[0]}x{sz[1]}x{sz[2]}",
                            sz, (1, 1), (1, 1), (0, 0), sparsity=sp, N=nn, test_var=tv,
                            avgpool=avgpool))
    # (1,1,1024*49) once per N / Var (the full cross product adds nothing but time)
    for nn in (1, 7):
        out.append(RefCase(f"perm_n{nn}_wideC", (1, 1, 1024 * 49), (1, 1), (1, 1), (0, 0),
                           sparsity=50, N=nn, test_var=bool(nn == 7)))
    return out


CASES = [
    RefCase("simple_2x3x2", (2, 3, 2), (2, 3), (3, 4)),
    RefCase("simple_5x5x1", (5, 5, 1), (3, 3), (1, 1)),
    RefCase("zero_block_count", (2, 2, 1), (1, 1), (1, 1), (0, 0), sparsity=100),
    RefCase("basic_2x2", (2, 2, 1), (1, 1), (1, 1), (0, 0), sparsity=0),
    RefCase("basic_2x2_n3", (2, 2, 1), (1, 1), (1, 1), (0, 0), sparsity=0, N=3),
    RefCase("basic_6x6", (6, 6, 1), (1, 1), (1, 1)),
    RefCase("overlap_3x3", (3, 3, 1), (2, 2), (1, 1), (0, 0), sparsity=0),
    RefCase("overlap_13x12", (13, 12, 1), (2, 3), (1, 2), (0, 0), sparsity=0.1),
] + [
    RefCase(f"sparsity_{sp}", (200, 300, 32), (3, 4), (2, 3), sparsity=sp, avgpool=True,
            use_atomics=True, big=(sp not in (50, 99)))
    for sp in (10, 20, 30, 40, 50, 70, 90, 99)
] + [
    RefCase("avg_holes_avg", (2, 3, 2), (2, 3), (3, 4), avgpool=True),
    RefCase("avg_holes_max", (2, 3, 2), (2, 3), (3, 4), avgpool=False),
] + [
    RefCase(f"channels_{cc}", (380, 480, cc), (18, 18), (18, 18), big=(cc not in (15, 16)))
    for cc in (15, 16, 24, 32, 48, 64)
] + [
    RefCase("channels_16x16", (200, 300, 32), (16, 16), (16, 16)),
] + _permutation_cases() + [
    RefCase("uneven_kernel", (8, 10, 7), (3, 4), (3, 4)),
    RefCase("gaps_1ch", (8, 10, 1), (3, 4), (4, 5)),
    RefCase("gaps_7ch", (8, 10, 7), (3, 4), (4, 5)),
    RefCase("uneven_boffs", (5, 5, 1), (3, 2), (3, 2), (-1, -2)),
    RefCase("uneven_nonoverlap_a", (5, 3, 1), (2, 3), (2, 3), (0, 0)),
    RefCase("uneven_nonoverlap_b", (5, 3, 1), (2, 3), (2, 3), (-1, -2)),
    RefCase("even_overlap", (3, 3, 1), (2, 2), (1, 1), (0, 0)),
    RefCase("holes", (3, 3, 1), (1, 1), (2, 2)),
    RefCase("large_blocks", (2048, 2048, 1), (1500, 490), (300, 390), use_atomics=True, big=True),
]

BY_NAME = {c.name: c for c in CASES}
assert len(BY_NAME) == len(CASES)
