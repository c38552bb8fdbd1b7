"""Shared bar for accumulating scatters over overlapping blocks: the CUDA result AND the CPU
checker's result must each lie within k rounded additions of the fp64 sum of base and addends, and
meet the relative bar (1e-6 fp32, 1e-3 for a single 16-bit addend) where nothing cancels
(``oracle/exact.py``).  That shows the two differ by summation order alone."""
import numpy as np

from oracle import exact


def cover_of(bsize, bstride):
    return -(-int(bsize[0]) // int(bstride[0])) * -(-int(bsize[1]) // int(bstride[1]))


def to_numpy(t):
    if isinstance(t, np.ndarray):
        return t
    if isinstance(t, (list, tuple, int)):
        return np.asarray(t)
    from cuda_ops import to_numpy as torch_to_numpy
    return torch_to_numpy(t)


def check_atomic_add(results, stack, count, indices, base, bsize, bstride, boffset, transpose=False):
    """``results``: {name: array} of outcomes of the same accumulating scatter (``base`` is the value
    before it).  Returns {name: (worst bound ratio, worst relative error)}."""
    stack, base, indices = to_numpy(stack), to_numpy(base), to_numpy(indices)
    nb = int(np.asarray(to_numpy(count)).reshape(-1)[0])
    ex, mag, k = exact.exact_add(stack, nb, indices, base, bsize, bstride, boffset, transpose)
    cover = cover_of(bsize, bstride)
    assert int(k.max(initial=0)) <= cover
    return {name: exact.check_add(to_numpy(r), ex, mag, k, base, cover, what=name) for name, r in results.items()}
