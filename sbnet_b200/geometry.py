"""Block-geometry calculus: from a convolution's input size, block size, kernel size, stride and
padding mode to the ``bsize / bstride / boffset / bcount / bsize_out`` the block ops take.

Integer restatement of the reference's ``calc_block_params`` family
(``benchmark/sparse_conv_lib.py:237-246,343-421``) and of the SAME/VALID size and padding arithmetic
it relies on (``benchmark/tf_conv_dims.py:94-279``), for static shapes.  4-vectors follow the
reference's conventions: ``in_size = [N, H, W, C]``, ``bsize = [1, bh, bw, 1]``,
``ksize = [kh, kw, cin, cout]``, ``strides = [1, sh, sw, 1]``.
"""
from __future__ import annotations

from collections import namedtuple
from typing import List, Sequence, Tuple

BlockParams = namedtuple("BlockParams", ["bsize", "bsize_out", "boffset", "bcount", "bstrides"])


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def _check(ksize: Sequence[int], strides: Sequence[int]) -> None:
    if len(ksize) != 4:
        raise ValueError("Expect `ksize` a list/tuple of length 4.")
    if len(strides) != 4:
        raise ValueError("Expect `strides` a list/tuple of length 4.")
    if strides[0] != 1 or strides[3] != 1:
        raise ValueError("Expect first and last dimension of `strides` = 1.")


def calc_out_size_1d(in_size: int, ksize: int, stride: int, padding: str) -> int:
    """Output extent of a convolution along one axis (``tf_conv_dims.py:263-279``)."""
    if padding == "VALID":
        return _ceil_div(in_size - ksize + 1, stride)
    if padding == "SAME":
        return _ceil_div(in_size, stride)
    raise ValueError(f'Unknown padding method "{padding}"')


def calc_out_size_4d(in_shape: Sequence[int], ksize: Sequence[int], strides: Sequence[int],
                     padding: str) -> List[int]:
    _check(ksize, strides)
    return [in_shape[0], calc_out_size_1d(in_shape[1], ksize[0], strides[1], padding),
            calc_out_size_1d(in_shape[2], ksize[1], strides[2], padding), ksize[3]]


def calc_padding_1d(in_size: int, out_size: int, ksize: int, stride: int, padding: str) -> int:
    """Total padding along one axis (``tf_conv_dims.py:133-155``)."""
    if padding == "VALID":
        return 0
    if padding == "SAME":
        return max((out_size - 1) * stride + ksize - in_size, 0)
    raise ValueError(f'Unknown padding method "{padding}"')


def calc_padding_4d(in_shape: Sequence[int], ksize: Sequence[int], strides: Sequence[int],
                    padding: str) -> Tuple[int, int, int, int]:
    """``(top, bottom, left, right)`` padding; the odd pixel goes to the bottom / right
    (``tf_conv_dims.py:94-130,158-181``)."""
    _check(ksize, strides)
    if padding == "VALID":
        return 0, 0, 0, 0
    if padding != "SAME":
        raise ValueError(f'Unknown padding method "{padding}"')
    out = []
    for axis, k, s in ((1, ksize[0], strides[1]), (2, ksize[1], strides[2])):
        total = calc_padding_1d(in_shape[axis], calc_out_size_1d(in_shape[axis], k, s, padding), k, s, padding)
        out += [total // 2, total - total // 2]
    return tuple(out)


def calc_block_strides(bsize: Sequence[int], ksize: Sequence[int], strides: Sequence[int]) -> List[int]:
    """Pitch of the blocks so that their convolution outputs tile the output exactly
    (``sparse_conv_lib.py:237-246``)."""
    return [1, bsize[1] - ksize[0] + strides[1], bsize[2] - ksize[1] + strides[2], 1]


def calc_block_params(in_size: Sequence[int], bsize: Sequence[int], ksize: Sequence[int],
                      strides: Sequence[int], padding: str) -> BlockParams:
    """Block parameters of one sparse convolution layer (``sparse_conv_lib.py:343-397``)."""
    _check(ksize, strides)
    if (bsize[1] - ksize[0]) % strides[1] != 0 or (bsize[2] - ksize[1]) % strides[2] != 0:
        raise ValueError("(bsize - ksize) must be a multiple of the stride in both dimensions")
    bstrides = calc_block_strides(bsize, ksize, strides)
    pad_h0, pad_h1, pad_w0, pad_w1 = calc_padding_4d(in_size, ksize, strides, padding)
    h, w = in_size[1], in_size[2]
    # extra bottom / right padding so that whole blocks cover the padded image
    pad_h1 += (-h + bsize[1]) % bstrides[1]
    pad_w1 += (-w + bsize[2]) % bstrides[2]
    padded = [in_size[0], h + pad_h0 + pad_h1, w + pad_w0 + pad_w1, in_size[3]]
    counts = calc_out_size_4d(padded, [bsize[1], bsize[2], 1, 1], bstrides, "VALID")
    out = calc_out_size_4d(bsize, ksize, strides, "VALID")
    params = BlockParams(bsize=[bsize[1], bsize[2]], bsize_out=[out[1], out[2]], boffset=[-pad_h0, -pad_w0],
                         bcount=[counts[1], counts[2]], bstrides=[bstrides[1], bstrides[2]])
    for i, size in enumerate((h, w)):   # the last block must still start inside the image
        if not params.boffset[i] + params.bstrides[i] * (params.bcount[i] - 1) < size:
            raise ValueError(f"last block starts outside the image: boffset {params.boffset[i]} "
                             f"bstrides {params.bstrides[i]} bcount {params.bcount[i]} size {size}")
    return params


def calc_block_params_res_block(in_size: Sequence[int], bsize: Sequence[int],
                                ksize_list: Sequence[Sequence[int]], strides: Sequence[int],
                                padding: str) -> BlockParams:
    """Block parameters of a residual block: the kernel is the block's receptive field
    (``sparse_conv_lib.py:400-421``)."""
    kh = 1 + sum(k[0] - 1 for k in ksize_list)
    kw = 1 + sum(k[1] - 1 for k in ksize_list)
    return calc_block_params(in_size, bsize, [kh, kw, 1, 1], strides, padding)
