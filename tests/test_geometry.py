"""Block-geometry calculus against the known answers the reference's tests hold
(benchmark/tf_conv_dims_tests.py:72-140, benchmark/sparse_conv_tests.py:437-460) and against the
geometries of the benchmark configurations."""
import pytest

from sbnet_b200 import configs as cfg
from sbnet_b200 import geometry as geo


def test_padding_known_answers():
    # tf_conv_dims_tests.py:74-81, :123-140
    assert geo.calc_padding_4d([1, 5, 6, 1], [2, 3, 1, 1], [1, 1, 1, 1], "SAME") == (0, 1, 1, 1)
    assert geo.calc_padding_4d([1, 5, 5, 1], [2, 3, 1, 1], [1, 1, 1, 1], "VALID") == (0, 0, 0, 0)
    assert geo.calc_padding_4d([1, 5, 6, 1], [2, 3, 1, 1], [1, 2, 2, 1], "SAME") == (0, 1, 0, 1)


def test_argument_errors():
    with pytest.raises(ValueError, match="length 4"):       # tf_conv_dims_tests.py:83-93
        geo.calc_padding_4d([1, 5, 6, 1], [2, 3, 1, 1, 1], [2, 1, 1, 1], "SAME")
    with pytest.raises(ValueError, match="first and last"):  # tf_conv_dims_tests.py:95-105
        geo.calc_padding_4d([1, 5, 6, 1], [2, 3, 1, 1], [2, 1, 1, 1], "SAME")
    with pytest.raises(ValueError, match="Unknown padding"):
        geo.calc_out_size_1d(5, 3, 1, "FULL")
    with pytest.raises(ValueError, match="multiple of the stride"):
        geo.calc_block_params([1, 10, 10, 1], [1, 4, 4, 1], [3, 3, 1, 1], [1, 2, 2, 1], "SAME")


@pytest.mark.parametrize("insize", [6, 7, 10, 11])
@pytest.mark.parametrize("ksize", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("stride", [1, 2, 3])
def test_out_size_matches_direct_count(insize, ksize, stride):
    if ksize > insize:
        return
    # SAME: every stride-th input position produces an output; VALID: windows that fit
    assert geo.calc_out_size_1d(insize, ksize, stride, "SAME") == len(range(0, insize, stride))
    assert geo.calc_out_size_1d(insize, ksize, stride, "VALID") == len(range(0, insize - ksize + 1, stride))


def test_block_params_of_the_hand_written_5x5_case():
    # sparse_conv_tests.py:437-460: bsize 3x3, ksize 3x3, stride 1, SAME on a 5x5 input
    p = geo.calc_block_params([1, 5, 5, 1], [1, 3, 3, 1], [3, 3, 1, 1], [1, 1, 1, 1], "SAME")
    assert p == geo.BlockParams(bsize=[3, 3], bsize_out=[1, 1], boffset=[-1, -1], bcount=[5, 5], bstrides=[1, 1])


def test_block_params_valid_8x8():
    # reduce_mask_tests.py:65-82: bsize 5x5, ksize 2x2, VALID on 8x8
    p = geo.calc_block_params([1, 8, 8, 1], [1, 5, 5, 1], [2, 2, 1, 1], [1, 1, 1, 1], "VALID")
    assert p.bstrides == [4, 4] and p.boffset == [0, 0] and p.bcount == [2, 2] and p.bsize_out == [4, 4]


@pytest.mark.parametrize("H,W", [(400, 352), (512, 512), (800, 704), (64, 48)])
def test_res_block_geometry_is_the_halo_geometry_of_the_benchmarks(H, W):
    p = geo.calc_block_params_res_block([1, H, W, 64], [1, 18, 18, 1], [[1, 1, 64, 16], [3, 3, 16, 16], [1, 1, 16, 64]],
                                        [1, 1, 1, 1], "SAME")
    g = cfg.halo_geom(H, W)
    assert tuple(p.bsize) == g.bsize and tuple(p.bstrides) == g.bstride
    assert tuple(p.boffset) == g.boffset and tuple(p.bcount) == g.bcount
    assert tuple(p.bsize_out) == cfg.inner_geom(H, W).bsize


def test_benchmark_geometries_cover_every_pixel():
    # The reference's extra bottom/right padding rounds (size - bsize) up to the block pitch without
    # counting the SAME padding, so full coverage is a property of the chosen sizes, not of the formula;
    # it holds for every benchmark geometry (block pitch 16, kernel 3, sizes multiple of 16).
    for H, W in [(400, 352), (512, 512), (800, 704)]:
        p = geo.calc_block_params([1, H, W, 1], [1, 18, 18, 1], [3, 3, 1, 1], [1, 1, 1, 1], "SAME")
        for size, i in ((H, 0), (W, 1)):
            covered = set()
            for blk in range(p.bcount[i]):
                covered.update(range(blk * p.bstrides[i], blk * p.bstrides[i] + p.bsize_out[i]))
            assert set(range(size)) <= covered
