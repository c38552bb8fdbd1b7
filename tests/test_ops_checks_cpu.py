"""Argument rules of the host-side op wrappers, checked without a GPU: every rule is a device-free
helper, and every wrapper -- synchronous, asynchronous and device-count -- raises ValueError before
anything could be launched (on this machine there is nothing to launch on)."""
import pytest
import torch

from sbnet_b200 import ops


def test_mask_rules():
    assert ops._check_mask(torch.zeros((2, 8, 12, 1))) == (2, 8, 12)
    assert ops._check_mask(torch.zeros((2, 8, 12))) == (2, 8, 12)
    with pytest.raises(ValueError, match="float32"):
        ops._check_mask(torch.zeros((2, 8, 12, 1), dtype=torch.float16))
    with pytest.raises(ValueError, match=r"\[N,H,W,1\]"):
        ops._check_mask(torch.zeros((2, 8, 12, 3)))
    with pytest.raises(ValueError, match=r"\[N,H,W,1\]"):
        ops._check_mask(torch.zeros((8, 12)))
    with pytest.raises(ValueError, match="contiguous"):
        ops._check_mask(torch.zeros((2, 12, 8)).transpose(1, 2))


def test_index_rules():
    good = torch.zeros((10, 3), dtype=torch.int16)
    ops._check_indices(good, 10)
    ops._check_indices(good, 0)
    with pytest.raises(ValueError, match="int16"):
        ops._check_indices(good.to(torch.int32), 4)
    with pytest.raises(ValueError, match="rows"):
        ops._check_indices(good, 11)
    with pytest.raises(ValueError, match=r"\[numBlocks, 3\]"):
        ops._check_indices(torch.zeros((10, 4), dtype=torch.int16), 4)
    with pytest.raises(ValueError, match=r"\[numBlocks, 3\]"):
        ops._check_indices(torch.zeros((3, 10), dtype=torch.int16).t(), 4)


def test_stack_and_image_rules():
    x = torch.zeros((1, 8, 8, 4))
    assert ops._check_image(x, "x") == (1, 8, 8, 4)
    with pytest.raises(ValueError, match="rank 4"):
        ops._check_image(torch.zeros((8, 8, 4)), "x")
    with pytest.raises(ValueError, match="dtype"):
        ops._check_image(torch.zeros((1, 8, 8, 4), dtype=torch.float64), "x")
    with pytest.raises(ValueError, match="contiguous"):
        ops._check_image(torch.zeros((1, 8, 4, 8)).transpose(2, 3), "x")
    ops._check_stack(torch.zeros((3, 2, 2, 4)), "out", 3, 16, x)
    with pytest.raises(ValueError, match="share a dtype"):
        ops._check_stack(torch.zeros((3, 2, 2, 4), dtype=torch.float16), "out", 3, 16, x)
    with pytest.raises(ValueError, match="needs 64"):
        ops._check_stack(torch.zeros((3, 2, 2, 4)), "out", 4, 16, x)
    with pytest.raises(ValueError, match="contiguous"):
        ops._check_stack(torch.zeros((3, 2, 4, 2)).transpose(2, 3), "out", 3, 16, x)


def test_device_count_rules():
    x = torch.zeros((1, 8, 8, 4))
    ops._check_count_dev(torch.zeros(1, dtype=torch.int32), x)
    with pytest.raises(ValueError, match="int32"):
        ops._check_count_dev(torch.zeros(1, dtype=torch.int64), x)
    with pytest.raises(ValueError, match="int32"):
        ops._check_count_dev(torch.zeros(0, dtype=torch.int32), x)
    with pytest.raises(ValueError, match="int32"):
        ops._check_count_dev(3, x)


@pytest.mark.parametrize("call", [
    lambda m: ops.reduce_mask(m, [2, 2], [4, 4], [4, 4], [0, 0], tol=0.5),
    lambda m: ops.reduce_mask_async(m, [2, 2], [4, 4], [4, 4], [0, 0], tol=0.5),
    lambda m: ops.reduce_mask_with_device_count(m, [2, 2], [4, 4], [4, 4], [0, 0], tol=0.5),
])
def test_every_reduce_mask_wrapper_rejects_a_host_mask(call):
    with pytest.raises(ValueError, match="CUDA tensor"):
        call(torch.zeros((1, 8, 8, 1), dtype=torch.float16))


def test_device_count_wrappers_reject_host_tensors():
    x = torch.zeros((1, 8, 8, 4))
    idx = torch.zeros((4, 3), dtype=torch.int16)
    cnt = torch.ones(1, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.sparse_gather_dyn(x, cnt, 4, idx, [4, 4], [4, 4], [0, 0])
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.sparse_scatter_var_dyn(torch.zeros((4, 4, 4, 4)), cnt, 4, idx, x, [4, 4], [4, 4], [0, 0], add=True)
