"""Checks that need no GPU: the C-ABI library loads, exports every symbol the public header
declares, and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def handle():
    from sbnet_b200 import build, lib
    build.build_library()
    return lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sbnet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sbnet_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(handle):
    from sbnet_b200 import lib
    names = declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert getattr(handle, n) is not None
    assert sorted(lib.SIGNATURES) == names


def test_version(handle):
    assert handle.sbnet_version() >= 100


def test_scatter_rejects_overlapping_add_without_atomics(handle):
    from sbnet_b200 import lib
    rc = handle.sbnet_sparse_scatter(None, 0, 1, 8, 8, 1, None, 0, 0, 2, 2, 1, 1, 4, None, 1, 0, 0, None)
    assert rc == -1
    assert b"non-overlapping" in handle.sbnet_last_error()
    with pytest.raises(ValueError):
        lib.check(rc)


@pytest.mark.parametrize("kwargs", [
    dict(N=0), dict(bSzH=0), dict(bStrW=0), dict(bCntH=40000), dict(N=40000), dict(bCntW=0),
])
def test_reduce_mask_rejects_bad_geometry(handle, kwargs):
    a = dict(N=1, H=8, W=8, bOffsH=0, bOffsW=0, bSzH=2, bSzW=2, bStrH=2, bStrW=2, bCntH=4, bCntW=4)
    a.update(kwargs)
    rc = handle.sbnet_reduce_mask(None, a["N"], a["H"], a["W"], 0.5, 0, a["bOffsH"], a["bOffsW"],
                                  a["bSzH"], a["bSzW"], a["bStrH"], a["bStrW"], a["bCntH"], a["bCntW"],
                                  None, None, None, 0, None)
    assert rc == -1 and handle.sbnet_last_error() != b""


def test_null_pointers_and_dtype_are_rejected(handle):
    assert handle.sbnet_reduce_mask(None, 1, 8, 8, 0.5, 0, 0, 0, 2, 2, 2, 2, 4, 4, None, None, None, 0, None) == -1
    assert handle.sbnet_sparse_gather(None, 7, 1, 8, 8, 1, None, 0, 0, 2, 2, 2, 2, 1, None, 0, None) == -1
    assert handle.sbnet_sparse_gather(None, 0, 1, 8, 8, 1, None, 0, 0, 2, 2, 2, 2, 1, None, 0, None) == -1
    # zero blocks: a successful no-op even with null buffers
    assert handle.sbnet_sparse_gather(None, 0, 1, 8, 8, 1, None, 0, 0, 2, 2, 2, 2, 0, None, 0, None) == 0
    assert handle.sbnet_copy_tensor(None, None, 0, None) == 0
    assert handle.sbnet_copy_tensor(None, None, 16, None) == -1


def test_pointers_off_their_element_boundary_are_rejected(handle):
    """A tensor pointer that is not a multiple of its element size would be a misaligned access on the device;
    the entry points turn it into an argument error before anything is launched (no GPU needed to see it)."""
    import ctypes as C
    P = lambda a: C.c_void_p(a)  # noqa: E731 - made-up addresses, never dereferenced
    ok = 0x10000
    for image, stack, idx, dtype in ((ok + 2, ok, ok, 0), (ok, ok + 1, ok, 0), (ok + 1, ok, ok, 1), (ok, ok, ok + 1, 1)):
        rc = handle.sbnet_sparse_gather(P(image), dtype, 1, 8, 8, 1, P(stack), 0, 0, 2, 2, 2, 2, 1, P(idx), 0, None)
        assert rc == -1 and b"aligned" in handle.sbnet_last_error(), (image, stack, idx, dtype)
    rc = handle.sbnet_sparse_scatter(P(ok + 2), 0, 1, 8, 8, 1, P(ok), 0, 0, 2, 2, 2, 2, 1, P(ok), 0, 0, 0, None)
    assert rc == -1 and b"aligned" in handle.sbnet_last_error()
    rc = handle.sbnet_reduce_mask(P(ok + 2), 1, 8, 8, 0.5, 0, 0, 0, 2, 2, 2, 2, 4, 4, P(ok), P(ok), None, 0, None)
    assert rc == -1 and b"aligned" in handle.sbnet_last_error()
    rc = handle.sbnet_reduce_mask(P(ok), 1, 8, 8, 0.5, 0, 0, 0, 2, 2, 2, 2, 4, 4, P(ok + 1), P(ok), None, 0, None)
    assert rc == -1 and b"aligned" in handle.sbnet_last_error()


def test_missing_library_fails_loudly(monkeypatch):
    from sbnet_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", "/nonexistent/libsbnet_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        lib.load()


def test_ops_refuse_cpu_tensors():
    import torch
    from sbnet_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.reduce_mask(torch.zeros(1, 4, 4, 1), [2, 2], [2, 2], [2, 2], [0, 0], tol=0.5)
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops.sparse_gather(torch.zeros(1, 4, 4, 1), [1], torch.zeros(1, 3, dtype=torch.int16), [2, 2],
                          [2, 2], [0, 0])


def test_product_package_never_touches_the_checker():
    """The CPU checker is test infrastructure: nothing under sbnet_b200/ may import, load or run it."""
    pkg = os.path.join(ROOT, "sbnet_b200")
    for dirpath, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".cc")):
                text = open(os.path.join(dirpath, name), errors="replace").read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, name)
