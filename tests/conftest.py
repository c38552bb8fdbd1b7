import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


import contextlib


@contextlib.contextmanager
def library_options(**values):
    """Sets process-wide switches of the CUDA library (``sbnet_set_option``) for the duration of a
    block and puts the previous values back."""
    from sbnet_b200 import lib
    saved = {k: lib.get_option(k) for k in values}
    try:
        for k, v in values.items():
            lib.set_option(k, v)
        yield
    finally:
        for k, v in saved.items():
            lib.set_option(k, v)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle_port():
    from oracle import oracle
    oracle.build(ref=False)
    return oracle.get("port")


@pytest.fixture(scope="session")
def oracle_ref():
    from oracle import oracle
    if not oracle.have_ref():
        try:
            oracle.build(ref=True)
        except Exception:
            pass
    if not oracle.have_ref():
        pytest.skip("reference CPU functors not built (no reference tree and no prebuilt library)")
    return oracle.get("ref")


@pytest.fixture(scope="session")
def cuda_ops():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sbnet_b200 import build
    build.build_library()
    from cuda_ops import CudaOps
    return CudaOps("cuda:0")
