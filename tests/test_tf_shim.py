"""The TensorFlow binding (sbnet_b200/csrc/tf_shim/sbnet_tf_ops.cc) without TensorFlow.

It is compiled against a small stand-in of the TensorFlow op API (tests/tf_stub/tf_stub.h) together
with a driver (tests/tf_stub/run_shim.cc):
* CPU: the ops and GPU kernels it registers are compared with the registrations extracted from the
  reference's own sources (tests/golden/tf_registrations.json, made by make_tf_registrations.py) --
  names, attrs with defaults, inputs, outputs and host-memory placement must be identical; the only
  difference allowed is `half` and `bfloat16` added to the element types of gather / scatter.
* GPU: every OpKernel::Compute is executed (ReduceMask -> SparseGather -> SparseScatter /
  SparseScatterVar, both layouts, timers, InvalidArgument paths) and checked against the CPU checker.
"""
import json
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STUB = os.path.join(ROOT, "tests", "tf_stub")
EXE = os.path.join(STUB, "_build", "run_shim")


@pytest.fixture(scope="module")
def run_shim(oracle_port):
    from sbnet_b200 import build
    build.build_library()
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    libdirs = [os.path.join(ROOT, "sbnet_b200"), os.path.join(ROOT, "oracle"), os.path.join(cuda, "lib64")]
    cmd = [cxx, "-std=c++17", "-O1", "-I", STUB, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include"),
           os.path.join(STUB, "run_shim.cc"), "-o", EXE, "-lsbnet_b200", "-lsbnet_oracle", "-lcudart"]
    for d in libdirs:
        cmd += ["-L", d, "-Wl,-rpath," + d]
    subprocess.run(cmd, check=True)
    return EXE


def test_registrations_match_the_reference(run_shim):
    dump = json.loads(subprocess.run([run_shim, "dump"], check=True, capture_output=True, text=True).stdout)
    with open(os.path.join(ROOT, "tests", "golden", "tf_registrations.json")) as f:
        ref = json.load(f)
    ours = {o["name"]: o for o in dump["ops"]}
    assert sorted(ours) == sorted(ref)
    for name, r in ref.items():
        attrs = list(r["attrs"])
        if name in ("SparseGather", "SparseScatter", "SparseScatterVar"):
            assert attrs[0] == "T: {float}"
            attrs[0] = "T: {float, half, bfloat16}"        # the one deliberate extension
        assert ours[name]["attrs"] == attrs
        assert ours[name]["inputs"] == r["inputs"]
        assert ours[name]["outputs"] == r["outputs"]
        kernels = [k for k in dump["kernels"] if k["op"] == name]
        assert kernels and all(k["device"] == "GPU" for k in kernels)
        for k in kernels:
            assert sorted(k["host_memory"]) == r["gpu_host_memory"]
    # float, half and bfloat16 kernels for the block ops (stand-in type codes 0, 1, 5), float only for ReduceMask
    types = {n: sorted(k["type"] for k in dump["kernels"] if k["op"] == n) for n in ours}
    assert types["ReduceMask"] == [0] and types["SparseGather"] == [0, 1, 5]
    assert types["SparseScatter"] == [0, 1, 5] and types["SparseScatterVar"] == [0, 1, 5]


@pytest.mark.gpu
def test_op_kernels_compute_on_gpu(run_shim, cuda_ops):
    res = subprocess.run([run_shim, "run"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and res.stdout.startswith("PASS"), res.stdout + res.stderr
