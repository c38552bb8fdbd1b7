"""The drop-in boundary used the way a foreign host uses it: ``include/sbnet_b200.h`` must be plain C, and a C99
program with nothing but the CUDA runtime and the shared library (``tests/c_abi/consumer.c``) runs the
mask -> gather -> scatter sequence of a sparse layer and checks it against the CPU checker it is linked with."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.join(ROOT, "tests", "c_abi")
BUILD = os.path.join(HERE, "_build")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _cc():
    for cand in ("/usr/bin/gcc", shutil.which("gcc"), shutil.which("cc")):
        if cand and os.path.exists(cand):
            return cand
    pytest.skip("no C compiler")


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, " ".join(cmd) + "\n" + res.stdout + res.stderr
    return res.stdout


def build_consumer():
    from sbnet_b200 import build
    lib = build.build_library()
    os.makedirs(BUILD, exist_ok=True)
    cc, exe = _cc(), os.path.join(BUILD, "consumer")
    _run([cc, "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"),
          "-isystem", os.path.join(CUDA, "include"), "-c", os.path.join(HERE, "consumer.c"), "-o", os.path.join(BUILD, "consumer.o")])
    _run([cc, "-O2", "-std=gnu11", "-c", os.path.join(ROOT, "oracle", "sbnet_oracle.c"), "-o", os.path.join(BUILD, "oracle.o")])
    libdir = os.path.dirname(lib)
    _run([cc, os.path.join(BUILD, "consumer.o"), os.path.join(BUILD, "oracle.o"), "-o", exe, "-L", libdir, "-lsbnet_b200",
          "-L", os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(CUDA, "lib64")])
    return exe


def test_header_is_plain_c():
    _run([_cc(), "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c",
          os.path.join(ROOT, "include", "sbnet_b200.h")])


def test_c_consumer_builds_against_the_shared_library():
    assert os.path.exists(build_consumer())


@pytest.mark.gpu
def test_c_consumer_runs_the_layer_sequence():
    out = _run([build_consumer()])
    assert out.startswith("PASS"), out
