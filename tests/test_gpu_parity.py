"""GPU parity: the CUDA library against the CPU checker on identical seeded inputs, through the C ABI.

* every case of the reference's op integration sweep (tests/ref_cases.py), with the reference's own
  assertions (sbnet_ops/tests/test_sparse_blocks.py:296-342): equal count, equal index set, sorted
  indices equal, gathered stacks bit-equal after sorting, transposed == numpy transpose of
  untransposed, scattered outputs bit-equal, empty mask -> one block (0,0,0);
* the benchmark-shaped cases (tests/config_cases.py): bit-exact except atomic adds over overlapping
  halos, where the CUDA result and the CPU checker's must both lie within k rounded additions of the
  fp64 sum and within 1e-6 relative (fp32) of it where nothing cancels (tests/atomic_check.py);
* the committed golden digests, which were produced by the reference's compiled CPU functors.
"""
import json
import os

import numpy as np
import pytest

import config_cases
from atomic_check import check_atomic_add
import pipeline
import ref_cases

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

@pytest.mark.parametrize("case", ref_cases.CASES, ids=[c.name for c in ref_cases.CASES])
def test_reference_sweep(cuda_ops, oracle_port, case):
    inputs = ref_cases.make_inputs(case)
    res = {}
    for transpose in (False, True):
        g = pipeline.run_case(cuda_ops, case, transpose, inputs)
        c = pipeline.run_case(oracle_port, case, transpose, inputs)
        assert g["count"] == c["count"]
        np.testing.assert_array_equal(g["indices"], c["indices"])
        np.testing.assert_array_equal(g["stack"], c["stack"])
        np.testing.assert_array_equal(g["y"], c["y"])
        if case.sparsity == 100:
            assert g["count"] == 1 and g["indices"][0].tolist() == [0, 0, 0]
        res[transpose] = g
    np.testing.assert_array_equal(res[True]["stack"], np.transpose(res[False]["stack"], [0, 3, 1, 2]))
    np.testing.assert_array_equal(res[True]["y"], res[False]["y"])


@pytest.mark.parametrize("name", config_cases.NAMES)
def test_config_cases(cuda_ops, oracle_port, name):
    g = config_cases.run(cuda_ops, name)
    c = config_cases.run(oracle_port, name)
    with open(os.path.join(GOLDEN, "config_cases.json")) as f:
        gold = json.load(f)[name]
    for key, exp in c["arrays"].items():
        got = g["arrays"][key]
        assert got.shape == exp.shape and got.dtype == exp.dtype
        if key in c["tol"]:
            at = c["atomic"]
            check_atomic_add({"cuda": got, "cpu checker": exp}, at["stack"], at["count"], at["indices"], at["base"],
                             at["geom"].bsize, at["geom"].bstride, at["geom"].boffset)
        else:
            np.testing.assert_array_equal(got, exp)
            assert g["digests"][key] == gold[key]
