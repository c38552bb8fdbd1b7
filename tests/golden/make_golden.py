"""Generates tests/golden/ref_cases.json from the reference's own CPU functors.

Run in a container where the reference tree is mounted:

    python -c "from oracle import oracle; oracle.build(ref=True)" && python tests/golden/make_golden.py

For every case of tests/ref_cases.py that is not marked ``big`` it runs
reduce_mask -> sparse_gather -> sparse_scatter[_var] through oracle/_ref/libsbnet_ref.so (the
reference functors compiled unchanged) for transpose False and True and records: the block count,
the sorted index list, and SHA-256 digests of the sorted gathered stack and of the scattered output.
Inputs are not stored; they are regenerated from the reference test's seed.  A second file,
config_cases.json, holds the same for the seeded benchmark-style inputs of sbnet_b200/configs.py at
reduced sizes (fp32 and fp16, add / atomic / transposed scatter).
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import oracle  # noqa: E402
import pipeline  # noqa: E402
import ref_cases  # noqa: E402
import config_cases  # noqa: E402


def main():
    ref = oracle.get("ref")
    ref.set_threads(1)
    out = {}
    for case in ref_cases.CASES:
        if case.big:
            continue
        inputs = ref_cases.make_inputs(case)
        rec = {}
        for transpose in (False, True):
            r = pipeline.run_case(ref, case, transpose, inputs)
            rec["T" if transpose else "N"] = dict(
                count=r["count"], indices=r["indices"].tolist() if r["count"] <= 64 else None,
                indices_sha=pipeline.digest(r["indices"]), stack_sha=pipeline.digest(r["stack"]),
                y_sha=pipeline.digest(r["y"]))
        out[case.name] = rec
    with open(os.path.join(HERE, "ref_cases.json"), "w") as f:
        json.dump(out, f, indent=0, sort_keys=True)
    print("ref_cases.json:", len(out), "cases")

    out = {}
    for name in config_cases.NAMES:
        out[name] = config_cases.run(ref, name)["digests"]
    with open(os.path.join(HERE, "config_cases.json"), "w") as f:
        json.dump(out, f, indent=0, sort_keys=True)
    print("config_cases.json:", len(out), "cases")


if __name__ == "__main__":
    main()
