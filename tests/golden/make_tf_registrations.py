"""Extracts the op and GPU-kernel registrations from the reference's sources into
tests/golden/tf_registrations.json (op name -> attrs / inputs / outputs / GPU host-memory arguments).

    python tests/golden/make_tf_registrations.py <reference tree>/sbnet_tensorflow/sbnet_ops

The TensorFlow binding of this repository must register exactly these interfaces
(tests/test_tf_shim.py); the one deliberate difference, `half` added to T, is applied by the test."""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def parse(src_dir):
    text = ""
    for name in ("reduce_mask.cc", "sparse_gather.cc"):
        with open(os.path.join(src_dir, name)) as f:
            text += re.sub(r"//[^\n]*", "", f.read()).replace("\\\n", "\n")
    ops = {}
    for m in re.finditer(r'REGISTER_OP\("(\w+)"\)(.*?);', text, flags=re.S):
        body = m.group(2)
        ops[m.group(1)] = dict(
            attrs=re.findall(r'\.Attr\("([^"]*)"\)', body),
            inputs=re.findall(r'\.Input\("([^"]*)"\)', body),
            outputs=re.findall(r'\.Output\("([^"]*)"\)', body),
            gpu_host_memory=[])
    for m in re.finditer(r'Name\("(\w+)"\)\s*\.Device\(DEVICE_GPU\)(.*?),\s*\w+<', text, flags=re.S):
        ops[m.group(1)]["gpu_host_memory"] = sorted(set(re.findall(r'\.HostMemory\("([^"]*)"\)', m.group(2))))
    return ops


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_tf_registrations.py <reference tree>/sbnet_tensorflow/sbnet_ops")
    src = sys.argv[1]
    out = parse(src)
    with open(os.path.join(HERE, "tf_registrations.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(json.dumps(out, indent=1, sort_keys=True))
