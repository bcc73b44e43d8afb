"""Import the reference project's own tiny-model test fixture as golden data.

Source: <reference>/tests/fixtures/glm_tiny/{config.json, model.safetensors, ref.json}, the
fixture of its tests/unit/test_glm_tiny.c. ref.json holds outputs of the transformers
implementation of the architecture (prompt ids, last-position logits, greedy continuation,
teacher-forced argmax at every position, and a 40-position run past the dense-attention limit),
so it pins both the CPU oracle and the GPU engine to something that neither of them produced.

Writes reference_tiny.npz (every tensor by engine name, raw storage: uint8 codes, uint16 BF16
bits, float32) and reference_tiny.json (config + the golden vectors).

    python tests/golden/make_reference_tiny.py [path of the reference tree]
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from __graft_entry__ import load_package  # noqa: E402

load_package()
import importlib  # noqa: E402

ck = importlib.import_module("glm53f_b200.checkpoint")


def main():
    from oracle import binding
    ref = sys.argv[1] if len(sys.argv) > 1 else binding.reference_tree()
    d = os.path.join(ref, "tests", "fixtures", "glm_tiny")
    tensors = ck.read_checkpoint(d)
    arrays, meta = {}, {}
    for name, (arr, dt, scale) in tensors.items():
        arrays[name] = arr
        meta[name] = dt
        if scale is not None:
            arrays[name + "_scale_inv"] = scale
    np.savez_compressed(os.path.join(HERE, "reference_tiny.npz"), **arrays)
    with open(os.path.join(d, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(d, "ref.json")) as f:
        golden = json.load(f)
    with open(os.path.join(HERE, "reference_tiny.json"), "w") as f:
        json.dump({"config": config, "dtypes": meta, "golden": golden}, f)
    print(f"{len(tensors)} tensors, golden keys {sorted(golden)}")


if __name__ == "__main__":
    main()
