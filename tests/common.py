"""Helpers shared by the test files."""
from __future__ import annotations

import json
import os

import numpy as np

import synth

pkg = synth.pkg
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_reference_tiny():
    """The reference project's unit-test model and its transformers-made golden vectors
    (tests/golden/make_reference_tiny.py). Returns (cfg, is_mla, is_dense, tensors, golden)."""
    import importlib
    ck = importlib.import_module("glm53f_b200.checkpoint")
    with open(os.path.join(GOLDEN, "reference_tiny.json")) as f:
        meta = json.load(f)
    cfg, is_mla, is_dense, _ = ck.read_config(meta["config"])
    z = np.load(os.path.join(GOLDEN, "reference_tiny.npz"))
    tensors = {}
    for name, dt in meta["dtypes"].items():
        scale = z[name + "_scale_inv"] if dt == pkg.DT_FP8 else None
        tensors[name] = (z[name], dt, scale)
    return cfg, is_mla, is_dense, tensors, meta["golden"]


def golden_tolerance_ratio(got, ref):
    """The reference test's logits criterion: |d| <= 1e-5 + 1e-4 |ref| (test_glm_tiny.c:77-86);
    returns the worst |d| / tolerance (<= 1 passes)."""
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(ref - got) / (1e-5 + 1e-4 * np.abs(ref))))


def rel_err(got, want):
    """max |got - want| / max |want|: the relative error the 1e-3 logits bar is stated in."""
    want = np.asarray(want, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - want)) / (np.max(np.abs(want)) + 1e-300))


def build_models(spec, tensors, cap, binding=None, engine=True, oracle=True, kv_mode=2, options=None):
    eng = orc = None
    if engine:
        eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, cap)
        for k, v in (options or {}).items():
            eng.set_option(k, v)
        eng.load_all(tensors)
        eng.finalize()
    if oracle:
        orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, cap, kv_mode)
        orc.load_all(tensors)
        orc.finalize()
    return eng, orc


def write_reference_tiny_checkpoint(directory):
    """Re-create the reference's test checkpoint directory (config.json, model.safetensors,
    ref.json) from the golden import, for programs that load it with the reference's own loader."""
    import importlib
    ck = importlib.import_module("glm53f_b200.checkpoint")
    with open(os.path.join(GOLDEN, "reference_tiny.json")) as f:
        meta = json.load(f)
    z = np.load(os.path.join(GOLDEN, "reference_tiny.npz"))
    st = {pkg.DT_F32: "F32", pkg.DT_BF16: "BF16", pkg.DT_FP8: "F8_E4M3"}
    out = {}
    for name, dt in meta["dtypes"].items():
        full = name if name == "lm_head.weight" else ck.PREFIX + name
        arr = z[name]
        if "conv1d" in name:
            arr = arr.reshape(arr.shape[0], 1, arr.shape[1])
        elif arr.ndim == 2 and arr.shape[1] == 1 and not name.endswith("proj.weight"):
            arr = arr.reshape(-1)
        out[full] = (arr, st[dt])
        if dt == pkg.DT_FP8:
            out[full + "_scale_inv"] = (z[name + "_scale_inv"], "F32")
    os.makedirs(directory, exist_ok=True)
    ck.write_safetensors(os.path.join(directory, "model.safetensors"), out)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(meta["config"], f)
    with open(os.path.join(directory, "ref.json"), "w") as f:
        json.dump(meta["golden"], f)
