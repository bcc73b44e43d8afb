"""The C-ABI library loads and exports every symbol include/glm53f_b200.h declares. No compute
call is made here, so this runs without a GPU."""
import ctypes
import os
import re

import synth

pkg = synth.pkg
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "glm53f_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(g5b_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(pkg.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 30
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_engine_refuses_without_a_device():
    """With no usable CUDA device the engine must refuse to exist: there is no CPU path."""
    L = pkg.lib()
    if L.g5b_device_count() > 0:
        return
    spec = synth.micro_spec()
    try:
        pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8)
    except RuntimeError as e:
        assert "not available" in str(e) or "no CPU path" in str(e)
    else:
        raise AssertionError("an engine was created without a GPU")


def test_config_struct_matches_header():
    """The ctypes mirror of g5b_config has the header's field order."""
    text = open(os.path.join(ROOT, "include", "glm53f_b200.h")).read()
    body = text[text.index("typedef struct g5b_config {"):text.index("} g5b_config;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for line in body.splitlines()[1:]:
        m = re.match(r"\s*(int32_t|float)\s+(.*);", line)
        if m:
            fields += [f.strip() for f in m.group(2).split(",")]
    assert fields == [f[0] for f in pkg.Config._fields_]


def test_checkpoint_reader_roundtrip(tmp_path):
    import importlib
    import numpy as np
    ck = importlib.import_module("glm53f_b200.checkpoint")
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    codes = np.arange(16, dtype=np.uint8).reshape(4, 4)
    conv = np.arange(8, dtype=np.uint16).reshape(2, 1, 4)
    ck.write_safetensors(str(tmp_path / "m.safetensors"), {
        ck.PREFIX + "layers.0.hc_attn_base": (a, "F32"),
        ck.PREFIX + "layers.0.mlp.gate_proj.weight": (codes, "F8_E4M3"),
        ck.PREFIX + "layers.0.mlp.gate_proj.weight_scale_inv": (np.ones((1, 1), np.float32), "F32"),
        ck.PREFIX + "layers.0.self_attn.q_conv1d.weight": (conv, "BF16"),
        "lm_head.weight": (a.astype(np.float32), "F32")})
    t = ck.read_checkpoint(str(tmp_path))
    assert set(t) == {"layers.0.hc_attn_base", "layers.0.mlp.gate_proj.weight",
                      "layers.0.self_attn.q_conv1d.weight", "lm_head.weight"}
    assert t["layers.0.mlp.gate_proj.weight"][2].shape == (1, 1)
    assert t["layers.0.self_attn.q_conv1d.weight"][0].shape == (2, 4)
