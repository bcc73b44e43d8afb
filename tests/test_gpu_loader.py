"""The C checkpoint loader: a safetensors directory streamed straight into the engine's HBM layout
gives the model that tensor-by-tensor loading gives, on one rank and on an expert-parallel rank
(which must skip the other ranks' experts), and refuses damaged checkpoints."""
import importlib
import json
import os

import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu


def _write_checkpoint(directory, tensors, shards=3):
    """The tensors as a sharded safetensors checkpoint with the released naming."""
    ck = importlib.import_module("glm53f_b200.checkpoint")
    st = {pkg.DT_F32: "F32", pkg.DT_BF16: "BF16", pkg.DT_FP8: "F8_E4M3"}
    files = [dict() for _ in range(shards)]
    for i, (name, (arr, dt, scale)) in enumerate(sorted(tensors.items())):
        full = name if name == "lm_head.weight" else ck.PREFIX + name
        if "conv1d" in name:
            arr = arr.reshape(arr.shape[0], 1, arr.shape[1])
        elif arr.ndim == 2 and arr.shape[1] == 1 and not name.endswith("proj.weight"):
            arr = arr.reshape(-1)
        files[i % shards][full] = (arr, st[dt])
        if dt == pkg.DT_FP8:
            files[(i + 1) % shards][full + "_scale_inv"] = (scale, "F32")      # the scale grid may sit in another shard
    os.makedirs(directory, exist_ok=True)
    for k, f in enumerate(files):
        ck.write_safetensors(os.path.join(directory, f"model-{k + 1:05d}-of-{shards:05d}.safetensors"), f)


def test_streamed_checkpoint_equals_tensor_by_tensor_loading(gpu_lib, tmp_path):
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=8)
    d = str(tmp_path / "ckpt")
    _write_checkpoint(d, tensors)
    ref = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
    ref.load_all(tensors); ref.finalize()
    ids = np.random.default_rng(3).integers(0, spec.cfg.vocab, 14).tolist()
    want, _ = ref.forward(ids)
    ref.close()
    for threads in (1, 5):
        eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
        eng.load_checkpoint(d, threads)
        eng.finalize()
        got, _ = eng.forward(ids)
        assert np.array_equal(got, want), threads
        eng.close()
    # an expert-parallel rank reads only its own experts and still finalizes
    ep = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32, 0, 1, 2)
    ep.load_checkpoint(d, 2)
    ep.finalize()
    ep.close()
    # a cut of the model (its first three layers) takes the layers it has and ignores the rest
    cut_cfg = spec.cfg.copy(); cut_cfg.n_layers = 3
    cut = pkg.Engine(cut_cfg, spec.is_mla[:3], spec.is_dense[:3], 32)
    cut.load_checkpoint(d, 2)
    cut.finalize()
    cut.close()


def test_loader_refuses_damaged_checkpoints(gpu_lib, tmp_path):
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=8)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
    with pytest.raises(RuntimeError, match="cannot open checkpoint directory"):
        eng.load_checkpoint(str(tmp_path / "nowhere"))
    empty = tmp_path / "empty"; empty.mkdir()
    with pytest.raises(RuntimeError, match="no .safetensors file"):
        eng.load_checkpoint(str(empty))
    eng.close()
    # a tensor of the wrong shape is refused by name, like the reference's bind
    bad = dict(tensors)
    arr, dt, sc = bad["layers.0.self_attn.q_proj.weight"]
    bad["layers.0.self_attn.q_proj.weight"] = (arr[:-1], dt, sc)
    d = str(tmp_path / "bad")
    _write_checkpoint(d, bad, shards=1)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
    with pytest.raises(RuntimeError, match="q_proj.weight is"):
        eng.load_checkpoint(d)
    eng.close()
    # a missing scale grid
    gone = {k: v for k, v in tensors.items()}
    d2 = str(tmp_path / "noscale")
    _write_checkpoint(d2, gone, shards=1)
    ck = importlib.import_module("glm53f_b200.checkpoint")
    path = os.path.join(d2, "model-00001-of-00001.safetensors")
    raw = ck.read_safetensors(path)
    victim = next(k for k in raw if k.endswith("_scale_inv"))
    del raw[victim]
    st = {pkg.DT_F32: "F32", pkg.DT_BF16: "BF16", pkg.DT_FP8: "F8_E4M3"}
    ck.write_safetensors(path, {k: (a, st[c]) for k, (a, c) in raw.items()})
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
    with pytest.raises(RuntimeError, match="scale_inv"):
        eng.load_checkpoint(d2)
    eng.close()
    # a truncated file: byte ranges beyond the end of the file come up short
    d3 = str(tmp_path / "short")
    _write_checkpoint(d3, tensors, shards=1)
    p3 = os.path.join(d3, "model-00001-of-00001.safetensors")
    size = os.path.getsize(p3)
    with open(p3, "r+b") as f:
        f.truncate(size - 4096)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32)
    with pytest.raises(RuntimeError):
        eng.load_checkpoint(d3)
    eng.close()
