"""Edge cases of the MoE layer at full-size shapes (hidden 4096, inter 2048; 32 resident experts keep
it small): activations that stress the exact two-term F16 split of the tensor-core kernels (all
zero, huge, tiny, one element dominating), and exact ties in the router, where the reference takes
the lowest expert index (src/core/glm53f_ops.c:955-966). Batch 1 runs the single decode kernel,
batch 5 the batched kernels; both must give the CPU path's output."""
import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu
SEED = 5


@pytest.fixture(scope="module")
def small_layer(gpu_lib, binding):
    spec, trunk, eng = synth.build_moe_layer_engine(SEED, n_experts=32)
    yield spec, trunk, eng
    eng.close()


def _inputs(cfg):
    rng = np.random.default_rng(77)
    E = cfg.hidden
    base = rng.standard_normal(E).astype(np.float32)
    spike = (base * 1e-3).astype(np.float32); spike[123] = 3.0e4
    return {
        "zeros": np.zeros(E, np.float32),
        "huge": (base * 1.0e4).astype(np.float32),
        "small": (base * 1.0e-3).astype(np.float32),
        "tiny": (base * 1.0e-12).astype(np.float32),
        "one element dominates": spike,
        "not bf16-representable": (base * np.float32(np.pi)).astype(np.float32),
    }


@pytest.mark.parametrize("T", [1, 5])
def test_extreme_activations(small_layer, binding, T):
    spec, trunk, eng = small_layer
    for name, v in _inputs(spec.cfg).items():
        x = np.tile(v, (T, 1)).astype(np.float32)
        if T > 1:
            x[1:] *= np.float32(0.5)                         # rows differ, same kind of extreme
        idx, _ = eng.op_router(0, x)
        orc = synth.oracle_moe_layer(binding, spec, trunk, SEED, idx.ravel())
        want_idx, want_w = orc.op_router(0, x)
        assert np.array_equal(idx, want_idx), name
        got, want = eng.op_moe(0, x), orc.op_moe(0, x)
        if not np.any(want):
            assert not np.any(got), name
        elif name == "tiny":
            # The tensor-core kernels keep silu(g) * u as two F16 terms times 2^8: products below
            # 2^-32 flush to zero. That is an absolute error (here the whole output, about 1e-20);
            # normalised activations never come near it.
            assert np.all(np.isfinite(got)) and np.abs(got - want).max() < 1e-12, name
        else:
            assert np.all(np.isfinite(got)), name
            assert common.rel_err(got, want) < 1e-5, name
        orc.close()


def test_router_ties_take_the_lowest_index(gpu_lib, binding):
    """Experts 2i and 2i+1 share their router row and bias, so every score ties exactly in pairs."""
    spec = synth.layer_spec("moe", n_experts=32)
    trunk = synth.moe_layer_trunk(spec, SEED)
    gate, dt, _ = trunk["layers.0.mlp.gate.weight"]
    gate = gate.copy(); gate[1::2] = gate[0::2]
    trunk["layers.0.mlp.gate.weight"] = (gate, dt, None)
    bias, bdt, _ = trunk["layers.0.mlp.gate.e_score_correction_bias"]
    bias = bias.copy(); bias[1::2] = bias[0::2]
    trunk["layers.0.mlp.gate.e_score_correction_bias"] = (bias, bdt, None)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8)
    eng.set_option("allow_partial", 1)
    eng.load_all(trunk)
    for ex in range(32):
        eng.fill_expert(0, ex, SEED, *synth.expert_scales(spec.cfg, 0, ex, SEED))
    eng.finalize()
    for T in (1, 3):
        x = synth.moe_inputs(spec.cfg, T, 11)
        idx, w = eng.op_router(0, x)
        orc = synth.oracle_moe_layer(binding, spec, trunk, SEED, idx.ravel())
        widx, ww = orc.op_router(0, x)
        assert np.array_equal(idx, widx)
        # the top-8 of 16 tied pairs: both members of the four best pairs, the even one first
        for t in range(T):
            picks = idx[t].tolist()
            assert all(picks[i + 1] == picks[i] + 1 and picks[i] % 2 == 0 for i in range(0, 8, 2)), picks
        assert common.rel_err(w, ww) < 1e-6
        assert common.rel_err(eng.op_moe(0, x), orc.op_moe(0, x)) < 1e-5      # the decode kernel selects for itself
        orc.close()
    eng.close()


def test_forward_refuses_what_the_reference_refuses(gpu_lib, binding):
    """Error behaviour of the forward pass: an empty call, a token outside the vocabulary and a call
    that would overrun the session's positions are refused with a message and leave the session
    where it was (the reference returns an error from glm53f_model_forward for the same inputs,
    src/model/glm53f_model.c:366-381); the next valid call continues from the same state."""
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=0, recipe="baseline")
    eng, orc = common.build_models(spec, tensors, 8, binding)
    ids = np.random.default_rng(3).integers(0, spec.cfg.vocab, 6)
    lg = eng.forward(ids)[0]
    assert eng.cached == 6
    for bad, word in (([], "at least one"), ([spec.cfg.vocab], "vocabulary"), ([-1], "vocabulary"),
                      ([1, 2, 3], "capacity")):
        with pytest.raises(RuntimeError, match=word):
            eng.forward(bad)
        assert eng.cached == 6
    lo = orc.forward(ids)[0]
    assert common.rel_err(lg, lo) < 1e-3
    nxt = [int(np.argmax(lo))]
    assert common.rel_err(eng.forward(nxt)[0], orc.forward(nxt)[0]) < 1e-3     # state intact after the refusals
    assert eng.cached == 7
    eng.close(); orc.close()


@pytest.mark.parametrize("T", [1, 5])
def test_moe_op_with_pinned_host_buffers(small_layer, T):
    """With a pinned, mapped output buffer the layer's last kernel writes the result straight into host
    memory (no device-to-host copy); the values are those of the staged path, bit for bit."""
    import torch
    spec, _, eng = small_layer
    L = pkg.lib()
    x = synth.moe_inputs(spec.cfg, T, 21)
    want = eng.op_moe(0, x)                                   # pageable numpy buffers: staged copies
    xp = torch.from_numpy(x).pin_memory()
    op = torch.full((T, spec.cfg.hidden), float("nan")).pin_memory()
    assert L.g5b_op_moe(eng.handle, 0, xp.numpy().ctypes.data, T, op.numpy().ctypes.data, 1) == 0, L.g5b_last_error()
    assert np.array_equal(op.numpy(), want)


def test_two_engines_on_two_devices_in_one_process(gpu_lib, binding):
    """Kernel set-up (the opt-in to large shared memory, SM counts, cooperative-launch support) is
    kept per device: a second engine on another GPU of the same process must give the CPU path's
    output too, in whichever order the two are used."""
    if gpu_lib.g5b_device_count() < 2:
        pytest.skip("needs two GPUs")
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=21, recipe="baseline")
    orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 32, 2)
    orc.load_all(tensors); orc.finalize()
    engines = []
    for dev in (0, 1):
        e = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32, dev)
        e.load_all(tensors); e.finalize()
        engines.append(e)
    ids = np.random.default_rng(2).integers(0, spec.cfg.vocab, 12).tolist()
    want, _ = orc.forward(ids)
    for e in (engines[1], engines[0], engines[1]):
        e.reset()
        got, _ = e.forward(ids)
        assert common.rel_err(got, want) < 1e-3 and int(np.argmax(got)) == int(np.argmax(want))
    for e in engines:
        e.close()
    orc.close()


def test_expert_parallel_group_inside_one_process(gpu_lib, binding):
    """Two engines of one process, one per device, wired without handles (peer access) and driven by one
    host thread each - what the adapter does when the reference's driver passes several devices
    (src/gpu/glm53f_gpu.h:44-46). Logits of both ranks against the CPU path, then greedy decode."""
    import threading
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=11, recipe="baseline")
    engines = []
    for r in range(2):
        e = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 32, r, r, 2)
        e.load_all(tensors); e.finalize()
        engines.append(e)
    with pytest.raises(RuntimeError, match="rank"):
        pkg.Engine.ep_connect_local(engines[::-1])
    pkg.Engine.ep_connect_local(engines)
    orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 32, 2)
    orc.load_all(tensors); orc.finalize()

    def on_all(fn):
        out, errs = [None, None], []

        def run(r):
            try:
                out[r] = fn(engines[r])
            except Exception as exc:                   # noqa: BLE001
                errs.append(repr(exc))
        ts = [threading.Thread(target=run, args=(r,)) for r in range(2)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        assert not errs, errs
        return out

    ids = np.random.default_rng(0).integers(0, spec.cfg.vocab, 18).tolist()
    lw, _ = orc.forward(ids)
    for lg, _ in on_all(lambda e: e.forward(ids)):
        assert common.rel_err(lg, lw) < 1e-3
    tok = int(np.argmax(lw))
    want = []
    t = tok
    for _ in range(6):
        lw, _ = orc.forward([t])
        t = int(np.argmax(lw)); want.append(t)
    for got in on_all(lambda e: e.decode_greedy(tok, 6)):
        assert got.tolist() == want
    for e in engines:
        e.close()
    orc.close()
