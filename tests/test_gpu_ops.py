"""GPU parity tests, op by op: the CUDA engine through its C ABI against the CPU oracle on the
same seeded inputs. Tolerances: indices (router, DSA selection) must be identical; floating point
must agree to 1e-4 relative per op or tighter (the end-to-end bar is 1e-3 relative on logits), and
the ops that repeat the reference's FP32 order are expected to agree to the last bit almost
everywhere."""
import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu


def gpu_matvec(arr, dt, scale, br, bc, x):
    import ctypes as C
    L = pkg.lib()
    t, keep = pkg.as_tensor(arr, dt, scale)
    x = np.ascontiguousarray(x, dtype=np.float32)
    T = x.shape[0] if x.ndim == 2 else 1
    y = np.zeros((T, arr.shape[0]), np.float32)
    rc = L.g5b_matvec_host(C.byref(t), br, bc, x.ctypes.data, T, y.ctypes.data, 0)
    assert rc == 0, L.g5b_last_error()
    return y if x.ndim == 2 else y[0]


def test_e4m3_decode_every_code(gpu_lib):
    """All 256 E4M3FN codes decode exactly, NaN codes included (reference test_fp8.c:157)."""
    codes = np.zeros((256, 16), np.uint8)
    codes[:, 0] = np.arange(256)
    x = np.zeros(16, np.float32); x[0] = 1.0
    y = gpu_matvec(codes, pkg.DT_FP8, np.ones((16, 1), np.float32), 16, 16, x)
    want = synth.E4M3_TABLE
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(y), nan)
    assert np.array_equal(y[~nan], want[~nan])


@pytest.mark.parametrize("rows,cols,br,bc", [(2048, 4096, 128, 128), (4096, 2048, 128, 128), (37, 1021, 16, 128),
                                               (9, 13, 4, 4), (64, 256, 128, 64), (24, 16384, 128, 128), (130, 1536, 128, 128)])
@pytest.mark.parametrize("T", [1, 3])
def test_fp8_matvec(gpu_lib, binding, rows, cols, br, bc, T):
    rng = np.random.default_rng(rows + cols + T)
    codes = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    codes[(codes & 0x7f) == 0x7f] ^= 1
    sr, sc = (rows + br - 1) // br, (cols + bc - 1) // bc
    scale = ((rng.integers(0, 1000, size=(sr, sc)) + 1) * 1e-6).astype(np.float32)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    got = gpu_matvec(codes, pkg.DT_FP8, scale, br, bc, x)
    want = binding.matvec_host("orc", codes, pkg.DT_FP8, scale, br, bc, x)
    assert common.rel_err(got, want) < 2e-6


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("rows,cols,T", [(8192, 4096, 1), (64, 4096, 2), (128, 4096, 5), (8192, 128, 1), (77, 1001, 3),
                                          (1024, 512, 4)])
def test_dense_matvec(gpu_lib, binding, dt, rows, cols, T):
    rng = np.random.default_rng(rows * 3 + cols + T)
    w = rng.standard_normal((rows, cols)).astype(np.float32)
    x = rng.standard_normal((T, cols)).astype(np.float32)
    arr, code = (synth.to_bf16_bits(w), pkg.DT_BF16) if dt == "bf16" else (w, pkg.DT_F32)
    got = gpu_matvec(arr, code, None, 0, 0, x)
    want = binding.matvec_host("orc", arr, code, None, 0, 0, x)
    assert common.rel_err(got, want) < 2e-6


def _mostly_bit_equal(got, want, frac=0.999, tol=1e-6):
    got, want = np.asarray(got), np.asarray(want)
    same = (got.view(np.uint32) == want.view(np.uint32)).mean()
    assert same >= frac, f"only {same:.5f} of the values are bit-equal"
    assert common.rel_err(got, want) < tol


def test_rmsnorm_swiglu_shortconv(gpu_lib, binding):
    import ctypes as C
    L, O = pkg.lib(), binding.oracle_lib()
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 4096)).astype(np.float32); w = rng.standard_normal(4096).astype(np.float32)
    a = np.zeros_like(x); b = np.zeros_like(x)
    assert L.g5b_rmsnorm_host(a.ctypes.data, x.ctypes.data, w.ctypes.data, 4096, 4, 1e-5, 0) == 0
    O.orc_rmsnorm_host(b.ctypes.data, x.ctypes.data, w.ctypes.data, 4096, 4, 1e-5)
    _mostly_bit_equal(a, b)
    gu = (rng.standard_normal((3, 2 * 2048)) * 6).astype(np.float32)
    a = np.zeros((3, 2048), np.float32); b = np.zeros_like(a)
    assert L.g5b_swiglu_host(a.ctypes.data, gu.ctypes.data, 2048, 3, 10.0, 0) == 0
    O.orc_swiglu_host(b.ctypes.data, gu.ctypes.data, 2048, 3, 10.0)
    _mostly_bit_equal(a, b)
    ch, k, T = 512, 4, 6
    xs = rng.standard_normal((T, ch)).astype(np.float32); ws = rng.standard_normal((ch, k)).astype(np.float32)
    s1 = rng.standard_normal((ch, k - 1)).astype(np.float32); s2 = s1.copy()
    a = np.zeros_like(xs); b = np.zeros_like(xs)
    assert L.g5b_shortconv_host(a.ctypes.data, xs.ctypes.data, ws.ctypes.data, s1.ctypes.data, ch, k, T, 0) == 0
    O.orc_shortconv_host(b.ctypes.data, xs.ctypes.data, ws.ctypes.data, s2.ctypes.data, ch, k, T)
    _mostly_bit_equal(a, b)
    assert np.array_equal(s1, s2)


@pytest.fixture(scope="module", params=["tiny", "micro"])
def pair(request, gpu_lib, binding):
    """(spec, engine, oracle) on the benchmark's tiny configuration (streaming kernels) and on the
    reference's unit-test shapes (any-shape kernels)."""
    spec = synth.tiny_spec() if request.param == "tiny" else synth.micro_spec()
    tensors = synth.make_model(spec, seed=1, recipe="spread")
    eng, orc = common.build_models(spec, tensors, 64, binding)
    yield spec, eng, orc
    eng.close(); orc.close()


def test_mhc_pre_and_post(pair):
    spec, eng, orc = pair
    rng = np.random.default_rng(11)
    h = rng.standard_normal((5, spec.cfg.hc_mult, spec.cfg.hidden)).astype(np.float32)
    for site in (0, 1):
        g, w = eng.op_hc_pre(1, site, h), orc.op_hc_pre(1, site, h)
        for a, b in zip(g, w):
            assert common.rel_err(a, b) < 1e-5
    x, post, comb = orc.op_hc_pre(1, 0, h)
    y = rng.standard_normal((5, spec.cfg.hidden)).astype(np.float32)
    _mostly_bit_equal(eng.op_hc_post(h, y, post, comb), orc.op_hc_post(h, y, post, comb))


def test_router_indices_identical(pair):
    spec, eng, orc = pair
    rng = np.random.default_rng(12)
    x = rng.standard_normal((40, spec.cfg.hidden)).astype(np.float32)
    layer = spec.is_dense.index(0)
    gi, gw = eng.op_router(layer, x)
    wi, ww = orc.op_router(layer, x)
    assert np.array_equal(gi, wi)
    assert common.rel_err(gw, ww) < 1e-6


@pytest.mark.parametrize("T", [1, 2, 5, 40])
def test_moe_layer(pair, T):
    spec, eng, orc = pair
    rng = np.random.default_rng(13 + T)
    x = rng.standard_normal((T, spec.cfg.hidden)).astype(np.float32)
    layer = spec.is_dense.index(0)
    assert common.rel_err(eng.op_moe(layer, x), orc.op_moe(layer, x)) < 1e-5
    assert common.rel_err(eng.op_moe(layer, x, False), orc.op_moe(layer, x, False)) < 1e-5


def test_dense_mlp(pair):
    spec, eng, orc = pair
    x = np.random.default_rng(14).standard_normal((3, spec.cfg.hidden)).astype(np.float32)
    layer = spec.is_dense.index(1)
    assert common.rel_err(eng.op_mlp(layer, x), orc.op_mlp(layer, x)) < 1e-5


def test_kda_layer_carries_state(pair):
    spec, eng, orc = pair
    rng = np.random.default_rng(15)
    layer = [i for i in range(spec.cfg.n_layers) if not spec.is_mla[i]][1]
    for T in (5, 1, 1, 3):
        x = rng.standard_normal((T, spec.cfg.hidden)).astype(np.float32)
        assert common.rel_err(eng.op_kda(layer, x), orc.op_kda(layer, x)) < 1e-5
    n = spec.cfg.kda_heads * spec.cfg.kda_head_dim ** 2
    assert common.rel_err(eng.state_read(layer, 0, 0, n), orc.state_read(layer, 0, 0, n)) < 1e-5


def test_mla_with_dsa_selection(pair):
    """40 positions with index_topk 16 / pool 4: past position 19 the indexer drops pools, so the
    selected positions must be identical and the attention output must agree."""
    spec, eng, orc = pair
    rng = np.random.default_rng(16)
    layer = spec.is_mla.index(1)
    x = rng.standard_normal((40, spec.cfg.hidden)).astype(np.float32)
    (g, gs), (w, ws) = eng.op_mla(layer, x, 0), orc.op_mla(layer, x, 0)
    assert ws is not None and gs is not None and np.array_equal(gs, ws)
    assert common.rel_err(g, w) < 1e-5
    for p in range(40, 46):                                    # decode steps, one position at a time
        x1 = rng.standard_normal((1, spec.cfg.hidden)).astype(np.float32)
        (g, gs), (w, ws) = eng.op_mla(layer, x1, p), orc.op_mla(layer, x1, p)
        assert np.array_equal(gs, ws)
        assert common.rel_err(g, w) < 1e-5


def test_decoder_layers(pair):
    spec, eng, orc = pair
    rng = np.random.default_rng(17)
    eng.reset(); orc.reset()
    h = rng.standard_normal((4, spec.cfg.hc_mult, spec.cfg.hidden)).astype(np.float32)
    for layer in range(spec.cfg.n_layers):
        g, w = eng.op_decoder_layer(layer, h, 46), orc.op_decoder_layer(layer, h, 46)
        assert common.rel_err(g, w) < 2e-5, layer


def test_engine_fails_loudly_on_bad_input(pair):
    spec, eng, orc = pair
    with pytest.raises(RuntimeError):
        eng.forward([spec.cfg.vocab + 5])
    with pytest.raises(RuntimeError):
        eng.load("layers.0.no_such_tensor", np.zeros((1, 1), np.float32), pkg.DT_F32)


def test_decoder_layer_with_fused_mhc_site(gpu_lib, binding):
    """Hidden 2048 with 4 streams is the smallest shape whose mHC site takes the one-launch path
    (norm factor + mixer product + gates + Sinkhorn + collapse + input RMSNorm in one kernel);
    the tiny model above takes the separate kernels. Both must give the CPU path's layer output."""
    c = pkg.Config(hidden=2048, n_layers=2, vocab=64, rms_eps=1e-5, hc_mult=4, hc_iters=20, hc_eps=1e-6,
                   kda_heads=4, kda_head_dim=64, conv_k=4, gate_lb=-5.0, mla_heads=4, q_lora=192, kv_lora=128,
                   qk_nope=64, v_head=64, index_topk=16, index_kpool=4, index_heads=4, index_dim=32,
                   n_experts=8, topk=2, n_shared=1, moe_inter=128, dense_inter=256, routed_scale=2.5,
                   norm_topk=1, swiglu_limit=10.0, fp8_block_r=128, fp8_block_c=128)
    spec = synth.Spec(c, [0, 1], [1, 0], with_head=False)
    for recipe in ("baseline", "spread"):
        tensors = synth.make_model(spec, seed=23, recipe=recipe)
        eng, orc = common.build_models(spec, tensors, 32, binding, options={"allow_partial": 1})
        rng = np.random.default_rng(29)
        for T in (1, 5):
            h = rng.standard_normal((T, c.hc_mult, c.hidden)).astype(np.float32)
            for layer in range(c.n_layers):
                g, w = eng.op_decoder_layer(layer, h, 0), orc.op_decoder_layer(layer, h, 0)
                assert common.rel_err(g, w) < 2e-5, (recipe, T, layer)
                h = w
        eng.close(); orc.close()
