"""The full-size architecture end to end on the GPU, cut to its first four layers so that it fits a
test (layers 0-2: KDA + dense MLP 12288; layer 3: MLA with the indexer + MoE with all 288 experts):
weights generated in HBM, prefill + greedy decode through the C ABI, then every layer against the
CPU path fed the GPU's own state (hidden 4096, four residual streams, one and five positions), the
vocabulary-sized head, and the same for a batch of positions through the multi-token projections."""
import numpy as np
import pytest

import common
import fullmodel
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu
SEED = 3
CAP = 64


@pytest.fixture(scope="module")
def model(gpu_lib):
    spec = synth.full_model_spec(4)
    # FP32 latents like the CPU path's: with the BF16 latent cache the position being appended is
    # rounded on the GPU and not on the CPU, which alone costs about 1e-4 on a 24-position context
    eng = fullmodel.build_engine(spec, SEED, CAP)
    yield spec, eng
    eng.close()


def test_generated_weights_match_the_cpu_replay(model, binding):
    """What the GPU generated is what the CPU regenerates: read a matrix back through a product
    with unit vectors (exact for BF16 weights) and compare with the replayed values."""
    spec, eng = model
    c = spec.cfg
    name = "layers.0.self_attn.b_proj.weight"                     # [64][4096] BF16
    mul = float(np.float32(0.02 / synth.BF16_UNIT))
    bits = binding.synth_matrix_bf16(SEED, name, mul, c.kda_heads * c.hidden).reshape(c.kda_heads, c.hidden)
    want = (bits.astype(np.uint32) << 16).view(np.float32)
    assert 0.019 < float(want.std()) < 0.021 and abs(float(want.mean())) < 1e-3
    cols = [0, 1, 77, 4095]
    x = np.zeros((len(cols), c.hidden), np.float32)
    for i, j in enumerate(cols):
        x[i, j] = 1.0
    got = eng.op_matvec(name, x)
    assert np.array_equal(got, want[:, cols].T)


def test_prefill_decode_and_every_layer_against_the_cpu_path(model, binding):
    spec, eng = model
    c = spec.cfg
    rng = np.random.default_rng(SEED)
    ids = rng.integers(0, c.vocab, 18).astype(np.int32)
    logits, _ = eng.forward(ids)
    assert np.isfinite(logits).all()
    toks = eng.decode_greedy(int(np.argmax(logits)), 6)
    assert eng.cached == 24 and toks.min() >= 0 and toks.max() < c.vocab
    # layer by layer at the position reached, one new position and then five: h ~ N(0, 1)
    for T in (1, 5):
        for layer in range(c.n_layers):
            h = rng.standard_normal((T, c.hc_mult, c.hidden)).astype(np.float32)
            r = fullmodel.layer_parity(eng, binding, spec, SEED, layer, h, eng.cached, CAP)
            assert r["rel_err"] < 1e-4, (T, layer, r["rel_err"])


def test_vocabulary_sized_head_and_dense_mlp(model, binding):
    """lm_head 154880 x 4096 (BF16) and the dense MLP at inter 12288 (FP8) at 1, 8, 33 and 64
    positions: the one-token kernels and whatever serves batches of positions."""
    spec, eng = model
    c = spec.cfg
    rng = np.random.default_rng(SEED + 1)
    mul = float(np.float32(0.02 / synth.BF16_UNIT))
    rows = 4096                                                    # compare a slice of the vocabulary rows on the CPU
    bits = binding.synth_matrix_bf16(SEED, "lm_head.weight", mul, c.vocab * c.hidden).reshape(c.vocab, c.hidden)
    pick = np.sort(rng.choice(c.vocab, rows, replace=False))
    w = (bits[pick].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    for T in (1, 8, 33, 64):
        x = rng.standard_normal((T, c.hidden)).astype(np.float32)
        got = eng.op_matvec("lm_head.weight", x)
        want = x.astype(np.float64) @ w.T
        # one to seven positions: FP32 sums in a fixed order; from eight on the tensor cores accumulate
        # (FP32 with their own rounding), a few 1e-6 on a 4096-long dot - the bar on logits is 1e-3
        assert common.rel_err(got[:, pick], want) < (2e-6 if T < 8 else 1e-5), T
    orc = synth.oracle_full_layer(binding, spec, SEED, 0, [], CAP)
    orc.finalize()
    for T in (1, 8, 33, 64):
        x = rng.standard_normal((T, c.hidden)).astype(np.float32)
        assert common.rel_err(eng.op_mlp(0, x), orc.op_mlp(0, x)) < 1e-5, T
    # the KDA projections (BF16) and the layer's other products at 8+ positions
    for name in ("layers.0.self_attn.q_proj.weight", "layers.0.self_attn.o_proj.weight", "layers.0.self_attn.g_b_proj.weight"):
        for T in (8, 33, 64):
            n_in = {"q_proj": c.hidden, "o_proj": c.kda_heads * c.kda_head_dim, "g_b_proj": c.kda_head_dim}[name.split(".")[3]]
            x = rng.standard_normal((T, n_in)).astype(np.float32)
            assert common.rel_err(eng.op_matvec(name, x), orc.op_matvec(name, x)) < 1e-5, (name, T)
    orc.close()


def test_two_full_size_decoder_layers_against_stored_cpu_results(gpu_lib):
    """KDA + MoE and MLA (8191 cached positions, indexer selecting) + MoE at hidden 4096 with all 288
    experts, against the CPU path's stored output (tests/golden/fullsize_layers.npz): the residual
    stream within 1e-4 relative, the router's picks identical."""
    golden = fullmodel.load_layer_case_golden()
    spec, eng, inputs = fullmodel.build_layer_case_engine()
    for layer in (0, 1):
        r = fullmodel.check_layer_case(eng, inputs, golden, layer)
        assert r["picks_equal"], layer
        assert r["rel_err"] < 1e-4, (layer, r["rel_err"])
    eng.close()


def test_mhc_sites_at_the_full_hidden_size(model, binding):
    """glm53f_hc_pre / glm53f_hc_post at hidden 4096 with four streams, one and five positions."""
    spec, eng = model
    c = spec.cfg
    orc = synth.oracle_full_layer(binding, spec, SEED, 0, [], CAP)
    orc.finalize()
    rng = np.random.default_rng(SEED + 2)
    for T in (1, 5):
        h = rng.standard_normal((T, c.hc_mult, c.hidden)).astype(np.float32)
        for site in (0, 1):
            gx, gp, gc = eng.op_hc_pre(0, site, h)
            wx, wp, wc = orc.op_hc_pre(0, site, h)
            assert common.rel_err(gx, wx) < 1e-5 and common.rel_err(gp, wp) < 1e-5 and common.rel_err(gc, wc) < 1e-5, (T, site)
            y = rng.standard_normal((T, c.hidden)).astype(np.float32)
            assert common.rel_err(eng.op_hc_post(h, y, wp, wc), orc.op_hc_post(h, y, wp, wc)) < 1e-6, (T, site)
    orc.close()
