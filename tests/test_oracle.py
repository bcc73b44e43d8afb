"""CPU tests of the oracle: the reference's golden vectors, its FP8 known-answer shapes, and
bit-equality with the reference itself where the reference objects were built."""
import numpy as np
import pytest

import common
import synth

pkg = synth.pkg


def _run_gates(model_factory):
    """The gates of the reference's tests/unit/test_glm_tiny.c (:72-136) on any model factory."""
    cfg, is_mla, is_dense, tensors, g = common.load_reference_tiny()
    nf = len(g["full_ids"])
    m = model_factory(cfg, is_mla, is_dense, tensors, nf)
    lg, _ = m.forward(g["prompt_ids"])
    assert common.golden_tolerance_ratio(lg, g["logits_last"]) <= 1.0          # GATE 1
    for i, want in enumerate(g["generated_ids"]):                              # GATE 2
        tok = int(np.argmax(lg))
        assert tok == want, f"greedy step {i}: {tok} != {want}"
        if i + 1 < len(g["generated_ids"]):
            lg, _ = m.forward([tok])
    last = lg.copy()
    m.reset()
    _, am = m.forward(g["full_ids"], want_logits=False, want_argmax=True)      # GATE 3
    assert am.tolist() == g["tf_argmax"]
    m.close()
    nl = len(g["long_ids"])                                                    # GATE 4: DSA selects
    m2 = model_factory(cfg, is_mla, is_dense, tensors, nl)
    lg2, am2 = m2.forward(g["long_ids"], want_argmax=True)
    assert am2.tolist() == g["long_tf_argmax"]
    assert common.golden_tolerance_ratio(lg2, g["long_logits_last"]) <= 1.0
    m2.close()
    return last, lg2


def _oracle_factory(binding, kv_mode=0):
    def make(cfg, is_mla, is_dense, tensors, cap):
        m = binding.OracleModel(cfg, is_mla, is_dense, cap, kv_mode)
        m.load_all(tensors); m.finalize()
        return m
    return make


def test_oracle_passes_reference_golden_gates(binding):
    _run_gates(_oracle_factory(binding))


def test_oracle_latent_cache_passes_golden_gates(binding):
    """The compressed-latent cache form (the one the GPU engine uses) against the same goldens."""
    _run_gates(_oracle_factory(binding, kv_mode=2))


def test_oracle_bit_identical_to_reference(binding):
    if not binding.have_ref():
        pytest.skip("reference objects not built here")

    def ref_factory(cfg, is_mla, is_dense, tensors, cap):
        m = binding.RefModel(cfg, is_mla, is_dense, cap, 0)
        m.load_all(tensors); m.finalize()
        return m
    a = _run_gates(_oracle_factory(binding))
    b = _run_gates(ref_factory)
    for x, y in zip(a, b):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


@pytest.mark.parametrize("rows,cols,br,bc,nan", [(2048, 4096, 128, 128, 0), (4096, 2048, 128, 128, 0),
                                                   (37, 1021, 16, 128, 0), (9, 13, 4, 4, 0), (64, 256, 128, 64, 1)])
def test_fp8_matvec_known_answer(binding, rows, cols, br, bc, nan):
    """Shapes of the reference's tests/unit/test_fp8.c:153-157 against an independent numpy
    evaluation of the same sum (eight float lanes per block, FP64 fold, block scale, FP64 total),
    and bit-equality with the reference's glm53f_mm where it was built."""
    rng = np.random.default_rng(rows * 31 + cols)
    codes = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
    codes.flat[:256] = np.arange(256, dtype=np.uint8)[: min(256, codes.size)]
    if not nan:
        codes[(codes & 0x7f) == 0x7f] ^= 1
    sr, sc = (rows + br - 1) // br, (cols + bc - 1) // bc
    scale = ((rng.integers(0, 1000, size=(sr, sc)) + 1) * 1e-6).astype(np.float32)
    x = ((rng.integers(0, 20001, size=cols) - 10000) * 1e-4).astype(np.float32)
    y = binding.matvec_host("orc", codes, pkg.DT_FP8, scale, br, bc, x)
    w = synth.E4M3_TABLE[codes]
    want = np.zeros(rows, np.float32)
    for r in range(0, rows, max(1, rows // 7)):               # a sample of rows, exact evaluation
        total = 0.0
        for b, c0 in enumerate(range(0, cols, bc)):
            c1 = min(cols, c0 + bc)
            lanes = np.zeros(8, np.float32)
            j = c0
            while j + 8 <= c1:
                prod = w[r, j:j + 8].astype(np.float64) * x[j:j + 8].astype(np.float64) + lanes.astype(np.float64)
                lanes = prod.astype(np.float32)               # fmaf: one rounding of the exact sum
                j += 8
            l = lanes.astype(np.float64)
            bs = ((l[0] + l[4]) + (l[2] + l[6])) + ((l[1] + l[5]) + (l[3] + l[7]))
            for jj in range(j, c1):
                bs += float(w[r, jj]) * float(x[jj])
            total += bs * float(scale[r // br, b])
        want[r] = np.float32(total)
        if np.isnan(want[r]):
            assert np.isnan(y[r])
        else:
            assert y[r] == want[r], (r, y[r], want[r])
    if binding.have_ref():
        z = binding.matvec_host("ref", codes, pkg.DT_FP8, scale, br, bc, x)
        assert np.array_equal(y.view(np.uint32)[~np.isnan(y)], z.view(np.uint32)[~np.isnan(z)])


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_dense_matvec_matches_reference(binding, dt):
    if not binding.have_ref():
        pytest.skip("reference objects not built here")
    rng = np.random.default_rng(5)
    w = rng.standard_normal((77, 1000)).astype(np.float32)
    x = rng.standard_normal((3, 1000)).astype(np.float32)
    arr, code = (synth.to_bf16_bits(w), pkg.DT_BF16) if dt == "bf16" else (w, pkg.DT_F32)
    a = binding.matvec_host("orc", arr, code, None, 0, 0, x)
    b = binding.matvec_host("ref", arr, code, None, 0, 0, x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_oracle_ops_bit_identical_to_reference_on_config1(binding):
    """Every op entry point, oracle against reference, on the benchmark's tiny configuration."""
    if not binding.have_ref():
        pytest.skip("reference objects not built here")
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=0, recipe="spread")
    cap = 48
    models = []
    for cls in (binding.OracleModel, binding.RefModel):
        m = cls(spec.cfg, spec.is_mla, spec.is_dense, cap, 2)
        m.load_all(tensors); m.finalize()
        models.append(m)
    o, r = models
    rng = np.random.default_rng(1)
    E, M = spec.cfg.hidden, spec.cfg.hc_mult
    h = rng.standard_normal((5, M, E)).astype(np.float32)
    x = rng.standard_normal((5, E)).astype(np.float32)
    same = lambda a, b: np.array_equal(np.asarray(a).view(np.uint32), np.asarray(b).view(np.uint32))
    for a, b in zip(o.op_hc_pre(1, 0, h), r.op_hc_pre(1, 0, h)):
        assert same(a, b)
    xo, po, co = o.op_hc_pre(1, 1, h)
    assert same(o.op_hc_post(h, x, po, co), r.op_hc_post(h, x, po, co))
    assert same(o.op_kda(1, x), r.op_kda(1, x))
    assert same(o.op_kda(1, x[:1]), r.op_kda(1, x[:1]))          # carried state
    io, wo = o.op_router(1, x); ir, wr = r.op_router(1, x)
    assert np.array_equal(io, ir) and same(wo, wr)
    assert same(o.op_moe(1, x), r.op_moe(1, x))
    assert same(o.op_moe(1, x, with_shared=False), r.op_moe(1, x, with_shared=False))
    assert same(o.op_mlp(0, x), r.op_mlp(0, x))
    xs = rng.standard_normal((40, E)).astype(np.float32)
    (ao, so), (ar, sr_) = o.op_mla(3, xs, 0), r.op_mla(3, xs, 0)  # 40 positions: DSA selects
    assert same(ao, ar) and so is not None and np.array_equal(so, sr_)
    assert same(o.op_decoder_layer(2, h, 0), r.op_decoder_layer(2, h, 0))
    ids = rng.integers(0, spec.cfg.vocab, 18)
    lo, _ = o.forward(ids); lr, _ = r.forward(ids)
    assert same(lo, lr)


@pytest.mark.parametrize("kv_mode", [1, 2])
def test_oracle_mtp_layer_bit_identical_to_reference(binding, kv_mode):
    """The multi-token-prediction layer (checkpoint layer n_layers): the oracle's restatement of
    glm53f_mtp_feed against the reference's own function, driven the way the reference's decode
    loop drives it (src/cli/glm53f_run.c:496-508): after the prompt the hidden states of all but
    the last position go in with the prompt's next tokens, then every step feeds one hidden state
    and the token the model just produced and takes a draft. Expanded and latent cache forms."""
    if not binding.have_ref():
        pytest.skip("reference objects not built here")
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=0, recipe="spread")
    tensors.update(synth.make_mtp_layer(spec, seed=0, recipe="spread"))
    cap = 40
    models = []
    for cls in (binding.OracleModel, binding.RefModel):
        m = cls(spec.cfg, spec.is_mla, spec.is_dense, cap, kv_mode)
        m.enable_mtp()
        m.load_all(tensors); m.finalize()
        models.append(m)
    same = lambda a, b: np.array_equal(np.asarray(a).view(np.uint32), np.asarray(b).view(np.uint32))
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, spec.cfg.vocab, 21).astype(np.int32)    # 21 + steps cross the indexer's dense limit of 19
    drafts = [[], []]
    nexts = [[], []]
    for k, m in enumerate(models):
        lg, _ = m.forward(prompt)
        nxt = int(np.argmax(lg))
        hid = m.mtp_hidden(0, prompt.size)
        _, x0 = m.mtp_feed(prompt[1:], hid[:-1], want_draft=False)
        d, x1 = m.mtp_feed([nxt], hid[-1:])
        keep = [x0, x1]
        drafts[k].append(d); nexts[k].append(nxt)
        for _ in range(6):
            lg, _ = m.forward([nxt])
            nxt = int(np.argmax(lg))
            d, x = m.mtp_feed([nxt])                                  # h = the state the forward call kept
            keep.append(x)
            drafts[k].append(d); nexts[k].append(nxt)
        m.keep = keep
    assert drafts[0] == drafts[1] and nexts[0] == nexts[1]
    for a, b in zip(models[0].keep, models[1].keep):
        assert same(a, b)
    for m in models:
        m.close()


def test_synthetic_codes_are_finite_and_spread(binding):
    c = binding.synth_codes(7, 3, 11, 1, 1 << 16)
    assert not np.any((c & 0x7f) == 0x7f)
    counts = np.bincount(c, minlength=256)
    assert counts[0x7f] == 0 and counts[0xff] == 0
    assert counts[counts > 0].min() > 150 and (counts > 0).sum() == 254
    assert not np.array_equal(c, binding.synth_codes(7, 3, 12, 1, 1 << 16))


def test_reference_checkpoint_roundtrip(binding, tmp_path):
    """The golden import written back as a checkpoint directory loads with the reference's own
    safetensors reader and bind, and gives the golden logits."""
    if not binding.have_ref():
        pytest.skip("reference objects not built here")
    cfg, is_mla, is_dense, tensors, g = common.load_reference_tiny()
    common.write_reference_tiny_checkpoint(str(tmp_path))
    m = binding.ref_open_dir(str(tmp_path), cfg, len(g["full_ids"]))
    lg, _ = m.forward(g["prompt_ids"])
    assert common.golden_tolerance_ratio(lg, g["logits_last"]) <= 1.0
    m.close()
