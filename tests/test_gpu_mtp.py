"""The multi-token-prediction layer (checkpoint layer n_layers) on the GPU against the CPU path,
driven the way the reference's decode loop drives it (src/cli/glm53f_run.c:496-508): the prompt's
hidden states with the prompt's next tokens, then one hidden state and the token just produced per
step, a draft after each. The CPU side is bit-identical to the reference's glm53f_mtp_feed
(tests/test_oracle.py)."""
import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu


def _models(binding, cap, latent_bf16=0):
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=0, recipe="spread")
    tensors.update(synth.make_mtp_layer(spec, seed=0, recipe="spread"))
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, cap)
    eng.enable_mtp()
    if latent_bf16:
        eng.set_option("latent_bf16", 1)
    eng.load_all(tensors); eng.finalize()
    orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, cap, 2)
    orc.enable_mtp()
    orc.load_all(tensors); orc.finalize()
    return spec, eng, orc


def test_mtp_layer_follows_the_cpu_path(gpu_lib, binding):
    spec, eng, orc = _models(binding, 48)
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, spec.cfg.vocab, 21).astype(np.int32)     # 21 + steps cross the indexer's dense limit of 19
    lg, _ = eng.forward(prompt); lw, _ = orc.forward(prompt)
    assert common.rel_err(lg, lw) < 1e-3
    nxt = int(np.argmax(lw))
    assert int(np.argmax(lg)) == nxt
    hg, hw = eng.mtp_hidden(0, prompt.size), orc.mtp_hidden(0, prompt.size)
    assert common.rel_err(hg, hw) < 1e-4
    # the prompt's positions but the last: 20 rows through the layer at once, fed from the host
    _, xg = eng.mtp_feed(prompt[1:], hw[:-1], want_draft=False)
    _, xw = orc.mtp_feed(prompt[1:], hw[:-1], want_draft=False)
    assert common.rel_err(xg, xw) < 1e-4
    dg, xg = eng.mtp_feed([nxt], hw[-1:]); dw, xw = orc.mtp_feed([nxt], hw[-1:])
    assert common.rel_err(xg, xw) < 1e-4 and dg == dw
    drafts, right = 1, 0
    for _ in range(8):
        lg, _ = eng.forward([nxt]); lw, _ = orc.forward([nxt])
        assert common.rel_err(lg, lw) < 1e-3
        tok = int(np.argmax(lw))
        assert int(np.argmax(lg)) == tok
        right += int(dg == tok)                                       # glm53f_mtp_score
        nxt = tok
        dg, xg = eng.mtp_feed([nxt])                                  # hidden state: the row the forward call kept
        dw, xw = orc.mtp_feed([nxt])
        assert common.rel_err(xg, xw) < 1e-3 and dg == dw
        drafts += 1
    assert drafts == 9 and 0 <= right <= 8
    # a new session forgets the fed positions
    eng.reset(); orc.reset()
    lg, _ = eng.forward(prompt[:5]); lw, _ = orc.forward(prompt[:5])
    dg, xg = eng.mtp_feed(prompt[1:6]); dw, xw = orc.mtp_feed(prompt[1:6])
    assert common.rel_err(xg, xw) < 1e-4 and dg == dw
    eng.close(); orc.close()


def test_mtp_layer_ops_and_limits(gpu_lib, binding):
    """The MTP layer is an ordinary layer slot: its attention and MoE blocks answer the op API at
    index n_layers; feeding without the layer enabled, or past the capacity, is refused."""
    spec, eng, orc = _models(binding, 24)
    L = spec.cfg.n_layers
    x = np.random.default_rng(2).standard_normal((5, spec.cfg.hidden)).astype(np.float32)
    assert common.rel_err(eng.op_moe(L, x), orc.op_moe(L, x)) < 1e-5
    (ag, _), (aw, _) = eng.op_mla(L, x, 0), orc.op_mla(L, x, 0)
    assert common.rel_err(ag, aw) < 1e-4
    eng.reset(); orc.reset()
    ids = np.arange(1, 25, dtype=np.int32)
    eng.forward(ids)
    eng.mtp_feed(ids)
    with pytest.raises(RuntimeError, match="exceed the capacity"):
        eng.mtp_feed(ids[:1])
    eng.close(); orc.close()
    plain = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8)
    plain.load_all(synth.make_model(spec, seed=0, recipe="spread")); plain.finalize()
    with pytest.raises(RuntimeError, match="not enabled"):
        plain.mtp_feed([1])
    plain.close()


SPEC_SEED = 9          # of seeds 0..15 the one with the widest arg-max margins (>= 5 % of the largest logit) and 7 of 17 drafts right


def _speculative_on_cpu(orc, prompt, n):
    """The speculative loop restated with the CPU path's calls: which drafts it makes, which it
    keeps, and the tokens (those of plain greedy decode)."""
    lw, _ = orc.forward(prompt)
    tok = int(np.argmax(lw))
    first = tok
    hid = orc.mtp_hidden(0, len(prompt))
    orc.mtp_feed(prompt[1:], hid[:-1], want_draft=False)
    h_last = hid[-1:]
    toks, drafts, right, passes = [], 0, 0, 0
    while len(toks) < n:
        d, _ = orc.mtp_feed([tok], h_last)
        drafts += 1
        lw, _ = orc.forward([tok])
        a0 = int(np.argmax(lw))
        h0 = orc.mtp_hidden(0, 1)
        if len(toks) + 1 >= n:
            toks.append(a0); passes += 1; right += int(a0 == d)
            break
        if a0 == d:
            lw, _ = orc.forward([a0])
            a1 = int(np.argmax(lw))
            h1 = orc.mtp_hidden(0, 1)
            orc.mtp_feed([a0], h0, want_draft=False)
            toks += [a0, a1]; right += 1; passes += 1
            tok, h_last = a1, h1
        else:
            toks.append(a0); passes += 1
            tok, h_last = a0, h0
    return first, toks, {"drafts": drafts, "accepted": right, "passes": passes}


def _four_token_models(binding, seed):
    """A tiny model with a vocabulary of four tokens, so that a draft is right often enough for
    both outcomes to occur within a few steps."""
    spec = synth.tiny_spec()
    spec.cfg.vocab = 4
    tensors = synth.make_model(spec, seed=seed, recipe="spread")
    tensors.update(synth.make_mtp_layer(spec, seed=seed, recipe="spread"))
    orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 64, 2)
    orc.enable_mtp()
    orc.load_all(tensors); orc.finalize()
    return spec, tensors, orc


def test_speculative_decode_gives_the_greedy_tokens(gpu_lib, binding):
    spec, tensors, orc = _four_token_models(binding, SPEC_SEED)
    prompt = np.random.default_rng(3).integers(0, 4, 9).astype(np.int32)
    first, want, want_stats = _speculative_on_cpu(orc, prompt, 24)
    assert 0 < want_stats["accepted"] < want_stats["drafts"], want_stats      # both outcomes occur (the seed is chosen for it)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 64)
    eng.enable_mtp()
    eng.load_all(tensors); eng.finalize()
    lg, _ = eng.forward(prompt)
    assert int(np.argmax(lg)) == first
    hid = eng.mtp_hidden(0, prompt.size)
    with pytest.raises(RuntimeError, match="feed it the hidden states"):
        eng.decode_speculative(first, 4)
    eng.mtp_feed(prompt[1:], hid[:-1], want_draft=False)
    got, stats = eng.decode_speculative(first, 24)
    assert got.tolist() == want
    assert stats == want_stats
    # and plain greedy decode of a fresh session gives the same tokens
    eng.reset()
    lg, _ = eng.forward(prompt)
    assert eng.decode_greedy(int(np.argmax(lg)), 24).tolist() == want
    eng.close(); orc.close()
