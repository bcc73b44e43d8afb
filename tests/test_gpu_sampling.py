"""Sampled decode: the device sampler against a numpy restatement of its definition on the same
logits, and the sampled decode loop against that restatement applied to the engine's own logits."""
import numpy as np
import pytest

import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu
M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def sample_restated(logits, temperature, top_p, seed, step):
    """The definition in csrc/sample.cu, in numpy."""
    l = np.asarray(logits, np.float32)
    t = np.float32(temperature)
    p = np.exp(((l - l.max()) / t).astype(np.float64)).astype(np.float32)
    z = p.astype(np.float64).sum()
    keep = np.ones(p.size, bool)
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order].astype(np.float64))
        k = int(np.searchsorted(cum, np.float64(np.float32(top_p)) * z, side="left"))
        tau = p[order[min(k, p.size - 1)]]
        keep = p >= tau
    u = (_mix64(seed ^ _mix64(step + 1)) >> 11) * 2.0 ** -53
    mass = np.where(keep, p, 0).astype(np.float64)
    run = np.cumsum(mass)
    idx = int(np.searchsorted(run, u * run[-1], side="right"))
    while not keep[min(idx, p.size - 1)]:
        idx += 1
    return min(idx, p.size - 1)


@pytest.mark.parametrize("V", [64, 1024, 154880])
def test_sampler_matches_its_definition(gpu_lib, V):
    rng = np.random.default_rng(V)
    for case in range(12):
        logits = (rng.standard_normal(V) * rng.choice([0.5, 2.0, 6.0])).astype(np.float32)
        temperature = float(rng.choice([0.3, 0.8, 1.0, 1.7]))
        top_p = float(rng.choice([0.1, 0.5, 0.9, 0.95, 1.0]))
        seed, step = int(rng.integers(1, 1 << 40)), int(rng.integers(0, 4096))
        got = pkg.sample_host(logits, temperature, top_p, seed, step)
        want = sample_restated(logits, temperature, top_p, seed, step)
        assert got == want, (V, case, temperature, top_p, got, want)


def test_sampler_statistics_follow_the_distribution(gpu_lib):
    """Many draws with different counters: the empirical frequencies follow softmax(logits / T)."""
    logits = np.array([2.0, 1.0, 0.0, -1.0, -30.0, 1.5, 0.5, -0.5], np.float32)
    n = 4000
    counts = np.zeros(logits.size)
    for step in range(n):
        counts[pkg.sample_host(logits, 1.0, 1.0, 12345, step)] += 1
    p = np.exp(logits - logits.max()); p /= p.sum()
    assert np.abs(counts / n - p).max() < 0.03
    assert counts[4] == 0


def test_sampled_decode_loop(gpu_lib):
    spec = synth.tiny_spec()
    tensors = synth.make_model(spec, seed=5)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, cap=48)
    eng.load_all(tensors); eng.finalize()
    ids = np.random.default_rng(1).integers(0, spec.cfg.vocab, 10).astype(np.int32)
    # temperature 0 is the greedy loop
    lg, _ = eng.forward(ids)
    first = int(np.argmax(lg))
    greedy = eng.decode_greedy(first, 6)
    eng.reset(); eng.forward(ids)
    assert np.array_equal(eng.decode_sampled(first, 6, 0.0, 1.0, 7), greedy)
    # a sampled run, then the same run step by step through forward() + the restated sampler
    eng.reset(); eng.forward(ids)
    toks = eng.decode_sampled(first, 8, 0.9, 0.8, 99)
    eng.reset(); eng.forward(ids)
    tok, pos = first, ids.size
    for i in range(8):
        lg, _ = eng.forward([tok])
        pos += 1
        tok = sample_restated(lg, 0.9, 0.8, 99, pos)
        assert tok == int(toks[i]), i
    # split into two calls: the same tokens (the generator is keyed by position, not by call)
    eng.reset(); eng.forward(ids)
    a = eng.decode_sampled(first, 3, 0.9, 0.8, 99)
    b = eng.decode_sampled(int(a[-1]), 5, 0.9, 0.8, 99)
    assert np.array_equal(np.concatenate([a, b]), toks)
    eng.close()
