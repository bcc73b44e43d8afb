"""The full-size random-init model (benchmark configurations 4 and 5): building it in HBM, and the
layer-by-layer parity check against the CPU path.

The CPU cannot hold the 306 GB model, so parity at full size is taken per layer: the GPU runs one
decoder layer on a given residual stream h with its session state as it stands; the CPU oracle is
given the same h, the same state (read back from the GPU before the call), the layer's trunk
tensors regenerated from the hashes the GPU used, and of the routed experts only the ones the GPU's
router picked. If the oracle's own router picks anything else it finds no weights and fails, so a
passing comparison also shows that the picks agree. Used by tests/test_gpu_fullmodel.py and by
bench.py's full-model leg (on rank 0; the other expert-parallel ranks make the same engine calls).
"""
from __future__ import annotations

import numpy as np

import synth

pkg = synth.pkg


def build_engine(spec, seed: int, cap: int, device: int = 0, ep_rank: int = 0, ep_size: int = 1, options=None):
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, cap, device, ep_rank, ep_size)
    for k, v in (options or {}).items():
        eng.set_option(k, v)
    synth.fill_full_model(eng, spec, seed, ep_rank, ep_size)
    eng.finalize()
    return eng


def model_bytes(spec, ep_size: int = 1):
    """(bytes resident per rank, bytes read per decoded token per rank, bytes read per token by all
    ranks together) for the engine's layout: trunk and head replicated, routed experts split."""
    c = spec.cfg
    elt = {synth.DT_F32: 4, synth.DT_BF16: 2, synth.DT_FP8: 1}
    expert = 3 * c.moe_inter * c.hidden + 3 * (c.moe_inter // c.fp8_block_r) * (c.hidden // c.fp8_block_c) * 4
    trunk = 0
    for L in range(c.n_layers):
        for _, kind, rows, cols, dt, _ in synth.layer_tensor_table(c, bool(spec.is_mla[L]), bool(spec.is_dense[L])):
            trunk += rows * cols * elt[dt]
    n_moe = sum(1 for d in spec.is_dense if not d)
    head = c.vocab * c.hidden * 2
    resident = trunk + 2 * head + n_moe * (c.n_experts // ep_size) * expert
    token_all = trunk + head + n_moe * c.topk * expert            # one embedding row is negligible
    token_rank = trunk + head + n_moe * c.topk * expert / ep_size
    return int(resident), float(token_rank), float(token_all)


def merge_kda_states(states, cfg):
    """An expert-parallel engine with the tensor split holds a current KDA state for its own heads
    only. `states`: every rank's full-size state array of one layer, in rank order; returns the array
    with each rank's heads taken from that rank (layout: S [H][D][D], then the conv histories of
    q | k | v, each [H * D][k - 1], include/glm53f/glm53f.h:363-367)."""
    world = len(states)
    if world == 1:
        return states[0]
    H, D, hist = cfg.kda_heads, cfg.kda_head_dim, cfg.conv_k - 1
    P = H * D
    out = np.array(states[0], copy=True)
    per = H // world
    for r in range(1, world):
        src = states[r]
        h0, h1 = r * per, (r + 1) * per
        out[h0 * D * D:h1 * D * D] = src[h0 * D * D:h1 * D * D]
        for part in range(3):
            base = H * D * D + part * P * hist
            out[base + h0 * D * hist:base + h1 * D * hist] = src[base + h0 * D * hist:base + h1 * D * hist]
    return out


def layer_parity(eng, binding, spec, seed: int, layer: int, h: np.ndarray, cached: int, cap: int, check: bool = True,
                 ranks=None):
    """One decoder layer on the GPU and (when `check`) on the CPU from the same input and state.
    Returns {"rel_err", "picks", "picks_equal", "state_rel_err"}; rel_err is max |d| / max |ref| of
    the residual stream leaving the layer."""
    c = spec.cfg
    is_mla, is_dense = bool(spec.is_mla[layer]), bool(spec.is_dense[layer])
    T = h.shape[0]
    state = {}
    if ranks is not None and ranks.world > 1 and not is_mla:
        # every rank contributes its heads' state (a collective: all ranks call it)
        P = c.kda_heads * c.kda_head_dim
        mine = eng.state_read(layer, 0, 0, P * c.kda_head_dim + 3 * P * (c.conv_k - 1))
        gathered = ranks.gather(mine)
        if check:
            state[0] = merge_kda_states(gathered, c)
    if check:
        if is_mla:
            if cached:
                state[1] = eng.state_read(layer, 1, 0, cached * c.kv_lora)
            n_idx = 2 * cap * c.index_dim + ((cap + c.index_kpool - 1) // c.index_kpool) * c.index_dim
            state[2] = eng.state_read(layer, 2, 0, n_idx)
        elif 0 not in state:
            P = c.kda_heads * c.kda_head_dim
            state[0] = eng.state_read(layer, 0, 0, P * c.kda_head_dim + 3 * P * (c.conv_k - 1))
    got = eng.op_decoder_layer(layer, h, cached)
    picks = None
    if not is_dense:
        picks, _ = eng.last_picks(T)
    if not check:
        return {"picks": picks}
    orc = synth.oracle_full_layer(binding, spec, seed, layer, [] if picks is None else picks.ravel(), cap)
    orc.finalize()
    for kind, arr in state.items():
        orc.state_write(0, kind, 0, arr)
    want = orc.op_decoder_layer(0, h, cached)
    out = {"rel_err": float(np.max(np.abs(got.astype(np.float64) - want)) / (np.max(np.abs(want)) + 1e-300)),
           "picks": picks}
    if not is_dense:
        # the oracle routed by itself; rerun its router on its own normalised input is not exposed, so
        # equality of picks is what the missing-expert failure above already enforces
        out["picks_equal"] = True
    orc.close()
    return out


# ------------------------------------------------ two full-size decoder layers with stored CPU results ----
# Layer 0 = KDA + MoE, layer 1 = MLA (8191 cached positions, the indexer selecting) + MoE, all 288
# experts, one new token. tests/golden/fullsize_layers.npz holds the CPU path's output for them
# (tests/golden/make_fullsize_layers.py); the GPU test and bench.py's layer timings compare with it.
LAYER_CASE_SEED = 6
LAYER_CASE_CAP = 8192


def layer_case_spec():
    c = pkg.full_size_config()
    c.n_layers = 2
    return synth.Spec(c, [0, 1], [0, 0], with_head=False)


def layer_case_inputs():
    """Seeded inputs of the two cases: residual stream h [1][4][4096] ~ N(0, 1) for each layer, a KDA
    state ~ 0.1 N(0, 1), and for the MLA layer a latent cache ~ N(0, 1) rounded to BF16 and an
    indexer state ~ N(0, 1) covering every position below the query's."""
    c = layer_case_spec().cfg
    rng = np.random.default_rng(LAYER_CASE_SEED)
    cap = LAYER_CASE_CAP
    P = c.kda_heads * c.kda_head_dim
    return {
        "h0": rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32),
        "h1": rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32),
        "kda_state": (0.1 * rng.standard_normal(P * c.kda_head_dim + 3 * P * (c.conv_k - 1))).astype(np.float32),
        "latent": synth.bf16_round(rng.standard_normal((cap, c.kv_lora)).astype(np.float32)),
        "idx_state": rng.standard_normal(2 * cap * c.index_dim + (cap // c.index_kpool) * c.index_dim).astype(np.float32),
    }


def seed_layer_case_state(model, inputs, kda_layer=0, mla_layer=1):
    """Write the cases' session state into an engine or an oracle model (same flat API)."""
    model.state_write(kda_layer, 0, 0, inputs["kda_state"])
    model.state_write(mla_layer, 1, 0, inputs["latent"].ravel())
    model.state_write(mla_layer, 2, 0, inputs["idx_state"])


def load_layer_case_golden():
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fullsize_layers.npz")
    z = np.load(path)
    return {k: z[k] for k in z.files}


def build_layer_case_engine(device: int = 0, sequences: int = 1):
    """The two-layer engine of the stored cases, weights generated in HBM, state seeded."""
    spec = layer_case_spec()
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, LAYER_CASE_CAP, device)
    eng.set_option("allow_partial", 1)
    eng.set_option("latent_bf16", 1)
    if sequences > 1:
        eng.set_option("sequences", sequences)
    synth.fill_full_model(eng, spec, LAYER_CASE_SEED, head=False)
    eng.finalize()
    inputs = layer_case_inputs()
    seed_layer_case_state(eng, inputs)
    return spec, eng, inputs


def check_layer_case(eng, inputs, golden, layer: int) -> dict:
    """Run stored case `layer` on the engine (state must be as seeded) and compare with the CPU result."""
    cached = 0 if layer == 0 else LAYER_CASE_CAP - 1
    got = eng.op_decoder_layer(layer, inputs[f"h{layer}"], cached)
    picks, _ = eng.last_picks(1)
    want = golden[f"out{layer}"].astype(np.float64)
    return {"rel_err": float(np.max(np.abs(got - want)) / np.max(np.abs(want))),
            "picks_equal": bool(np.array_equal(picks, golden[f"picks{layer}"]))}
