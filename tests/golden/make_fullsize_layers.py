"""CPU results for two full-size decoder layers, stored as golden data.

Runs this repository's CPU oracle (oracle/, itself held bit for bit to the unmodified reference by
tests/test_oracle.py) on the two cases tests/fullmodel.py defines: a KDA + MoE layer and an MLA +
MoE layer (8191 cached positions, the indexer selecting 2048 + 3 of them), hidden 4096, four
residual streams, 288 routed experts, one new token. Weights are the synthetic full-size model's
(regenerated from the hashes the GPU fills HBM with), so only the experts the router picks are
ever materialised: a first pass walks the layer op by op to learn the picks, a second pass runs
glm53f_decoder_layer's restatement as a whole on a fresh state.

Writes fullsize_layers.npz: out0 / out1 (the residual streams leaving the layers), picks0 / picks1
(router choices), sel1 (the DSA-selected positions of the MLA case).

    python tests/golden/make_fullsize_layers.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import fullmodel  # noqa: E402
import synth  # noqa: E402
from oracle import binding  # noqa: E402


def rmsnorm(x, w_bits, eps):
    w = (w_bits.astype(np.uint32).ravel() << 16).view(np.float32)
    return binding.rmsnorm_host("orc", x, w, eps)


def picks_of(spec, seed, layer, h, cached, cap, inputs):
    """Walk the layer op by op (no routed expert needed up to the router) and return its picks."""
    c = spec.cfg
    orc = synth.oracle_full_layer(binding, spec, seed, layer, [], cap)
    orc.finalize()
    if spec.is_mla[layer]:
        orc.state_write(0, 1, 0, inputs["latent"].ravel()); orc.state_write(0, 2, 0, inputs["idx_state"])
    else:
        orc.state_write(0, 0, 0, inputs["kda_state"])
    x, post, comb = orc.op_hc_pre(0, 0, h)
    w_in, _ = synth.synth_vector(seed, f"layers.{layer}.input_layernorm.weight", c.hidden, synth.DT_BF16, "norm")
    xn = rmsnorm(x, w_in, c.rms_eps)
    sel = None
    if spec.is_mla[layer]:
        y, sel = orc.op_mla(0, xn, cached)
    else:
        y = orc.op_kda(0, xn)
    h1 = orc.op_hc_post(h, y, post, comb)
    x2, _, _ = orc.op_hc_pre(0, 1, h1)
    w_post, _ = synth.synth_vector(seed, f"layers.{layer}.post_attention_layernorm.weight", c.hidden, synth.DT_BF16, "norm")
    idx, _ = orc.op_router(0, rmsnorm(x2, w_post, c.rms_eps))
    orc.close()
    return idx, sel


def main():
    spec = fullmodel.layer_case_spec()
    seed, cap = fullmodel.LAYER_CASE_SEED, fullmodel.LAYER_CASE_CAP
    inputs = fullmodel.layer_case_inputs()
    out = {}
    for layer, cached in ((0, 0), (1, cap - 1)):
        h = inputs[f"h{layer}"]
        idx, sel = picks_of(spec, seed, layer, h, cached, cap, inputs)
        orc = synth.oracle_full_layer(binding, spec, seed, layer, idx.ravel(), cap)
        orc.finalize()
        if spec.is_mla[layer]:
            orc.state_write(0, 1, 0, inputs["latent"].ravel()); orc.state_write(0, 2, 0, inputs["idx_state"])
        else:
            orc.state_write(0, 0, 0, inputs["kda_state"])
        out[f"out{layer}"] = orc.op_decoder_layer(0, h, cached)
        out[f"picks{layer}"] = idx
        if sel is not None:
            out[f"sel{layer}"] = sel
        orc.close()
        print(f"layer {layer}: picks {idx.ravel().tolist()}, |out| max {np.abs(out[f'out{layer}']).max():.4g}")
    np.savez_compressed(os.path.join(HERE, "fullsize_layers.npz"), **out)


if __name__ == "__main__":
    main()
