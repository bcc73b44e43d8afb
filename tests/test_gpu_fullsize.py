"""GPU parity at the benchmark's full sizes: one MoE layer with 288 experts (batch 1, 8, 64), one
KDA layer (32 and 64 heads), one MLA layer at contexts 2048 / 8192 / 32768."""
import numpy as np
import pytest

import common
import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu
SEED = 0


@pytest.fixture(scope="module")
def moe_layer(gpu_lib):
    spec, trunk, eng = synth.build_moe_layer_engine(SEED)
    yield spec, trunk, eng
    eng.close()


@pytest.mark.parametrize("B", [1, 8, 64])
def test_full_size_moe_layer(moe_layer, binding, B):
    """Router indices identical to the CPU path; layer output within 1e-4 relative. The CPU side
    regenerates only the experts the router picked, from the same counter-based hash."""
    spec, trunk, eng = moe_layer
    x = synth.moe_inputs(spec.cfg, B, SEED)
    gi, gw = eng.op_router(0, x)
    orc = synth.oracle_moe_layer(binding, spec, trunk, SEED, gi.ravel())
    wi, ww = orc.op_router(0, x)
    assert np.array_equal(gi, wi)
    assert common.rel_err(gw, ww) < 1e-6
    got, want = eng.op_moe(0, x), orc.op_moe(0, x)
    assert np.isfinite(got).all()
    assert common.rel_err(got, want) < 1e-4
    # linearity of the routed sum in the router weights is a size-independent property: the
    # output without the shared expert plus the shared expert alone equals the full output
    routed = eng.op_moe(0, x, with_shared=False)
    assert common.rel_err(routed, orc.op_moe(0, x, with_shared=False)) < 1e-4
    orc.close()


@pytest.mark.parametrize("H", [32, 64])
def test_full_size_kda_layer(gpu_lib, binding, H):
    spec = synth.layer_spec("kda", kda_heads=H)
    tensors = synth.make_model(spec, seed=4, recipe="baseline")
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8)
    eng.set_option("allow_partial", 1)
    eng.load_all(tensors); eng.finalize()
    orc = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 8, 2)
    orc.load_all(tensors); orc.finalize()
    rng = np.random.default_rng(4)
    D = spec.cfg.kda_head_dim
    n = H * D * D + 3 * H * D * (spec.cfg.conv_k - 1)
    state = (rng.standard_normal(n) * 0.1).astype(np.float32)
    eng.state_write(0, 0, 0, state); orc.state_write(0, 0, 0, state)
    for T in (1, 1, 4):
        x = synth.bf16_round(rng.standard_normal((T, spec.cfg.hidden)).astype(np.float32))
        assert common.rel_err(eng.op_kda(0, x), orc.op_kda(0, x)) < 1e-4
    assert common.rel_err(eng.state_read(0, 0, 0, n), orc.state_read(0, 0, 0, n)) < 1e-5
    eng.close(); orc.close()


@pytest.mark.parametrize("latent_bf16", [0, 1])
def test_full_size_mla_layer(gpu_lib, binding, latent_bf16):
    """Contexts 2048 (dense regime: 512 pools fit the budget), 8192 and 32768 (the indexer keeps
    512 pools = 2048 positions + tail). Caches are seeded directly, BF16-representable values."""
    spec = synth.layer_spec("mla")
    c = spec.cfg
    cap = 32768
    tensors = synth.make_model(spec, seed=5, recipe="spread")
    eng = pkg.Engine(c, spec.is_mla, spec.is_dense, cap)
    eng.set_option("allow_partial", 1)
    eng.set_option("latent_bf16", latent_bf16)
    eng.load_all(tensors); eng.finalize()
    orc = binding.OracleModel(c, spec.is_mla, spec.is_dense, cap, 2)
    orc.load_all(tensors); orc.finalize()
    rng = np.random.default_rng(5)
    lat = synth.bf16_round(rng.standard_normal((cap, c.kv_lora)).astype(np.float32))
    idx = rng.standard_normal(2 * cap * c.index_dim + (cap // c.index_kpool) * c.index_dim).astype(np.float32)
    for m in (eng, orc):
        m.state_write(0, 1, 0, lat)
        m.state_write(0, 2, 0, idx)
    for ctx in (2048, 8192, 32768):
        x = synth.bf16_round(rng.standard_normal((1, c.hidden)).astype(np.float32))
        (g, gs), (w, ws) = eng.op_mla(0, x, ctx - 1), orc.op_mla(0, x, ctx - 1)
        if ctx == 2048:
            assert gs is None and ws is None
        else:
            assert len(ws) in (2048, 2049, 2050, 2051) and np.array_equal(gs, ws), ctx
        assert common.rel_err(g, w) < (3e-3 if latent_bf16 else 1e-4), ctx
        if latent_bf16:
            # the attention core on the tensor cores (the default with a BF16 cache) against the FP64
            # kernels on the same cache: same selection, output within the FP32 accumulation's reach
            eng.set_option("mla_tensor", 0)
            g64, gs64 = eng.op_mla(0, x, ctx - 1)
            eng.set_option("mla_tensor", 1)
            assert (gs is None and gs64 is None) or np.array_equal(gs, gs64)
            assert common.rel_err(g, g64) < 2e-5, ctx
    eng.close(); orc.close()


def test_expert_kernel_variants_agree(moe_layer, binding):
    """Batch 1 has three implementations: register-streaming CUDA-core kernels (the path odd shapes
    take), bulk-copy streamed tensor-core kernels as three launches, and the whole layer as one
    cooperative kernel (the default). All must give the CPU path's output."""
    spec, trunk, eng = moe_layer
    x = synth.moe_inputs(spec.cfg, 1, SEED + 3)
    # a general FP32 activation too, not only BF16-representable values
    x2 = (np.random.default_rng(5).standard_normal((1, spec.cfg.hidden)) * 3.7).astype(np.float32)
    for xin in (x, x2):
        idx, _ = eng.op_router(0, xin)
        orc = synth.oracle_moe_layer(binding, spec, trunk, SEED, idx.ravel())
        want = orc.op_moe(0, xin)
        outs = []
        for mode in (0, 1, 2):
            eng.set_option("expert_path", mode)
            outs.append(eng.op_moe(0, xin))
            assert common.rel_err(outs[-1], want) < 1e-5, mode
            assert common.rel_err(eng.op_moe(0, xin, False), orc.op_moe(0, xin, False)) < 1e-5, mode
        eng.set_option("expert_path", 2)
        for _ in range(3):
            assert np.array_equal(outs[2], eng.op_moe(0, xin))      # deterministic, counters carry over
        orc.close()
