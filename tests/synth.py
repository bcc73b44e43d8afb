"""Seeded synthetic models and layer inputs for the tests, the smoke check and the benchmark.

Nothing here comes from a dataset: the reference project measures on prompts that are not in its
repository, so every input is random with the shapes and value distributions its configs state
(hidden sizes, FP8 128x128 block scales, BF16 trunk, N(0, 0.02) weights, ...). torch is used
only for the FP8 / BF16 casts.
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass, field

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

pkg = load_package()
DT_F32, DT_BF16, DT_FP8 = pkg.DT_F32, pkg.DT_BF16, pkg.DT_FP8


@dataclass
class Spec:
    cfg: "pkg.Config"
    is_mla: list
    is_dense: list
    with_head: bool = True
    only: str = ""          # "", "moe", "kda", "mla": which sub-block a single-layer spec carries
    extra: dict = field(default_factory=dict)


def tiny_spec() -> Spec:
    """The tiny model of the benchmark's first configuration: hidden 256, 6 layers (layer 0
    dense inter 512, layers 1-5 MoE with 16 experts of inter 128, top-4, one shared expert),
    KDA in layers 0,1,2,4,5 (4 heads x 64, conv 4), MLA in layer 3 (4 heads, latent 128, pool 4 /
    top-16), 4 mHC streams with 20 Sinkhorn iterations, vocabulary 1024, FP8 blocks 128x128.
    Sizes the configuration leaves open: q_lora 192, qk_nope = v_head = 64, indexer 4 heads x 32.
    The KDA low-rank gates have rank head_dim (64): the reference binds f_a / g_a as
    [head_dim][hidden] (src/model/glm53f_bind.c:183,188), so a rank-16 gate could not be loaded."""
    c = pkg.Config(hidden=256, n_layers=6, vocab=1024, rms_eps=1e-5, hc_mult=4, hc_iters=20, hc_eps=1e-6,
                   kda_heads=4, kda_head_dim=64, conv_k=4, gate_lb=-5.0, mla_heads=4, q_lora=192, kv_lora=128,
                   qk_nope=64, v_head=64, index_topk=16, index_kpool=4, index_heads=4, index_dim=32,
                   n_experts=16, topk=4, n_shared=1, moe_inter=128, dense_inter=512, routed_scale=2.5,
                   norm_topk=1, swiglu_limit=10.0, fp8_block_r=128, fp8_block_c=128)
    return Spec(c, [0, 0, 0, 1, 0, 0], [1, 0, 0, 0, 0, 0])


def micro_spec() -> Spec:
    """Shapes of the reference's own unit-test model (hidden 32, FP8 blocks 4x4, head_dim 8, swiglu
    limit 0.5 so that the clamp binds): nothing is a multiple of 16 bytes, so every product takes
    the engine's any-shape kernels."""
    c = pkg.Config(hidden=32, n_layers=5, vocab=64, rms_eps=1e-5, hc_mult=4, hc_iters=20, hc_eps=1e-6,
                   kda_heads=2, kda_head_dim=8, conv_k=4, gate_lb=-5.0, mla_heads=2, q_lora=12, kv_lora=8,
                   qk_nope=8, v_head=8, index_topk=16, index_kpool=4, index_heads=2, index_dim=8,
                   n_experts=6, topk=2, n_shared=1, moe_inter=8, dense_inter=24, routed_scale=2.5,
                   norm_topk=1, swiglu_limit=0.5, fp8_block_r=4, fp8_block_c=4)
    return Spec(c, [0, 0, 1, 0, 1], [1, 0, 0, 0, 0])


def layer_spec(only: str, kda_heads: int = 64, n_experts: int = 288, hidden: int = 4096,
               moe_inter: int = 2048) -> Spec:
    """One full-size layer carrying a single sub-block (the benchmark's second and third
    configurations): only = 'moe' | 'kda' | 'mla'."""
    c = pkg.full_size_config()
    c.n_layers = 1
    c.kda_heads = kda_heads
    c.n_experts = n_experts
    c.hidden = hidden
    c.moe_inter = moe_inter
    return Spec(c, [1 if only == "mla" else 0], [0], with_head=False, only=only)


# ------------------------------------------------------------------ casts ----
def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 values that are exactly representable in BF16."""
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float()
    return t.numpy().copy()


def fp8_quant(w: np.ndarray, br: int, bc: int):
    """Per-block max-abs scaling to E4M3 (the released checkpoint's recipe): returns uint8 codes
    and the FP32 `scale_inv` grid. Ragged edge blocks are scaled by their own maximum."""
    rows, cols = w.shape
    sr, sc = (rows + br - 1) // br, (cols + bc - 1) // bc
    pad = np.zeros((sr * br, sc * bc), np.float32)
    pad[:rows, :cols] = w
    t = torch.from_numpy(pad).reshape(sr, br, sc, bc)
    mx = t.abs().amax(dim=(1, 3))
    scale = torch.where(mx > 0, 448.0 / torch.where(mx > 0, mx, torch.ones_like(mx)), torch.ones_like(mx))
    q = torch.clamp(t * scale[:, None, :, None], -448.0, 448.0).to(torch.float8_e4m3fn)
    codes = q.reshape(sr * br, sc * bc).view(torch.uint8).numpy()[:rows, :cols].copy()
    inv = (1.0 / scale).float().numpy().copy()
    return codes, inv


E4M3_TABLE = np.array(
    [(-1.0 if b >> 7 else 1.0) * (np.nan if (b & 0x7f) == 0x7f else
     ((b & 7) / 8.0 * 2.0 ** -6 if ((b >> 3) & 15) == 0 else (1 + (b & 7) / 8.0) * 2.0 ** (((b >> 3) & 15) - 7)))
     for b in range(256)], dtype=np.float32)


# ------------------------------------------------------------------ models ----
def make_model(spec: Spec, seed: int = 0, recipe: str = "baseline", experts: bool = True) -> dict:
    """{tensor name: (array, dtype, scale-or-None)} for every tensor the spec implies.

    recipe 'baseline': every matrix N(0, 0.02) and correction bias N(0, 0.1), norm weights
    1 + N(0, 0.02), mHC base N(0, 0.02) and scale 1, A_log and dt_bias N(0, 0.02).
    recipe 'spread': wider values so that every mechanism moves the output: matrices
    N(0, 0.5/sqrt(cols)), norm weights 1 + 0.3 N, mHC scale U(0.5, 1.5) and base N(0,1), A_log and
    dt_bias N(0,1)."""
    c = spec.cfg
    rng = np.random.default_rng(seed)
    out = {}
    E, M = c.hidden, c.hc_mult
    MIX = (2 + M) * M

    def mat_vals(rows, cols):
        std = 0.02 if recipe == "baseline" else 0.5 / np.sqrt(cols)
        return (rng.standard_normal((rows, cols)) * std).astype(np.float32)

    def bf(name, rows, cols):
        out[name] = (to_bf16_bits(mat_vals(rows, cols)), DT_BF16, None)

    def f8(name, rows, cols):
        codes, inv = fp8_quant(mat_vals(rows, cols), c.fp8_block_r, c.fp8_block_c)
        out[name] = (codes, DT_FP8, inv)

    def vec_bf(name, n, kind):
        if kind == "norm":
            v = 1.0 + (0.02 if recipe == "baseline" else 0.3) * rng.standard_normal(n)
        else:
            v = (0.02 if recipe == "baseline" else 0.3) * rng.standard_normal(n)
        out[name] = (to_bf16_bits(v.astype(np.float32)).reshape(n, 1), DT_BF16, None)

    def vec_f32(name, n, vals):
        out[name] = (np.ascontiguousarray(vals, dtype=np.float32).reshape(n, 1), DT_F32, None)

    wide = recipe != "baseline"
    if spec.with_head:
        bf("embed_tokens.weight", c.vocab, E)
        vec_bf("norm.weight", E, "norm")
        bf("lm_head.weight", c.vocab, E)
    for L in range(c.n_layers):
        p = f"layers.{L}."
        vec_bf(p + "input_layernorm.weight", E, "norm")
        vec_bf(p + "post_attention_layernorm.weight", E, "norm")
        for site in ("attn", "ffn"):
            bf(p + f"hc_{site}_fn", MIX, M * E)
            vec_f32(p + f"hc_{site}_base", MIX, rng.standard_normal(MIX) * (1.0 if wide else 0.02))
            vec_f32(p + f"hc_{site}_scale", 3, 0.5 + rng.random(3) if wide else np.ones(3))
        if spec.only in ("", "mla", "kda"):
            if spec.is_mla[L]:
                H, IH, ID = c.mla_heads, c.index_heads, c.index_dim
                f8(p + "self_attn.q_a_proj.weight", c.q_lora, E)
                vec_bf(p + "self_attn.q_a_layernorm.weight", c.q_lora, "norm")
                f8(p + "self_attn.q_b_proj.weight", H * c.qk_nope, c.q_lora)
                f8(p + "self_attn.kv_a_proj_with_mqa.weight", c.kv_lora, E)
                vec_bf(p + "self_attn.kv_a_layernorm.weight", c.kv_lora, "norm")
                bf(p + "self_attn.kv_b_proj.weight", H * (c.qk_nope + c.v_head), c.kv_lora)
                f8(p + "self_attn.o_proj.weight", E, H * c.v_head)
                bf(p + "self_attn.indexer.wq_b.weight", IH * ID, c.q_lora)
                bf(p + "self_attn.indexer.wk.weight", ID, E)
                vec_bf(p + "self_attn.indexer.k_norm.weight", ID, "norm")
                vec_bf(p + "self_attn.indexer.k_norm.bias", ID, "bias")
                bf(p + "self_attn.indexer.weights_proj.weight", IH, E)
                bf(p + "self_attn.indexer.index_kpool_compress_gate", ID, E)
                out[p + "self_attn.indexer.index_kpool_compress_ape"] = (
                    to_bf16_bits(mat_vals(c.index_kpool, ID)), DT_BF16, None)
            else:
                H, D = c.kda_heads, c.kda_head_dim
                P = H * D
                for n in ("q", "k", "v"):
                    bf(p + f"self_attn.{n}_proj.weight", P, E)
                    out[p + f"self_attn.{n}_conv1d.weight"] = (
                        to_bf16_bits((rng.standard_normal((P, c.conv_k)) * (0.3 if wide else 0.02)).astype(np.float32)),
                        DT_BF16, None)
                bf(p + "self_attn.f_a_proj.weight", D, E)
                bf(p + "self_attn.f_b_proj.weight", P, D)
                vec_f32(p + "self_attn.A_log", H, rng.standard_normal(H) * (1.0 if wide else 0.02))
                vec_f32(p + "self_attn.dt_bias", P, rng.standard_normal(P) * (1.0 if wide else 0.02))
                bf(p + "self_attn.b_proj.weight", H, E)
                bf(p + "self_attn.g_a_proj.weight", D, E)
                bf(p + "self_attn.g_b_proj.weight", P, D)
                vec_bf(p + "self_attn.o_norm.weight", D, "norm")
                bf(p + "self_attn.o_proj.weight", E, P)
        if spec.only in ("", "moe"):
            if spec.is_dense[L]:
                f8(p + "mlp.gate_proj.weight", c.dense_inter, E)
                f8(p + "mlp.up_proj.weight", c.dense_inter, E)
                f8(p + "mlp.down_proj.weight", E, c.dense_inter)
            else:
                SI = c.moe_inter * c.n_shared
                out[p + "mlp.gate.weight"] = (
                    to_bf16_bits((rng.standard_normal((c.n_experts, E)) * (0.02 if not wide else 0.5 / np.sqrt(E))
                                  ).astype(np.float32)), DT_BF16, None)
                vec_f32(p + "mlp.gate.e_score_correction_bias", c.n_experts, 0.1 * rng.standard_normal(c.n_experts))
                f8(p + "mlp.shared_experts.gate_proj.weight", SI, E)
                f8(p + "mlp.shared_experts.up_proj.weight", SI, E)
                f8(p + "mlp.shared_experts.down_proj.weight", E, SI)
                if experts:
                    for ex in range(c.n_experts):
                        f8(p + f"mlp.experts.{ex}.gate_proj.weight", c.moe_inter, E)
                        f8(p + f"mlp.experts.{ex}.up_proj.weight", c.moe_inter, E)
                        f8(p + f"mlp.experts.{ex}.down_proj.weight", E, c.moe_inter)
    return out


def make_mtp_layer(spec: Spec, seed: int = 0, recipe: str = "spread") -> dict:
    """The tensors of checkpoint layer n_layers, the multi-token-prediction layer: an MLA + MoE layer
    of the model's shapes without mHC tensors, plus enorm, hnorm, shared_head.norm and eh_proj
    [hidden][2 hidden] (the reference's plan_mtp, src/model/glm53f_bind.c:208-249). Drawn from a
    generator of its own, so the trunk made by make_model with the same seed is unchanged."""
    c = spec.cfg
    L = c.n_layers
    one = Spec(cfg=c, is_mla=np.array([1], np.uint8), is_dense=np.array([0], np.uint8), with_head=False)
    cfg1 = c.copy()
    cfg1.n_layers = 1
    one.cfg = cfg1
    layer = make_model(one, seed=seed + 7919, recipe=recipe)
    out = {}
    for name, v in layer.items():
        rest = name[len("layers.0."):]
        if rest.startswith("hc_"):
            continue
        out[f"layers.{L}.{rest}"] = v
    rng = np.random.default_rng(seed + 104729)
    E = c.hidden
    amp = 0.02 if recipe == "baseline" else 0.3
    for nm in ("enorm.weight", "hnorm.weight", "shared_head.norm.weight"):
        out[f"layers.{L}.{nm}"] = (to_bf16_bits((1.0 + amp * rng.standard_normal(E)).astype(np.float32)).reshape(E, 1), DT_BF16, None)
    std = 0.02 if recipe == "baseline" else 0.5 / np.sqrt(2 * E)
    out[f"layers.{L}.eh_proj.weight"] = (to_bf16_bits((rng.standard_normal((E, 2 * E)) * std).astype(np.float32)), DT_BF16, None)
    return out


# ------------------------------------------------- full-size MoE layer (config 2) ----
def expert_scales(cfg, layer: int, expert: int, seed: int):
    """FP32 block scales log-uniform in [2^-12, 2^-6] for the three matrices of one expert."""
    rng = np.random.default_rng([seed, layer, expert, 77])
    br, bc = cfg.fp8_block_r, cfg.fp8_block_c
    gs = ((cfg.moe_inter + br - 1) // br, (cfg.hidden + bc - 1) // bc)
    ds = ((cfg.hidden + br - 1) // br, (cfg.moe_inter + bc - 1) // bc)
    mk = lambda shape: np.exp2(-12.0 + 6.0 * rng.random(shape)).astype(np.float32)
    return mk(gs), mk(gs), mk(ds)


def moe_layer_trunk(spec: Spec, seed: int) -> dict:
    """Router (BF16, N(0, 0.02)), correction bias (FP32, N(0, 0.1)), shared expert (uniform finite
    codes, log-uniform scales) and the layer's norms / mHC tensors: everything of the full-size
    MoE layer except the routed experts, which are generated on the GPU."""
    c = spec.cfg
    t = make_model(spec, seed, "baseline", experts=False)
    rng = np.random.default_rng([seed, 4242])
    p = "layers.0.mlp.shared_experts."
    for n, (r, cc) in (("gate", (c.moe_inter, c.hidden)), ("up", (c.moe_inter, c.hidden)),
                       ("down", (c.hidden, c.moe_inter))):
        codes = rng.integers(0, 254, size=(r, cc), dtype=np.uint8)
        codes = (codes + (codes >= 127)).astype(np.uint8)
        sr, sc = (r + c.fp8_block_r - 1) // c.fp8_block_r, (cc + c.fp8_block_c - 1) // c.fp8_block_c
        t[p + f"{n}_proj.weight"] = (codes, DT_FP8, np.exp2(-12.0 + 6.0 * rng.random((sr, sc))).astype(np.float32))
    return t


def moe_inputs(cfg, T: int, seed: int) -> np.ndarray:
    """Activations ~ N(0, 1) rounded to BF16 (held as float32), [T][hidden]."""
    rng = np.random.default_rng([seed, T, 9])
    return bf16_round(rng.standard_normal((T, cfg.hidden)).astype(np.float32))


def build_moe_layer_engine(seed: int = 0, n_experts: int = 288, device: int = 0, options=None):
    """The benchmark's second configuration on the GPU: one full-size MoE layer (hidden 4096,
    inter 2048, `n_experts` routed + 1 shared, top-8); routed experts are generated on the device.
    Returns (spec, trunk tensors, engine)."""
    spec = layer_spec("moe", n_experts=n_experts)
    trunk = moe_layer_trunk(spec, seed)
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8, device)
    eng.set_option("allow_partial", 1)
    for k, v in (options or {}).items():
        eng.set_option(k, v)
    eng.load_all(trunk)
    for ex in range(n_experts):
        eng.fill_expert(0, ex, seed, *expert_scales(spec.cfg, 0, ex, seed))
    eng.finalize()
    return spec, trunk, eng


def oracle_moe_layer(binding, spec: Spec, trunk: dict, seed: int, experts):
    """The same layer on the CPU with only `experts` materialised (regenerated from the hash)."""
    c = spec.cfg
    orc = binding.OracleModel(c, spec.is_mla, spec.is_dense, 8, 2)
    keep = ("mlp.gate.weight", "mlp.gate.e_score_correction_bias", "mlp.shared_experts")
    for name, (arr, dt, sc) in trunk.items():
        if any(k in name for k in keep):
            orc.load(name, arr, dt, sc)
    n = c.moe_inter * c.hidden
    for ex in sorted(set(int(e) for e in experts)):
        gs, us, ds = expert_scales(c, 0, ex, seed)
        for which, (nm, shape, sc) in enumerate((("gate", (c.moe_inter, c.hidden), gs),
                                                 ("up", (c.moe_inter, c.hidden), us),
                                                 ("down", (c.hidden, c.moe_inter), ds))):
            codes = binding.synth_codes(seed, 0, ex, which, n).reshape(shape)
            orc.load(f"layers.0.mlp.experts.{ex}.{nm}_proj.weight", codes, DT_FP8, sc)
    return orc


# ------------------------------------------- full-size model (configs 4 and 5) ----
BF16_UNIT = 37837.2       # standard deviation of the device generator's BF16 values at mul = 1


def full_model_spec(n_layers: int = 45) -> Spec:
    """The released architecture (45 layers: MLA at 3, 7, ..., 43, KDA elsewhere; dense MLP in
    layers 0-2, MoE from 3 on), optionally cut to its first `n_layers` layers the way the
    reference's --layers option does (src/model/glm53f_model.c:77)."""
    c = pkg.full_size_config()
    c.n_layers = n_layers
    is_mla = [1 if l % 4 == 3 else 0 for l in range(n_layers)]
    is_dense = [1 if l < 3 else 0 for l in range(n_layers)]
    return Spec(c, is_mla, is_dense)


def layer_tensor_table(c, is_mla: bool, is_dense: bool):
    """[(name below 'layers.L.', 'mat' | 'vec', rows, cols, dtype, what)] of one decoder layer, routed
    experts excluded: names and shapes as the reference binds them (src/model/glm53f_bind.c:139-206).
    `what` tells the generators which distribution a vector gets."""
    E, M = c.hidden, c.hc_mult
    MIX = (2 + M) * M
    t = [("input_layernorm.weight", "vec", E, 1, DT_BF16, "norm"),
         ("post_attention_layernorm.weight", "vec", E, 1, DT_BF16, "norm")]
    for site in ("attn", "ffn"):
        t += [(f"hc_{site}_fn", "mat", MIX, M * E, DT_BF16, ""), (f"hc_{site}_base", "vec", MIX, 1, DT_F32, "small"),
              (f"hc_{site}_scale", "vec", 3, 1, DT_F32, "one")]
    a = "self_attn."
    if is_mla:
        H, IH, ID = c.mla_heads, c.index_heads, c.index_dim
        t += [(a + "q_a_proj.weight", "mat", c.q_lora, E, DT_FP8, ""), (a + "q_a_layernorm.weight", "vec", c.q_lora, 1, DT_BF16, "norm"),
              (a + "q_b_proj.weight", "mat", H * c.qk_nope, c.q_lora, DT_FP8, ""),
              (a + "kv_a_proj_with_mqa.weight", "mat", c.kv_lora, E, DT_FP8, ""),
              (a + "kv_a_layernorm.weight", "vec", c.kv_lora, 1, DT_BF16, "norm"),
              (a + "kv_b_proj.weight", "mat", H * (c.qk_nope + c.v_head), c.kv_lora, DT_BF16, ""),
              (a + "o_proj.weight", "mat", E, H * c.v_head, DT_FP8, ""),
              (a + "indexer.wq_b.weight", "mat", IH * ID, c.q_lora, DT_BF16, ""),
              (a + "indexer.wk.weight", "mat", ID, E, DT_BF16, ""),
              (a + "indexer.k_norm.weight", "vec", ID, 1, DT_BF16, "norm"), (a + "indexer.k_norm.bias", "vec", ID, 1, DT_BF16, "small"),
              (a + "indexer.weights_proj.weight", "mat", IH, E, DT_BF16, ""),
              (a + "indexer.index_kpool_compress_gate", "mat", ID, E, DT_BF16, ""),
              (a + "indexer.index_kpool_compress_ape", "vec", c.index_kpool * ID, 1, DT_BF16, "small")]
    else:
        H, D = c.kda_heads, c.kda_head_dim
        P = H * D
        for n in ("q", "k", "v"):
            t += [(a + f"{n}_proj.weight", "mat", P, E, DT_BF16, ""), (a + f"{n}_conv1d.weight", "vec", P * c.conv_k, 1, DT_BF16, "small")]
        t += [(a + "f_a_proj.weight", "mat", D, E, DT_BF16, ""), (a + "f_b_proj.weight", "mat", P, D, DT_BF16, ""),
              (a + "A_log", "vec", H, 1, DT_F32, "small"), (a + "dt_bias", "vec", P, 1, DT_F32, "small"),
              (a + "b_proj.weight", "mat", H, E, DT_BF16, ""), (a + "g_a_proj.weight", "mat", D, E, DT_BF16, ""),
              (a + "g_b_proj.weight", "mat", P, D, DT_BF16, ""), (a + "o_norm.weight", "vec", D, 1, DT_BF16, "norm"),
              (a + "o_proj.weight", "mat", E, P, DT_BF16, "")]
    if is_dense:
        t += [("mlp.gate_proj.weight", "mat", c.dense_inter, E, DT_FP8, ""), ("mlp.up_proj.weight", "mat", c.dense_inter, E, DT_FP8, ""),
              ("mlp.down_proj.weight", "mat", E, c.dense_inter, DT_FP8, "")]
    else:
        SI = c.moe_inter * c.n_shared
        t += [("mlp.gate.weight", "mat", c.n_experts, E, DT_BF16, ""), ("mlp.gate.e_score_correction_bias", "vec", c.n_experts, 1, DT_F32, "bias"),
              ("mlp.shared_experts.gate_proj.weight", "mat", SI, E, DT_FP8, ""), ("mlp.shared_experts.up_proj.weight", "mat", SI, E, DT_FP8, ""),
              ("mlp.shared_experts.down_proj.weight", "mat", E, SI, DT_FP8, "")]
    return t


def synth_vector(seed: int, name: str, n: int, dtype: int, what: str):
    """A small vector of the full-size synthetic model, made on the host: norm weights 1 + N(0, 0.02),
    correction bias N(0, 0.1), mHC scale 1, everything else N(0, 0.02). Seeded by (seed, name)."""
    import zlib
    rng = np.random.default_rng([seed, zlib.crc32(name.encode())])
    v = {"norm": lambda: 1.0 + 0.02 * rng.standard_normal(n), "bias": lambda: 0.1 * rng.standard_normal(n),
         "one": lambda: np.ones(n), "small": lambda: 0.02 * rng.standard_normal(n)}[what]().astype(np.float32)
    if dtype == DT_BF16:
        return to_bf16_bits(v).reshape(n, 1), DT_BF16
    return v.reshape(n, 1), DT_F32


E4M3_UNIFORM_RMS = 100.058      # root mean square of the 254 finite E4M3 values, each equally likely


def synth_scale_grid(c, seed: int, name: str, rows: int, cols: int) -> np.ndarray:
    """FP32 block scales of a synthetic FP8 matrix of the full-size model: log-uniform over a factor
    of four around 0.02 / (RMS of uniform codes), so that the matrix as a whole has the N(0, 0.02)
    magnitude of the other random-init weights and every sub-block's output stays O(1)."""
    import zlib
    rng = np.random.default_rng([seed, zlib.crc32(name.encode()), 5])
    sr, sc = (rows + c.fp8_block_r - 1) // c.fp8_block_r, (cols + c.fp8_block_c - 1) // c.fp8_block_c
    return (0.02 / E4M3_UNIFORM_RMS * np.exp2(-1.0 + 2.0 * rng.random((sr, sc)))).astype(np.float32)


def full_expert_scales(c, layer: int, expert: int, seed: int):
    """The three scale grids (gate, up, down) of a routed expert of the full-size synthetic model."""
    p = f"layers.{layer}.mlp.experts.{expert}."
    return (synth_scale_grid(c, seed, p + "gate_proj.weight", c.moe_inter, c.hidden),
            synth_scale_grid(c, seed, p + "up_proj.weight", c.moe_inter, c.hidden),
            synth_scale_grid(c, seed, p + "down_proj.weight", c.hidden, c.moe_inter))


def model_level_tensors(c):
    return [("embed_tokens.weight", "mat", c.vocab, c.hidden, DT_BF16, ""), ("norm.weight", "vec", c.hidden, 1, DT_BF16, "norm"),
            ("lm_head.weight", "mat", c.vocab, c.hidden, DT_BF16, "")]


def fill_full_model(eng, spec: Spec, seed: int, ep_rank: int = 0, ep_size: int = 1, head: bool = True):
    """Random-init weights of the full-size architecture straight into HBM: matrices are generated on
    the GPU (g5b_engine_fill_matrix / fill_expert), vectors and scale grids on the host. BF16
    matrices ~ N(0, 0.02); FP8 matrices uniform finite codes with block scales that give them the
    same overall magnitude."""
    c = spec.cfg
    mul = np.float32(0.02 / BF16_UNIT)

    def put(name, kind, rows, cols, dt, what):
        if kind == "vec":
            arr, vdt = synth_vector(seed, name, rows, dt, what)
            eng.load(name, arr, vdt)
        elif dt == DT_BF16:
            eng.fill_matrix(name, DT_BF16, seed, rows, mul=float(mul))
        else:
            eng.fill_matrix(name, DT_FP8, seed, rows, scale_inv=synth_scale_grid(c, seed, name, rows, cols))

    if head:
        for row in model_level_tensors(c):
            put(*row)
    per = c.n_experts // ep_size
    for L in range(c.n_layers):
        for name, kind, rows, cols, dt, what in layer_tensor_table(c, bool(spec.is_mla[L]), bool(spec.is_dense[L])):
            put(f"layers.{L}." + name, kind, rows, cols, dt, what)
        if not spec.is_dense[L]:
            for ex in range(ep_rank * per, (ep_rank + 1) * per):
                eng.fill_expert(L, ex, seed, *full_expert_scales(c, L, ex, seed))


def oracle_full_layer(binding, spec: Spec, seed: int, layer: int, experts, cap: int, kv_mode: int = 2):
    """Layer `layer` of the synthetic full-size model on the CPU, as a one-layer model: every trunk
    tensor of the layer is regenerated from the same hashes the GPU used, and of the routed experts
    only those in `experts` (the ones the GPU's router picked) are materialised."""
    c = spec.cfg.copy()
    c.n_layers = 1
    mul = np.float32(0.02 / BF16_UNIT)
    orc = binding.OracleModel(c, [spec.is_mla[layer]], [spec.is_dense[layer]], cap, kv_mode)
    for name, kind, rows, cols, dt, what in layer_tensor_table(c, bool(spec.is_mla[layer]), bool(spec.is_dense[layer])):
        src = f"layers.{layer}." + name
        if kind == "vec":
            arr, vdt = synth_vector(seed, src, rows, dt, what)
            orc.load("layers.0." + name, arr, vdt)
        elif dt == DT_BF16:
            orc.load("layers.0." + name, binding.synth_matrix_bf16(seed, src, float(mul), rows * cols).reshape(rows, cols), DT_BF16)
        else:
            orc.load("layers.0." + name, binding.synth_matrix_codes(seed, src, rows * cols).reshape(rows, cols), DT_FP8,
                     synth_scale_grid(spec.cfg, seed, src, rows, cols))
    if not spec.is_dense[layer]:
        n = c.moe_inter * c.hidden
        for ex in sorted(set(int(e) for e in experts)):
            gs, us, ds = full_expert_scales(c, layer, ex, seed)
            for which, (nm, shape, sc) in enumerate((("gate", (c.moe_inter, c.hidden), gs), ("up", (c.moe_inter, c.hidden), us),
                                                     ("down", (c.hidden, c.moe_inter), ds))):
                codes = binding.synth_codes(seed, layer, ex, which, n).reshape(shape)
                orc.load(f"layers.0.mlp.experts.{ex}.{nm}_proj.weight", codes, DT_FP8, sc)
    return orc
