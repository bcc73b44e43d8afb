"""Benchmark of the decode hot path: one full-size MoE layer of the GLM-5.3-Flash architecture
(hidden 4096, 288 routed experts + 1 shared of inter 2048, top-8 sigmoid router, FP8 E4M3 codes
with 128x128 block scales), batch 1 - the configuration the expert-GEMV roofline is quoted on.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one pass of the layer over one token. Prints ONE JSON line:
  value        decode tokens/s through the layer with inputs resident in HBM (CUDA events on the
               engine's stream around each step, L2 flushed before each step)
  e2e          the same through the host-buffer C-ABI call (pinned host memory in and out)
  roofline     the layer's kernel: algorithmic bytes / its event-timed duration against the
               measured HBM copy bandwidth; in_layer = the same inside a whole decoder layer
  cpu_baseline the reference's own CPU implementation (glm53f_moe) on this box's host cores (N = 1)
  extra        batch 8 / 64, the attention layers, whole decoder layers, and the full-size
               random-init model (as many of its 45 layers as the GPUs hold) decoded greedily
With N > 1 (launched by torchrun, one rank per GPU) the N GPUs serve ONE token stream together:
the layer is expert parallel (288 / N routed experts per rank, rows exchanged over NVLink peer
mappings inside the layer's kernel), so the scaling is strong; the time is the maximum over ranks.
Before timing, the expert-parallel output is compared with the one-GPU engine's on the same inputs
(extra.expert_parallel.parity). N independent replicas are reported under extra.replicas.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

SEED = 0
EXPERT_BYTES = 3 * 2048 * 4096 + 3 * 16 * 32 * 4            # codes + block scales of one expert
GATEUP_BYTES = 2 * 2048 * 4096 + 2 * 16 * 32 * 4            # what the gate/up kernel reads per expert
ROUTER_BYTES = 288 * 4096 * 2                               # BF16 router matrix
FLUSH_BYTES = 512 << 20                                     # two halves, each > 126 MB of L2: write one, read the other
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up launch at batch 1 (profiles/), or None
# DRAM bytes (read + write) per launch from the ncu captures summarised under profiles/
GATEUP_TRAFFIC_NCU = None
DECODE_TRAFFIC_NCU = 233.9e6      # moe_decode_kernel: 231.8 MB captured with 32 resident experts + 2.1 MB for 256 more router rows


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def wait_first(self, timeout=8.0):
        """nvidia-smi takes a second or so to print its first line; the timed region is short, so wait
        for the sampler to be running before the region starts and drop what it saw until then."""
        t0 = time.time()
        while self.proc and not self.rows and time.time() - t0 < timeout:
            time.sleep(0.02)
        self.rows.clear()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_moe(steps: int, warmup: int, batch: int = 1, threads: int | None = None):
    """The reference's glm53f_moe (oracle/_ref, built from the unmodified reference sources) on the
    host cores, on the same layer: `steps` calls on a rotating set of 4 seeded inputs. Falls back to
    this repo's CPU restatement when the reference objects are absent. Returns a dict."""
    import synth
    from oracle import binding
    spec = synth.layer_spec("moe")
    trunk = synth.moe_layer_trunk(spec, SEED)
    xs = [synth.moe_inputs(spec.cfg, batch, SEED + i) for i in range(4)]
    kind = "reference" if binding.have_ref() else "port"
    router = binding.OracleModel(spec.cfg, spec.is_mla, spec.is_dense, 8, 2)
    for name, (arr, dt, sc) in trunk.items():
        if "mlp.gate." in name:
            router.load(name, arr, dt, sc)
    chosen = np.concatenate([router.op_router(0, x)[0].ravel() for x in xs])
    router.close()
    cls = binding.RefModel if kind == "reference" else binding.OracleModel
    m = cls(spec.cfg, spec.is_mla, spec.is_dense, 8, 2)
    keep = ("mlp.gate.weight", "mlp.gate.e_score_correction_bias", "mlp.shared_experts")
    for name, (arr, dt, sc) in trunk.items():
        if any(k in name for k in keep):
            m.load(name, arr, dt, sc)
    c = spec.cfg
    for ex in sorted(set(int(e) for e in chosen)):
        gs, us, ds = synth.expert_scales(c, 0, ex, SEED)
        for which, (nm, shape, sc) in enumerate((("gate", (c.moe_inter, c.hidden), gs), ("up", (c.moe_inter, c.hidden), us),
                                                 ("down", (c.hidden, c.moe_inter), ds))):
            codes = binding.synth_codes(SEED, 0, ex, which, c.moe_inter * c.hidden).reshape(shape)
            m.load(f"layers.0.mlp.experts.{ex}.{nm}_proj.weight", codes, synth.DT_FP8, sc)
    cores = threads or os.cpu_count() or 1
    try:                                            # the thread count of the OpenMP runtime the CPU library uses
        C.CDLL("libgomp.so.1", mode=C.RTLD_GLOBAL).omp_set_num_threads(cores)
    except OSError:
        pass
    for i in range(warmup):
        m.op_moe(0, xs[i % 4])
    t0 = time.perf_counter()
    for i in range(steps):
        m.op_moe(0, xs[i % 4])
    dt = time.perf_counter() - t0
    m.close()
    return {"value": batch * steps / dt, "unit": "tokens/s", "cores": cores, "kind": kind,
            "ms_per_step": 1e3 * dt / steps,
            "sample": f"{steps} calls of glm53f_moe at batch {batch} on 4 rotating seeded inputs, "
                      f"{len(set(chosen.tolist()))} distinct routed experts + shared resident in RAM"}


METRIC = "decode tokens/s through one full-size MoE layer, batch 1"
DTYPE = "fp8_e4m3 weights, f32 activations and accumulation"


def bench_config(world: int) -> dict:
    """The `config` object of the JSON line: the same for this repo's arm and the reference arm."""
    return {"workload": "config 2: single MoE layer decode, hidden 4096, inter 2048, 288+1 experts, top-8, batch 1",
            "l2": f"GPU arm: flushed before every step ({FLUSH_BYTES >> 21} MiB written, then {FLUSH_BYTES >> 21} MiB "
                  "read so that no dirty line is left), the timed steps dealt over 16 different tokens; CPU arm: 4 rotating "
                  "inputs, 226 MB of weights per step",
            "parallelism": "one GPU" if world == 1 else
                           f"expert parallel over {world} GPUs: one token stream, {288 // world} routed experts per rank"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    warmup = max(3, args.warmup)
    r = cpu_reference_moe(args.steps, warmup)
    line = {"impl": "reference", "metric": METRIC,
            "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup,
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic", "config": bench_config(max(1, args.gpus)),
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def time_batch(pkg, eng, torch, B, steps, warmup, flush=FLUSH_BYTES, phases=True, inputs=1):
    """Device-resident timing of the MoE layer at batch B: (ms per step list, phase ms, launches, output, ms
    per input). `inputs` > 1: the `steps` timed steps are dealt over that many different seeded inputs
    (different routings: with expert parallelism a step takes what the busiest rank takes, which depends on
    how the token's eight picks fall on the ranks)."""
    import synth
    L = pkg.lib()
    inputs = max(1, min(inputs, steps))
    xs = [torch.from_numpy(synth.moe_inputs(eng.cfg, B, SEED + 1000 * k)).cuda() for k in range(inputs)]
    out = torch.empty_like(xs[0])
    torch.cuda.synchronize()
    each = np.zeros(max(steps, warmup, 1), np.float32)
    tot = C.c_float(0)
    assert L.g5b_time_op(eng.handle, b"moe", 0, xs[0].data_ptr(), B, 0, out.data_ptr(), warmup, flush,
                         C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
    ms4 = (C.c_float * 8)()
    cnt = C.c_long(0)
    n0 = L.g5b_launch_count()
    timed, per_input = [], []
    for k, x in enumerate(xs):
        share = steps // inputs + (1 if k < steps % inputs else 0)          # exactly `steps` timed steps in all
        assert L.g5b_time_op(eng.handle, b"moe", 0, x.data_ptr(), B, 0, out.data_ptr(), share, flush,
                             C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        timed += each[:share].astype(float).tolist()
        per_input.append(float(np.mean(each[:share])))
    launches = L.g5b_launch_count() - n0 - (2 * steps if flush else 0)
    timed = np.asarray(timed)
    if not phases:
        return timed, [0.0] * 4, int(launches), out, per_input
    # per-phase times in a separate short pass: the phase events make the host wait inside every
    # step, which would inflate the step time measured above
    eng.set_option("profile", 1)
    L.g5b_engine_profile_read(eng.handle, ms4, 8, C.byref(cnt), 1)
    scratch = np.zeros(32, np.float32)
    assert L.g5b_time_op(eng.handle, b"moe", 0, xs[0].data_ptr(), B, 0, out.data_ptr(), min(20, max(3, steps)), flush,
                         C.byref(tot), scratch.ctypes.data) == 0, L.g5b_last_error()
    L.g5b_engine_profile_read(eng.handle, ms4, 8, C.byref(cnt), 1)
    eng.set_option("profile", 0)
    phases = [ms4[i] / max(1, cnt.value) for i in range(4)]
    return timed, phases, int(launches), out, per_input


def time_attention_layers(pkg, torch, steps: int, peak: float, device: int = 0):
    """The third benchmark configuration: one full-size KDA layer (32 and 64 heads) and one MLA layer
    with the indexer at contexts 2048 / 8192 / 32768, one new token, device-resident, L2 flushed
    before every call. Bytes = the layer's weights as stored + recurrent state read and written
    (KDA) or the latent rows and pooled keys read (MLA)."""
    import synth
    L = pkg.lib()
    out = {}

    def weight_bytes(tensors):
        return int(sum(a.nbytes + (0 if sc is None else sc.nbytes) for a, _, sc in tensors.values()))

    def run(eng, op, x, cached, n):
        xd = torch.from_numpy(x).cuda(); od = torch.empty_like(xd)
        each = np.zeros(max(n, 3), np.float32); tot = C.c_float(0)
        for k in (3, n):
            assert L.g5b_time_op(eng.handle, op, 0, xd.data_ptr(), x.shape[0], cached, od.data_ptr(), k, FLUSH_BYTES,
                                 C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        return float(np.mean(each[:n]))

    rng = np.random.default_rng(SEED)
    for H in (32, 64):
        spec = synth.layer_spec("kda", kda_heads=H)
        tensors = synth.make_model(spec, seed=4, recipe="baseline")
        eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8, device)
        eng.set_option("allow_partial", 1)
        eng.load_all(tensors); eng.finalize()
        D = spec.cfg.kda_head_dim
        state_bytes = 4 * (H * D * D + 3 * H * D * (spec.cfg.conv_k - 1))
        x = synth.bf16_round(rng.standard_normal((1, spec.cfg.hidden)).astype(np.float32))
        ms = run(eng, b"kda", x, 0, steps)
        nbytes = weight_bytes(tensors) + 2 * state_bytes
        out[f"kda_H{H}"] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_GBps": nbytes / (ms * 1e-3) / 1e9,
                            "frac": nbytes / (ms * 1e-3) / 1e9 / peak}
        if H == 64:
            # the same layer over a prefill chunk: 64 positions of one sequence
            x64 = synth.bf16_round(rng.standard_normal((64, spec.cfg.hidden)).astype(np.float32))
            out["kda_H64_64_positions"] = {"ms": run(eng, b"kda", x64, 0, max(3, steps // 4))}
        eng.close()
    spec = synth.layer_spec("mla")
    c = spec.cfg
    cap = 32768
    tensors = synth.make_model(spec, seed=5, recipe="spread")
    eng = pkg.Engine(c, spec.is_mla, spec.is_dense, cap, device)
    eng.set_option("allow_partial", 1)
    eng.set_option("latent_bf16", 1)
    eng.load_all(tensors); eng.finalize()
    lat = synth.bf16_round(rng.standard_normal((cap, c.kv_lora)).astype(np.float32))
    idx = rng.standard_normal(2 * cap * c.index_dim + (cap // c.index_kpool) * c.index_dim).astype(np.float32)
    eng.state_write(0, 1, 0, lat)
    eng.state_write(0, 2, 0, idx)
    x = synth.bf16_round(rng.standard_normal((1, c.hidden)).astype(np.float32))
    for ctx in (2048, 8192, 32768):
        ms = run(eng, b"mla", x, ctx - 1, steps)
        visible = min(ctx, c.index_topk + c.index_kpool - 1)
        nbytes = weight_bytes(tensors) + visible * c.kv_lora * 2 + (ctx // c.index_kpool) * c.index_dim * 4
        out[f"mla_ctx{ctx}"] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_GBps": nbytes / (ms * 1e-3) / 1e9,
                                "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "latent": "bf16"}
    eng.close()
    return out


def time_mhc_site(pkg, torch, steps: int, device: int = 0):
    """One mHC site of a full-size layer on its own (gates, Sinkhorn, collapse, the sub-block's
    RMSNorm in one launch), without and with the previous sub-block's stream expansion riding along,
    for 1 and 64 tokens. The engine holds one KDA + MoE layer with 16 routed experts (0.5 GB): small
    enough for a profiler capture."""
    import synth
    L = pkg.lib()
    c = pkg.full_size_config()
    c.n_layers = 1
    c.n_experts = 16
    spec = synth.Spec(c, [0], [0], with_head=False)
    tensors = synth.make_model(spec, seed=6, recipe="baseline", experts=False)
    eng = pkg.Engine(c, spec.is_mla, spec.is_dense, 8, device)
    eng.set_option("allow_partial", 1)
    eng.set_option("sequences", 64)
    eng.load_all(tensors)
    for ex in range(c.n_experts):
        eng.fill_expert(0, ex, SEED, *synth.expert_scales(c, 0, ex, SEED))
    eng.finalize()
    rng = np.random.default_rng(SEED)
    out = {}
    for T in (1, 64):
        h = torch.from_numpy(rng.standard_normal((T, c.hc_mult, c.hidden)).astype(np.float32)).cuda()
        for op in (b"hc_site", b"hc_site_post"):
            hd = h.clone()
            each = np.zeros(max(steps, 3), np.float32); tot = C.c_float(0)
            for k in (3, steps):
                hd.copy_(h)
                assert L.g5b_time_op(eng.handle, op, 0, hd.data_ptr(), T, 0, hd.data_ptr(), k, FLUSH_BYTES,
                                     C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
            out[f"{op.decode()}_T{T}_us"] = float(np.mean(each[:steps])) * 1e3
    eng.close()
    return out


def time_decoder_layers(pkg, torch, steps: int, device: int = 0):
    """Two whole full-size decoder layers, one new token: layer 0 = KDA + MoE, layer 1 = MLA (8191
    cached positions, indexer selecting) + MoE, each with its two mHC sites and norms; weights
    generated in HBM. Before anything is timed each layer's output is compared with the CPU path's
    stored result for the same seeded input and state (tests/golden/fullsize_layers.npz)."""
    import fullmodel
    L = pkg.lib()
    golden = fullmodel.load_layer_case_golden()
    spec, eng, inputs = fullmodel.build_layer_case_engine(device, sequences=64)
    c, cap = spec.cfg, fullmodel.LAYER_CASE_CAP
    out = {"parity_vs_stored_cpu_result": {name: fullmodel.check_layer_case(eng, inputs, golden, layer)
                                           for layer, name in ((0, "kda_moe_layer"), (1, "mla_moe_layer_ctx8192"))}}
    rng = np.random.default_rng(SEED)
    h = torch.from_numpy(rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32)).cuda()

    def timed(op, layer, hsrc, T, cached, n):
        hd = hsrc.clone()
        each = np.zeros(max(n, 3), np.float32); tot = C.c_float(0)
        for k in (3, n):
            hd.copy_(hsrc)
            assert L.g5b_time_op(eng.handle, op, layer, hd.data_ptr(), T, cached, hd.data_ptr(), k, FLUSH_BYTES,
                                 C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        return {"ms": float(np.mean(each[:n])), "finite": bool(torch.isfinite(hd).all().item())}

    out["kda_moe_layer"] = timed(b"layer", 0, h, 1, 0, steps)
    out["mla_moe_layer_ctx8192"] = timed(b"layer", 1, h, 1, cap - 1, steps)
    # both layers in one pass (the second layer's first mHC site applies the first layer's pending
    # stream expansion inside its own launch, as in the whole model)
    out["kda_moe_then_mla_moe_layers"] = timed(b"layers", 0, h, 1, cap - 1, steps)
    # the same two layers advancing 64 sequences by one token each (state and caches per sequence,
    # weights read once per batch)
    h64 = torch.from_numpy(rng.standard_normal((64, c.hc_mult, c.hidden)).astype(np.float32)).cuda()
    out["kda_moe_layer_batch64"] = timed(b"layer_batch", 0, h64, 64, 0, max(3, steps // 2))
    out["mla_moe_layer_ctx8192_batch64"] = timed(b"layer_batch", 1, h64, 64, cap - 1, max(3, steps // 2))
    eng.close()
    return out


def time_head_and_dense(pkg, torch, steps: int, device: int = 0):
    """The vocabulary-sized head (mean of the streams, final norm, lm_head 154880 x 4096 BF16, arg-max)
    and one dense MLP (inter 12288, FP8) of the full-size model, one token, L2 flushed."""
    import fullmodel
    L = pkg.lib()
    spec = synth_mod().full_model_spec(1)                         # layer 0: KDA + dense MLP
    eng = fullmodel.build_engine(spec, SEED, 8, device)
    c = spec.cfg
    rng = np.random.default_rng(SEED)
    h = torch.from_numpy(rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((1, c.hidden)).astype(np.float32)).cuda()
    y = torch.empty_like(x)
    out = {}
    for op, src, dst, nbytes in ((b"head", h, h, c.vocab * c.hidden * 2),
                                 (b"mlp", x, y, 3 * c.dense_inter * c.hidden + 3 * (c.dense_inter // 128) * (c.hidden // 128) * 4)):
        each = np.zeros(max(steps, 3), np.float32); tot = C.c_float(0)
        for k in (3, steps):
            assert L.g5b_time_op(eng.handle, op, 0, src.data_ptr(), 1, 0, dst.data_ptr(), k, FLUSH_BYTES,
                                 C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        ms = float(np.mean(each[:steps]))
        out[op.decode()] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_GBps": nbytes / (ms * 1e-3) / 1e9}
    eng.close()
    return out


def time_projection(pkg, torch, name: str, T: int, steps: int, device: int = 0):
    """One matrix of the full-size model times T positions (the path the forward pass takes for that
    many positions: one-token kernels below 8, the tcgen05 kernel from 8 on), L2 flushed before every
    launch. The engine holds layer 0 (KDA + dense MLP) and, for lm_head, the head: a small case for ncu."""
    import synth
    L = pkg.lib()
    spec = synth.full_model_spec(1)
    head = name in ("lm_head.weight", "embed_tokens.weight")
    spec.with_head = head
    eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 16, device)
    eng.set_option("allow_partial", 1)
    synth.fill_full_model(eng, spec, SEED, head=head)
    eng.finalize()
    table = {"layers.0." + n: (r, c, dt) for n, kind, r, c, dt, _ in synth.layer_tensor_table(spec.cfg, False, True) if kind == "mat"}
    table.update({n: (r, c, dt) for n, kind, r, c, dt, _ in synth.model_level_tensors(spec.cfg) if kind == "mat"})
    rows, cols, dt = table[name]
    x = torch.randn(T, cols, device="cuda"); y = torch.empty(T, rows, device="cuda")
    each = np.zeros(max(steps, 3), np.float32)
    for k in (3, steps):
        assert L.g5b_time_matvec(eng.handle, name.encode(), x.data_ptr(), T, y.data_ptr(), k, FLUSH_BYTES,
                                 each.ctypes.data) == 0, L.g5b_last_error()
    ms = float(np.median(each[:steps]))
    nbytes = rows * cols * {synth.DT_F32: 4, synth.DT_BF16: 2, synth.DT_FP8: 1}[dt]
    peak, _ = measured_peaks()
    eng.close()
    return {"matrix": name, "rows": rows, "cols": cols, "positions": T, "ms": ms, "algorithmic_bytes": nbytes,
            "achieved_GBps": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak}


def synth_mod():
    import synth
    return synth


def expert_parallel_parity(pkg, one, ep, ranks, rank: int):
    """The expert-parallel layer against the one-GPU engine of the same rank on the same seeded
    inputs (batch 1 four times, batch 8 once): outputs must be bit-equal, because the contribution
    rows and the top-k-ordered FP64 combine are the same arithmetic wherever the rows were computed.
    Returns the `parity` object; every rank makes the same calls."""
    import synth
    worst, bit_equal, idx_equal = 0.0, True, True
    err = ""
    try:
        for B, seed in ((1, SEED), (1, SEED + 1), (1, SEED + 2), (1, SEED + 3), (8, SEED + 4)):
            x = synth.moe_inputs(one.cfg, B, seed)
            a, b = one.op_moe(0, x), ep.op_moe(0, x)
            ia, _ = one.op_router(0, x)
            ib, _ = ep.op_router(0, x)
            bit_equal = bit_equal and bool(np.array_equal(a, b))
            idx_equal = idx_equal and bool(np.array_equal(ia, ib))
            worst = max(worst, float(np.max(np.abs(a.astype(np.float64) - b)) / (np.max(np.abs(a)) + 1e-300)))
    except Exception as exc:                                       # noqa: BLE001
        err = repr(exc)[:300]
    ok = ranks.all_ok(not err)
    res = {"max_rel_err": ranks.reduce(worst, "max"), "bit_equal": ranks.all_ok(bit_equal),
           "router_idx_equal": ranks.all_ok(idx_equal), "cases": "batch 1 x 4 seeds, batch 8 x 1 seed, against the one-GPU engine on every rank"}
    if not ok:
        res["error"] = err or "another rank failed"
    return res


def time_e2e(L, eng, torch, ranks, steps: int, warmup: int):
    """The layer through the host-buffer C-ABI call: pinned host memory in and out, copies inside the
    timed region, L2 flushed before every step. Returns (seconds of the slowest rank, bytes in, bytes out)."""
    import synth
    xh = torch.from_numpy(synth.moe_inputs(eng.cfg, 1, SEED)).pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    xn, on = xh.numpy(), oh.numpy()
    for _ in range(warmup):
        assert L.g5b_op_moe(eng.handle, 0, xn.ctypes.data, 1, on.ctypes.data, 1) == 0, L.g5b_last_error()
    flush = torch.empty(FLUSH_BYTES // 8, dtype=torch.float32, device="cuda")
    clean = torch.zeros(FLUSH_BYTES // 8, dtype=torch.float32, device="cuda")
    total = 0.0
    ranks.barrier()
    for _ in range(steps):
        flush.zero_()
        clean.sum()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert L.g5b_op_moe(eng.handle, 0, xn.ctypes.data, 1, on.ctypes.data, 1) == 0, L.g5b_last_error()
        total += time.perf_counter() - t0
    return ranks.reduce(total, "max"), int(xn.nbytes), int(on.nbytes)


def run_full_model(pkg, torch, ranks, local: int, rank: int, world: int, peak: float, layers_cap: int,
                   new_tokens: int = 256):
    """Benchmark configuration 4: the full-size random-init model (45 layers, 288 experts per MoE
    layer, vocabulary 154880) resident across the ranks, expert parallel (trunk replicated): prefill
    an 18-token random-id prompt, then decode `new_tokens` tokens greedily at batch 1 without
    returning to the host between steps. With fewer GPUs than the 306 GB need, the first layers that
    fit are run (the reference's --layers cut). Then layers 0, 3 and the last one are compared with
    the CPU path on the GPU's own state (rank 0 checks; every rank makes the same engine calls)."""
    import fullmodel
    import synth
    res, err, eng = {}, "", None
    free = torch.cuda.mem_get_info()[0]
    n_layers = 0
    for n in range(min(45, layers_cap), 0, -1):
        resident, _, _ = fullmodel.model_bytes(synth.full_model_spec(n), world)
        if resident + (6 << 30) <= free * 0.94:
            n_layers = n
            break
    n_layers = int(ranks.reduce(n_layers, "min"))
    if n_layers < 4:
        return {"error": "not enough free device memory for four layers"}
    spec = synth.full_model_spec(n_layers)
    c = spec.cfg
    cap = 18 + new_tokens + 30
    resident, token_rank, token_all = fullmodel.model_bytes(spec, world)
    t0 = time.perf_counter()
    try:
        eng = fullmodel.build_engine(spec, SEED, cap, local, rank, world, options={"latent_bf16": 1})
    except Exception as exc:                                       # noqa: BLE001
        err = repr(exc)[:300]
    build_s = time.perf_counter() - t0
    if not ranks.all_ok(not err):
        if eng is not None:
            eng.close()
        return {"error": err or "another rank could not build the model"}
    handles = ranks.gather(eng.ep_export() if world > 1 else b"")
    toks = None
    try:
        if world > 1:
            eng.ep_connect(handles)
    except Exception as exc:                                       # noqa: BLE001
        err = repr(exc)[:300]
    if not ranks.all_ok(not err):
        eng.close()
        return {"error": err or "another rank could not connect"}
    ids = np.random.default_rng(SEED).integers(0, c.vocab, 18).astype(np.int32)
    prefill_s = decode_s = 0.0
    try:
        # warm-up: the same prefill and a few decode steps, then forget them
        lg, _ = eng.forward(ids)
        eng.decode_greedy(int(np.argmax(lg)), 8)
        eng.reset()
        ranks.barrier()
        t0 = time.perf_counter()
        lg, _ = eng.forward(ids)
        prefill_s = time.perf_counter() - t0
        first = int(np.argmax(lg))
        ranks.barrier()
        t0 = time.perf_counter()
        toks = eng.decode_greedy(first, new_tokens)
        decode_s = time.perf_counter() - t0
    except Exception as exc:                                       # noqa: BLE001
        err = repr(exc)[:300]
    ok = ranks.all_ok(not err)
    decode_s = ranks.reduce(decode_s, "max")
    prefill_s = ranks.reduce(prefill_s, "max")
    all_toks = ranks.gather(None if toks is None else toks.tolist())
    if not ok:
        eng.close()
        return {"error": err or "another rank failed while decoding"}
    ms = 1e3 * decode_s / new_tokens
    res = {"layers": n_layers, "of_layers": 45, "n_gpus": world, "new_tokens": new_tokens, "prompt_tokens": 18,
           "trunk": ("one GPU" if world == 1 else "KDA and MLA layers split by heads over the ranks (partial output rows summed in rank order), "
                     "head split by vocabulary rows for the arg-max, mHC sites and norms replicated"), "experts_per_rank": c.n_experts // world,
           "resident_bytes_per_rank": resident, "build_s": build_s, "prefill_ms": 1e3 * prefill_s,
           "ms_per_token": ms, "tokens_per_s": 1e3 / ms,
           "algorithmic_bytes_per_token": token_all, "bytes_read_per_token_per_rank": token_rank,
           "frac_of_aggregate_roofline": token_all / (ms * 1e-3) / 1e9 / (world * peak),
           "frac_of_one_rank_roofline_for_its_own_reads": token_rank / (ms * 1e-3) / 1e9 / peak,
           "tokens_equal_on_all_ranks": all(t == all_toks[0] for t in all_toks),
           "first_tokens": all_toks[0][:8]}
    # per-layer parity at the position reached (rank 0 holds the CPU side)
    parity, perr = {}, ""
    rng = np.random.default_rng(SEED + 11)
    for layer in sorted({0, 3, n_layers - 1}):
        h = rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32)
        try:
            if rank == 0:
                from oracle import binding
                r = fullmodel.layer_parity(eng, binding, spec, SEED, layer, h, eng.cached, cap, ranks=ranks)
                parity[f"layer{layer}"] = {"rel_err": r["rel_err"], "picks": None if r["picks"] is None else r["picks"].ravel().tolist()}
            else:
                fullmodel.layer_parity(eng, None, spec, SEED, layer, h, eng.cached, cap, check=False, ranks=ranks)
        except Exception as exc:                                   # noqa: BLE001
            perr = repr(exc)[:300]
        if not ranks.all_ok(not perr):
            parity["error"] = perr or "another rank failed"
            break
    res["layer_parity_vs_cpu"] = parity
    eng.close()
    return res


def run_batch_decode(pkg, torch, ranks, local: int, rank: int, world: int, layers_cap: int, sequences: int = 64,
                     context: int = 4096, new_tokens: int = 128, prefill_tokens: int = 2048):
    """Benchmark configuration 5: the full-size random-init model with `sequences` concurrent
    sequences at a context of `context` positions each (their KDA states, latent caches and indexer
    states filled on the device: a stand-in for the prompts' prefill), decoding `new_tokens` tokens
    per sequence in lockstep; routed experts split over the ranks. Two arms at N > 1: every sequence's
    attention on every rank (tokens replicated), and the sequences split over the ranks - each rank
    runs attention and all other per-token work for sequences / N of them, MoE layers gather the
    ranks' tokens and send contribution rows to the rank a token lives on. Both arms start from the
    same synthetic state, so the split arm must reproduce the first arm's tokens. Then one
    `prefill_tokens`-token prompt through the prefill path of sequence 0 (chunks of 64 positions).
    As many layers as the GPUs hold."""
    import fullmodel
    import synth
    c0 = pkg.full_size_config()
    cap = context + new_tokens + 8
    # session state per sequence and layer (FP32 KDA state and indexer state, BF16 latents)
    P = c0.kda_heads * c0.kda_head_dim
    kda_bytes = 4 * (P * c0.kda_head_dim + 3 * P * (c0.conv_k - 1))
    mla_bytes = cap * c0.kv_lora * 2 + 4 * (2 * cap * c0.index_dim + ((cap + c0.index_kpool - 1) // c0.index_kpool) * c0.index_dim)
    free = torch.cuda.mem_get_info()[0]
    n_layers = 0
    for n in range(min(45, layers_cap), 0, -1):
        spec = synth.full_model_spec(n)
        resident, _, _ = fullmodel.model_bytes(spec, world)
        state = sequences * sum(mla_bytes if m else kda_bytes for m in spec.is_mla)
        if resident + state + (8 << 30) <= free * 0.94:
            n_layers = n
            break
    n_layers = int(ranks.reduce(n_layers, "min"))
    if n_layers < 4:
        return {"error": "not enough free device memory for four layers"}
    spec = synth.full_model_spec(n_layers)
    c = spec.cfg
    all_ids = np.random.default_rng(SEED).integers(0, c.vocab, sequences).astype(np.int32)
    steps = new_tokens - 3

    def arm(split: bool, with_prefill: bool):
        own = sequences // world if split else sequences
        eng, err = None, ""
        opts = {"latent_bf16": 1, "sequences": own}
        if split:
            opts["sequence_split"] = 1
        try:
            eng = fullmodel.build_engine(spec, SEED, cap, local, rank, world, options=opts)
        except Exception as exc:                                       # noqa: BLE001
            err = repr(exc)[:300]
        if not ranks.all_ok(not err):
            if eng is not None:
                eng.close()
            return {"error": err or "another rank could not build the model"}, None, None
        handles = ranks.gather(eng.ep_export() if world > 1 else b"")
        try:
            if world > 1:
                eng.ep_connect(handles)
        except Exception as exc:                                       # noqa: BLE001
            err = repr(exc)[:300]
        if not ranks.all_ok(not err):
            eng.close()
            return {"error": err or "another rank could not connect"}, None, None
        decode_s = prefill_s = 0.0
        toks = early = None
        try:
            eng.synth_session(SEED, context)
            ids = all_ids[rank * own:(rank + 1) * own] if split else all_ids
            for _ in range(3):                                         # warm-up steps (they advance the sequences too)
                _, ids = eng.decode_batch(ids, want_logits=False)
            early = ids.tolist()
            ranks.barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                _, ids = eng.decode_batch(ids, want_logits=False)
            decode_s = time.perf_counter() - t0
            toks = ids.tolist()
            if with_prefill:
                # prefill throughput: one prompt through sequence 0 from an empty session
                eng.reset()
                prompt = np.random.default_rng(SEED + 1).integers(0, c.vocab, prefill_tokens).astype(np.int32)
                eng.use_sequence(0)
                eng.forward(prompt[:128], want_logits=False)           # warm-up chunk pair
                eng.reset()
                eng.use_sequence(0)
                ranks.barrier()
                t0 = time.perf_counter()
                eng.forward(prompt, want_logits=False)
                prefill_s = time.perf_counter() - t0
        except Exception as exc:                                       # noqa: BLE001
            err = repr(exc)[:300]
        ok = ranks.all_ok(not err)
        decode_s = ranks.reduce(decode_s, "max")
        prefill_s = ranks.reduce(prefill_s, "max")
        all_toks = ranks.gather(toks)
        all_early = ranks.gather(early)
        eng.close()
        if not ok:
            return {"error": err or "another rank failed"}, None, None
        res = {"sequences_per_rank": own, "timed_steps": steps, "ms_per_step": 1e3 * decode_s / steps,
               "tokens_per_s": sequences * steps / decode_s, "tokens_per_s_per_sequence": steps / decode_s}
        if with_prefill:
            res["prefill"] = {"tokens": prefill_tokens, "ms": 1e3 * prefill_s, "tokens_per_s": prefill_tokens / prefill_s, "chunk": 64}
        return res, all_toks, all_early

    out = {"layers": n_layers, "of_layers": 45, "n_gpus": world, "sequences": sequences, "context": context,
           "state": "synthetic session state at the stated context (filled on the device), no prompts run"}
    rep, rep_toks, rep_early = arm(False, True)
    if "error" in rep:
        return rep
    out.update(rep)
    out["attention"] = "every sequence on every rank (no sequence parallelism); routed experts split over the ranks"
    out["tokens_equal_on_all_ranks"] = all(t == rep_toks[0] for t in rep_toks)
    if world > 1 and sequences % world == 0:
        sp, sp_toks, sp_early = arm(True, False)
        if "error" not in sp:
            sp["attention"] = ("sequences split over the ranks: attention and every per-token kernel for sequences / N per rank; MoE "
                               "layers gather the ranks' tokens over peer stores (dispatch) and send contribution rows to the token's rank (combine)")
            flat = [t for ts in sp_toks for t in ts]
            # (the unsplit arm sums the KDA output projection over the ranks, this arm does not: a last-bit
            # difference can flip an arg-max of a random-init model's near-uniform logits after many steps)
            sp["sequences_with_the_unsplit_arm_s_token_after_3_steps"] = int(sum(
                a == b for a, b in zip([t for ts in sp_early for t in ts], rep_early[0])))
            sp["sequences_with_the_unsplit_arm_s_token_after_%d_steps" % new_tokens] = int(sum(a == b for a, b in zip(flat, rep_toks[0])))
        out["sequence_split"] = sp
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--experts", type=int, default=288,
                    help="routed experts resident in the layer (288 = the stated config; fewer only to keep "
                         "an ncu capture small: the batch-1 kernels touch 8 routed + 1 shared either way)")
    ap.add_argument("--batches", default="8,64", help="extra batch sizes reported under 'extra'")
    ap.add_argument("--no-expert-parallel", action="store_true",
                    help="N > 1: run N independent replicas only (no expert-parallel engine)")
    ap.add_argument("--only-attention-layers", action="store_true",
                    help="run only the KDA / MLA single-layer timings and print them (a small case for ncu)")
    ap.add_argument("--no-decoder-layers", action="store_true",
                    help="with --only-attention-layers: skip the two whole decoder layers (15 GB of experts), "
                         "which keeps an ncu capture of the KDA / MLA kernels small")
    ap.add_argument("--only-mhc-site", action="store_true",
                    help="run only the timing of one mHC site of a full-size layer and print it (a small case for ncu)")
    ap.add_argument("--no-attention-layers", action="store_true",
                    help="skip the KDA / MLA single-layer and decoder-layer timings reported under 'extra'")
    ap.add_argument("--only-projection", default="",
                    help="time one matrix of the full-size model (e.g. layers.0.mlp.gate_proj.weight, lm_head.weight) "
                         "times --positions positions and print it (a small case for ncu)")
    ap.add_argument("--positions", type=int, default=64)
    ap.add_argument("--mma-rate", action="store_true",
                    help="print the cycles per tcgen05.mma instruction (M = 128) for N = 16..256, both kinds, and exit")
    ap.add_argument("--no-full-model", action="store_true", help="skip the full-size model's greedy decode")
    ap.add_argument("--no-batch-decode", action="store_true", help="skip the 64-sequence decode of the full-size model")
    ap.add_argument("--only-full-model", action="store_true", help="run only the full-size model's greedy decode and print it")
    ap.add_argument("--full-model-layers", type=int, default=45, help="upper limit on the layers of the full-size model")
    ap.add_argument("--full-model-tokens", type=int, default=256)
    ap.add_argument("--expert-path", type=int, default=-1,
                    help="batch-1 expert kernels: 0 register-streaming, 1 tensor-core kernels as three launches, 2 whole layer in one kernel (default)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import synth
    from __graft_entry__ import load_package
    pkg = load_package()
    L = pkg.lib()                                   # raises when the CUDA library is missing
    if not torch.cuda.is_available() or L.g5b_device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)

    if args.mma_rate:
        # cycles per tcgen05.mma instruction, one issuing thread per SM, operands that never change
        import ctypes as C
        L.g5b_debug_mma_rate.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double)]
        sms = torch.cuda.get_device_properties(local).multi_processor_count
        rows = []
        for fp8 in (0, 1):
            for n in (16, 32, 64, 128, 192, 256):
                cyc = (C.c_double * 2)()
                if L.g5b_debug_mma_rate(n, fp8, 1, sms, 2000, cyc) != 0:
                    raise SystemExit("the instruction-rate probe failed")
                rows.append({"kind": "f8f6f4, K = 32" if fp8 else "f16, K = 16", "M": 128, "N": n,
                             "cycles_per_instruction_issued": cyc[0], "cycles_per_instruction_complete": cyc[1]})
        print(json.dumps({"tcgen05_mma_rate": rows, "ctas": sms, "instructions_per_cta": 8000}))
        return

    # the CPU baseline first: one rank, before any other rank's process competes for the host cores
    cpu = None
    if world == 1 and not args.no_cpu_baseline and args.experts == 288 and not (
            args.only_mhc_site or args.only_attention_layers or args.only_full_model or args.only_projection):
        cpu = cpu_reference_moe(steps=60, warmup=2)
        one = cpu_reference_moe(steps=30, warmup=1, threads=1)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        cpu["one_thread_value"] = one["value"]

    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import importlib
    ranks = importlib.import_module("glm53f_b200.ranks").Ranks(dist if world > 1 else None, "cuda")
    peak, peak_kind = measured_peaks()
    warmup = max(3, args.warmup)

    if args.only_projection:
        print(json.dumps({"projection": time_projection(pkg, torch, args.only_projection, args.positions, max(3, args.steps), local)}),
              flush=True)
        return
    if args.only_mhc_site:
        print(json.dumps({"mhc_site": time_mhc_site(pkg, torch, max(3, args.steps), local)}), flush=True)
        return
    if args.only_attention_layers:
        res = {"config3": time_attention_layers(pkg, torch, max(3, args.steps), peak, local)}
        if not args.no_decoder_layers:
            res["decoder_layers"] = time_decoder_layers(pkg, torch, max(3, args.steps), local)
        print(json.dumps(res), flush=True)
        return
    if args.only_full_model:
        res = {"full_model": run_full_model(pkg, torch, ranks, local, rank, world, peak, args.full_model_layers, args.full_model_tokens)}
        if not args.no_batch_decode:
            res["batch_decode"] = run_batch_decode(pkg, torch, ranks, local, rank, world, args.full_model_layers)
        if rank == 0:
            print(json.dumps(res), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    opts = {}
    if args.expert_path >= 0:
        opts["expert_path"] = args.expert_path
    # every rank holds a whole copy of the layer (the one-GPU engine): the headline at N = 1, the
    # reference for the expert-parallel parity check and the replica figure at N > 1
    spec, trunk, one_eng = synth.build_moe_layer_engine(SEED, n_experts=args.experts, device=local, options=opts)
    use_ep = world > 1 and args.experts % world == 0 and not args.no_expert_parallel
    extra = {}
    ep_eng, ep_err = None, ""
    if use_ep:
        try:
            ep_eng = pkg.Engine(spec.cfg, spec.is_mla, spec.is_dense, 8, local, rank, world)
            ep_eng.set_option("allow_partial", 1)
            for k, v in opts.items():
                ep_eng.set_option(k, v)
            ep_eng.load_all(trunk)
            for ex in range(args.experts):
                ep_eng.fill_expert(0, ex, SEED, *synth.expert_scales(spec.cfg, 0, ex, SEED))
            ep_eng.finalize()
        except Exception as exc:                               # noqa: BLE001
            ep_err = repr(exc)[:300]
        handles = ranks.gather(ep_eng.ep_export() if not ep_err else b"")
        if not ep_err:
            try:
                ep_eng.ep_connect(handles)
            except Exception as exc:                           # noqa: BLE001
                ep_err = repr(exc)[:300]
        if not ranks.all_ok(not ep_err):
            raise SystemExit(f"expert-parallel engine could not be set up: {ep_err or 'another rank failed'}")
        extra["expert_parallel"] = {"ranks": world, "routed_experts_per_rank": args.experts // world,
                                    "parity": expert_parallel_parity(pkg, one_eng, ep_eng, ranks, rank)}
    eng = ep_eng if use_ep else one_eng
    sampler = ClockSampler(local)

    # ---- headline: batch 1, device resident
    sampler.start()
    sampler.wait_first()
    ranks.barrier()
    HEADLINE_INPUTS = 16          # different tokens, i.e. different routings, share the timed steps
    each, phases, launches, _, per_input = time_batch(pkg, eng, torch, 1, args.steps, warmup, phases=not use_ep,
                                                      inputs=HEADLINE_INPUTS)
    ranks.barrier()
    if use_ep:
        # how the eight picks of each of those tokens fall on the ranks: a step takes what the busiest rank takes
        per = args.experts // world
        busiest = []
        for k in range(len(per_input)):
            idx, _ = one_eng.op_router(0, synth.moe_inputs(spec.cfg, 1, SEED + 1000 * k))
            busiest.append(int(np.bincount(idx.ravel() // per, minlength=world).max()))
        slowest = ranks.gather(per_input)
        extra["expert_parallel"]["tokens_timed"] = len(per_input)
        extra["expert_parallel"]["picks_on_the_busiest_rank_per_token"] = busiest
        extra["expert_parallel"]["ms_per_token_slowest_rank"] = [float(max(r[k] for r in slowest)) for k in range(len(per_input))]
    local_ms_per_step = float(each.sum()) / args.steps
    ms_per_step = ranks.reduce(local_ms_per_step, "max")        # the slowest rank's
    # expert parallel: all ranks serve the same token; replicas only when asked for: one stream per rank
    streams = 1 if (use_ep or world == 1) else world
    value = streams * 1e3 / ms_per_step

    # ---- end to end: host buffers (pinned) through the C-ABI op, H2D and D2H inside the timing
    e2e_s, h2d, d2h = time_e2e(L, eng, torch, ranks, args.steps, warmup)
    clocks = sampler.stop()       # sampled over the device-timed and the end-to-end regions
    e2e = {"value": streams * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s / args.steps}

    # ---- roofline of the dominant kernel
    router_bytes = args.experts * 4096 * 2
    layer_bytes = 9 * EXPERT_BYTES + router_bytes
    one_launch = launches == args.steps
    if use_ep:
        # every rank reads the router matrix and the shared expert, and the routed picks it owns
        all_bytes = world * (EXPERT_BYTES + router_bytes) + 8 * EXPERT_BYTES
        roofline = {"bound": "hbm", "kernel": "moe_decode_kernel, expert parallel (router + top-8 + own picks + shared expert + "
                                              "row exchange over peer mappings + combine, batch 1)",
                    "achieved": all_bytes / (ms_per_step * 1e-3) / 1e9, "peak": world * peak,
                    "peak_kind": f"{world} x the {peak_kind} copy bandwidth", "unit": "GB/s",
                    "frac": all_bytes / (ms_per_step * 1e-3) / 1e9 / (world * peak), "traffic": None,
                    "algorithmic_bytes_per_launch": all_bytes, "ms_per_launch": ms_per_step,
                    "note": "bytes all ranks read per step (each rank: router + shared expert; the 8 picks once), "
                            "against the ranks' combined bandwidth"}
    else:
        layer = {"algorithmic_bytes_per_step": layer_bytes, "achieved": layer_bytes / (local_ms_per_step * 1e-3) / 1e9,
                 "frac": layer_bytes / (local_ms_per_step * 1e-3) / 1e9 / peak}
        if one_launch:
            roofline = {"bound": "hbm", "kernel": "moe_decode_kernel (router + top-8 + 8 routed and 1 shared expert + combine, batch 1)",
                        "achieved": layer["achieved"], "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                        "frac": layer["frac"], "traffic": DECODE_TRAFFIC_NCU, "algorithmic_bytes_per_launch": layer_bytes,
                        "ms_per_launch": local_ms_per_step, "layer": layer}
        else:
            gateup_ms = phases[1]
            achieved = 9 * GATEUP_BYTES / (gateup_ms * 1e-3) / 1e9 if gateup_ms > 0 else 0.0
            roofline = {"bound": "hbm", "kernel": "gate/up + SwiGLU kernel of the chosen expert path (8 routed + 1 shared expert, batch 1)",
                        "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                        "frac": achieved / peak, "traffic": GATEUP_TRAFFIC_NCU,
                        "algorithmic_bytes_per_launch": 9 * GATEUP_BYTES, "ms_per_launch": gateup_ms, "layer": layer}

    if not use_ep:
        extra["phase_ms_b1"] = ({"moe_decode_kernel": phases[0]} if one_launch else
                                {"router+plan": phases[0], "gate_up": phases[1], "down": phases[2], "combine": phases[3]})
    if use_ep:
        # N independent replicas of the layer, one token stream each (no data-path collective)
        ranks.barrier()
        r_each, _, _, _, _ = time_batch(pkg, one_eng, torch, 1, args.steps, warmup, phases=False)
        r_ms = ranks.reduce(float(r_each.sum()) / args.steps, "max")
        extra["replicas"] = {"ranks": world, "tokens_per_s": world * 1e3 / r_ms, "ms_per_step": r_ms,
                             "note": "one whole copy of the layer and one token stream per rank"}
        ep_eng.close()
    if rank == 0 and world == 1:
        for B in [int(b) for b in args.batches.split(",") if b]:
            eb, ph, _, _, _ = time_batch(pkg, one_eng, torch, B, max(10, args.steps // 10), 3)
            idx, _ = one_eng.op_router(0, synth.moe_inputs(spec.cfg, B, SEED))
            distinct = int(len(set(idx.ravel().tolist())))
            ms = float(eb.mean())
            extra[f"batch{B}"] = {"tokens_per_s": B * 1e3 / ms, "ms_per_step": ms, "distinct_experts": distinct,
                                  "achieved_GBps": ((distinct + 1) * EXPERT_BYTES + ROUTER_BYTES) / (ms * 1e-3) / 1e9,
                                  "phase_ms": ph}
    one_eng.close()
    if world == 1 and not args.no_attention_layers and args.experts == 288:
        n = max(10, args.steps // 10)
        extra["config3"] = time_attention_layers(pkg, torch, n, peak, local)
        extra["decoder_layers"] = time_decoder_layers(pkg, torch, n, local)
        extra["head_and_dense_mlp"] = time_head_and_dense(pkg, torch, n, local)
        extra["mhc_site"] = time_mhc_site(pkg, torch, n, local)
        if not use_ep and one_launch:
            # the same kernel inside a whole decoder layer (after other kernels, cold instruction cache)
            kda_layer_bytes = 286048984 + layer_bytes + 2 * 786432
            ms = extra["decoder_layers"]["kda_moe_layer"]["ms"]
            roofline["in_layer"] = {"what": "whole KDA + MoE decoder layer, one token: weights + state read and written",
                                    "ms": ms, "algorithmic_bytes": kda_layer_bytes,
                                    "frac": kda_layer_bytes / (ms * 1e-3) / 1e9 / peak}

    # ---- the full-size model, as many layers as the GPUs hold (all 45 from four GPUs on)
    if not args.no_full_model and args.experts == 288:
        try:
            extra["full_model"] = run_full_model(pkg, torch, ranks, local, rank, world, peak, args.full_model_layers,
                                                 args.full_model_tokens)
        except Exception as exc:                                   # noqa: BLE001
            extra["full_model"] = {"error": repr(exc)[:300]}

    if not args.no_full_model and not args.no_batch_decode and args.experts == 288:
        try:
            extra["batch_decode"] = run_batch_decode(pkg, torch, ranks, local, rank, world, args.full_model_layers)
        except Exception as exc:                                   # noqa: BLE001
            extra["batch_decode"] = {"error": repr(exc)[:300]}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong" if (use_ep or world == 1) else "weak", "vs_baseline": None,
                "dtype": DTYPE, "data": "synthetic", "config": bench_config(world) if (use_ep or world == 1) else
                dict(bench_config(1), parallelism=f"{world} independent replicas, one token stream each"),
                "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
                "extra": extra}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
