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
                  "read so that no dirty line is left); CPU arm: 4 rotating inputs, 226 MB of weights per step",
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


def time_batch(pkg, eng, torch, B, steps, warmup, flush=FLUSH_BYTES, phases=True):
    """Device-resident timing of the MoE layer at batch B: (ms per step list, phase ms, launches)."""
    import synth
    L = pkg.lib()
    x = torch.from_numpy(synth.moe_inputs(eng.cfg, B, SEED)).cuda()
    out = torch.empty_like(x)
    torch.cuda.synchronize()
    each = np.zeros(max(steps, warmup, 1), np.float32)
    tot = C.c_float(0)
    assert L.g5b_time_op(eng.handle, b"moe", 0, x.data_ptr(), B, 0, out.data_ptr(), warmup, flush,
                         C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
    ms4 = (C.c_float * 8)()
    cnt = C.c_long(0)
    n0 = L.g5b_launch_count()
    assert L.g5b_time_op(eng.handle, b"moe", 0, x.data_ptr(), B, 0, out.data_ptr(), steps, flush,
                         C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
    launches = L.g5b_launch_count() - n0 - (2 * steps if flush else 0)
    timed = each[:steps].astype(float)
    if not phases:
        return timed, [0.0] * 4, int(launches), out
    # per-phase times in a separate short pass: the phase events make the host wait inside every
    # step, which would inflate the step time measured above
    eng.set_option("profile", 1)
    L.g5b_engine_profile_read(eng.handle, ms4, 8, C.byref(cnt), 1)
    scratch = np.zeros(32, np.float32)
    assert L.g5b_time_op(eng.handle, b"moe", 0, x.data_ptr(), B, 0, out.data_ptr(), min(20, max(3, steps)), flush,
                         C.byref(tot), scratch.ctypes.data) == 0, L.g5b_last_error()
    L.g5b_engine_profile_read(eng.handle, ms4, 8, C.byref(cnt), 1)
    eng.set_option("profile", 0)
    phases = [ms4[i] / max(1, cnt.value) for i in range(4)]
    return timed, phases, int(launches), out


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
            assert L.g5b_time_op(eng.handle, op, 0, xd.data_ptr(), 1, cached, od.data_ptr(), k, FLUSH_BYTES,
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
    """Two whole full-size decoder layers, one new token: layer 0 = KDA + MoE, layer 1 = MLA (8192
    cached positions, indexer selecting) + MoE, each with its two mHC sites and norms. From the two
    times the full model's batch-1 token time on ONE GPU's worth of bandwidth is extrapolated
    (34 KDA layers + 11 MLA layers + the 1.27 GB head at the KDA layer's measured GB/s) - the
    306 GB model itself needs 8 GPUs."""
    import synth
    L = pkg.lib()
    c = pkg.full_size_config()
    c.n_layers = 2
    spec = synth.Spec(c, [0, 1], [0, 0], with_head=False)
    tensors = synth.make_model(spec, seed=6, recipe="baseline", experts=False)
    cap = 8192
    eng = pkg.Engine(c, spec.is_mla, spec.is_dense, cap, device)
    eng.set_option("allow_partial", 1)
    eng.set_option("latent_bf16", 1)
    eng.set_option("sequences", 64)
    eng.load_all(tensors)
    for layer in range(2):
        for ex in range(c.n_experts):
            eng.fill_expert(layer, ex, SEED, *synth.expert_scales(c, layer, ex, SEED))
    eng.finalize()
    rng = np.random.default_rng(SEED)
    h = torch.from_numpy(rng.standard_normal((1, c.hc_mult, c.hidden)).astype(np.float32)).cuda()
    out = {}
    for layer, cached, name in ((0, 0, "kda_moe_layer"), (1, cap - 1, "mla_moe_layer_ctx8192")):
        hd = h.clone()
        each = np.zeros(max(steps, 3), np.float32); tot = C.c_float(0)
        for k in (3, steps):
            hd.copy_(h)
            assert L.g5b_time_op(eng.handle, b"layer", layer, hd.data_ptr(), 1, cached, hd.data_ptr(), k, FLUSH_BYTES,
                                 C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        out[name] = {"ms": float(np.mean(each[:steps])), "finite": bool(torch.isfinite(hd).all().item())}
    # both layers in one pass (the second layer's first mHC site applies the first layer's pending
    # stream expansion inside its own launch, as in the whole model)
    hd = h.clone()
    each = np.zeros(max(steps, 3), np.float32); tot = C.c_float(0)
    for k in (3, steps):
        hd.copy_(h)
        assert L.g5b_time_op(eng.handle, b"layers", 0, hd.data_ptr(), 1, cap - 1, hd.data_ptr(), k, FLUSH_BYTES,
                             C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
    out["kda_moe_then_mla_moe_layers"] = {"ms": float(np.mean(each[:steps])), "finite": bool(torch.isfinite(hd).all().item())}
    # the same two layers advancing 64 sequences by one token each (state and caches per sequence,
    # weights read once per batch)
    h64 = torch.from_numpy(rng.standard_normal((64, c.hc_mult, c.hidden)).astype(np.float32)).cuda()
    for layer, cached, name in ((0, 0, "kda_moe_layer_batch64"), (1, cap - 1, "mla_moe_layer_ctx8192_batch64")):
        hd = h64.clone()
        n = max(3, steps // 2)
        each = np.zeros(max(n, 3), np.float32); tot = C.c_float(0)
        for k in (2, n):
            hd.copy_(h64)
            assert L.g5b_time_op(eng.handle, b"layer_batch", layer, hd.data_ptr(), 64, cached, hd.data_ptr(), k, FLUSH_BYTES,
                                 C.byref(tot), each.ctypes.data) == 0, L.g5b_last_error()
        out[name] = {"ms": float(np.mean(each[:n])), "finite": bool(torch.isfinite(hd).all().item())}
    eng.close()
    b64_ms = 34 * out["kda_moe_layer_batch64"]["ms"] + 11 * out["mla_moe_layer_ctx8192_batch64"]["ms"]
    out["full_model_batch64_tokens_per_s_extrapolated"] = 64e3 / b64_ms
    kda_bytes = 286048984 + 228907008 + 2 * 786432
    rate = kda_bytes / (out["kda_moe_layer"]["ms"] * 1e-3)
    head_ms = 154880 * 4096 * 2 / rate * 1e3
    token_ms = 34 * out["kda_moe_layer"]["ms"] + 11 * out["mla_moe_layer_ctx8192"]["ms"] + head_ms
    out["full_model_token_ms_extrapolated"] = token_ms
    out["full_model_tokens_per_s_extrapolated"] = 1e3 / token_ms
    out["note"] = ("extrapolated: 34 x KDA+MoE layer + 11 x MLA+MoE layer + lm_head at the KDA+MoE layer's measured "
                   "rate; the three dense-MLP layers counted as MoE layers; one GPU's bandwidth, weights of 8 GPUs")
    return out


def time_expert_parallel(pkg, torch, dist, synth, rep, args, local, rank, world, warmup):
    """N > 1: the same layer expert-parallel (288 / N routed experts per rank, activations and the
    shared expert replicated, contribution rows exchanged over peer mappings inside the decode
    kernel): one token stream served by all ranks together, i.e. the latency side of the N-GPU
    trade-off. Returns the entry for `extra`. Every rank takes part in every collective here
    whatever happens on it, and the ranks agree on each stage's outcome before the next."""
    def all_ok(flag: bool) -> bool:
        t = torch.tensor([1.0 if flag else 0.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item() > 0.5)

    ep, err, handle = None, "", b""
    try:
        spec_ep = synth.layer_spec("moe", n_experts=args.experts)
        trunk_ep = synth.moe_layer_trunk(spec_ep, SEED)
        ep = pkg.Engine(spec_ep.cfg, spec_ep.is_mla, spec_ep.is_dense, 8, local, rank, world)
        ep.set_option("allow_partial", 1)
        ep.load_all(trunk_ep)
        for ex in range(args.experts):
            ep.fill_expert(0, ex, SEED, *synth.expert_scales(spec_ep.cfg, 0, ex, SEED))
        ep.finalize()
        handle = ep.ep_export()
    except Exception as exc:                                   # noqa: BLE001
        err = repr(exc)[:300]
    handles = [None] * world
    dist.all_gather_object(handles, handle)
    if not err:
        try:
            ep.ep_connect(handles)
        except Exception as exc:                               # noqa: BLE001
            err = repr(exc)[:300]
    ep_ms = 0.0
    if all_ok(not err):
        try:
            ep_each, _, _, _ = time_batch(pkg, ep, torch, 1, args.steps, warmup, phases=False)
            ep_ms = float(ep_each.mean())
        except Exception as exc:                               # noqa: BLE001
            err = repr(exc)[:300]
    ok = all_ok(not err)
    ep_ms = rep.max_over_ranks(ep_ms, dist, "cuda")
    if ep is not None:
        ep.close()
    if not ok or ep_ms <= 0:
        return {"ranks": world, "error": err or "another rank failed"}
    return {"ranks": world, "ms_per_step": ep_ms, "tokens_per_s": 1e3 / ep_ms,
            "routed_experts_per_rank": args.experts // world}


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
                    help="N > 1: skip the expert-parallel timing of the layer reported under 'extra'")
    ap.add_argument("--only-attention-layers", action="store_true",
                    help="run only the KDA / MLA single-layer timings and print them (a small case for ncu)")
    ap.add_argument("--no-decoder-layers", action="store_true",
                    help="with --only-attention-layers: skip the two whole decoder layers (15 GB of experts), "
                         "which keeps an ncu capture of the KDA / MLA kernels small")
    ap.add_argument("--only-mhc-site", action="store_true",
                    help="run only the timing of one mHC site of a full-size layer and print it (a small case for ncu)")
    ap.add_argument("--no-attention-layers", action="store_true",
                    help="skip the KDA / MLA single-layer timings reported under 'extra'")
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
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    warmup = max(3, args.warmup)
    if args.only_mhc_site:
        print(json.dumps({"mhc_site": time_mhc_site(pkg, torch, max(3, args.steps), local)}), flush=True)
        return
    if args.only_attention_layers:
        peak, _ = measured_peaks()
        res = {"config3": time_attention_layers(pkg, torch, max(3, args.steps), peak, local)}
        if not args.no_decoder_layers:
            res["decoder_layers"] = time_decoder_layers(pkg, torch, max(3, args.steps), local)
        print(json.dumps(res), flush=True)
        return
    opts = {}
    if args.expert_path >= 0:
        opts["expert_path"] = args.expert_path
    spec, trunk, eng = synth.build_moe_layer_engine(SEED, n_experts=args.experts, device=local, options=opts)
    sampler = ClockSampler(local)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- headline: batch 1, device resident
    sampler.start()
    sampler.wait_first()
    barrier()
    each, phases, launches, _ = time_batch(pkg, eng, torch, 1, args.steps, warmup)
    barrier()
    import importlib
    rep = importlib.import_module("glm53f_b200.replicas")
    local_ms_per_step = float(each.sum()) / args.steps
    job = rep.whole_job_rate(units_local=args.steps, seconds_local=float(each.sum()) * 1e-3,
                             dist=dist if world > 1 else None, device="cuda")
    ms_per_step = job["seconds"] * 1e3 / args.steps          # the slowest rank's
    value = job["rate"]                                      # tokens of all ranks / slowest rank's time

    # ---- end to end: host buffers (pinned) through the C-ABI op, H2D and D2H inside the timing
    xh = torch.from_numpy(synth.moe_inputs(spec.cfg, 1, SEED)).pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    xn, on = xh.numpy(), oh.numpy()
    for _ in range(warmup):
        assert L.g5b_op_moe(eng.handle, 0, xn.ctypes.data, 1, on.ctypes.data, 1) == 0
    flush = torch.empty(FLUSH_BYTES // 8, dtype=torch.float32, device="cuda")
    clean = torch.zeros(FLUSH_BYTES // 8, dtype=torch.float32, device="cuda")
    e2e_s = 0.0
    barrier()
    for _ in range(args.steps):
        flush.zero_()
        clean.sum()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert L.g5b_op_moe(eng.handle, 0, xn.ctypes.data, 1, on.ctypes.data, 1) == 0
        e2e_s += time.perf_counter() - t0
    e2e_job = rep.whole_job_rate(units_local=args.steps, seconds_local=e2e_s, dist=dist if world > 1 else None,
                                 device="cuda")
    e2e_s = e2e_job["seconds"]
    clocks = sampler.stop()       # sampled over the device-timed and the end-to-end regions
    e2e = {"value": e2e_job["rate"], "unit": "tokens/s", "h2d_bytes_per_step": int(xn.nbytes),
           "d2h_bytes_per_step": int(on.nbytes), "ms_per_step": 1e3 * e2e_s / args.steps}

    # ---- roofline of the dominant kernel
    router_bytes = args.experts * 4096 * 2
    layer_bytes = 9 * EXPERT_BYTES + router_bytes
    peak, peak_kind = measured_peaks()
    layer = {"algorithmic_bytes_per_step": layer_bytes, "achieved": layer_bytes / (local_ms_per_step * 1e-3) / 1e9,
             "frac": layer_bytes / (local_ms_per_step * 1e-3) / 1e9 / peak}
    if launches == args.steps:
        # one launch per step: the whole layer (router matrix, 8 routed + 1 shared expert) in one kernel
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

    if launches == args.steps:
        extra = {"phase_ms_b1": {"moe_decode_kernel": phases[0]}}
    else:
        extra = {"phase_ms_b1": {"router+plan": phases[0], "gate_up": phases[1], "down": phases[2], "combine": phases[3]}}
    if rank == 0:
        for B in [int(b) for b in args.batches.split(",") if b]:
            eb, ph, _, _ = time_batch(pkg, eng, torch, B, max(10, args.steps // 10), 3)
            idx, _ = eng.op_router(0, synth.moe_inputs(spec.cfg, B, SEED))
            distinct = int(len(set(idx.ravel().tolist())))
            ms = float(eb.mean())
            extra[f"batch{B}"] = {"tokens_per_s": B * 1e3 / ms, "ms_per_step": ms, "distinct_experts": distinct,
                                  "achieved_GBps": ((distinct + 1) * EXPERT_BYTES + ROUTER_BYTES) / (ms * 1e-3) / 1e9,
                                  "phase_ms": ph}
    eng.close()
    if rank == 0 and not args.no_attention_layers and args.experts == 288:
        extra["config3"] = time_attention_layers(pkg, torch, max(10, args.steps // 10), peak, local)
        extra["decoder_layers"] = time_decoder_layers(pkg, torch, max(10, args.steps // 10), local)
        extra["mhc_site"] = time_mhc_site(pkg, torch, max(10, args.steps // 10), local)

    # ---- N > 1: the same layer expert-parallel (288 / N routed experts per rank, activations and the
    # shared expert replicated, contribution rows exchanged over peer mappings): one token stream
    # served by all ranks together, i.e. the latency side of the N-GPU trade-off
    if world > 1 and 288 % world == 0 and not args.no_expert_parallel:
        # the headline above does not depend on this extra: a failure here is reported, not fatal
        try:
            extra["expert_parallel_b1"] = time_expert_parallel(pkg, torch, dist, synth, rep, args, local, rank, world,
                                                               warmup)
        except Exception as exc:                               # noqa: BLE001
            extra["expert_parallel_b1"] = {"ranks": world, "error": repr(exc)[:300]}

    cpu = None
    if rank == 0 and not args.no_cpu_baseline and args.experts == 288:
        cpu = cpu_reference_moe(steps=60, warmup=2)
        one = cpu_reference_moe(steps=30, warmup=1, threads=1)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        cpu["one_thread_value"] = one["value"]

    if rank == 0:
        line = {"metric": "decode tokens/s through one full-size MoE layer, batch 1", "value": value, "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "fp8_e4m3 weights, f32 activations and accumulation", "data": "synthetic",
                "config": {"workload": "config 2: single MoE layer decode, hidden 4096, inter 2048, 288+1 experts, "
                                       "top-8, batch 1", "l2": f"flushed before every step ({FLUSH_BYTES >> 21} MiB written, then {FLUSH_BYTES >> 21} MiB read so that no dirty line is left)",
                           "parallelism": f"{world} independent replica(s), one token stream each"},
                "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
                "extra": extra}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
