// moe.cu - sigmoid router with correction bias and top-k, and the routed + shared experts.
//
// Reference: glm53f_router (src/core/glm53f_ops.c:945-976) and moe_chunk (:1144-1342). The
// reference never ran these on a GPU: routed experts stayed on the CPU behind an SSD cache
// (src/gpu/glm53f_gpu.c:1024-1040). Here every expert is HBM resident and a MoE layer is
//   router_scores -> router_topk -> (moe_plan when T > 1) -> gate/up + clamped SwiGLU -> down
//   -> combine,
// with no host involvement: the expert ids stay on the device and the expert kernels index the
// weight table with them.
//
// Expert-major like the reference: each distinct expert's weights are streamed once for all
// (token, slot) pairs that chose it, every pair keeps its own output row, and the rows are
// summed per token in top-k order in FP64 (:1329-1337), the shared expert added last in FP32.
#include "dot_rows.cuh"
#include "kernels.h"

namespace g5b {

constexpr int MOE_THREADS = 256;
constexpr int MOE_WARPS = MOE_THREADS / 32;

// ------------------------------------------------------------------ router ----
// One launch routes a chunk of tokens: every warp takes the FP64 dot product of one router row
// with one token (16-byte loads of the BF16 or FP32 row), writes sigmoid((float) sum), and the
// CTA that finishes last (a counter in device memory, no spinning) selects the top-k of every
// token and groups the (token, slot) pairs by expert for the expert kernels.
//
// Selection: top-k of (score + bias) by repeated arg-max with strict '>' so that the lowest
// index wins ties; weights from the unbiased scores, normalised in FP64, times the routed scale
// (reference glm53f_router, src/core/glm53f_ops.c:945-976).
constexpr int RT_WARPS = 4;
constexpr int RT_MAX_TOKENS = 64;            // tokens per launch (the engine's pass size)

struct RouterArgs {
    int *idx; float *w; float *score;
    const float *x; int ldx;
    const void *gate; int gate_dt;
    const float *bias;
    int NE, E, K, T, norm_topk;
    float routed_scale;
    MoePlan p;
    int n_local0, n_local, with_shared;
    int *counter;
    int sh_t0, sh_n;                 // the shared expert's slot takes tokens [sh_t0, sh_t0 + sh_n)
};

// Order-preserving key of a selection score; 0 = not selectable (NaN, -inf, already taken).
__device__ __forceinline__ uint32_t choice_key(float v)
{
    if (!(v > -INFINITY)) return 0u;
    const uint32_t u = __float_as_uint(__fadd_rn(v, 0.f));     // -0 -> +0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Top-k of one token by one warp, scores and keys in registers (expert lane + 32 i in slot i): K
// rounds of "largest key of the warp, then the lowest expert holding it" with warp reductions.
template <int PER>
__device__ void topk_one_token(const RouterArgs &a, int t, int lane)
{
    const float *scp = a.score + (size_t)t * a.NE;
    float sc[PER];
    uint32_t key[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int e = lane + 32 * i;
        sc[i] = e < a.NE ? __ldcg(scp + e) : 0.f;
        key[i] = e < a.NE ? choice_key(__fadd_rn(sc[i], a.bias[e])) : 0u;
    }
    int pick0 = 0, pick1 = 0;                      // lane l keeps picks l and l + 32 (K <= 64)
    float w0 = 0.f, w1 = 0.f;
    for (int j = 0; j < a.K; j++) {
        uint32_t m = 0u;
#pragma unroll
        for (int i = 0; i < PER; i++) m = max(m, key[i]);
        m = __reduce_max_sync(0xffffffffu, m);
        uint32_t cand = 0xffffffffu;
#pragma unroll
        for (int i = 0; i < PER; i++) cand = min(cand, key[i] == m ? (uint32_t)(lane + 32 * i) : 0xffffffffu);
        uint32_t bi = __reduce_min_sync(0xffffffffu, cand);
        if (m == 0u) bi = 0u;                      // nothing selectable is left (the reference aborts here)
        float wsel = 0.f;
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (bi == (uint32_t)(lane + 32 * i)) { wsel = sc[i]; key[i] = 0u; }
        wsel = __shfl_sync(0xffffffffu, wsel, bi & 31);
        if (lane == (j & 31)) {
            if (j < 32) { pick0 = (int)bi; w0 = wsel; } else { pick1 = (int)bi; w1 = wsel; }
        }
    }
    if (a.norm_topk) {
        double tot = 0.0;
        for (int j = 0; j < a.K; j++) tot += (double)__shfl_sync(0xffffffffu, j < 32 ? w0 : w1, j & 31);
        w0 = (float)((double)w0 / (tot + 1e-20));
        w1 = (float)((double)w1 / (tot + 1e-20));
    }
    if (lane < a.K) {
        a.idx[(size_t)t * a.K + lane] = pick0;
        a.w[(size_t)t * a.K + lane] = __fmul_rn(w0, a.routed_scale);
    }
    if (lane + 32 < a.K) {
        a.idx[(size_t)t * a.K + lane + 32] = pick1;
        a.w[(size_t)t * a.K + lane + 32] = __fmul_rn(w1, a.routed_scale);
    }
}

__global__ void __launch_bounds__(RT_WARPS * 32) router_kernel(const RouterArgs a)
{
    __shared__ int sidx_buf[RT_MAX_TOKENS * G5B_MAX_TOPK];
    __shared__ int cnt[G5B_MAX_EXPERTS], off[G5B_MAX_EXPERTS];
    __shared__ int psum[RT_WARPS * 32], ssum[RT_WARPS * 32];
    __shared__ int is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int e = blockIdx.x * RT_WARPS + warp, t = blockIdx.y;
    if (e < a.NE) {
        const float *xt = a.x + (size_t)t * a.ldx;
        double acc = 0.0;
        if (a.gate_dt == DT_BF16 && (a.E & 7) == 0 && (a.ldx & 3) == 0) {
            const uint16_t *row = static_cast<const uint16_t *>(a.gate) + (size_t)e * a.E;
#pragma unroll 4
            for (int c = lane * 8; c < a.E; c += 256) {
                const uint4 wv = ld_stream16(row + c);
                const float4 x0 = *reinterpret_cast<const float4 *>(xt + c), x1 = *reinterpret_cast<const float4 *>(xt + c + 4);
                float w[8];
                bf16x2_to_f32(wv.x, w[0], w[1]); bf16x2_to_f32(wv.y, w[2], w[3]);
                bf16x2_to_f32(wv.z, w[4], w[5]); bf16x2_to_f32(wv.w, w[6], w[7]);
                acc = fma((double)w[0], (double)x0.x, acc); acc = fma((double)w[1], (double)x0.y, acc);
                acc = fma((double)w[2], (double)x0.z, acc); acc = fma((double)w[3], (double)x0.w, acc);
                acc = fma((double)w[4], (double)x1.x, acc); acc = fma((double)w[5], (double)x1.y, acc);
                acc = fma((double)w[6], (double)x1.z, acc); acc = fma((double)w[7], (double)x1.w, acc);
            }
        } else if (a.gate_dt == DT_BF16) {
            const uint16_t *row = static_cast<const uint16_t *>(a.gate) + (size_t)e * a.E;
            for (int i = lane; i < a.E; i += 32) acc = fma((double)bf16_to_f32(row[i]), (double)xt[i], acc);
        } else {
            const float *row = static_cast<const float *>(a.gate) + (size_t)e * a.E;
            for (int i = lane; i < a.E; i += 32) acc = fma((double)row[i], (double)xt[i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) a.score[(size_t)t * a.NE + e] = sigmoid_host((float)acc);
    }
    // The CTA that finishes a token's rows last (one counter per token, no spinning) selects that
    // token's experts, so the tokens of a batch are selected in parallel; the CTA that finishes
    // the last selection then groups the pairs.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(a.counter + 1 + t, 1);
        is_last = prev == (int)gridDim.x - 1;
        if (is_last) a.counter[1 + t] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (warp == 0) {
        if (a.NE <= 512) topk_one_token<16>(a, t, lane);
        else             topk_one_token<32>(a, t, lane);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(a.counter, 1);
        is_last = prev == (int)gridDim.y - 1;
        if (is_last) *a.counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (!a.p.n_slots) return;

    // Group the (token, slot) pairs by expert. Slots are numbered in expert order; the shared
    // expert, when asked for, is the last slot and takes every token. Which pair of an expert
    // lands where inside its slot does not matter: every pair has its own output row.
    const int n = a.T * a.K, nth = RT_WARPS * 32;
    int *sidx = sidx_buf;                                     // [T*K] ids
    for (int i = tid; i < n; i += nth) sidx[i] = __ldcg(a.idx + i);
    for (int le = tid; le < a.n_local; le += nth) cnt[le] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += nth) {
        const int le = sidx[i] - a.n_local0;
        if (le >= 0 && le < a.n_local) atomicAdd(&cnt[le], 1);
    }
    __syncthreads();
    const int per = (a.n_local + nth - 1) / nth;              // consecutive experts per thread
    int pairs = 0, slots = 0;
    for (int k = 0; k < per; k++) {
        const int le = tid * per + k;
        if (le < a.n_local && cnt[le]) { pairs += cnt[le]; slots++; }
    }
    psum[tid] = pairs; ssum[tid] = slots;
    __syncthreads();
    for (int o = 1; o < nth; o <<= 1) {                       // inclusive scans over the threads
        const int pv = tid >= o ? psum[tid - o] : 0, sv = tid >= o ? ssum[tid - o] : 0;
        __syncthreads();
        psum[tid] += pv; ssum[tid] += sv;
        __syncthreads();
    }
    int pbase = psum[tid] - pairs, sbase = ssum[tid] - slots;
    const int total_pairs = psum[nth - 1], total_slots = ssum[nth - 1];
    for (int k = 0; k < per; k++) {
        const int le = tid * per + k;
        if (le >= a.n_local) break;
        off[le] = pbase;
        if (cnt[le]) {
            a.p.slot_expert[sbase] = le; a.p.slot_off[sbase] = pbase; a.p.slot_cnt[sbase] = cnt[le];
            pbase += cnt[le]; sbase++;
        }
    }
    __syncthreads();
    for (int le = tid; le < a.n_local; le += nth) cnt[le] = 0;    // reused as the write cursor of each expert
    __syncthreads();
    for (int i = tid; i < n; i += nth) {
        const int le = sidx[i] - a.n_local0;
        if (le < 0 || le >= a.n_local) continue;
        const int pos = off[le] + atomicAdd(&cnt[le], 1);
        a.p.pair_tok[pos] = i / a.K;
        a.p.pair_dst[pos] = i;
    }
    const bool shared = a.with_shared && a.sh_n > 0;
    if (shared) {
        if (tid == 0) { a.p.slot_expert[total_slots] = a.n_local; a.p.slot_off[total_slots] = total_pairs; a.p.slot_cnt[total_slots] = a.sh_n; }
        for (int tt = tid; tt < a.sh_n; tt += nth) { a.p.pair_tok[total_pairs + tt] = a.sh_t0 + tt; a.p.pair_dst[total_pairs + tt] = n + a.sh_t0 + tt; }
    }
    if (tid == 0) *a.p.n_slots = total_slots + (shared ? 1 : 0);
}

// p may be null-planned (p.n_slots == nullptr) when only the routing is wanted.
void router_plan(cudaStream_t st, int *idx, float *w, float *score, const float *x, int ldx, const void *gate,
                 int gate_dt, const float *bias, int T, const MoeShape &s, const MoePlan &p, int with_shared,
                 int *counter, int shared_t0, int shared_n)
{
    RouterArgs a{idx, w, score, x, ldx, gate, gate_dt, bias, s.NE, s.E, s.K, T, s.norm_topk, s.routed_scale,
                 p, s.n_local0, s.n_local, with_shared, counter, shared_t0, shared_n < 0 ? T : shared_n};
    G5B_LAUNCH(router_kernel, dim3((s.NE + RT_WARPS - 1) / RT_WARPS, T), RT_WARPS * 32, 0, st, a);
}

// ----------------------------------------------------------------- experts ----
__device__ __forceinline__ float swiglu_clamped(float g, float u, float lim)
{
    g = g > lim ? lim : g;
    u = u > lim ? lim : (u < -lim ? -lim : u);
    return __fmul_rn(__fmul_rn(g, sigmoid_host(g)), u);
}

struct ExpertArgs {
    const ExpertW *experts;
    MoePlan p;
    const float *x;      // gate/up: layer input [T][ldx]; down: activations [pairs][I]
    float *y;            // gate/up: activations [pairs][I]; down: contributions [T*K (+T)][E]
    int ldx, E, I, br, bc, dt;
    float limit;
};

// Rows of one token tile. gate/up: the warp holds gate rows r, r+1 and up rows r, r+1 and writes
// the clamped SwiGLU of the pair; down: four consecutive output rows.
template <int TT, bool GATEUP>
__device__ __forceinline__ void expert_tile(const ExpertArgs &a, const void *const (&wrow)[RW],
                                            const float *const (&srow)[RW], int off, int i0, int cnt,
                                            int r, int rows_total, int C, int lane)
{
    const float *xp[TT];
    float xinv[TT];
    int pair[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) {
        pair[t] = off + min(i0 + t, cnt - 1);
        xp[t] = GATEUP ? a.x + (size_t)a.p.pair_tok[pair[t]] * a.ldx : a.x + (size_t)pair[t] * a.I;
        xinv[t] = 1.f;
    }
    float acc[RW][TT];
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
        for (int t = 0; t < TT; t++) acc[q][t] = 0.f;
    dot_rows<TT>(acc, a.dt, wrow, srow, a.bc, xp, xinv, nullptr, false, 0, C / piece_elems(a.dt), lane);
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
        for (int t = 0; t < TT; t++) acc[q][t] = warp_sum(acc[q][t]);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (i0 + t >= cnt) break;
            if (GATEUP) {
                float *dst = a.y + (size_t)pair[t] * a.I;
                dst[r] = swiglu_clamped(acc[0][t], acc[2][t], a.limit);
                if (r + 1 < rows_total) dst[r + 1] = swiglu_clamped(acc[1][t], acc[3][t], a.limit);
            } else {
                float *dst = a.y + (size_t)a.p.pair_dst[pair[t]] * a.E;
#pragma unroll
                for (int q = 0; q < RW; q++)
                    if (r + q < rows_total) dst[r + q] = acc[q][t];
            }
        }
    }
}

// MAXTT = 1 is the decode instantiation (one token per expert, half the registers, two CTAs per
// SM); MAXTT = 4 serves batches.
template <bool GATEUP, int MAXTT>
__global__ void __launch_bounds__(MOE_THREADS, MAXTT == 1 ? 2 : 1) expert_kernel(const ExpertArgs a)
{
    const int s = blockIdx.y;
    if (s >= *a.p.n_slots) return;
    const ExpertW ew = a.experts[a.p.slot_expert[s]];
    const int off = a.p.slot_off[s], cnt = a.p.slot_cnt[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = GATEUP ? a.E : a.I;                       // columns of the matrices multiplied
    const int rows_total = GATEUP ? a.I : a.E;
    const int scols = (C + a.bc - 1) / (a.bc > 0 ? a.bc : 1);
    const size_t rb = (size_t)C * (a.dt == DT_FP8 ? 1 : a.dt == DT_BF16 ? 2 : 4);
    const int r = (blockIdx.x * MOE_WARPS + warp) * (GATEUP ? 2 : RW);
    if (r >= rows_total) return;

    const void  *wrow[RW];
    const float *srow[RW];
    if (GATEUP) {
        const int r1 = min(r + 1, rows_total - 1);
        wrow[0] = ew.gate + (size_t)r * rb;  wrow[1] = ew.gate + (size_t)r1 * rb;
        wrow[2] = ew.up + (size_t)r * rb;    wrow[3] = ew.up + (size_t)r1 * rb;
        if (a.dt == DT_FP8) {
            srow[0] = ew.gate_s + (size_t)(r / a.br) * scols;  srow[1] = ew.gate_s + (size_t)(r1 / a.br) * scols;
            srow[2] = ew.up_s + (size_t)(r / a.br) * scols;    srow[3] = ew.up_s + (size_t)(r1 / a.br) * scols;
        } else { srow[0] = srow[1] = srow[2] = srow[3] = nullptr; }
    } else {
#pragma unroll
        for (int q = 0; q < RW; q++) {
            const int rq = min(r + q, rows_total - 1);
            wrow[q] = ew.down + (size_t)rq * rb;
            srow[q] = a.dt == DT_FP8 ? ew.down_s + (size_t)(rq / a.br) * scols : nullptr;
        }
    }
    // Token tiles: the weights stream once per tile of up to four tokens of this expert.
    for (int i0 = 0; i0 < cnt;) {
        const int rem = cnt - i0;
        if (MAXTT >= 4 && rem >= 3)      { expert_tile<MAXTT >= 4 ? 4 : 1, GATEUP>(a, wrow, srow, off, i0, cnt, r, rows_total, C, lane); i0 += 4; }
        else if (MAXTT >= 2 && rem == 2) { expert_tile<MAXTT >= 2 ? 2 : 1, GATEUP>(a, wrow, srow, off, i0, cnt, r, rows_total, C, lane); i0 += 2; }
        else                             { expert_tile<1, GATEUP>(a, wrow, srow, off, i0, cnt, r, rows_total, C, lane); i0 += 1; }
    }
}

// Any shape / block size: a warp per output row and pair, FP64 sums (test fixtures).
template <bool GATEUP>
__global__ void __launch_bounds__(MOE_THREADS) expert_any_kernel(const ExpertArgs a)
{
    const int s = blockIdx.y;
    if (s >= *a.p.n_slots) return;
    const ExpertW ew = a.experts[a.p.slot_expert[s]];
    const int off = a.p.slot_off[s], cnt = a.p.slot_cnt[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int C = GATEUP ? a.E : a.I, rows_total = GATEUP ? a.I : a.E;
    const int scols = (C + a.bc - 1) / (a.bc > 0 ? a.bc : 1);
    const int r = blockIdx.x * MOE_WARPS + warp;
    if (r >= rows_total) return;
    const int nm = GATEUP ? 2 : 1;
    for (int i = 0; i < cnt; i++) {
        const int pair = off + i;
        const float *x = GATEUP ? a.x + (size_t)a.p.pair_tok[pair] * a.ldx : a.x + (size_t)pair * a.I;
        double acc[2] = {0.0, 0.0};
        for (int m = 0; m < nm; m++) {
            const void *W = GATEUP ? (m ? ew.up : ew.gate) : ew.down;
            const float *S = GATEUP ? (m ? ew.up_s : ew.gate_s) : ew.down_s;
            for (int c = lane; c < C; c += 32) {
                double wv;
                if (a.dt == DT_FP8)
                    wv = (double)e4m3_to_f32(static_cast<const uint8_t *>(W)[(size_t)r * C + c]) *
                         (double)S[(size_t)(r / a.br) * scols + c / a.bc];
                else if (a.dt == DT_BF16) wv = (double)bf16_to_f32(static_cast<const uint16_t *>(W)[(size_t)r * C + c]);
                else wv = (double)static_cast<const float *>(W)[(size_t)r * C + c];
                acc[m] += wv * (double)x[c];
            }
            acc[m] = warp_sum(acc[m]);
        }
        if (lane == 0) {
            if (GATEUP) a.y[(size_t)pair * a.I + r] = swiglu_clamped((float)acc[0], (float)acc[1], a.limit);
            else        a.y[(size_t)a.p.pair_dst[pair] * a.E + r] = (float)acc[0];
        }
    }
}

static bool experts_fast(const MoeShape &s, int C)
{
    if (C % piece_elems(s.dt)) return false;
    if (s.dt == DT_FP8 && (s.bc % 16 || s.br < 1)) return false;
    return true;
}

static int plan_slots(const MoePlan &p, int T, const MoeShape &s)
{
    int m = T * s.K < s.n_local ? T * s.K : s.n_local;
    m += 1;
    return m < p.max_slots ? m : p.max_slots;
}

void moe_gateup(cudaStream_t st, float *act, const float *x, int ldx, const ExpertW *experts,
                const MoePlan &p, int T, const MoeShape &s)
{
    ExpertArgs a{experts, p, x, act, ldx, s.E, s.I, s.br, s.bc, s.dt, s.limit};
    const int slots = plan_slots(p, T, s);
    const dim3 grid((s.I + 2 * MOE_WARPS - 1) / (2 * MOE_WARPS), slots);
    if (experts_fast(s, s.E) && (ldx % 4) == 0) {
        if (T == 1) G5B_LAUNCH((expert_kernel<true, 1>), grid, MOE_THREADS, 0, st, a);
        else        G5B_LAUNCH((expert_kernel<true, 4>), grid, MOE_THREADS, 0, st, a);
    } else
        G5B_LAUNCH(expert_any_kernel<true>, dim3((s.I + MOE_WARPS - 1) / MOE_WARPS, slots), MOE_THREADS, 0, st, a);
}

void moe_down(cudaStream_t st, float *contrib, const float *act, const ExpertW *experts,
              const MoePlan &p, int T, const MoeShape &s)
{
    ExpertArgs a{experts, p, act, contrib, s.I, s.E, s.I, s.br, s.bc, s.dt, s.limit};
    const int slots = plan_slots(p, T, s);
    const dim3 grid((s.E + RW * MOE_WARPS - 1) / (RW * MOE_WARPS), slots);
    if (experts_fast(s, s.I) && (s.I % 4) == 0) {
        if (T == 1) G5B_LAUNCH((expert_kernel<false, 1>), grid, MOE_THREADS, 0, st, a);
        else        G5B_LAUNCH((expert_kernel<false, 4>), grid, MOE_THREADS, 0, st, a);
    } else
        G5B_LAUNCH(expert_any_kernel<false>, dim3((s.E + MOE_WARPS - 1) / MOE_WARPS, slots), MOE_THREADS, 0, st, a);
}

// out[t][d] = (float) sum_j w[t][j] * contrib[t*K+j][d]  (FP64, top-k order)  (+ shared, FP32).
__global__ void moe_combine_kernel(float *out, int ldo, const float *contrib, const float *w, int T, int K,
                                   int E, int with_shared)
{
    const int t = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= E) return;
    double s = 0.0;
    for (int j = 0; j < K; j++)
        s += (double)w[(size_t)t * K + j] * (double)contrib[((size_t)t * K + j) * E + d];
    float o = (float)s;
    if (with_shared) o = __fadd_rn(o, contrib[((size_t)T * K + t) * E + d]);
    out[(size_t)t * ldo + d] = o;
}

void moe_combine(cudaStream_t st, float *out, int ldo, const float *contrib, const float *w, int T,
                 const MoeShape &s, int with_shared)
{
    G5B_LAUNCH(moe_combine_kernel, dim3((s.E + 255) / 256, T), 256, 0, st, out, ldo, contrib, w, T, s.K, s.E,
               with_shared);
}

}  // namespace g5b
