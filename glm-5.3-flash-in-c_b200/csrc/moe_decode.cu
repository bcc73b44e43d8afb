// moe_decode.cu - one MoE layer for one token in ONE persistent kernel: router, top-k, gate/up
// with clamped SwiGLU, down, and the combine.
//
// Why one kernel: as three launches (router, gate/up, down) the layer spent about a third of its
// time outside the streaming loops - launch gaps, each kernel's prologue (barrier set-up, plan and
// pointer loads, activation split), and a 20 us router whose tail ran on a single CTA. Here all
// 148 SMs start streaming at once: the shared expert does not depend on routing, so its gate/up
// rows are in flight while the router rows are being multiplied; every CTA then selects the top-k
// itself from the 288 scores (identical everywhere), and the weight pipeline never drains between
// gate/up and down because the down weights of a CTA's first row tiles are prefetched before the
// grid-wide point where the activations become visible.
//
// Launched cooperatively (all CTAs co-resident, one per SM). The two grid-wide points are counters
// in device memory that only ever grow (the host passes the value each launch starts from); every
// wait - on them, on the shared-memory mbarriers - is bounded, and a wait that runs out records a
// code in mapped host memory and unwinds the CTA after draining its copies.
//
// Work items: gate/up item = 16 gate rows + the same 16 up rows (two stages of 2048 columns);
// down item = 32 output rows (one stage, plus the expert's activation terms). Items are numbered
// shared expert first, then the routed experts in top-k order, and dealt round-robin to the CTAs.
// Arithmetic is that of moe_mma.cu (tensor-core products of E4M3 codes with the activation split
// into two F16 terms); selection and combine follow the reference (src/core/glm53f_ops.c:945-976,
// 1329-1340).
#include "kernels.h"
#include "mma_stage.cuh"
#include "stage_timers.cuh"

namespace g5b {

constexpr int DEC_SPIN_LIMIT = 1 << 21;
constexpr int DEC_PER = 16;                  // experts per lane of the selecting warp: NE <= 512

struct DecodeArgs {
    const ExpertW *experts;     // [NE + 1], shared expert last
    const float *x;             // [E]
    const void *gate; int gate_dt;
    const float *bias;
    float *score;               // [NE] scratch
    int *idx; float *w;         // [K] outputs (also used by the combine)
    __half *act;                // [K + 1][2][I] scratch
    float *contrib;             // [K + 1][E] scratch
    float *out;                 // [E]
    int E, I, NE, K, br, bc, with_shared, norm_topk;
    float limit, routed_scale;
    unsigned long long *sync;   // [2] grid-wide counters
    unsigned long long base;    // value of both counters when this launch starts
    int *tile_done;
    int *err;
    // expert parallel (ep_size > 1): this rank owns experts [n_local0, n_local0 + n_local); experts[]
    // is indexed by local expert, shared expert last; peers[r] is rank r's exchange region: ep_size
    // step words (the multi-token exchange kernel's), ep_size arrival counters (this kernel's: word
    // ep_size + q counts the CTAs of rank q that have delivered, over all launches), then at rows_off
    // this step's row buffer [K][E]
    int ep_rank, ep_size, n_local0, n_local;
    void *const *peers;
    size_t rows_off;
    unsigned long long ep_launch;      // expert-parallel launches of this kernel so far, this one included
    unsigned long long ep_wait_ns;
};

__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Wait until every CTA of the grid has arrived at counter `which`; bounded. Called by a whole warp:
// every lane polls the same word (one transaction), so the loop is uniform and the warp leaves
// it converged - a single polling lane left the warp split for the code that follows, which
// then ran several times slower.
__device__ __forceinline__ bool grid_wait(const DecodeArgs &a, int which, int code)
{
    const unsigned long long target = a.base + gridDim.x;
    bool seen = false;
    for (int i = 0; i < DEC_SPIN_LIMIT && !seen; i++) {
        seen = ld_acquire(a.sync + which) >= target;
        if (!seen) __nanosleep(40);
    }
    seen = __all_sync(0xffffffffu, seen);
    if (!seen && (threadIdx.x & 31) == 0) atomicExch(a.err, code);
    __syncwarp();
    return seen;
}

// Order-preserving key of a selection score; 0 = not selectable (NaN, -inf, already taken).
__device__ __forceinline__ uint32_t choice_key(float v)
{
    if (!(v > -INFINITY)) return 0u;
    const uint32_t u = __float_as_uint(__fadd_rn(v, 0.f));     // -0 -> +0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(MM_THREADS, 1) moe_decode_kernel(const DecodeArgs a)
{
    const float act_sc = act_term_scale(a.limit), act_inv = 1.0f / act_sc;   // powers of two
    DT_BEGIN();
    extern __shared__ __align__(128) uint8_t smem[];
    const int tps_g = a.I / 16;                 // gate/up items per expert
    const int tps_d = a.E / MM_ROWS;            // down items per expert
    const int nsl = a.K + (a.with_shared ? 1 : 0);
    const int sh_g = a.with_shared ? tps_g : 0;   // gate/up items of the shared expert: known before the plan
    const int n_dn_all = nsl * tps_d;             // down items when every pick is this GPU's
    const int scols_g = a.E / a.bc, scols_d = a.I / a.bc;
    const size_t scale_off = (size_t)MM_ROWS * MM_PITCH;
    const size_t stage_bytes = scale_off + 512;
    uint8_t *stages = smem;
    uint8_t *actring = smem + MM_NS * stage_bytes;                  // [NS][2][I] F16; gate/up phase: x terms [2][E]
    const size_t act_bytes = (size_t)a.I * 4;
    __half *x_h = reinterpret_cast<__half *>(actring);
    float *red = reinterpret_cast<float *>(actring + MM_NS * act_bytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(red) + MM_CONS * 16 * 4);
    uint64_t *empty = full + MM_NS;
    uint64_t *plan_ready = empty + MM_NS;       // the router weights of the picks are in s_w
    uint64_t *sel_ready = plan_ready + 1;        // the picks' expert pointers and s_local are written
    __shared__ ExpertW s_ew[MM_MAX_SLOTS];       // slot j < K: j-th routed pick; slot K: shared expert
    __shared__ float s_w[MM_MAX_SLOTS];
    __shared__ int s_lslot[MM_MAX_SLOTS];        // the picks whose experts live on this rank, in top-k order
    __shared__ int s_nloc;                       // how many (K on a single GPU)
    __shared__ int s_flag;
    __shared__ int my_tiles[MM_MAX_ITEMS], my_last[MM_MAX_ITEMS];
    __shared__ float wmax[MM_THREADS / 32];
    __shared__ float x_scale[2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < MM_NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], MM_CONS); }
        mbar_init(plan_ready, 1);
        mbar_init(sel_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x == 32 && a.with_shared) s_ew[a.K] = a.experts[a.n_local];
    __syncthreads();

    // Work items are numbered over the picks this rank owns only, so that the round-robin deal stays
    // even when other ranks own some of the picks. Gate/up: the shared expert's row tiles first (they
    // need no plan), then the local picks in top-k order. Down: the local picks, then the shared
    // expert. (s_lslot / s_nloc are valid once the plan is made; on one GPU they are the identity.)
    auto gu_slot = [&](int g, int &slot, int &rt) {
        if (g < sh_g) { slot = a.K; rt = g; }
        else {
            const int j = (g - sh_g) / tps_g;
            slot = a.ep_size > 1 ? s_lslot[j] : j;
            rt = (g - sh_g) % tps_g;
        }
    };
    auto dn_slot = [&](int g, int nloc, int &slot, int &rt) {
        const int j = g / tps_d;
        rt = g % tps_d;
        slot = j < nloc ? (a.ep_size > 1 ? s_lslot[j] : j) : a.K;
    };
    bool ok = true;

    if (warp == MM_CONS) {
        // ================================================================ producer ====
        int it = 0;
        bool have_plan = false;
        float plan_w = 0.f;                          // lane j < K: router score of the j-th pick
        float bias_r[DEC_PER];                       // the selection bias does not depend on the scores: fetch it now
#pragma unroll
        for (int i = 0; i < DEC_PER; i++) bias_r[i] = lane + 32 * i < a.NE ? a.bias[lane + 32 * i] : 0.f;
        asm volatile("bar.sync 2, %0;" ::"r"((MM_CONS + 1) * 32) : "memory");   // the consumers' router loads are issued
        // The producer selects the experts (every CTA for itself; the result is the same everywhere)
        // while the consumers multiply what is already in flight: wait for all router rows, then
        // top-k of score + bias by repeated arg-max, lowest index on ties.
        auto make_plan = [&]() -> bool {
            if (!grid_wait(a, 0, 6)) return false;
            DT_MARK_P(9);
            // scores and choices stay in registers (expert lane + 32 i in slot i): one round of loads,
            // no shared-memory traffic between the rounds
            float sc[DEC_PER];
            uint32_t key[DEC_PER];
#pragma unroll
            for (int i = 0; i < DEC_PER; i++) {
                const int e = lane + 32 * i;
                sc[i] = e < a.NE ? __ldcg(a.score + e) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < DEC_PER; i++) key[i] = lane + 32 * i < a.NE ? choice_key(__fadd_rn(sc[i], bias_r[i])) : 0u;
            int my_pick = 0;
            float my_w = 0.f;
            // K rounds of arg-max: the largest key of the warp, then the lowest expert holding it
            for (int j = 0; j < a.K; j++) {
                uint32_t m = 0u;
#pragma unroll
                for (int i = 0; i < DEC_PER; i++) m = max(m, key[i]);
                m = __reduce_max_sync(0xffffffffu, m);
                uint32_t cand = 0xffffffffu;
#pragma unroll
                for (int i = 0; i < DEC_PER; i++) cand = min(cand, key[i] == m ? (uint32_t)(lane + 32 * i) : 0xffffffffu);
                uint32_t bi = __reduce_min_sync(0xffffffffu, cand);
                if (m == 0u) bi = 0u;                                  // nothing selectable is left
                float wsel = 0.f;
#pragma unroll
                for (int i = 0; i < DEC_PER; i++)
                    if (bi == (uint32_t)(lane + 32 * i)) { wsel = sc[i]; key[i] = 0u; }
                wsel = __shfl_sync(0xffffffffu, wsel, bi & 31);
                if (lane == j) { my_pick = (int)bi; my_w = wsel; }
            }
            DT_MARK_P(13);
            {                                         // the K pointer records are fetched side by side
                const int le = my_pick - a.n_local0;
                const bool local = lane < a.K && le >= 0 && le < a.n_local;
                if (local) s_ew[lane] = a.experts[le];
                if (lane < a.K && blockIdx.x == 0) a.idx[lane] = my_pick;
                const unsigned lm = __ballot_sync(0xffffffffu, local);
                if (local) s_lslot[__popc(lm & ((1u << lane) - 1u))] = lane;
                if (lane == 0) s_nloc = __popc(lm);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sel_ready);
            DT_MARK_P(14);
            plan_w = my_w;                            // normalised after the last copy is issued (below)
            __syncwarp();
            DT_MARK_P(1);
            return true;
        };
        // Router weights of the picks (reference: normalise in FP64, scale). Only the combine needs
        // them, so the FP64 division stays off the path to the first routed copy.
        auto finish_weights = [&]() {
            float w = plan_w;
            if (a.norm_topk) {
                double tot = 0.0;
                for (int j = 0; j < a.K; j++) tot += (double)__shfl_sync(0xffffffffu, w, j);
                w = (float)((double)w / (tot + 1e-20));
            }
            w = __fmul_rn(w, a.routed_scale);
            if (lane < a.K) {
                s_w[lane] = w;
                if (blockIdx.x == 0) a.w[lane] = w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(plan_ready);
        };
        int n_gu = sh_g;                               // until the plan is made only the shared expert's items exist
        for (int g = blockIdx.x; ok; g += gridDim.x) {
            if (g >= sh_g && !have_plan) {
                ok = make_plan();
                if (!ok) break;
                have_plan = true;
                n_gu = sh_g + s_nloc * tps_g;
            }
            if (g >= n_gu) break;
            int slot, rt;
            gu_slot(g, slot, rt);
            const ExpertW ew = s_ew[slot];
            for (int kh = 0; kh < a.E / MM_CB && ok; kh++, it++) {
                const int s = it % MM_NS;
                if (it >= MM_NS) ok = mbar_wait(&empty[s], ((it / MM_NS) - 1) & 1, a.err, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t *st = stages + (size_t)s * stage_bytes;
                if (lane == 0) mbar_expect_tx(&full[s], MM_ROWS * MM_CB + 2 * scols_g * 4);
                __syncwarp();
                const uint8_t *src = (lane < 16 ? ew.gate : ew.up) + (size_t)(rt * 16 + (lane & 15)) * a.E + (size_t)kh * MM_CB;
                bulk_g2s(st + (size_t)lane * MM_PITCH, src, MM_CB, &full[s]);
                if (lane == 0) {
                    bulk_g2s(st + scale_off, ew.gate_s + (size_t)((rt * 16) / a.br) * scols_g, scols_g * 4, &full[s]);
                    bulk_g2s(st + scale_off + 256, ew.up_s + (size_t)((rt * 16) / a.br) * scols_g, scols_g * 4, &full[s]);
                }
            }
        }
        // down: weights are prefetched before the activations exist; their copy follows the grid point
        bool acts_visible = false;
        int pending = 0, pend_stage[MM_NS], pend_slot[MM_NS];
        const int nloc_p = ok ? s_nloc : 0;
        const int n_dn = ok ? (nloc_p + (a.with_shared ? 1 : 0)) * tps_d : 0;
        // this CTA's last down item
        const int last_g = (int)blockIdx.x < n_dn ? (int)blockIdx.x + ((n_dn - 1 - (int)blockIdx.x) / (int)gridDim.x) * (int)gridDim.x : -1;
        for (int g = blockIdx.x; g < n_dn && ok; g += gridDim.x) {
            int slot, rt;
            dn_slot(g, nloc_p, slot, rt);
            const ExpertW ew = s_ew[slot];
            const int s = it % MM_NS;
            if (it >= MM_NS) ok = mbar_wait(&empty[s], ((it / MM_NS) - 1) & 1, a.err, 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            uint8_t *st = stages + (size_t)s * stage_bytes;
            if (lane == 0) mbar_expect_tx(&full[s], MM_ROWS * MM_CB + scols_d * 4 + (uint32_t)act_bytes);
            __syncwarp();
            bulk_g2s(st + (size_t)lane * MM_PITCH, ew.down + (size_t)(rt * MM_ROWS + lane) * a.I, MM_CB, &full[s]);
            if (lane == 0)
                bulk_g2s(st + scale_off, ew.down_s + (size_t)((rt * MM_ROWS) / a.br) * scols_d, scols_d * 4, &full[s]);
            pend_stage[pending] = s; pend_slot[pending] = slot; pending++;
            const bool last = g == last_g;
            it++;
            if (!acts_visible && (pending == MM_NS || last)) {
                ok = grid_wait(a, 1, 7);
                if (!ok) break;
                acts_visible = true;
            }
            if (acts_visible) {
                if (lane == 0)
                    for (int k = 0; k < pending; k++)
                        bulk_g2s(actring + (size_t)pend_stage[k] * act_bytes,
                                 reinterpret_cast<const uint8_t *>(a.act) + (size_t)pend_slot[k] * act_bytes,
                                 (uint32_t)act_bytes, &full[pend_stage[k]]);
                pending = 0;
            }
        }
        if (ok) finish_weights();
        if (!ok) {
            // Copies in flight must land before shared memory goes away. A stage whose activation
            // copy was never issued cannot complete; give it its missing bytes from the buffer
            // (whatever it holds) so that the barrier closes, then wait for every stage in flight.
            if (lane == 0)
                for (int k = 0; k < pending; k++)
                    bulk_g2s(actring + (size_t)pend_stage[k] * act_bytes, reinterpret_cast<const uint8_t *>(a.act),
                             (uint32_t)act_bytes, &full[pend_stage[k]]);
            for (int k = 0; k < MM_NS && k < it; k++) {
                const int j = it - 1 - k;
                mbar_wait(&full[j % MM_NS], (j / MM_NS) & 1, a.err, 3);
            }
        }
    } else {
        // =============================================================== consumers ====
        const int mt = warp & 1, kq = warp >> 1;
        const int g8 = lane >> 2, t4 = lane & 3;
        const int ctid = threadIdx.x;                     // 0..255
        // ---- router rows first (every CTA waits for all of them): two rows per pass, each row split
        // over four warps so that all of its loads are in flight at once; FP64 partial sums are
        // added in a fixed order, then the float sigmoid. (Compensated FP32 sums were 0.5 us faster
        // with a warm instruction cache and 1 us slower after other kernels: four times the code.)
        {
            double *rsum = reinterpret_cast<double *>(red);           // [8] partial sums, red is idle here
            const int quarter = warp & 3, which = warp >> 2, span = a.E / 4;
            bool released = false;                                // the producer may start copying
            for (int e0 = blockIdx.x; e0 < a.NE; e0 += 2 * gridDim.x) {
                const int e = e0 + which * gridDim.x;
                double acc = 0.0;
                if (a.gate_dt == DT_BF16 && span == 1024) {
                    // all loads of the row quarter first, then the hand-over to the producer, then the
                    // arithmetic: the router's few loads enter the memory queues ahead of the 200 KB
                    // of bulk copies each SM is about to issue instead of behind them
                    const int ee = e < a.NE ? e : a.NE - 1;
                    const uint16_t *row = static_cast<const uint16_t *>(a.gate) + (size_t)ee * a.E + (size_t)quarter * span;
                    const float *xq = a.x + (size_t)quarter * span;
                    uint4 wv[4];
                    float4 x0[4], x1[4];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int c = lane * 8 + k * 256;
                        wv[k] = ld_stream16(row + c);
                        x0[k] = *reinterpret_cast<const float4 *>(xq + c);
                        x1[k] = *reinterpret_cast<const float4 *>(xq + c + 4);
                    }
                    if (!released) { asm volatile("bar.arrive 2, %0;" ::"r"((MM_CONS + 1) * 32) : "memory"); released = true; }
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        float w[8];
                        bf16x2_to_f32(wv[k].x, w[0], w[1]); bf16x2_to_f32(wv[k].y, w[2], w[3]);
                        bf16x2_to_f32(wv[k].z, w[4], w[5]); bf16x2_to_f32(wv[k].w, w[6], w[7]);
                        acc = fma((double)w[0], (double)x0[k].x, acc); acc = fma((double)w[1], (double)x0[k].y, acc);
                        acc = fma((double)w[2], (double)x0[k].z, acc); acc = fma((double)w[3], (double)x0[k].w, acc);
                        acc = fma((double)w[4], (double)x1[k].x, acc); acc = fma((double)w[5], (double)x1[k].y, acc);
                        acc = fma((double)w[6], (double)x1[k].z, acc); acc = fma((double)w[7], (double)x1[k].w, acc);
                    }
                } else if (e < a.NE) {
                    if (!released) { asm volatile("bar.arrive 2, %0;" ::"r"((MM_CONS + 1) * 32) : "memory"); released = true; }
                    if (a.gate_dt == DT_BF16) {
                        const uint16_t *row = static_cast<const uint16_t *>(a.gate) + (size_t)e * a.E + (size_t)quarter * span;
                        const float *xq = a.x + (size_t)quarter * span;
                        for (int i = lane; i < span; i += 32) acc = fma((double)bf16_to_f32(row[i]), (double)xq[i], acc);
                    } else {
                        const float *row = static_cast<const float *>(a.gate) + (size_t)e * a.E + (size_t)quarter * span;
                        const float *xq = a.x + (size_t)quarter * span;
                        for (int i = lane; i < span; i += 32) acc = fma((double)row[i], (double)xq[i], acc);
                    }
                }
                acc = warp_sum(acc);
                if (lane == 0) rsum[warp] = acc;
                asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
                if (ctid < 2 && e0 + ctid * (int)gridDim.x < a.NE) {
                    const double t = ((rsum[4 * ctid] + rsum[4 * ctid + 1]) + rsum[4 * ctid + 2]) + rsum[4 * ctid + 3];
                    a.score[e0 + ctid * gridDim.x] = sigmoid_host((float)t);
                }
                asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            }
            if (!released) asm volatile("bar.arrive 2, %0;" ::"r"((MM_CONS + 1) * 32) : "memory");
            if (ctid == 0) { __threadfence(); atomicAdd(a.sync + 0, 1ull); }
        }
        DT_MARK(0);
        // ---- activation split (power-of-two scale so that the largest element sits near 2^14)
        {
            float m = 0.f;
            for (int c = ctid * 4; c < a.E; c += MM_CONS * 32 * 4) {
                const float4 v = *reinterpret_cast<const float4 *>(a.x + c);
                m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (lane == 0) wmax[warp] = m;
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            if (ctid == 0) {
                float mm = 0.f;
                for (int i = 0; i < MM_CONS; i++) mm = fmaxf(mm, wmax[i]);
                int ex = 0;
                if (mm > 0.f && mm < INFINITY) frexpf(mm, &ex);
                x_scale[0] = ldexpf(1.0f, 14 - ex);
                x_scale[1] = ldexpf(1.0f, ex - 14);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            const float sc = x_scale[0];
            for (int c = ctid; c < a.E; c += MM_CONS * 32) {
                __half hi, mid;
                split_f16(a.x[c] * sc, hi, mid);
                x_h[c] = hi;
                x_h[a.E + c] = mid;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        }
        DT_MARK(6);
        int it = 0;
        bool seen_routed = false;

        // ---- gate/up items
        bool have_sel = false;
        int n_gu = a.ep_size > 1 ? sh_g : sh_g + a.K * tps_g;     // expert parallel: the local picks are not known yet
        for (int g = blockIdx.x; ok; g += gridDim.x) {
            if (a.ep_size > 1 && g >= sh_g && !have_sel) {       // which of the picks are this rank's
                ok = mbar_wait_warp(sel_ready, 0, a.err, 10);
                if (!ok) break;
                have_sel = true;
                n_gu = sh_g + s_nloc * tps_g;
            }
            if (g >= n_gu) break;
            int slot, rt;
            gu_slot(g, slot, rt);
            float accf[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kh = 0; kh < a.E / MM_CB && ok; kh++, it++) {
                const int s = it % MM_NS;
                ok = mbar_wait_warp(&full[s], (it / MM_NS) & 1, a.err, 2);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (it == 0) DT_MARK(7);
                if (slot != a.K && !seen_routed) { DT_MARK(8); seen_routed = true; }
                const uint8_t *st = stages + (size_t)s * stage_bytes;
                const float *sc = reinterpret_cast<const float *>(st + scale_off) + (mt ? 64 : 0);
                mma_consume_stage(accf, st, sc, x_h + (size_t)g8 * a.E, kh * MM_CB, a.bc, mt, kq, g8, t4);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            if (t4 == 0) {
                red[warp * 16 + g8] = accf[0] + accf[1] * (1.0f / 2048.0f);
                red[warp * 16 + g8 + 8] = accf[2] + accf[3] * (1.0f / 2048.0f);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            if (ctid < 16) {
                const int r = ctid;
                float gsum = 0.f, usum = 0.f;
#pragma unroll
                for (int q = 0; q < 4; q++) { gsum += red[(2 * q) * 16 + r]; usum += red[(2 * q + 1) * 16 + r]; }
                const float inv = x_scale[1];
                float gv = gsum * inv, uv = usum * inv;
                gv = gv > a.limit ? a.limit : gv;
                uv = uv > a.limit ? a.limit : (uv < -a.limit ? -a.limit : uv);
                const float act = __fmul_rn(__fmul_rn(gv, sigmoid_host(gv)), uv);
                __half hi, mid;
                split_f16(act * act_sc, hi, mid);
                __half *dst = a.act + (size_t)slot * 2 * a.I;
                dst[rt * 16 + r] = hi;
                dst[a.I + rt * 16 + r] = mid;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        }
        // ---- grid point 1: this CTA's activations are written
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        if (ctid == 0) atomicAdd(a.sync + 1, 1ull);
        DT_MARK(2);
        bool first_down = true;

        // ---- down items (the stage's full barrier covers the activation terms too)
        if (ok && a.ep_size > 1 && !have_sel) { ok = mbar_wait_warp(sel_ready, 0, a.err, 10); have_sel = ok; }
        const int nloc_c = a.ep_size > 1 ? (ok ? s_nloc : 0) : a.K;
        const int n_dn = ok ? (nloc_c + (a.with_shared ? 1 : 0)) * tps_d : 0;
        for (int g = blockIdx.x; g < n_dn && ok; g += gridDim.x) {
            int slot, rt;
            dn_slot(g, nloc_c, slot, rt);
            const int s = it % MM_NS;
            ok = mbar_wait_warp(&full[s], (it / MM_NS) & 1, a.err, 2);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            it++;
            if (first_down) { DT_MARK(3); first_down = false; }
            const uint8_t *st = stages + (size_t)s * stage_bytes;
            const float *sc = reinterpret_cast<const float *>(st + scale_off);
            const __half *xt = reinterpret_cast<const __half *>(actring + (size_t)s * act_bytes) + (size_t)g8 * a.I;
            float accf[4] = {0.f, 0.f, 0.f, 0.f};
            mma_consume_stage(accf, st, sc, xt, 0, a.bc, mt, kq, g8, t4);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (t4 == 0) {
                red[warp * 16 + g8] = accf[0] + accf[1] * (1.0f / 2048.0f);
                red[warp * 16 + g8 + 8] = accf[2] + accf[3] * (1.0f / 2048.0f);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            if (ctid < 32) {
                const int r = ctid, m2 = r >> 4, rr = r & 15;
                float v = 0.f;
#pragma unroll
                for (int q = 0; q < 4; q++) v += red[(2 * q + m2) * 16 + rr];
                v *= act_inv;
                const size_t at = (size_t)slot * a.E + rt * MM_ROWS + r;
                if (a.ep_size > 1 && slot != a.K) {
                    // a routed pick's row goes straight into every rank's exchange buffer (peer stores)
                    for (int q = 0; q < a.ep_size; q++)
                        reinterpret_cast<float *>(static_cast<uint8_t *>(a.peers[q]) + a.rows_off)[at] = v;
                } else {
                    a.contrib[at] = v;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        }
        DT_MARK(4);
        if (ok) {                                  // the combine needs the router weights of the plan
            ok = mbar_wait_warp(plan_ready, 0, a.err, 8);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && a.ep_size > 1) {
            // ---- expert parallel: this CTA's rows are on their way into every rank's buffer. One
            // release-add per rank (system scope; through the barrier before it, it covers the stores
            // of every thread of the CTA) counts this CTA as done on that rank - no election of a last
            // CTA and no second fence. A rank is complete on a peer when its counter there has grown
            // by one per CTA; only the CTAs that hold a share of the combine wait for that.
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            const int cnt0 = a.ep_size;                             // the counters follow the step words
            if (ctid < a.ep_size)
                red_release_sys_add(reinterpret_cast<unsigned long long *>(a.peers[ctid]) + cnt0 + a.ep_rank, 1ull);
            DT_MARK(15);
            if ((int)blockIdx.x * MM_CONS * 32 < a.E) {
                if (ctid == 0) s_flag = 1;
                asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
                if (ctid < a.ep_size) {
                    const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(a.peers[a.ep_rank]) + cnt0 + ctid;
                    const bool seen = wait_word_sys(mine, a.ep_launch * gridDim.x, a.ep_wait_ns);
                    if (!seen) { atomicExch(a.err, 20 + ctid); s_flag = 0; }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
                DT_MARK(12);
                if (s_flag) {
                    const float *rows = reinterpret_cast<const float *>(static_cast<const uint8_t *>(a.peers[a.ep_rank]) + a.rows_off);
                    for (int d = blockIdx.x * MM_CONS * 32 + ctid; d < a.E; d += gridDim.x * MM_CONS * 32) {
                        double sum = 0.0;
                        for (int j = 0; j < a.K; j++) sum += (double)s_w[j] * (double)__ldcg(rows + (size_t)j * a.E + d);
                        float o = (float)sum;
                        if (a.with_shared) o = __fadd_rn(o, __ldcg(a.contrib + (size_t)a.K * a.E + d));
                        a.out[d] = o;
                    }
                }
            }
        } else if (ok) {
            // ---- combine: report every row tile this CTA wrote; whoever completes a tile sums its K
            // contributions in top-k order in FP64 and adds the shared expert in FP32
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            int mine = 0;
            for (int g = blockIdx.x; g < n_dn_all; g += gridDim.x) mine++;
            if (mine > MM_MAX_ITEMS) { if (ctid == 0) atomicExch(a.err, 4); mine = 0; }
            if (ctid < mine) {
                const int rt = (blockIdx.x + ctid * gridDim.x) % tps_d;
                const int prev = atomicAdd(&a.tile_done[rt], 1);
                my_tiles[ctid] = rt;
                my_last[ctid] = prev == nsl - 1;
                if (prev == nsl - 1) a.tile_done[rt] = 0;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            __threadfence();
            for (int k = warp; k < mine; k += MM_CONS) {
                if (!my_last[k]) continue;
                const int d = my_tiles[k] * MM_ROWS + lane;
                double sum = 0.0;
                for (int j = 0; j < a.K; j++) sum += (double)s_w[j] * (double)__ldcg(a.contrib + (size_t)j * a.E + d);
                float o = (float)sum;
                if (a.with_shared) o = __fadd_rn(o, __ldcg(a.contrib + (size_t)a.K * a.E + d));
                a.out[d] = o;
            }
        }
        DT_MARK(5);
    }
    DT_END();
}

DT_EXPORT()

static size_t decode_smem_bytes(int I)
{
    return MM_NS * ((size_t)MM_ROWS * MM_PITCH + 512) + MM_NS * (size_t)I * 4 + MM_CONS * 16 * 4 + 8 * sizeof(uint64_t) + 64;
}

// Needs: the shapes of moe_mma_supported, two stages per gate/up item (so that the last stage is
// idle while the plan is made), the activation terms of the gate/up phase fitting the down
// phase's activation ring, all experts on this GPU, and a device that can launch cooperatively
// with every SM available to this process.
bool moe_decode_supported(const MoeShape &s, int T)
{
    if (!moe_mma_supported(s, T)) return false;
    if (s.NE > 32 * DEC_PER || s.K > 32 || s.K + 1 > MM_MAX_SLOTS) return false;
    if (s.E / MM_CB > MM_NS - 1 || s.I != MM_CB) return false;
    if ((size_t)s.E * 4 > MM_NS * (size_t)s.I * 4) return false;
    if (decode_smem_bytes(s.I) > 226 * 1024) return false;
    // per device: the opt-in to this much shared memory, and whether one CTA per SM is resident
    static SmemGrant grant;
    static int fits[G5B_MAX_DEVICES];                       // 0 not asked yet, 1 yes, -1 no
    const int dev = dev_now();
    if (!dev_cooperative()) return false;
    if (!dev_opt_in_smem((const void *)moe_decode_kernel, decode_smem_bytes(s.I), grant)) return false;
    if (fits[dev] == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, moe_decode_kernel, MM_THREADS, decode_smem_bytes(s.I)) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        fits[dev] = n >= 1 ? 1 : -1;
    }
    return fits[dev] == 1;
}

int moe_decode(cudaStream_t st, float *out, const float *x, const void *gate, int gate_dt, const float *bias,
               const ExpertW *experts, float *score, int *idx, float *w, void *act, float *contrib,
               const MoeShape &s, int with_shared, unsigned long long *sync, unsigned long long *launches,
               int *tile_done, int *err, const DecodeEp *ep)
{
    const int sms = dev_sms();
    DecodeArgs a{experts, x, gate, gate_dt, bias, score, idx, w, static_cast<__half *>(act), contrib, out,
                 s.E, s.I, s.NE, s.K, s.br, s.bc, with_shared, s.norm_topk, s.limit, s.routed_scale,
                 sync, (*launches) * (unsigned long long)sms, tile_done, err,
                 ep ? ep->rank : 0, ep ? ep->size : 1, s.n_local0, s.n_local, ep ? ep->peers : nullptr,
                 ep ? ep->rows_off : 0, ep ? ep->launch : 0ull, ep ? ep->wait_ns : 0ull};
    void *params[] = {&a};
    cudaError_t rc;
    rc = cudaLaunchCooperativeKernel((const void *)moe_decode_kernel, dim3(sms), dim3(MM_THREADS), params,
                                     decode_smem_bytes(s.I), st);
    if (rc != cudaSuccess) { cudaGetLastError(); return -1; }
    ++(*launches);
    ++g_launches;
    return 0;
}

}  // namespace g5b
