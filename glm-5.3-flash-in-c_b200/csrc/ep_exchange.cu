// ep_exchange.cu - the exchange step of an expert-parallel MoE layer, fused with the combine.
//
// Every rank (one process per GPU) holds the replicated activations and 1/ep_size of the routed
// experts, routes every token itself (same inputs, same picks on every rank) and computes the
// contribution rows of the picks whose experts it owns. This kernel then
//   1. stores each of those rows into the exchange buffer of EVERY rank (its own included) with
//      plain 16-byte stores over NVLink peer mappings - an all-gather of contribution rows with no
//      library call and no staging copy,
//   2. publishes "rank r has delivered step s" as one 64-bit word in every rank's flag array
//      (system-scope fence, then the store, by the last CTA to finish its rows),
//   3. waits - bounded - until every rank's word for this step has arrived here, and
//   4. combines: out[t][d] = (float) sum_j w[t][j] * row[t*K+j][d] in FP64 in top-k order, plus the
//      shared expert's row (computed on every rank) in FP32: the arithmetic of the one-GPU combine
//      and of the reference (src/core/glm53f_ops.c:1329-1340), so the result does not depend on
//      the number of ranks.
//
// Two exchange buffers alternate by step parity: a rank can be at most one step ahead of a peer
// (its next combine needs that peer's next word), so rows of step s+1 never land in a buffer
// that a slower peer still reads for step s. The wait is limited in wall-clock time (engine option
// "ep_wait_ms", default 5 s): a wait that runs out sets the error word in mapped host memory and
// the CTA returns without combining; nothing is left in flight. After such a failure the ranks
// no longer agree on the step number (this rank counted the step, a slower peer may still
// complete it), so the group must be re-aligned with g5b_engine_ep_resync before its next step.
#include "kernels.h"
#include "common.cuh"

namespace g5b {

__global__ void __launch_bounds__(256) ep_exchange_combine_kernel(const EpExchange a)
{
    __shared__ int s_flag;                                      // this CTA finished last
    const int tid = threadIdx.x;
    const size_t row_f4 = (size_t)a.E / 4;
    const int routed_rows = a.T * a.K;
    const int ns = *a.plan.n_slots;
    const int total = ns > 0 ? a.plan.slot_off[ns - 1] + a.plan.slot_cnt[ns - 1] : 0;

    // ---- 1. deliver this rank's rows to every rank
    for (int p = blockIdx.x; p < total; p += gridDim.x) {
        const int row = a.plan.pair_dst[p];
        if (row >= routed_rows) continue;                       // the shared expert's rows stay local
        const float4 *src = reinterpret_cast<const float4 *>(a.contrib + (size_t)row * a.E);
        for (int r = 0; r < a.size; r++) {
            float4 *dst = reinterpret_cast<float4 *>(static_cast<uint8_t *>(a.peers[r]) + a.rows_off) + (size_t)row * row_f4;
            for (size_t i = tid; i < row_f4; i += blockDim.x) dst[i] = src[i];
        }
    }
    // ---- 2. the last CTA to finish publishes this rank's word on every rank
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(a.arrive, 1);
        s_flag = prev == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (s_flag) {
        if (tid == 0) *a.arrive = 0;
        __threadfence_system();
        if (tid < a.size) {
            unsigned long long *flags = reinterpret_cast<unsigned long long *>(a.peers[tid]);
            st_release_sys(flags + a.rank, a.step);
        }
    }
    // ---- 3. wait for every rank's word (bounded); thread r watches rank r
    bool seen = true;
    if (tid < a.size) {
        const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(a.peers[a.rank]);
        seen = wait_word_sys(mine + tid, a.step, a.wait_ns);
        if (!seen) atomicExch(a.err, 20 + tid);                 // which rank never delivered
    }
    if (!__syncthreads_and(seen)) return;
    // ---- 4. combine from the local exchange buffer
    const float *rows = reinterpret_cast<const float *>(static_cast<const uint8_t *>(a.peers[a.rank]) + a.rows_off);
    const size_t n = (size_t)a.T * a.E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / a.E), d = (int)(i % a.E);
        double s = 0.0;
        for (int j = 0; j < a.K; j++)
            s += (double)a.w[(size_t)t * a.K + j] * (double)__ldcg(rows + ((size_t)t * a.K + j) * a.E + d);
        float o = (float)s;
        if (a.with_shared) o = __fadd_rn(o, a.contrib[((size_t)routed_rows + t) * a.E + d]);
        a.out[(size_t)t * a.ldo + d] = o;
    }
}

// The all-reduce of a column-split trunk product (TsReduce, kernels.h). CTA b owns the float4s
// b, b + gridDim.x, ... of the [T][E] block: it stores them into slot `rank` of every rank's buffer,
// counts itself done on every rank (release-add, covering the CTA's stores through the barrier
// before it), waits for every rank's counter to reach launch x CTAs and adds the slots of its own
// float4s in rank order. All ranks run the same grid.
constexpr int TS_CTAS = 8, TS_GATHER_CTAS = 32;
__global__ void __launch_bounds__(256) ts_allreduce_kernel(const TsReduce a)
{
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    const size_t n4 = (size_t)a.T * a.E / 4, row4 = (size_t)a.E / 4, slot4 = (size_t)a.max_t * row4;
    const float4 *src = reinterpret_cast<const float4 *>(a.partial);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = src[i];
        for (int r = 0; r < a.size; r++)
            (reinterpret_cast<float4 *>(static_cast<uint8_t *>(a.peers[r]) + a.area_off) + (size_t)a.rank * slot4)[i] = v;
    }
    __syncthreads();
    if (tid < a.size) red_release_sys_add(reinterpret_cast<unsigned long long *>(a.peers[tid]) + a.cnt0 + a.rank, 1ull);
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < a.size) {
        const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(a.peers[a.rank]) + a.cnt0 + tid;
        if (!wait_word_sys(mine, a.launch * gridDim.x, a.wait_ns)) { atomicExch(a.err, 40 + tid); s_ok = 0; }
    }
    __syncthreads();
    if (!s_ok || a.gather_only) return;
    const float4 *slots = reinterpret_cast<const float4 *>(static_cast<const uint8_t *>(a.peers[a.rank]) + a.area_off);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 s = __ldcg(slots + i);
        for (int r = 1; r < a.size; r++) {
            const float4 v = __ldcg(slots + (size_t)r * slot4 + i);
            s.x = __fadd_rn(s.x, v.x); s.y = __fadd_rn(s.y, v.y); s.z = __fadd_rn(s.z, v.z); s.w = __fadd_rn(s.w, v.w);
        }
        const size_t t = i / row4, c = (i % row4) * 4;
        *reinterpret_cast<float4 *>(a.out + t * a.ldo + c) = s;
    }
}

// The exchange of a MoE layer with the sequences split over the ranks (SeqExchange, kernels.h).
__global__ void __launch_bounds__(256) seq_exchange_kernel(const SeqExchange a)
{
    __shared__ int s_flag;
    const int tid = threadIdx.x;
    const size_t row_f4 = (size_t)a.E / 4;
    const int routed_rows = a.m * a.K;
    const int ns = *a.plan.n_slots;
    const int total = ns > 0 ? a.plan.slot_off[ns - 1] + a.plan.slot_cnt[ns - 1] : 0;

    // ---- 1. every routed row goes to the rank its token lives on
    for (int p = blockIdx.x; p < total; p += gridDim.x) {
        const int row = a.plan.pair_dst[p];
        if (row >= routed_rows) continue;                       // the shared expert's rows stay local
        const int g = a.g0 + row / a.K, pick = row % a.K;
        const int home = g / a.n, lt = g % a.n;
        const float4 *src = reinterpret_cast<const float4 *>(a.contrib + (size_t)row * a.E);
        float4 *dst = reinterpret_cast<float4 *>(static_cast<uint8_t *>(a.peers[home]) + a.rows_off) + ((size_t)lt * a.K + pick) * row_f4;
        for (size_t i = tid; i < row_f4; i += blockDim.x) dst[i] = src[i];
    }
    if (!a.finish) return;
    // ---- 2. the last CTA to finish publishes this rank's word on every rank; the release is
    // cumulative, so it covers the rows that the earlier groups' launches of this call delivered
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(a.arrive, 1);
        s_flag = prev == (int)gridDim.x - 1;
    }
    __syncthreads();
    if (s_flag) {
        if (tid == 0) *a.arrive = 0;
        __threadfence_system();
        if (tid < a.size) st_release_sys(reinterpret_cast<unsigned long long *>(a.peers[tid]) + a.rank, a.step);
    }
    // ---- 3. wait for every rank's word
    bool seen = true;
    if (tid < a.size) {
        const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(a.peers[a.rank]);
        seen = wait_word_sys(mine + tid, a.step, a.wait_ns);
        if (!seen) atomicExch(a.err, 20 + tid);
    }
    if (!__syncthreads_and(seen)) return;
    // ---- 4. combine the own tokens from the local exchange buffer (the one-GPU arithmetic)
    const float *rows = reinterpret_cast<const float *>(static_cast<const uint8_t *>(a.peers[a.rank]) + a.rows_off);
    const int own0 = a.rank * a.n - a.g0;                       // first own token inside the group
    const size_t n = (size_t)a.n * a.E;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / a.E), d = (int)(i % a.E);
        double s = 0.0;
        for (int j = 0; j < a.K; j++)
            s += (double)a.w[(size_t)(own0 + t) * a.K + j] * (double)__ldcg(rows + ((size_t)t * a.K + j) * a.E + d);
        float o = (float)s;
        if (a.with_shared) o = __fadd_rn(o, a.contrib[((size_t)routed_rows + own0 + t) * a.E + d]);
        a.out[(size_t)t * a.ldo + d] = o;
    }
}

void seq_exchange(cudaStream_t st, const SeqExchange &a, int ctas)
{
    G5B_LAUNCH(seq_exchange_kernel, dim3(ctas), 256, 0, st, a);
}

// (value, index) of every rank's best vocabulary row, exchanged and reduced to the first maximum in
// index order (HeadPick, kernels.h). One warp; lane r serves rank r.
__global__ void __launch_bounds__(32) head_pick_kernel(const HeadPick a)
{
    const int lane = threadIdx.x;
    const int parity = (int)(a.launch & 1ull);
    const int li = a.local_idx[0];
    const float v = a.logits[li];
    const unsigned long long word_v = (unsigned long long)__float_as_uint(v), word_i = (unsigned long long)(a.row0 + li);
    if (lane < a.size) {
        unsigned long long *base = reinterpret_cast<unsigned long long *>(a.peers[lane]) + a.word0;
        unsigned long long *slot = base + ((size_t)parity * 8 + a.rank) * 2;
        slot[0] = word_v; slot[1] = word_i;
        __threadfence_system();
        red_release_sys_add(base + 32 + a.rank, 1ull);
    }
    bool seen = true;
    const unsigned long long *mine = reinterpret_cast<const unsigned long long *>(a.peers[a.rank]) + a.word0;
    if (lane < a.size) {
        seen = wait_word_sys(mine + 32 + lane, a.launch, a.wait_ns);
        if (!seen) atomicExch(a.err, 50 + lane);
    }
    if (!__all_sync(0xffffffffu, seen)) return;
    if (lane == 0) {
        float best = 0.f; int bi = -1;
        for (int r = 0; r < a.size; r++) {                      // rank order = index order; strict > keeps the first maximum
            const unsigned long long *slot = mine + ((size_t)parity * 8 + r) * 2;
            const float vr = __uint_as_float((unsigned)ld_acquire_sys(slot));
            const int ir = (int)ld_acquire_sys(slot + 1);
            if (bi < 0 || vr > best) { best = vr; bi = ir; }
        }
        a.local_idx[0] = bi;
    }
}

void head_pick_exchange(cudaStream_t st, const HeadPick &a)
{
    G5B_LAUNCH(head_pick_kernel, 1, 32, 0, st, a);
}

// Every launch of a group must use the same grid: the arrival counters count launches x CTAs.
void ts_allreduce(cudaStream_t st, const TsReduce &a)
{
    G5B_LAUNCH(ts_allreduce_kernel, a.gather_only ? TS_GATHER_CTAS : TS_CTAS, 256, 0, st, a);
}

void ep_exchange_combine(cudaStream_t st, const EpExchange &a, int ctas)
{
    G5B_LAUNCH(ep_exchange_combine_kernel, dim3(ctas), 256, 0, st, a);
}

}  // namespace g5b
