// tc_gemm.cu - weight matrices times 8..64 positions at once on the 5th-generation tensor cores:
// y[t][r] = sum_c W[r][c] * x'[t][c], W in its checkpoint format (FP8 E4M3 codes with FP32 scales
// per 128 x 128 block, or BF16), activations FP32, every weight byte read from HBM once.
//
// Reference: glm53f_mm_batch / matmul_f8_batch / matmul_bf16 (src/core/glm53f_ops.c:101-154,
// 378-444), which decode each block of codes once for up to 64 inputs. The one-token kernels of
// this engine re-read the weights for every four positions; this kernel keeps all positions
// resident as the B operand of tcgen05.mma and streams the weights through shared memory once.
//
// Shape of the computation (one CTA per SM, persistent over tiles of 128 weight rows):
//   A operand  = 128 rows of W, K-major, 128-byte swizzled tiles in shared memory, loaded by TMA
//                (cp.async.bulk.tensor, no multicast). BF16 weights are multiplied as stored. FP8
//                codes are turned into F16 (exact: every E4M3 value is an F16 value) by four
//                converter warps on their way from the TMA tile to the MMA tile.
//   B operand  = the activations as exact sums of 16-bit terms: x' = hi + mid / 2048 in F16 (after a
//                per-position power-of-two scaling) against FP8 weights, hi + mid + lo in BF16 against
//                BF16 weights, so that products are exact and only the FP32 accumulation rounds.
//                Term-major rows [term * Tp + t][C] of a buffer in global memory (L2 resident),
//                loaded by TMA chunk by chunk beside the weights.
//   D          = FP32 accumulators in tensor memory: 128 lanes (weight rows) x N columns (terms of
//                the positions). FP8: one accumulator per 128-column block of W, four in flight;
//                the epilogue warps multiply each by the block's scale and add it to a running sum
//                in registers (block scales are scalars per tile: tiles are aligned to the 128-row
//                scale blocks). BF16: one accumulator per 512 columns, two in flight, summed in registers
//                the same way (the tensor cores truncate when they accumulate: after 4096 columns in one
//                accumulator the result is 5e-6 off, in pieces of 512 it is 1e-6).
//
// Warps: 0-3 epilogue (tcgen05.ld needs warp w on lanes 32w..32w+31), 4 TMA producer, 5 MMA issue
// and tensor-memory allocation, 6-9 FP8 -> F16 conversion (FP8 kernel only). All hand-offs are
// mbarriers; every wait is bounded, and a wait that runs out records a code in mapped host memory,
// lets every role drain, frees the tensor memory and returns.
#include <cuda.h>

#include <map>
#include <tuple>

#include "kernels.h"
#include "mma_stage.cuh"

namespace g5b {

constexpr int TC_BM = 128;                 // weight rows per tile = UMMA M
constexpr int TC_ATOM_K = 64;              // 16-bit elements per 128-byte swizzle row
constexpr int TC_ATOM_BYTES = TC_BM * 128; // one A atom: 128 rows x 128 bytes
constexpr int TC_EPI_WARPS = 4;
constexpr int TC_MAX_T = 64;
constexpr int TC_SEG_CHUNKS = 8;            // BF16: 64-column chunks summed inside the tensor cores before the FP32 registers take over

// ------------------------------------------------------------------ PTX wrappers ----
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Eight consecutive FP32 columns of this thread's lane.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8])
{
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile in the canonical 128-byte-swizzled layout: rows
// of 128 bytes, groups of eight rows 1024 bytes apart (the stride field), 16-byte chunks of row r
// stored at chunk ^ (r & 7). The tile base is 1024-byte aligned; a step of 16 elements along K
// inside the row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t tc_smem_desc(const void *p)
{
    const uint64_t addr = (uint64_t)(smem_u32(p) >> 4) & 0x3fffu;
    return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: FP32 accumulation, A and B of format `fmt` (0 F16, 1 BF16), both K-major,
// M = 128, N = n.
__device__ __forceinline__ uint32_t tc_idesc(int fmt, int n)
{
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

// ------------------------------------------------------------- activation terms ----
// Row term * Tp + t of `terms` = term of x'[t], x' = x (or xw * (x * xinv) for a fused RMSNorm).
// FP8 form: F16 terms of x' * 2^e with 2^e chosen per position so that the largest element sits
// near 2^14; inv[t] = 2^-e. Rows of the padding positions T..Tp-1 are zero.
__global__ void __launch_bounds__(256) tc_split_f16_kernel(__half *terms, float *inv, const float *x, int ldx,
                                                           const float *xinv, const float *xw, int C, int T, int Tp)
{
    __shared__ float wmax[8];
    __shared__ float sc;
    const int t = blockIdx.x;
    __half *hi = terms + (size_t)t * C, *mid = terms + ((size_t)Tp + t) * C;
    if (t >= T) {
        for (int c = threadIdx.x; c < C; c += blockDim.x) { hi[c] = __float2half_rn(0.f); mid[c] = __float2half_rn(0.f); }
        return;
    }
    const float *xt = x + (size_t)t * ldx;
    const float rinv = xinv ? xinv[t] : 1.0f;
    auto value = [&](int c) {
        float v = xt[c];
        if (xinv) { v = __fmul_rn(v, rinv); if (xw) v = __fmul_rn(xw[c], v); }
        return v;
    };
    float m = 0.f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) m = fmaxf(m, fabsf(value(c)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.f;
        for (int i = 0; i < 8; i++) mm = fmaxf(mm, wmax[i]);
        int ex = 0;
        if (mm > 0.f && mm < INFINITY) frexpf(mm, &ex);
        sc = ldexpf(1.0f, 14 - ex);
        inv[t] = ldexpf(1.0f, ex - 14);
    }
    __syncthreads();
    const float s = sc;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float v = value(c) * s;
        const __half h = __float2half_rn(v);
        hi[c] = h;
        mid[c] = __float2half_rn((v - __half2float(h)) * 2048.0f);
    }
}

// BF16 form: x' = hi + mid + lo exactly (24 bits), no scaling (BF16 has FP32's exponent range).
__global__ void __launch_bounds__(256) tc_split_bf16_kernel(__nv_bfloat16 *terms, const float *x, int ldx, const float *xinv,
                                                            const float *xw, int C, int T, int Tp)
{
    const int t = blockIdx.x;
    __nv_bfloat16 *r0 = terms + (size_t)t * C, *r1 = terms + ((size_t)Tp + t) * C, *r2 = terms + ((size_t)2 * Tp + t) * C;
    if (t >= T) {
        const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
        for (int c = threadIdx.x; c < C; c += blockDim.x) { r0[c] = z; r1[c] = z; r2[c] = z; }
        return;
    }
    const float *xt = x + (size_t)t * ldx;
    const float rinv = xinv ? xinv[t] : 1.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = xt[c];
        if (xinv) { v = __fmul_rn(v, rinv); if (xw) v = __fmul_rn(xw[c], v); }
        const __nv_bfloat16 hi = __float2bfloat16_rn(v);
        const float e1 = v - __bfloat162float(hi);                  // exact
        const __nv_bfloat16 mid = __float2bfloat16_rn(e1);
        const float e2 = e1 - __bfloat162float(mid);                // exact
        r0[c] = hi; r1[c] = mid; r2[c] = __float2bfloat16_rn(e2);
    }
}

#ifdef G5B_TC_TRACE
__device__ unsigned long long g_tc_trace[8][64];
#define TC_TRACE(role, it) do { if (blockIdx.x == 0 && (it) < 64) g_tc_trace[role][it] = clock64(); } while (0)
extern "C" int g5b_debug_tc_trace(unsigned long long *dst) { return cudaMemcpyFromSymbol(dst, g_tc_trace, sizeof g_tc_trace) == cudaSuccess ? 0 : -1; }
#else
#define TC_TRACE(role, it) do { } while (0)
#endif

// ----------------------------------------------------------------------- kernel ----
struct TcArgs {
    const float *S;        // FP8: block scales [R / 128][scols]
    int scols;
    float *y; int ldy;     // [T][ldy]
    const float *inv;      // FP8: per-position 2^-e of the term scaling
    int R, C, T, Tp, N;    // N = MMA columns: terms * Tp rounded up to 16
    int KS;                // the columns of W are split over KS work items per row tile
    float *part;           // KS > 1: partial results [KS][T][R]
    int *cnt;              // KS > 1: arrivals per row tile, zero between launches
    int a_stages, b_stages;
    int *err;
};

template <bool FP8> struct TcCfg;
template <> struct TcCfg<true> {
    // warps: 0-3 epilogue, 4 TMA producer, 5 MMA, 6-9 converters
    static constexpr int CONV_BUFS = 2, ACCS = 4, THREADS = 10 * 32, TERMS = 2;
};
template <> struct TcCfg<false> {
    // warps: 0-3 epilogue, 4 producer, 5 MMA
    static constexpr int ACCS = 2, THREADS = 6 * 32, TERMS = 3;
};
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_MAX_SPLIT = 8;            // work items a row tile's columns may be split over

// Shared memory, FP8 kernel: raw FP8 tiles [a_stages][16 KB] | converted F16 tiles [2][2 atoms x 16
// KB] | B stages [b_stages][2 atoms x N x 128 B] | barriers. BF16 kernel: stages of (A atom 16 KB | B
// atom N x 128 B) | barriers. Every tile starts on a 1024-byte boundary.
static void tc_stage_plan(bool fp8, int N, int &a_stages, int &b_stages, size_t &bytes)
{
    const size_t budget = 226 * 1024 - 1024 - 1024;          // alignment slack, barriers
    const size_t batom = (size_t)N * 128;
    if (fp8) {
        size_t left = budget - 2 * 2 * 16384;
        // weights come from HBM (about 1.5 us away), activation terms from L2 (about half that): grow
        // the two rings in turns, weights first
        b_stages = 2; a_stages = 3;
        left -= (size_t)b_stages * 2 * batom + (size_t)a_stages * 16384;
        auto grow = [&](int &n, int upto, size_t unit) { while (n < upto && left >= unit) { n++; left -= unit; } };
        grow(a_stages, 4, 16384);
        grow(b_stages, 3, 2 * batom);
        grow(a_stages, 6, 16384);
        grow(b_stages, TC_MAX_STAGES, 2 * batom);
        grow(a_stages, TC_MAX_STAGES, 16384);
        bytes = 1024 + (size_t)a_stages * 16384 + 2 * 2 * 16384 + (size_t)b_stages * 2 * batom + 1024;
    } else {
        const size_t stage = 16384 + ((batom + 1023) & ~(size_t)1023);
        a_stages = (int)(budget / stage);
        if (a_stages > TC_MAX_STAGES) a_stages = TC_MAX_STAGES;
        b_stages = a_stages;
        bytes = 1024 + (size_t)a_stages * stage + 1024;
    }
}

// Partial results of a row tile whose columns were split: the last work item to finish adds them
// in the order of the splits (so the result does not depend on which finished when) and writes y.
// Called by the 128 epilogue threads; acc[t] holds this item's partial sums of row `row`.
__device__ __forceinline__ void tc_finish_tile(const TcArgs &a, int tile, int split, int row, const float (&acc)[TC_MAX_T], int *s_last)
{
    const bool live = tile * TC_BM + row < a.R;                  // rows of a ragged last tile beyond R do not exist
    float *yr = a.y + (size_t)tile * TC_BM + row;
    if (a.KS == 1) {
#pragma unroll
        for (int t = 0; t < TC_MAX_T; t++)
            if (t < a.T && live) yr[(size_t)t * a.ldy] = acc[t];
        return;
    }
    float *pr = a.part + (size_t)split * a.T * a.R + (size_t)tile * TC_BM + row;
#pragma unroll
    for (int t = 0; t < TC_MAX_T; t++)
        if (t < a.T && live) __stcg(pr + (size_t)t * a.R, acc[t]);
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(a.cnt + tile, 1);
        *s_last = prev == a.KS - 1;
        if (prev == a.KS - 1) a.cnt[tile] = 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*s_last && live) {
        __threadfence();
        const float *p0 = a.part + (size_t)tile * TC_BM + row;
        // eight positions at a time, all of their partial sums requested before the first is used
        for (int t0 = 0; t0 < a.T; t0 += 8) {
            float v[8][TC_MAX_SPLIT];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int k = 0; k < TC_MAX_SPLIT; k++)
                    v[i][k] = (k < a.KS && t0 + i < a.T) ? __ldcg(p0 + ((size_t)k * a.T + t0 + i) * a.R) : 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float sum = v[i][0];
#pragma unroll
                for (int k = 1; k < TC_MAX_SPLIT; k++) if (k < a.KS) sum = __fadd_rn(sum, v[i][k]);
                if (t0 + i < a.T) yr[(size_t)(t0 + i) * a.ldy] = sum;
            }
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <bool FP8>
__global__ void __launch_bounds__(TcCfg<FP8>::THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const TcArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_items = ((a.R + TC_BM - 1) / TC_BM) * a.KS;
    const int N = a.N;
    const size_t batom = (size_t)N * 128;
    const int AS = a.a_stages, BS = a.b_stages;
    __shared__ uint32_t s_tmem;
    __shared__ int s_last;
    bool ok = true;
    // the K range of a work item, in units of `unit` columns (FP8: 128-column blocks; BF16: segments
    // of TC_SEG_CHUNKS 64-column chunks)
    auto item_range = [&](int item, int units, int &tile, int &split, int &u0, int &u1) {
        tile = item / a.KS; split = item % a.KS;
        u0 = (int)((long)split * units / a.KS);
        u1 = (int)((long)(split + 1) * units / a.KS);
    };

    if constexpr (FP8) {
        using Cf = TcCfg<true>;
        uint8_t *raw = smem;                                             // [AS][16384]
        uint8_t *conv = raw + (size_t)AS * 16384;                        // [CONV_BUFS][2][16384]
        uint8_t *bst = conv + Cf::CONV_BUFS * 2 * TC_ATOM_BYTES;         // [BS][2][batom]
        uint64_t *bars = reinterpret_cast<uint64_t *>(bst + (size_t)BS * 2 * batom);
        uint64_t *raw_full = bars, *raw_empty = raw_full + TC_MAX_STAGES;
        uint64_t *b_full = raw_empty + TC_MAX_STAGES, *b_empty = b_full + TC_MAX_STAGES;
        uint64_t *a_full = b_empty + TC_MAX_STAGES, *a_empty = a_full + Cf::CONV_BUFS;
        uint64_t *acc_full = a_empty + Cf::CONV_BUFS, *acc_empty = acc_full + Cf::ACCS;
        if (threadIdx.x == 0) {
            for (int i = 0; i < TC_MAX_STAGES; i++) {
                mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4);
                mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1);
            }
            for (int i = 0; i < Cf::CONV_BUFS; i++) { mbar_init(&a_full[i], 4); mbar_init(&a_empty[i], 1); }
            for (int i = 0; i < Cf::ACCS; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], TC_EPI_WARPS); }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        if (warp == 5) tmem_alloc(&s_tmem, 512);
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        const uint32_t tmem = s_tmem;
        const int KB = a.C / 128;                                         // 128-column blocks of W

        if (warp == 4) {
            // --------------------- weights: HBM -> raw FP8 tiles; activation terms: L2 -> B stages ----
            if (lane == 0) {
                long it = 0;
                for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                    int tile, split, kb0, kb1;
                    item_range(item, KB, tile, split, kb0, kb1);
                    for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                        const int rs = (int)(it % AS), bs = (int)(it % BS);
                        if (it >= AS) ok = mbar_wait(&raw_empty[rs], (uint32_t)((it / AS) - 1) & 1, a.err, 31);
                        if (!ok) break;
                        mbar_expect_tx(&raw_full[rs], 16384);
                        tma_load_2d(raw + (size_t)rs * 16384, &mapA, kb * 128, tile * TC_BM, &raw_full[rs]);
                        TC_TRACE(0, it);
                        if (it >= BS) ok = mbar_wait(&b_empty[bs], (uint32_t)((it / BS) - 1) & 1, a.err, 32);
                        if (!ok) break;
                        mbar_expect_tx(&b_full[bs], (uint32_t)(2 * batom));
                        tma_load_2d(bst + (size_t)bs * 2 * batom, &mapB, kb * 128, 0, &b_full[bs]);
                        tma_load_2d(bst + (size_t)bs * 2 * batom + batom, &mapB, kb * 128 + 64, 0, &b_full[bs]);
                        TC_TRACE(1, it);
                    }
                }
                // copies in flight must land before shared memory goes away
                if (!ok) {
                    for (long j = it - 1; j >= 0 && j >= it - AS; j--) mbar_wait(&raw_full[j % AS], (uint32_t)(j / AS) & 1, a.err, 33);
                    for (long j = it - 1; j >= 0 && j >= it - BS; j--) mbar_wait(&b_full[j % BS], (uint32_t)(j / BS) & 1, a.err, 33);
                }
            }
        } else if (warp == 5) {
            // ------------------------------------------------------------------ MMA issue ----
            if (lane == 0) {
                const uint32_t idesc = tc_idesc(0, N);
                long it = 0;
                for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                    int tile, split, kb0, kb1;
                    item_range(item, KB, tile, split, kb0, kb1);
                    for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                        const int aj = (int)(it % Cf::CONV_BUFS), bs = (int)(it % BS), ai = (int)(it % Cf::ACCS);
                        if (it >= Cf::ACCS) ok = mbar_wait(&acc_empty[ai], (uint32_t)((it / Cf::ACCS) - 1) & 1, a.err, 34);
                        if (ok) ok = mbar_wait(&b_full[bs], (uint32_t)(it / BS) & 1, a.err, 36);
                        if (ok) ok = mbar_wait(&a_full[aj], (uint32_t)(it / Cf::CONV_BUFS) & 1, a.err, 35);
                        if (!ok) break;
                        tc_fence_after();
                        TC_TRACE(4, it);
                        const uint32_t d = tmem + (uint32_t)(ai * N);
#pragma unroll
                        for (int atom = 0; atom < 2; atom++) {
                            const uint64_t ad = tc_smem_desc(conv + ((size_t)aj * 2 + atom) * TC_ATOM_BYTES);
                            const uint64_t bd = tc_smem_desc(bst + (size_t)bs * 2 * batom + atom * batom);
#pragma unroll
                            for (int k = 0; k < 4; k++) tc_mma_f16(d, ad + 2 * k, bd + 2 * k, idesc, (atom | k) ? 1u : 0u);
                        }
                        tc_commit(&a_empty[aj]);
                        tc_commit(&b_empty[bs]);
                        tc_commit(&acc_full[ai]);
                    }
                }
            }
        } else if (warp >= 6) {
            // -------------------------------------------------- FP8 codes -> F16, tile by tile ----
            const int r = threadIdx.x - 6 * 32;                          // the row this thread converts
            long it = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tile, split, kb0, kb1;
                item_range(item, KB, tile, split, kb0, kb1);
                for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                    const int rs = (int)(it % AS), aj = (int)(it % Cf::CONV_BUFS);
                    ok = mbar_wait_warp(&raw_full[rs], (uint32_t)(it / AS) & 1, a.err, 37);
                    if (!ok) break;
                    if (threadIdx.x == 6 * 32) TC_TRACE(2, it);
                    const uint8_t *src = raw + (size_t)rs * 16384 + (size_t)r * 128;
                    uint4 w[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) w[c] = *reinterpret_cast<const uint4 *>(src + ((c ^ (r & 7)) << 4));
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[rs]);          // the codes are in registers
                    if (it >= Cf::CONV_BUFS) ok = mbar_wait_warp(&a_empty[aj], (uint32_t)((it / Cf::CONV_BUFS) - 1) & 1, a.err, 38);
                    if (!ok) break;
                    uint8_t *dst = conv + (size_t)aj * 2 * TC_ATOM_BYTES + (size_t)r * 128;
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        uint4 lo, hi;
                        lo.x = e4m3x2_to_f16x2(w[c].x); lo.y = e4m3x2_to_f16x2(w[c].x >> 16);
                        lo.z = e4m3x2_to_f16x2(w[c].y); lo.w = e4m3x2_to_f16x2(w[c].y >> 16);
                        hi.x = e4m3x2_to_f16x2(w[c].z); hi.y = e4m3x2_to_f16x2(w[c].z >> 16);
                        hi.z = e4m3x2_to_f16x2(w[c].w); hi.w = e4m3x2_to_f16x2(w[c].w >> 16);
                        uint8_t *atom = dst + (size_t)(c >> 2) * TC_ATOM_BYTES;
                        const int q = (c & 3) * 2;
                        *reinterpret_cast<uint4 *>(atom + ((q ^ (r & 7)) << 4)) = lo;
                        *reinterpret_cast<uint4 *>(atom + (((q + 1) ^ (r & 7)) << 4)) = hi;
                    }
                    fence_proxy_async();                                 // generic-proxy stores, read by the MMA
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[aj]);
                    if (threadIdx.x == 6 * 32) TC_TRACE(3, it);
                }
            }
        } else {
            // ------------------------------- epilogue: scale each block's product, sum, store ----
            const int row = warp * 32 + lane;                            // lane of tensor memory = row of the tile
            const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
            long it = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tile, split, kb0, kb1;
                item_range(item, KB, tile, split, kb0, kb1);
                float acc[TC_MAX_T];
#pragma unroll
                for (int i = 0; i < TC_MAX_T; i++) acc[i] = 0.f;
                const float *srow = a.S + (size_t)tile * a.scols;
                for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                    const int ai = (int)(it % Cf::ACCS);
                    const float sv = __ldg(srow + kb);
                    ok = mbar_wait_warp(&acc_full[ai], (uint32_t)(it / Cf::ACCS) & 1, a.err, 39);
                    if (!ok) break;
                    tc_fence_after();
                    if (threadIdx.x == 0) TC_TRACE(5, it);
                    const uint32_t base = lane_addr + (uint32_t)(ai * N);
#pragma unroll
                    for (int g = 0; g < TC_MAX_T / 8; g++) {
                        if (g * 8 < a.Tp) {
                            float hi[8], mid[8];
                            tmem_ld8(base + g * 8, hi);
                            tmem_ld8(base + a.Tp + g * 8, mid);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 8; i++) acc[g * 8 + i] = fmaf(hi[i] + mid[i] * (1.0f / 2048.0f), sv, acc[g * 8 + i]);
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ai]);
                    if (threadIdx.x == 0) TC_TRACE(6, it);
                }
                if (!ok) break;
#pragma unroll
                for (int t = 0; t < TC_MAX_T; t++) acc[t] *= (t < a.T ? __ldg(a.inv + t) : 0.f);
                tc_finish_tile(a, tile, split, row, acc, &s_last);
            }
        }
        tc_fence_before();
        __syncthreads();
        if (warp == 5) { __syncwarp(); tmem_dealloc(tmem, 512); }
    } else {
        using Cf = TcCfg<false>;
        const size_t bpad = (batom + 1023) & ~(size_t)1023;
        const size_t stage = 16384 + bpad;
        uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)AS * stage);
        uint64_t *full = bars, *empty = full + TC_MAX_STAGES, *acc_full = empty + TC_MAX_STAGES, *acc_empty = acc_full + Cf::ACCS;
        if (threadIdx.x == 0) {
            for (int i = 0; i < TC_MAX_STAGES; i++) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
            for (int i = 0; i < Cf::ACCS; i++) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], TC_EPI_WARPS); }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        if (warp == 5) tmem_alloc(&s_tmem, 512);
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        const uint32_t tmem = s_tmem;
        const int KC = a.C / TC_ATOM_K;                                   // 64-column chunks of W
        const int SEGS = (KC + TC_SEG_CHUNKS - 1) / TC_SEG_CHUNKS;        // segments: one accumulator each
        const int acc_cols = 256;                                         // columns between the two accumulators (N <= 192)

        if (warp == 4) {
            if (lane == 0) {
                long it = 0;
                for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                    int tile, split, sg0, sg1;
                    item_range(item, SEGS, tile, split, sg0, sg1);
                    const int kc1 = sg1 * TC_SEG_CHUNKS < KC ? sg1 * TC_SEG_CHUNKS : KC;
                    for (int kc = sg0 * TC_SEG_CHUNKS; kc < kc1 && ok; kc++, it++) {
                        const int s = (int)(it % AS);
                        if (it >= AS) ok = mbar_wait(&empty[s], (uint32_t)((it / AS) - 1) & 1, a.err, 41);
                        if (!ok) break;
                        mbar_expect_tx(&full[s], (uint32_t)(16384 + batom));
                        tma_load_2d(smem + (size_t)s * stage, &mapA, kc * TC_ATOM_K, tile * TC_BM, &full[s]);
                        tma_load_2d(smem + (size_t)s * stage + 16384, &mapB, kc * TC_ATOM_K, 0, &full[s]);
                    }
                }
                if (!ok) for (long j = it - 1; j >= 0 && j >= it - AS; j--) mbar_wait(&full[j % AS], (uint32_t)(j / AS) & 1, a.err, 43);
            }
        } else if (warp == 5) {
            if (lane == 0) {
                const uint32_t idesc = tc_idesc(1, N);
                long it = 0, scount = 0;
                for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                    int tile, split, sg0, sg1;
                    item_range(item, SEGS, tile, split, sg0, sg1);
                    for (int sg = sg0; sg < sg1 && ok; sg++, scount++) {
                        const int ab = (int)(scount % Cf::ACCS);
                        if (scount >= Cf::ACCS) ok = mbar_wait(&acc_empty[ab], (uint32_t)((scount / Cf::ACCS) - 1) & 1, a.err, 44);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t d = tmem + (uint32_t)(ab * acc_cols);
                        const int kc0 = sg * TC_SEG_CHUNKS, kc1 = kc0 + TC_SEG_CHUNKS < KC ? kc0 + TC_SEG_CHUNKS : KC;
                        for (int kc = kc0; kc < kc1 && ok; kc++, it++) {
                            const int s = (int)(it % AS);
                            ok = mbar_wait(&full[s], (uint32_t)(it / AS) & 1, a.err, 45);
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t ad = tc_smem_desc(smem + (size_t)s * stage);
                            const uint64_t bd = tc_smem_desc(smem + (size_t)s * stage + 16384);
#pragma unroll
                            for (int k = 0; k < 4; k++) tc_mma_f16(d, ad + 2 * k, bd + 2 * k, idesc, ((kc - kc0) | k) ? 1u : 0u);
                            tc_commit(&empty[s]);
                        }
                        if (ok) tc_commit(&acc_full[ab]);
                    }
                }
            }
        } else if (warp < TC_EPI_WARPS) {
            const int row = warp * 32 + lane;
            const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
            long scount = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int tile, split, sg0, sg1;
                item_range(item, SEGS, tile, split, sg0, sg1);
                float acc[TC_MAX_T];
#pragma unroll
                for (int i = 0; i < TC_MAX_T; i++) acc[i] = 0.f;
                for (int sg = sg0; sg < sg1 && ok; sg++, scount++) {
                    const int ab = (int)(scount % Cf::ACCS);
                    ok = mbar_wait_warp(&acc_full[ab], (uint32_t)(scount / Cf::ACCS) & 1, a.err, 46);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = lane_addr + (uint32_t)(ab * acc_cols);
#pragma unroll
                    for (int g = 0; g < TC_MAX_T / 8; g++) {
                        if (g * 8 < a.Tp) {
                            float h[8], m[8], l[8];
                            tmem_ld8(base + g * 8, h);
                            tmem_ld8(base + a.Tp + g * 8, m);
                            tmem_ld8(base + 2 * a.Tp + g * 8, l);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 8; i++) acc[g * 8 + i] = __fadd_rn(acc[g * 8 + i], __fadd_rn(__fadd_rn(h[i], m[i]), l[i]));
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ab]);
                }
                if (!ok) break;
                tc_finish_tile(a, tile, split, row, acc, &s_last);
            }
        }
        tc_fence_before();
        __syncthreads();
        if (warp == 5) { __syncwarp(); tmem_dealloc(tmem, 512); }
    }
}

// ------------------------------------------------------------------------- host ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

// A [rows][cols] row-major matrix of `elt`-byte elements, copied in boxes of box_rows x 128 bytes
// with the 128-byte swizzle. Rows past `rows` read as zero.
static bool make_map(CUtensorMap *m, const void *base, CUtensorMapDataType dt, int elt, size_t rows, size_t cols, int box_rows,
                     size_t pitch = 0)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)(pitch ? pitch : cols) * elt};
    const cuuint32_t box[2] = {(cuuint32_t)(128 / elt), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(m, dt, 2, const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct TcGemm {
    void *terms = nullptr;          // [3 * 64][max_c] 16-bit
    float *inv = nullptr;           // [64]
    int max_c = 0;
    // what the terms buffer holds (several matrices share one input)
    const float *x = nullptr, *xinv = nullptr, *xw = nullptr;
    int ldx = 0, C = 0, T = 0, kind = -1;
    std::map<std::tuple<const void *, int, int, int, int>, CUtensorMap> amaps;   // weights by (pointer, rows, cols, pitch, dt)
    SmemGrant grant_fp8, grant_bf16;
    float *part = nullptr;          // split-K partial results [TC_MAX_SPLIT][64][part_rows]
    int *cnt = nullptr;             // arrivals per row tile
    int *err = nullptr;
};
constexpr int TC_PART_ROWS = 16384;

TcGemm *tc_gemm_create(int max_c, int *err)
{
    if (!encode_fn()) return nullptr;
    TcGemm *g = new TcGemm;
    g->max_c = max_c; g->err = err;
    if (cudaMalloc(&g->terms, (size_t)3 * TC_MAX_T * max_c * 2) != cudaSuccess || cudaMalloc((void **)&g->inv, TC_MAX_T * 4) != cudaSuccess ||
        cudaMalloc((void **)&g->part, (size_t)TC_MAX_SPLIT * TC_MAX_T * TC_PART_ROWS * 4) != cudaSuccess ||
        cudaMalloc((void **)&g->cnt, (TC_PART_ROWS / TC_BM) * 4) != cudaSuccess) {
        cudaGetLastError();
        tc_gemm_free(g);
        return nullptr;
    }
    cudaMemset(g->terms, 0, (size_t)3 * TC_MAX_T * max_c * 2);
    cudaMemset(g->cnt, 0, (TC_PART_ROWS / TC_BM) * 4);
    return g;
}

void tc_gemm_free(TcGemm *g)
{
    if (!g) return;
    if (g->terms) cudaFree(g->terms);
    if (g->inv) cudaFree(g->inv);
    if (g->part) cudaFree(g->part);
    if (g->cnt) cudaFree(g->cnt);
    delete g;
}

void tc_gemm_new_input(TcGemm *g) { if (g) g->x = nullptr; }

bool tc_gemm_takes(const TcGemm *g, const GemvSeg &s, int T)
{
    // (the last row tile may be ragged: rows beyond R are filled with zeros by the copy and never stored)
    if (!g || T < 8 || T > TC_MAX_T || s.C > g->max_c || s.R < 16) return false;
    if (s.dt == DT_FP8 && s.R % TC_BM) return false;
    if ((reinterpret_cast<uintptr_t>(s.W) & 15) || (((size_t)s.ldw * (s.dt == DT_FP8 ? 1 : 2)) & 15)) return false;
    if (s.dt == DT_FP8) return s.C % 128 == 0 && s.br == 128 && s.bc == 128 && s.S != nullptr;
    if (s.dt == DT_BF16) return s.C % TC_ATOM_K == 0;
    return false;
}

int tc_gemm_run(TcGemm *g, cudaStream_t st, const GemvSeg &s, int T)
{
    const bool fp8 = s.dt == DT_FP8;
    const int terms = fp8 ? 2 : 3;
    const int Tp = (T + 7) & ~7;
    const int N = (terms * Tp + 15) & ~15;
    if (g->x != s.x || g->xinv != s.xinv || g->xw != s.xw || g->ldx != s.ldx || g->C != s.C || g->T != T || g->kind != (int)fp8) {
        if (fp8) G5B_LAUNCH(tc_split_f16_kernel, Tp, 256, 0, st, static_cast<__half *>(g->terms), g->inv, s.x, s.ldx, s.xinv, s.xw, s.C, T, Tp);
        else     G5B_LAUNCH(tc_split_bf16_kernel, Tp, 256, 0, st, static_cast<__nv_bfloat16 *>(g->terms), s.x, s.ldx, s.xinv, s.xw, s.C, T, Tp);
        g->x = s.x; g->xinv = s.xinv; g->xw = s.xw; g->ldx = s.ldx; g->C = s.C; g->T = T; g->kind = (int)fp8;
    }
    const auto key = std::make_tuple(s.W, s.R, s.C, s.ldw, s.dt);
    auto it = g->amaps.find(key);
    if (it == g->amaps.end()) {
        CUtensorMap m;
        if (!make_map(&m, s.W, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, fp8 ? 1 : 2, (size_t)s.R, (size_t)s.C, TC_BM, (size_t)s.ldw))
            return -1;
        it = g->amaps.emplace(key, m).first;
    }
    CUtensorMap mb;
    if (!make_map(&mb, g->terms, fp8 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (size_t)terms * Tp, (size_t)s.C, N))
        return -1;
    // Fewer row tiles than SMs: split the columns over several work items per tile. The split is chosen
    // by a small model of the launch in microseconds: waves x (pipeline fill + the item's share of the
    // K units) + what the partial results cost (a fixed part and a pass per split). Units: a 128-column
    // block of an FP8 matrix, a 512-column segment of a BF16 one. (With more than half of the SMs busy
    // anyway a split measured no gain: 12288 x 4096 FP8 at 64 positions 91 us whole, 95 us in three.)
    const int tiles = (s.R + TC_BM - 1) / TC_BM, sms = dev_sms();
    const int units = fp8 ? s.C / 128 : (s.C / TC_ATOM_K + TC_SEG_CHUNKS - 1) / TC_SEG_CHUNKS;
    int KS = 1;
    if (2 * tiles <= sms && s.R <= TC_PART_ROWS) {
        const double fill = 3.0, unit = fp8 ? 1.5 : 3.0;
        double best = 1e30;
        for (int k = 1; k <= TC_MAX_SPLIT && k <= units; k++) {
            const int items = tiles * k, waves = (items + sms - 1) / sms;
            const double t = waves * (fill + unit * ((units + k - 1) / k)) + (k > 1 ? 2.0 + 0.5 * k : 0.0);
            if (t < best - 1e-9) { best = t; KS = k; }
        }
    }
    int a_stages, b_stages;
    size_t smem;
    tc_stage_plan(fp8, N, a_stages, b_stages, smem);
    TcArgs a{s.S, s.scols, s.y, s.ldy, g->inv, s.R, s.C, T, Tp, N, KS, g->part, g->cnt, a_stages, b_stages, g->err};
    const int items = tiles * KS;
    const int grid = items < sms ? items : sms;
    if (fp8) {
        if (!dev_opt_in_smem((const void *)tc_gemm_kernel<true>, smem, g->grant_fp8)) return -1;
        tc_gemm_kernel<true><<<grid, TcCfg<true>::THREADS, smem, st>>>(it->second, mb, a);
    } else {
        if (!dev_opt_in_smem((const void *)tc_gemm_kernel<false>, smem, g->grant_bf16)) return -1;
        tc_gemm_kernel<false><<<grid, TcCfg<false>::THREADS, smem, st>>>(it->second, mb, a);
    }
    ++g_launches;
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

// ------------------------------------------------------------ instruction-rate probe ----
// What one tcgen05.mma costs when nothing else uses the SM: one thread issues `reps` groups of four
// instructions (the four K steps of a 128-byte swizzle row) on shared-memory tiles that never
// change, M = 128, N as given, rotating over `accs` accumulators; then one commit and a bounded
// wait. out[0] = cycles until the last instruction was issued, out[1] = until all had completed, of
// CTA 0. The design of tc_gemm_kernel rests on these figures (an instruction costs what its 128-row
// A operand costs, whatever N is).
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

__global__ void __launch_bounds__(64) tc_mma_rate_kernel(int N, int reps, int accs, int fp8, long long *out, int *err)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ __align__(8) uint64_t bar;
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *A = base, *B = base + TC_ATOM_BYTES;                  // A: 128 rows x 128 B; B: up to 256 rows x 128 B
    for (int i = threadIdx.x; i < (TC_ATOM_BYTES + 256 * 128) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(base)[i] = fp8 ? 0x38383838u : 0x3c003c00u;      // ones
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    __syncthreads();
    if (threadIdx.x < 32) tmem_alloc(&s_tmem, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s_tmem;
    if (threadIdx.x == 32) {
        const uint32_t idesc = tc_idesc(0, N);                     // format code 0: F16, or E4M3 for the 8-bit kind
        const uint64_t ad = tc_smem_desc(A), bd = tc_smem_desc(B);
        const long long t0 = clock64();
        for (int r = 0; r < reps; r++) {
            const uint32_t d = tm + (uint32_t)((r % accs) * N);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (fp8) tc_mma_f8(d, ad + 2 * k, bd + 2 * k, idesc, (r >= accs || k) ? 1u : 0u);
                else     tc_mma_f16(d, ad + 2 * k, bd + 2 * k, idesc, (r >= accs || k) ? 1u : 0u);
            }
        }
        const long long t1 = clock64();
        tc_commit(&bar);
        const bool ok = mbar_wait(&bar, 0, err, 61);               // bounded; a wait that runs out records code 61
        const long long t2 = clock64();
        if (blockIdx.x == 0 && ok) { out[0] = t1 - t0; out[1] = t2 - t0; }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tm, 512);
}

}  // namespace g5b

// Cycles per tcgen05.mma (M = 128; K = 16 for kind::f16, 32 for kind::f8f6f4) with `ctas` CTAs
// running: cycles[0] until issued, cycles[1] until complete. Measurement aid, no counterpart in
// the reference.
extern "C" int g5b_debug_mma_rate(int n, int fp8, int accs, int ctas, int reps, double *cycles)
{
    using namespace g5b;
    if (n < 16 || n > 256 || (n & 15) || accs < 1 || accs * n > 512 || ctas < 1 || reps < 1) return -1;
    long long *out = nullptr;
    int *err = nullptr;
    if (cudaMalloc((void **)&out, 16) != cudaSuccess || cudaMalloc((void **)&err, 4) != cudaSuccess) { cudaFree(out); return -1; }
    cudaMemset(out, 0, 16); cudaMemset(err, 0, 4);
    const size_t smem = TC_ATOM_BYTES + 256 * 128 + 1024;
    static SmemGrant grant;
    int rc = -1;
    if (dev_opt_in_smem((const void *)tc_mma_rate_kernel, smem, grant)) {
        tc_mma_rate_kernel<<<ctas, 64, smem>>>(n, reps, accs, fp8, out, err);
        long long h[2] = {0, 0};
        int e = 0;
        if (cudaDeviceSynchronize() == cudaSuccess && cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost) == cudaSuccess &&
            cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost) == cudaSuccess && e == 0) {
            cycles[0] = (double)h[0] / (4.0 * reps);
            cycles[1] = (double)h[1] / (4.0 * reps);
            rc = 0;
        }
    }
    cudaFree(out); cudaFree(err);
    return rc;
}
