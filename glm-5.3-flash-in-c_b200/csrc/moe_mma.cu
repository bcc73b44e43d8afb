// moe_mma.cu - batch-1 expert kernels: FP8 weights streamed by the bulk-copy engine and multiplied
// by the tensor cores straight from their E4M3 codes.
//
// Why tensor cores for a matrix-VECTOR product: with CUDA-core arithmetic every weight byte costs
// about four issued instructions (two conversions E4M3 -> F16 -> F32, an FMA, and its share of the
// loads); ncu showed the streamed CUDA-core kernel at 51 % issue utilisation at only 51 % of DRAM
// throughput, i.e. issue-bound below the HBM roofline. Here a byte costs about one instruction:
// a pair of codes becomes an F16 pair with ONE conversion, and mma.sync.m16n8k16 does the
// multiplies and the FP32 accumulation. The product stays a GEMV: the B operand holds the single
// activation vector, split EXACTLY into two F16 terms (x * 2^k = hi + 2^-11 mid, 22 significant
// bits), one term per B column; the other six columns are zero. Products of a 4-bit E4M3
// significand and an 11-bit F16 significand are exact in the tensor core, sums are FP32.
//
// Stage = 32 weight rows x 2048 columns (rows 64 bytes apart beyond their length so that the
// eight row groups of a warp read shared memory without bank conflicts). Eight consumer warps:
// warp = (M tile of 16 rows) x (quarter of the stage's columns); the four column quarters of a
// row are added at the end of a work item in a fixed order. Block scales are applied every 128
// columns in FP32, as the reference factors its FP8 product (src/core/glm53f_ops.c:185-228).
#include "kernels.h"
#include "mma_stage.cuh"

namespace g5b {

struct MmaArgs {
    const ExpertW *experts;
    MoePlan p;
    const void *x;         // gate/up: float [E]; down: F16 terms [pairs][2][I]
    void *y;               // gate/up: F16 terms [pairs][2][I]; down: contributions float [K(+1)][E]
    int E, I, br, bc;
    float limit;
    float *out;            // down: combined layer output, or nullptr
    const float *w;
    int K, with_shared;
    int *tile_done;
    int *err;
};

template <bool GATEUP>
__global__ void __launch_bounds__(MM_THREADS, 1) moe_mma_kernel(const MmaArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int C = GATEUP ? a.E : a.I;
    const int rows_total = GATEUP ? a.I : a.E;
    const float act_sc = act_term_scale(a.limit), act_inv = 1.0f / act_sc;   // powers of two
    const int KH = C / MM_CB;
    const int scols = C / a.bc;
    const int rows_per_item = GATEUP ? MM_ROWS / 2 : MM_ROWS;
    const int tps = rows_total / rows_per_item;
    // stage: weights [32][PITCH] | two scale rows (64 floats each) | down: activation terms [2][I] F16
    const size_t scale_off = (size_t)MM_ROWS * MM_PITCH;
    const size_t act_off = scale_off + 512;
    const size_t stage_bytes = act_off + (GATEUP ? 0 : (size_t)a.I * 4);
    uint8_t *stages = smem;
    uint8_t *tail = smem + MM_NS * stage_bytes;
    __half *x_h = reinterpret_cast<__half *>(tail);                       // gate/up: [2][E]
    float *red = reinterpret_cast<float *>(tail + (GATEUP ? (size_t)a.E * 4 : 0));   // [8][16]
    uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(red) + MM_CONS * 16 * 4);
    uint64_t *empty = full + MM_NS;
    __shared__ int my_tiles[MM_MAX_ITEMS], my_last[MM_MAX_ITEMS];
    __shared__ ExpertW s_ew[MM_MAX_SLOTS];
    __shared__ int s_pair[MM_MAX_SLOTS], s_dst[MM_MAX_SLOTS], s_nslots;
    __shared__ float wmax[MM_THREADS / 32];
    __shared__ float x_scale[2];                                          // scale, 1/scale

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < MM_NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], MM_CONS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // The plan and the expert pointer table are read ONCE per CTA into shared memory: they sit
    // behind two dependent loads, which per work item would stall the producer for microseconds.
    if (warp == 0) {
        int n = *a.p.n_slots;
        n = n < 0 ? 0 : (n > MM_MAX_SLOTS ? MM_MAX_SLOTS : n);
        for (int i = lane; i < n; i += 32) {
            const int off = a.p.slot_off[i];
            s_ew[i] = a.experts[a.p.slot_expert[i]];
            s_pair[i] = off;
            s_dst[i] = a.p.pair_dst[off];
        }
        if (lane == 0) s_nslots = n;
    }
    if (GATEUP) {
        // scale the activation by a power of two so that its largest element sits near 2^14, then
        // split every element into two F16 terms
        const float *x = static_cast<const float *>(a.x);
        float m = 0.f;
        for (int c = threadIdx.x; c < a.E; c += MM_THREADS) m = fmaxf(m, fabsf(x[c]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) wmax[warp] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            float mm = 0.f;
            for (int i = 0; i < MM_THREADS / 32; i++) mm = fmaxf(mm, wmax[i]);
            int ex = 0;
            if (mm > 0.f && mm < INFINITY) frexpf(mm, &ex);
            x_scale[0] = ldexpf(1.0f, 14 - ex);
            x_scale[1] = ldexpf(1.0f, ex - 14);
        }
        __syncthreads();
        const float sc = x_scale[0];
        for (int c = threadIdx.x; c < a.E; c += MM_THREADS) {
            __half hi, mid;
            split_f16(x[c] * sc, hi, mid);
            x_h[c] = hi;
            x_h[a.E + c] = mid;
        }
    }
    __syncthreads();

    const int n_items = s_nslots * tps;
    bool ok = true;

    if (warp == MM_CONS) {
        // ---------------------------------------------------------------- producer ----
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int slot = item / tps, rt = item % tps;
            const ExpertW ew = s_ew[slot];
            const int pair = s_pair[slot];
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % MM_NS;
                if (it >= MM_NS) ok = mbar_wait(&empty[s], ((it / MM_NS) - 1) & 1, a.err, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t *st = stages + (size_t)s * stage_bytes;
                const uint32_t bytes = MM_ROWS * MM_CB + (GATEUP ? 2 : 1) * scols * 4 + (GATEUP ? 0 : a.I * 4);
                if (lane == 0) mbar_expect_tx(&full[s], bytes);
                __syncwarp();
                const uint8_t *src;
                if (GATEUP) src = (lane < 16 ? ew.gate : ew.up) + (size_t)(rt * 16 + (lane & 15)) * C + (size_t)kh * MM_CB;
                else        src = ew.down + (size_t)(rt * MM_ROWS + lane) * C + (size_t)kh * MM_CB;
                bulk_g2s(st + (size_t)lane * MM_PITCH, src, MM_CB, &full[s]);
                if (lane == 0) {
                    const int r0 = rt * rows_per_item;
                    if (GATEUP) {
                        bulk_g2s(st + scale_off, ew.gate_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                        bulk_g2s(st + scale_off + 256, ew.up_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                    } else {
                        bulk_g2s(st + scale_off, ew.down_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                        bulk_g2s(st + act_off, static_cast<const uint8_t *>(a.x) + (size_t)pair * a.I * 4, a.I * 4, &full[s]);
                    }
                }
            }
        }
        if (!ok) {                       // copies in flight must land before shared memory goes away
            for (int k = 0; k < MM_NS && k < it; k++) {
                const int j = it - 1 - k;
                mbar_wait(&full[j % MM_NS], (j / MM_NS) & 1, a.err, 3);
            }
        }
    } else {
        // --------------------------------------------------------------- consumers ----
        const int mt = warp & 1, kq = warp >> 1;          // M tile (16 rows), column quarter of the stage
        const int g = lane >> 2, t = lane & 3;
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int slot = item / tps, rt = item % tps;
            const int pair = s_pair[slot];
            float accf[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % MM_NS;
                ok = mbar_wait_warp(&full[s], (it / MM_NS) & 1, a.err, 2);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint8_t *st = stages + (size_t)s * stage_bytes;
                const float *sc = reinterpret_cast<const float *>(st + scale_off) + ((GATEUP && mt) ? 64 : 0);
                const __half *xt = GATEUP ? x_h + (size_t)g * a.E : reinterpret_cast<const __half *>(st + act_off) + (size_t)g * a.I;
                mma_consume_stage(accf, st, sc, xt, kh * MM_CB, a.bc, mt, kq, g, t);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            // columns 0 (hi) and 1 (mid) of the accumulator tile live in the lanes with t == 0
            if (t == 0) {
                red[warp * 16 + g] = accf[0] + accf[1] * (1.0f / 2048.0f);
                red[warp * 16 + g + 8] = accf[2] + accf[3] * (1.0f / 2048.0f);
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            if (GATEUP) {
                if (threadIdx.x < 16) {
                    const int r = threadIdx.x;
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
                    __half *dst = static_cast<__half *>(a.y) + (size_t)pair * 2 * a.I;
                    dst[rt * 16 + r] = hi;
                    dst[a.I + rt * 16 + r] = mid;
                }
            } else if (threadIdx.x < 32) {
                const int r = threadIdx.x, m2 = r >> 4, rr = r & 15;
                float v = 0.f;
#pragma unroll
                for (int q = 0; q < 4; q++) v += red[(2 * q + m2) * 16 + rr];
                static_cast<float *>(a.y)[(size_t)s_dst[slot] * a.E + rt * MM_ROWS + r] = v * act_inv;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        }
        if (!GATEUP && a.out && ok) {
            // Combine once per CTA: report every row tile this CTA wrote; whoever completes a tile
            // sums its K contributions in top-k order in FP64 and adds the shared expert
            // (reference: src/core/glm53f_ops.c:1329-1340).
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            const int n = s_nslots;
            int mine = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x) mine++;
            if (mine > MM_MAX_ITEMS) { if (threadIdx.x == 0) atomicExch(a.err, 4); mine = 0; }
            if ((int)threadIdx.x < mine) {
                const int rt = (blockIdx.x + threadIdx.x * gridDim.x) % tps;
                const int prev = atomicAdd(&a.tile_done[rt], 1);
                my_tiles[threadIdx.x] = rt;
                my_last[threadIdx.x] = prev == n - 1;
                if (prev == n - 1) a.tile_done[rt] = 0;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            __threadfence();
            const float *contrib = static_cast<const float *>(a.y);
            for (int k = warp; k < mine; k += MM_CONS) {
                if (!my_last[k]) continue;
                const int d = my_tiles[k] * MM_ROWS + lane;
                double sum = 0.0;
                for (int j = 0; j < a.K; j++) sum += (double)a.w[j] * (double)__ldcg(contrib + (size_t)j * a.E + d);
                float o = (float)sum;
                if (a.with_shared) o = __fadd_rn(o, __ldcg(contrib + (size_t)a.K * a.E + d));
                a.out[d] = o;
            }
        }
    }
}

static size_t mma_smem_bytes(bool gateup, int E, int I)
{
    const size_t stage = (size_t)MM_ROWS * MM_PITCH + 512 + (gateup ? 0 : (size_t)I * 4);
    return MM_NS * stage + (gateup ? (size_t)E * 4 : 0) + MM_CONS * 16 * 4 + 2 * MM_NS * sizeof(uint64_t) + 64;
}

bool moe_mma_supported(const MoeShape &s, int T)
{
    if (T != 1 || s.dt != DT_FP8 || s.K + 1 > MM_MAX_SLOTS) return false;
    if (s.E % MM_CB || s.I % MM_CB || s.I % 16 || s.E % MM_ROWS) return false;
    if (s.bc < 64 || 512 % s.bc || s.br % MM_ROWS || s.E / s.bc > 64 || s.I / s.bc > 64) return false;
    if ((s.E / s.bc) % 4 || (s.I / s.bc) % 4) return false;          // scale rows are copied in 16-byte units
    if (!(s.limit > 0.f) || s.limit * s.limit > 60000.f) return false;   // activations must fit F16
    if (mma_smem_bytes(true, s.E, s.I) > 226 * 1024 || mma_smem_bytes(false, s.E, s.I) > 226 * 1024) return false;
    return true;
}

template <bool GATEUP>
static void launch_mma(cudaStream_t st, const MmaArgs &a, size_t smem)
{
    static SmemGrant grant;
    if (!dev_opt_in_smem((const void *)moe_mma_kernel<GATEUP>, smem, grant)) return;
    G5B_LAUNCH(moe_mma_kernel<GATEUP>, dev_sms(), MM_THREADS, smem, st, a);
}

void moe_mma_gateup(cudaStream_t st, void *act_terms, const float *x, const ExpertW *experts, const MoePlan &p,
                    const MoeShape &s, int *err)
{
    MmaArgs a{experts, p, x, act_terms, s.E, s.I, s.br, s.bc, s.limit, nullptr, nullptr, s.K, 0, nullptr, err};
    launch_mma<true>(st, a, mma_smem_bytes(true, s.E, s.I));
}

void moe_mma_down(cudaStream_t st, float *out, float *contrib, const void *act_terms, const float *w,
                  const ExpertW *experts, const MoePlan &p, const MoeShape &s, int with_shared, int *tile_done,
                  int *err)
{
    MmaArgs a{experts, p, act_terms, contrib, s.E, s.I, s.br, s.bc, s.limit, out, w, s.K, with_shared, tile_done, err};
    launch_mma<false>(st, a, mma_smem_bytes(false, s.E, s.I));
}

}  // namespace g5b
