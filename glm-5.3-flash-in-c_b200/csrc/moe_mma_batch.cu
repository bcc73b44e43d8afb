// moe_mma_batch.cu - expert kernels for batches (2..64 tokens per pass): the bulk-copy pipeline and
// tensor-core consumer of moe_mma.cu with FOUR activation vectors per weight stage.
//
// At batch B the router's picks spread over many experts (measured 48 distinct experts at B = 8,
// 119 at B = 64 with the stated input distributions), a few tokens each, so the work is still
// weight streaming: every byte of an expert that has any token must be read once. The batch-1
// kernel leaves six of the eight B columns of mma.sync.m16n8k16 empty; here they carry three more
// tokens (column 2p = hi term of token p, 2p + 1 = its mid term), at the same tensor-pipe cost.
// An expert with more than four tokens is streamed once per group of four (its second pass hits
// L2 when it follows closely).
//
// Work item = (token tile of <= 4 pairs of one expert slot, row tile); a stage carries 32 weight
// rows x 2048 columns, their scale rows, AND the matching 2048-column slice of the tile's
// activation terms (8 rows of F16, copied from an L2-resident buffer that a small kernel fills
// with every token's two terms first) - so stages are self-contained and nothing is re-staged
// when consecutive items belong to different experts. Two stages of 99 KB in flight per SM.
#include "kernels.h"
#include "mma_stage.cuh"

namespace g5b {

constexpr int MB_NS = 2;                       // stages
constexpr int MB_TILE = 4;                     // pairs per pass
constexpr int MB_MAX_TILES = 448;              // 289 slots + (64 x 8 + 64) / 4 extra tiles at most
constexpr int MB_MAX_SLOTS = 296;

struct MmaBatchArgs {
    const ExpertW *experts;
    MoePlan p;
    const __half *xterms;        // gate/up: [T][2][E] terms of the scaled activations; down: [pairs][2][I]
    const float *xinv;           // gate/up: 1 / scale of token t
    void *y;                     // gate/up: F16 terms [pairs][2][I]; down: contributions float [rows][E]
    int E, I, br, bc, T;
    float limit;
    int *err;
};

// ---- every token's activation as two F16 terms of x * 2^k (k per token: max |x| near 2^14)
__global__ void __launch_bounds__(256) split_terms_kernel(__half *xterms, float *xinv, const float *x, int ldx, int E)
{
    __shared__ float wmax[8];
    __shared__ float scale;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *xt = x + (size_t)t * ldx;
    float m = 0.f;
    for (int c = threadIdx.x; c < E; c += blockDim.x) m = fmaxf(m, fabsf(xt[c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.f;
        for (int i = 0; i < 8; i++) mm = fmaxf(mm, wmax[i]);
        int ex = 0;
        if (mm > 0.f && mm < INFINITY) frexpf(mm, &ex);
        scale = ldexpf(1.0f, 14 - ex);
        xinv[t] = ldexpf(1.0f, ex - 14);
    }
    __syncthreads();
    const float sc = scale;
    __half *dst = xterms + (size_t)t * 2 * E;
    for (int c = threadIdx.x; c < E; c += blockDim.x) {
        __half hi, mid;
        split_f16(xt[c] * sc, hi, mid);
        dst[c] = hi;
        dst[E + c] = mid;
    }
}

template <bool GATEUP>
__global__ void __launch_bounds__(MM_THREADS, 1) moe_mma_batch_kernel(const MmaBatchArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int C = GATEUP ? a.E : a.I;
    const int rows_total = GATEUP ? a.I : a.E;
    const float act_sc = act_term_scale(a.limit), act_inv = 1.0f / act_sc;   // powers of two
    const int KH = C / MM_CB;
    const int scols = C / a.bc;
    const int rows_per_item = GATEUP ? MM_ROWS / 2 : MM_ROWS;
    const int tps = rows_total / rows_per_item;
    // stage: weights [32][MM_PITCH] | two scale rows (64 floats each) | activation tile [8][XT_PITCH]
    const size_t scale_off = (size_t)MM_ROWS * MM_PITCH;
    const size_t x_off = scale_off + 512;
    const size_t stage_bytes = x_off + (size_t)8 * XT_PITCH;
    uint8_t *stages = smem;
    uint8_t *tail = smem + MB_NS * stage_bytes;
    float *red = reinterpret_cast<float *>(tail);                                   // [8 warps][16 rows][4 pairs]
    uint64_t *full = reinterpret_cast<uint64_t *>(tail + MM_CONS * 16 * MB_TILE * 4);
    uint64_t *empty = full + MB_NS;
    ExpertW *s_ew = reinterpret_cast<ExpertW *>(empty + MB_NS);                     // [MB_MAX_SLOTS]
    int *tile_slot = reinterpret_cast<int *>(s_ew + MB_MAX_SLOTS);                  // [MB_MAX_TILES]
    int *tile_off = tile_slot + MB_MAX_TILES;                                       // first pair of the tile
    int *tile_cnt = tile_off + MB_MAX_TILES;
    __shared__ int s_ntiles;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < MB_NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], MM_CONS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // plan -> shared memory, once per CTA: expert pointers per slot, and the list of token tiles
    int nslots = *a.p.n_slots;
    nslots = nslots < 0 ? 0 : (nslots > MB_MAX_SLOTS ? MB_MAX_SLOTS : nslots);
    for (int i = threadIdx.x; i < nslots; i += blockDim.x) s_ew[i] = a.experts[a.p.slot_expert[i]];
    if (threadIdx.x == 0) {
        int n = 0;
        for (int i = 0; i < nslots; i++) {
            const int off = a.p.slot_off[i], cnt = a.p.slot_cnt[i];
            for (int q = 0; q < cnt && n < MB_MAX_TILES; q += MB_TILE) {
                tile_slot[n] = i; tile_off[n] = off + q; tile_cnt[n] = cnt - q < MB_TILE ? cnt - q : MB_TILE;
                n++;
            }
        }
        s_ntiles = n;
    }
    __syncthreads();

    const int n_items = s_ntiles * tps;
    bool ok = true;

    if (warp == MM_CONS) {
        // ---------------------------------------------------------------- producer ----
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int tile = item / tps, rt = item % tps;
            const ExpertW ew = s_ew[tile_slot[tile]];
            const int pair0 = tile_off[tile], np = tile_cnt[tile];
            // lanes 0..7 each fetch one row of the activation tile: pair lane / 2, term lane % 2
            const uint8_t *xsrc = nullptr;
            if (lane < 2 * np) {
                const int pr = pair0 + (lane >> 1), term = lane & 1;
                if (GATEUP) xsrc = reinterpret_cast<const uint8_t *>(a.xterms + ((size_t)a.p.pair_tok[pr] * 2 + term) * a.E);
                else        xsrc = reinterpret_cast<const uint8_t *>(a.xterms + ((size_t)pr * 2 + term) * a.I);
            }
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % MB_NS;
                if (it >= MB_NS) ok = mbar_wait(&empty[s], ((it / MB_NS) - 1) & 1, a.err, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t *st = stages + (size_t)s * stage_bytes;
                const uint32_t bytes = MM_ROWS * MM_CB + (GATEUP ? 2 : 1) * scols * 4 + 2 * np * MM_CB * 2;
                if (lane == 0) mbar_expect_tx(&full[s], bytes);
                __syncwarp();
                const uint8_t *src;
                if (GATEUP) src = (lane < 16 ? ew.gate : ew.up) + (size_t)(rt * 16 + (lane & 15)) * C + (size_t)kh * MM_CB;
                else        src = ew.down + (size_t)(rt * MM_ROWS + lane) * C + (size_t)kh * MM_CB;
                bulk_g2s(st + (size_t)lane * MM_PITCH, src, MM_CB, &full[s]);
                if (xsrc) bulk_g2s(st + x_off + (size_t)lane * XT_PITCH, xsrc + (size_t)kh * MM_CB * 2, MM_CB * 2, &full[s]);
                if (lane == 0) {
                    const int r0 = rt * rows_per_item;
                    if (GATEUP) {
                        bulk_g2s(st + scale_off, ew.gate_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                        bulk_g2s(st + scale_off + 256, ew.up_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                    } else {
                        bulk_g2s(st + scale_off, ew.down_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                    }
                }
            }
        }
        if (!ok) {                       // copies in flight must land before shared memory goes away
            for (int k = 0; k < MB_NS && k < it; k++) {
                const int j = it - 1 - k;
                mbar_wait(&full[j % MB_NS], (j / MB_NS) & 1, a.err, 3);
            }
        }
    } else {
        // --------------------------------------------------------------- consumers ----
        const int mt = warp & 1, kq = warp >> 1;          // M tile (16 rows), column quarter of the stage
        const int g = lane >> 2, t = lane & 3;
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int tile = item / tps, rt = item % tps;
            const int pair0 = tile_off[tile], np = tile_cnt[tile];
            float accf[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % MB_NS;
                ok = mbar_wait_warp(&full[s], (it / MB_NS) & 1, a.err, 2);
                if (!ok) break;
                const uint8_t *st = stages + (size_t)s * stage_bytes;
                const float *sc = reinterpret_cast<const float *>(st + scale_off) + ((GATEUP && mt) ? 64 : 0);
                mma_consume_stage_x4(accf, st, sc, st + x_off, kh * MM_CB, a.bc, mt, kq, g, t);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
            // lane (g, t) holds rows g and g + 8 of pair t: hi + mid / 2048
            red[(warp * 16 + g) * MB_TILE + t] = accf[0] + accf[1] * (1.0f / 2048.0f);
            red[(warp * 16 + g + 8) * MB_TILE + t] = accf[2] + accf[3] * (1.0f / 2048.0f);
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
            if (GATEUP) {
                if (threadIdx.x < 16 * MB_TILE) {
                    const int r = threadIdx.x >> 2, pr = threadIdx.x & 3;
                    if (pr < np) {
                        float gsum = 0.f, usum = 0.f;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            gsum += red[((2 * q) * 16 + r) * MB_TILE + pr];
                            usum += red[((2 * q + 1) * 16 + r) * MB_TILE + pr];
                        }
                        const float inv = a.xinv[a.p.pair_tok[pair0 + pr]];
                        float gv = gsum * inv, uv = usum * inv;
                        gv = gv > a.limit ? a.limit : gv;
                        uv = uv > a.limit ? a.limit : (uv < -a.limit ? -a.limit : uv);
                        const float act = __fmul_rn(__fmul_rn(gv, sigmoid_host(gv)), uv);
                        __half hi, mid;
                        split_f16(act * act_sc, hi, mid);
                        __half *dst = static_cast<__half *>(a.y) + (size_t)(pair0 + pr) * 2 * a.I;
                        dst[rt * 16 + r] = hi;
                        dst[a.I + rt * 16 + r] = mid;
                    }
                }
            } else if (threadIdx.x < 32 * MB_TILE) {
                const int r = threadIdx.x >> 2, pr = threadIdx.x & 3, m2 = r >> 4, rr = r & 15;
                if (pr < np) {
                    float v = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; q++) v += red[((2 * q + m2) * 16 + rr) * MB_TILE + pr];
                    static_cast<float *>(a.y)[(size_t)a.p.pair_dst[pair0 + pr] * a.E + rt * MM_ROWS + r] = v * act_inv;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"r"(MM_CONS * 32) : "memory");
        }
    }
}

static size_t mmab_smem_bytes()
{
    const size_t stage = (size_t)MM_ROWS * MM_PITCH + 512 + (size_t)8 * XT_PITCH;
    return MB_NS * stage + MM_CONS * 16 * MB_TILE * 4 + 2 * MB_NS * sizeof(uint64_t) + MB_MAX_SLOTS * sizeof(ExpertW) +
           3 * MB_MAX_TILES * sizeof(int) + 64;
}

bool moe_mma_batch_supported(const MoeShape &s, int T)
{
    if (T < 1 || T > 64 || s.dt != DT_FP8) return false;
    if (s.n_local + 1 > MB_MAX_SLOTS || (T * s.K + T + MB_TILE - 1) / MB_TILE + s.n_local + 1 > MB_MAX_TILES) return false;
    if (s.E % MM_CB || s.I % MM_CB || s.I % 16 || s.E % MM_ROWS) return false;
    if (s.bc < 64 || 512 % s.bc || s.br % MM_ROWS || s.E / s.bc > 64 || s.I / s.bc > 64) return false;
    if ((s.E / s.bc) % 4 || (s.I / s.bc) % 4) return false;          // scale rows are copied in 16-byte units
    if (!(s.limit > 0.f) || s.limit * s.limit > 60000.f) return false;   // activations must fit F16
    return mmab_smem_bytes() <= 226 * 1024;
}

template <bool GATEUP>
static void launch_mmab(cudaStream_t st, const MmaBatchArgs &a)
{
    static SmemGrant grant;
    if (!dev_opt_in_smem((const void *)moe_mma_batch_kernel<GATEUP>, mmab_smem_bytes(), grant)) return;
    G5B_LAUNCH(moe_mma_batch_kernel<GATEUP>, dev_sms(), MM_THREADS, mmab_smem_bytes(), st, a);
}

void moe_mma_batch_gateup(cudaStream_t st, void *act_terms, void *xterms, float *xinv, const float *x, int ldx,
                          const ExpertW *experts, const MoePlan &p, int T, const MoeShape &s, int *err)
{
    G5B_LAUNCH(split_terms_kernel, T, 256, 0, st, static_cast<__half *>(xterms), xinv, x, ldx, s.E);
    MmaBatchArgs a{experts, p, static_cast<const __half *>(xterms), xinv, act_terms, s.E, s.I, s.br, s.bc, T, s.limit, err};
    launch_mmab<true>(st, a);
}

void moe_mma_batch_down(cudaStream_t st, float *contrib, const void *act_terms, const ExpertW *experts,
                        const MoePlan &p, int T, const MoeShape &s, int *err)
{
    MmaBatchArgs a{experts, p, static_cast<const __half *>(act_terms), nullptr, contrib, s.E, s.I, s.br, s.bc, T, s.limit, err};
    launch_mmab<false>(st, a);
}

}  // namespace g5b
