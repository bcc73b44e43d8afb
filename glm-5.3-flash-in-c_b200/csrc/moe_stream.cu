// moe_stream.cu - the batch-1 (decode) expert kernels: weights streamed HBM -> shared memory by
// the bulk-copy engine (cp.async.bulk + mbarrier), multiplied out of shared memory.
//
// Why: at one token per expert a warp-per-rows kernel keeps at most ~64 KB of loads in flight per
// SM (registers bound it) and measured 40 % of DRAM throughput on B200, stalled on the scoreboard.
// Here one producer warp keeps two 64 KB stages in flight per SM with no register cost while eight
// consumer warps decode and multiply the third, so the memory system stays saturated.
//
//   gate/up  stage = 16 gate rows + the same 16 up rows, 2048 columns of each (two stages cover the
//            4096 columns); a consumer warp owns two row pairs and writes SwiGLU(gate, up).
//   down     stage = 32 output rows x 2048 columns plus the expert's activation vector; the CTA that
//            finishes the last expert of a row tile also combines the K routed contributions in
//            top-k order in FP64 and adds the shared expert (reference: src/core/glm53f_ops.c:
//            1329-1340), so no separate combine launch is needed.
//
// Persistent grid: one CTA per SM walks work items blockIdx.x, +gridDim.x, ... Every wait on an
// mbarrier is bounded; a wait that runs out records an error code in device memory, the CTA drains
// the copies it has in flight (again bounded) and returns, and the host reports failure.
#include "bulk.cuh"
#include "kernels.h"

namespace g5b {

constexpr int ST_ROWS = 32;                  // weight rows per stage
constexpr int ST_CB = 2048;                  // bytes of each row per stage
constexpr int ST_NS = 3;                     // stages
constexpr int ST_MAX_ITEMS = 32;
constexpr int ST_MAX_SLOTS = 17;             // experts per token (top-k + shared) this path serves
//             // work items one CTA may own (down: combine bookkeeping)

// Position of column c in the activation layout the consumers read without bank conflicts: the
// 16 columns a lane multiplies with one 16-byte piece of codes are stored as four float4 that are
// `pieces` float4 apart, so that the 32 lanes of a warp read 32 consecutive float4.
__host__ __device__ inline int perm_index(int c, int pieces)
{
    return (((c & 15) >> 2) * pieces + (c >> 4)) * 4 + (c & 3);
}

struct StreamArgs {
    const ExpertW *experts;
    MoePlan p;
    const float *x;        // gate/up: the token's activation [E]; down: activations [pairs][I] (permuted)
    float *y;              // gate/up: activations [pairs][I] (permuted); down: contributions [K(+1)][E]
    int E, I, br, bc;
    float limit;
    // combine (down only)
    float *out;
    const float *w;
    int K, with_shared;
    int *tile_done;        // [rows_total / ST_ROWS] arrivals per row tile, zeroed by the last arrival
    int *err;
};

__device__ __forceinline__ float swiglu_clamped_s(float g, float u, float lim)
{
    g = g > lim ? lim : g;
    u = u > lim ? lim : (u < -lim ? -lim : u);
    return __fmul_rn(__fmul_rn(g, sigmoid_host(g)), u);
}

// NW consumer warps share the 32 rows of a stage (4 rows each at NW = 8, 2 at NW = 16); warp NW is
// the producer.
template <bool GATEUP, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) moe_stream_kernel(const StreamArgs a)
{
    constexpr int ST_CONS = NW, ST_THREADS = (NW + 1) * 32, RPW = ST_ROWS / NW;
    extern __shared__ __align__(128) uint8_t smem[];
    const int C = GATEUP ? a.E : a.I;                 // columns of the matrices
    const int rows_total = GATEUP ? a.I : a.E;
    const int KH = C / ST_CB;                         // stages per work item
    const int pieces = C / 16;
    const int scols = C / a.bc;
    const int rows_per_item = GATEUP ? ST_ROWS / 2 : ST_ROWS;
    const int tps = rows_total / rows_per_item;       // work items per expert
    // stage layout: weights | scale rows (2 x 64 floats) | activation vector (down only)
    const size_t scale_off = (size_t)ST_ROWS * ST_CB;
    const size_t act_off = scale_off + 512;
    const size_t stage_bytes = act_off + (GATEUP ? 0 : (size_t)a.I * 4);
    uint8_t *stages = smem;
    float *x_s = reinterpret_cast<float *>(smem + ST_NS * stage_bytes);          // gate/up only: [E] permuted
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ST_NS * stage_bytes + (GATEUP ? (size_t)a.E * 4 : 0));
    uint64_t *empty = full + ST_NS;
    __shared__ int my_tiles[ST_MAX_ITEMS], my_last[ST_MAX_ITEMS];
    __shared__ ExpertW s_ew[ST_MAX_SLOTS];
    __shared__ int s_pair[ST_MAX_SLOTS], s_dst[ST_MAX_SLOTS], s_nslots;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < ST_NS; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], ST_CONS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // The plan and the expert pointer table are read ONCE per CTA into shared memory: they sit
    // behind two dependent loads, which per work item would stall the producer for microseconds.
    if (warp == 0) {
        int n = *a.p.n_slots;
        n = n < 0 ? 0 : (n > ST_MAX_SLOTS ? ST_MAX_SLOTS : n);
        for (int i = lane; i < n; i += 32) {
            const int off = a.p.slot_off[i];
            s_ew[i] = a.experts[a.p.slot_expert[i]];
            s_pair[i] = off;
            s_dst[i] = a.p.pair_dst[off];
        }
        if (lane == 0) s_nslots = n;
    }
    if (GATEUP) {
        for (int c = threadIdx.x; c < a.E; c += ST_THREADS) x_s[perm_index(c, pieces)] = a.x[c];
    }
    __syncthreads();

    const int n_items = s_nslots * tps;
    bool ok = true;

    if (warp == ST_CONS) {
        // ---------------------------------------------------------------- producer ----
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int slot = item / tps, rt = item % tps;
            const ExpertW ew = s_ew[slot];
            const int pair = s_pair[slot];
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % ST_NS;
                if (it >= ST_NS) ok = mbar_wait(&empty[s], ((it / ST_NS) - 1) & 1, a.err, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t *st = stages + (size_t)s * stage_bytes;
                const uint32_t bytes = ST_ROWS * ST_CB + (GATEUP ? 2 : 1) * scols * 4 + (GATEUP ? 0 : a.I * 4);
                if (lane == 0) mbar_expect_tx(&full[s], bytes);
                __syncwarp();
                const uint8_t *src;
                if (GATEUP) src = (lane < 16 ? ew.gate : ew.up) + (size_t)(rt * 16 + (lane & 15)) * C + (size_t)kh * ST_CB;
                else        src = ew.down + (size_t)(rt * ST_ROWS + lane) * C + (size_t)kh * ST_CB;
                bulk_g2s(st + (size_t)lane * ST_CB, src, ST_CB, &full[s]);
                if (lane == 0) {
                    const int r0 = rt * rows_per_item;
                    if (GATEUP) {
                        bulk_g2s(st + scale_off, ew.gate_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                        bulk_g2s(st + scale_off + 256, ew.up_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                    } else {
                        bulk_g2s(st + scale_off, ew.down_s + (size_t)(r0 / a.br) * scols, scols * 4, &full[s]);
                        bulk_g2s(st + act_off, a.x + (size_t)pair * a.I, a.I * 4, &full[s]);
                    }
                }
            }
        }
        // copies in flight must land before the CTA's shared memory goes away
        if (!ok) {
            for (int k = 0; k < ST_NS && k < it; k++) {
                const int j = it - 1 - k;
                mbar_wait(&full[j % ST_NS], (j / ST_NS) & 1, a.err, 3);
            }
        }
    } else {
        // --------------------------------------------------------------- consumers ----
        int it = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int slot = item / tps, rt = item % tps;
            const int pair = s_pair[slot];
            float acc[RPW];
#pragma unroll
            for (int q = 0; q < RPW; q++) acc[q] = 0.f;
            for (int kh = 0; kh < KH && ok; kh++, it++) {
                const int s = it % ST_NS;
                ok = mbar_wait_warp(&full[s], (it / ST_NS) & 1, a.err, 2);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint8_t *st = stages + (size_t)s * stage_bytes;
                const float *sc = reinterpret_cast<const float *>(st + scale_off);
                const float *xv = GATEUP ? x_s : reinterpret_cast<const float *>(st + act_off);
                // gate/up: the first RPW/2 rows of a warp are gate rows, the rest the same up rows
                const uint8_t *wp[RPW];
#pragma unroll
                for (int q = 0; q < RPW; q++) {
                    const int row = GATEUP ? (q < RPW / 2 ? (RPW / 2) * warp + q : 16 + (RPW / 2) * warp + (q - RPW / 2))
                                           : RPW * warp + q;
                    wp[q] = st + (size_t)row * ST_CB;
                }
#pragma unroll
                for (int j = 0; j < ST_CB / 16 / 32; j++) {
                    const int piece = lane + 32 * j;                       // within this stage
                    const int gpiece = kh * (ST_CB / 16) + piece;          // within the row
                    float xr[16];
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float4 v = *reinterpret_cast<const float4 *>(xv + ((size_t)k * pieces + gpiece) * 4);
                        xr[4 * k] = v.x; xr[4 * k + 1] = v.y; xr[4 * k + 2] = v.z; xr[4 * k + 3] = v.w;
                    }
                    const int cb = (gpiece * 16) / a.bc;
                    const float s_a = sc[cb], s_b = GATEUP ? sc[64 + cb] : s_a;
#pragma unroll
                    for (int q = 0; q < RPW; q++) {
                        const uint4 wv = *reinterpret_cast<const uint4 *>(wp[q] + (size_t)piece * 16);
                        float w[16];
                        e4m3x4_to_f32(wv.x, w[0], w[1], w[2], w[3]);
                        e4m3x4_to_f32(wv.y, w[4], w[5], w[6], w[7]);
                        e4m3x4_to_f32(wv.z, w[8], w[9], w[10], w[11]);
                        e4m3x4_to_f32(wv.w, w[12], w[13], w[14], w[15]);
                        float s0 = 0.f, s1 = 0.f;
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            s0 = fmaf(w[e], xr[e], s0);
                            s1 = fmaf(w[e + 1], xr[e + 1], s1);
                        }
                        acc[q] = fmaf(s0 + s1, (GATEUP && q >= RPW / 2) ? s_b : s_a, acc[q]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (!ok) break;
#pragma unroll
            for (int q = 0; q < RPW; q++) acc[q] = warp_sum(acc[q]);
            if (GATEUP) {
                if (lane == 0) {
                    float *dst = a.y + (size_t)pair * a.I;
                    const int ap = a.I / 16;
#pragma unroll
                    for (int q = 0; q < RPW / 2; q++) {
                        const int r = rt * 16 + (RPW / 2) * warp + q;
                        dst[perm_index(r, ap)] = swiglu_clamped_s(acc[q], acc[RPW / 2 + q], a.limit);
                    }
                }
            } else {
                const int r = rt * ST_ROWS + RPW * warp;
                if (lane == 0) {
#pragma unroll
                    for (int q = 0; q < RPW; q++) a.y[(size_t)s_dst[slot] * a.E + r + q] = acc[q];
                }
            }
        }
        if (!GATEUP && a.out && ok) {
            // Combine, once per CTA after all of its items: every item reports its row tile; the CTA
            // whose report completes a tile (all experts of the token have written it) sums the K
            // contributions of that tile in top-k order in FP64 and adds the shared expert.
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"r"(ST_CONS * 32) : "memory");
            const int n = s_nslots;
            int mine = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x) mine++;
            if (mine > ST_MAX_ITEMS) { if (threadIdx.x == 0) atomicExch(a.err, 4); mine = 0; }
            if ((int)threadIdx.x < mine) {
                const int rt = (blockIdx.x + threadIdx.x * gridDim.x) % tps;
                const int prev = atomicAdd(&a.tile_done[rt], 1);
                my_tiles[threadIdx.x] = rt;
                my_last[threadIdx.x] = prev == n - 1;
                if (prev == n - 1) a.tile_done[rt] = 0;
            }
            asm volatile("bar.sync 1, %0;" ::"r"(ST_CONS * 32) : "memory");
            __threadfence();
            for (int k = warp; k < mine; k += ST_CONS) {
                if (!my_last[k]) continue;
                const int d = my_tiles[k] * ST_ROWS + lane;
                double sum = 0.0;
                for (int j = 0; j < a.K; j++) sum += (double)a.w[j] * (double)__ldcg(a.y + (size_t)j * a.E + d);
                float o = (float)sum;
                if (a.with_shared) o = __fadd_rn(o, __ldcg(a.y + (size_t)a.K * a.E + d));
                a.out[d] = o;
            }
        }
    }
}

size_t stream_smem_bytes(bool gateup, int E, int I)
{
    const size_t stage = (size_t)ST_ROWS * ST_CB + 512 + (gateup ? 0 : (size_t)I * 4);
    return ST_NS * stage + (gateup ? (size_t)E * 4 : 0) + 2 * ST_NS * sizeof(uint64_t) + 64;
}

// The streamed path serves FP8 experts whose shapes tile evenly; everything else keeps the
// register-streaming kernels of moe.cu.
bool moe_stream_supported(const MoeShape &s, int T)
{
    if (T != 1 || s.dt != DT_FP8 || s.K + 1 > ST_MAX_SLOTS) return false;
    if (s.E % ST_CB || s.I % ST_CB || s.I % 16 || s.E % ST_ROWS) return false;
    if (s.bc < 16 || s.bc % 16 || s.br % ST_ROWS || s.E / s.bc > 64 || s.I / s.bc > 64) return false;
    if ((s.E / s.bc) % 4 || (s.I / s.bc) % 4) return false;          // scale rows copied in 16-byte units
    if (stream_smem_bytes(true, s.E, s.I) > 227 * 1024 || stream_smem_bytes(false, s.E, s.I) > 227 * 1024) return false;
    return true;
}

static int g_sms = 0;
static int sm_count()
{
    if (!g_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
        if (g_sms < 1) g_sms = 148;
    }
    return g_sms;
}

template <bool GATEUP, int NW>
static void launch_stream(cudaStream_t st, const StreamArgs &a, size_t smem)
{
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(moe_stream_kernel<GATEUP, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr = true;
    }
    G5B_LAUNCH((moe_stream_kernel<GATEUP, NW>), sm_count(), (NW + 1) * 32, smem, st, a);
}

void moe_stream_gateup(cudaStream_t st, float *act, const float *x, const ExpertW *experts, const MoePlan &p,
                       const MoeShape &s, int *err, int warps)
{
    StreamArgs a{experts, p, x, act, s.E, s.I, s.br, s.bc, s.limit, nullptr, nullptr, s.K, 0, nullptr, err};
    const size_t smem = stream_smem_bytes(true, s.E, s.I);
    if (warps == 8) launch_stream<true, 8>(st, a, smem);
    else            launch_stream<true, 16>(st, a, smem);
}

void moe_stream_down(cudaStream_t st, float *out, float *contrib, const float *act, const float *w,
                     const ExpertW *experts, const MoePlan &p, const MoeShape &s, int with_shared,
                     int *tile_done, int *err, int warps)
{
    StreamArgs a{experts, p, act, contrib, s.E, s.I, s.br, s.bc, s.limit, out, w, s.K, with_shared, tile_done, err};
    const size_t smem = stream_smem_bytes(false, s.E, s.I);
    if (warps == 8) launch_stream<false, 8>(st, a, smem);
    else            launch_stream<false, 16>(st, a, smem);
}

}  // namespace g5b
