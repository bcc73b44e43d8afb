// mhc.cu - manifold-constrained hyper-connections: the 4-stream residual of the architecture.
//
// Reference: glm53f_hc_pre / glm53f_hc_post (src/core/glm53f_ops.c:560-625) and the device
// kernels k_hc_mix / k_hc_collapse / k_hc_post (src/gpu/glm53f_gpu_kernels.cu:455-535), where one
// thread per token ran the whole Sinkhorn normalisation and two more launches collapsed and
// expanded the streams. Here one launch per site does gates, Sinkhorn and the collapse: warp 0
// normalises the mixer while the other warps collapse the streams, which only need `pre`.
#include "acc2.cuh"
#include "common.cuh"
#include "kernels.h"

namespace g5b {

constexpr int HC_THREADS = 256;

__global__ void __launch_bounds__(HC_THREADS) hc_finish_kernel(
    float *x, float *post, float *comb, const float *h, const float *mix, const float *base,
    const float *scale, int M, int E, int iters, float epsf)
{
    __shared__ double pre[G5B_MAX_HC];
    __shared__ double cm[G5B_MAX_HC * G5B_MAX_HC];
    const int t = blockIdx.x, tid = threadIdx.x;
    const int MIX = (2 + M) * M;
    const float *mx = mix + (size_t)t * MIX;
    const double eps = (double)epsf;

    if (tid >= 32 && tid < 32 + M) {
        const int i = tid - 32;
        pre[i] = (double)sigmoid_host(mul_add_unfused(mx[i], scale[0], base[i])) + eps;
        post[(size_t)t * M + i] = __fmul_rn(2.0f, sigmoid_host(mul_add_unfused(mx[M + i], scale[1], base[M + i])));
    }
    __syncthreads();

    if (tid < 32) {
        // Row softmax + eps, then column / row normalisations, each dividing by (sum + eps) with
        // the sum taken in index order (src/core/glm53f_ops.c:577-598).
        const int MM = M * M;
        for (int e = tid; e < MM; e += 32) {
            const int i = e / M, j = e % M;
            double top = -INFINITY, z = 0.0, mine = 0.0;
            for (int jj = 0; jj < M; jj++) {
                const int k = 2 * M + i * M + jj;
                const double l = (double)mul_add_unfused(mx[k], scale[2], base[k]);
                if (l > top) top = l;
            }
            for (int jj = 0; jj < M; jj++) {
                const int k = 2 * M + i * M + jj;
                const double l = (double)mul_add_unfused(mx[k], scale[2], base[k]);
                const double ex = exp(l - top);
                z += ex;
                if (jj == j) mine = ex;
            }
            cm[e] = mine / z + eps;
        }
        __syncwarp();
        for (int pass = 0; pass < 2 * iters - 1; pass++) {
            const bool by_col = (pass & 1) == 0;
            double nv[2];
            int n = 0;
            for (int e = tid; e < MM; e += 32, n++) {
                const int i = e / M, j = e % M;
                double s = 0.0;
                for (int b = 0; b < M; b++) s += by_col ? cm[b * M + j] : cm[i * M + b];
                nv[n] = cm[e] / (s + eps);
            }
            __syncwarp();
            n = 0;
            for (int e = tid; e < MM; e += 32, n++) cm[e] = nv[n];
            __syncwarp();
        }
        for (int e = tid; e < MM; e += 32) comb[(size_t)t * MM + e] = (float)cm[e];
    } else {
        // x[d] = sum_i pre[i] * h[i][d] in FP64 (src/core/glm53f_ops.c:603-607)
        const float *ht = h + (size_t)t * M * E;
        for (int d = tid - 32; d < E; d += HC_THREADS - 32) {
            double s = 0.0;
            for (int i = 0; i < M; i++) s += pre[i] * (double)ht[(size_t)i * E + d];
            x[(size_t)t * E + d] = (float)s;
        }
    }
}

void hc_finish(cudaStream_t st, float *x, float *post, float *comb, const float *h, const float *mix,
               const HcW &w, int T, int M, int E, int iters, float eps)
{
    G5B_LAUNCH(hc_finish_kernel, T, HC_THREADS, 0, st, x, post, comb, h, mix, w.base, w.scale, M, E, iters, eps);
}

// ---- one launch per site for the decoder layer: RMSNorm0 factor + mixer product + gates + Sinkhorn
// + collapse + the sub-block's input RMSNorm.
// As separate launches these were six kernels of one to six CTAs each, about 60 us per site and
// two sites per layer - more than the attention or the MoE block they wrap. Here HCF_SLICES CTAs
// per token each take a slice of the flattened streams: the slice's sum of squares and its part
// of the (2+M)M mixer dot products, in FP64. The CTA that finishes a token last (a counter, no
// spinning) adds the parts in slice order, applies the norm factor to the dots (the mixer's input
// is RMSNorm0(h) = h * inv without a weight, src/core/glm53f_ops.c:563-569), then runs the code of
// hc_finish_kernel above and finally normalises the collapsed vector with the layer's norm weight
// (glm53f_rmsnorm, src/core/glm53f_ops.c:473-480), so the sub-block reads its input directly.
// 1 / d for d > 0 to within an ulp or two: the hardware's 20-bit estimate and two Newton steps.
// The Sinkhorn passes below are a chain of 39 dependent divisions per site; the exact division
// sequence made that chain 7 us long, and the mixer is rounded to float at the end anyway.
__device__ __forceinline__ double recip_newton(double d)
{
    double r;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(d));
    r = fma(r, fma(-d, r, 1.0), r);
    r = fma(r, fma(-d, r, 1.0), r);
    return r;
}

constexpr int HCF_SLICES = 32, HCF_MAX_E = 8192, HCF_MAX_MIX = (2 + G5B_MAX_HC) * G5B_MAX_HC;

struct HcFused {
    float *xn, *post, *comb;
    float *h;                       // [T][M][E]; rewritten in place when y is given
    const float *y;                 // optional: the previous sub-block's output [T][E] - its hc_post
                                    // (with the post / comb still in the arrays above) is applied first
    const uint16_t *fn;             // BF16 [(2+M)M][M*E]
    const float *base, *scale, *norm_w;
    double *part;                   // [T][HCF_SLICES][(2+M)M + 1]
    int *counters;                  // [T], zero between launches
    int M, E, iters;
    float hc_eps, rms_eps;
};

__global__ void __launch_bounds__(HC_THREADS) hc_pre_fused_kernel(const HcFused a)
{
    __shared__ float hs[HCF_MAX_E * G5B_MAX_HC / HCF_SLICES];   // this CTA's slice of the streams; later reused
    __shared__ float xs[HCF_MAX_E];                              // collapsed vector (last CTA)
    __shared__ double red[32];
    __shared__ double dots[HCF_MAX_MIX + 1];
    __shared__ float mx[HCF_MAX_MIX];
    __shared__ double pre[G5B_MAX_HC];
    __shared__ double cm[G5B_MAX_HC * G5B_MAX_HC];
    __shared__ int is_last;
    const int t = blockIdx.y, cta = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = a.M, E = a.E, ME = M * E, MIX = (2 + M) * M;
    const int W = E / HCF_SLICES, d0 = cta * W;                 // this CTA's columns, of every stream
    float *ht = a.h + (size_t)t * ME;

    // ---- every CTA: its columns of the M streams
    for (int i = tid; i < M * W; i += HC_THREADS) hs[i] = ht[(size_t)(i / W) * E + d0 + (i % W)];
    __syncthreads();
    if (a.y) {
        // the pending hc_post of the previous site: h'[j][d] = post[j] y[d] + sum_i comb[i][j] h[i][d]
        // in FP64 (src/core/glm53f_ops.c:612-625), written back and used below
        float nv[G5B_MAX_HC];
        if (tid < W) {
            const double yv = (double)a.y[(size_t)t * E + d0 + tid];
            const float *cb = a.comb + (size_t)t * M * M, *po = a.post + (size_t)t * M;
            for (int j = 0; j < M; j++) {
                double sj = (double)po[j] * yv;
                for (int i = 0; i < M; i++) sj += (double)cb[i * M + j] * (double)hs[i * W + tid];
                nv[j] = (float)sj;
            }
        }
        __syncthreads();
        if (tid < W)
            for (int j = 0; j < M; j++) {
                hs[j * W + tid] = nv[j];
                ht[(size_t)j * E + d0 + tid] = nv[j];
            }
        __syncthreads();
    }
    double ss = 0.0;
    for (int i = tid; i < M * W; i += HC_THREADS) ss += (double)hs[i] * (double)hs[i];
    ss = block_sum(ss, red);
    double *mine = a.part + ((size_t)t * HCF_SLICES + cta) * (MIX + 1);
    if (tid == 0) mine[MIX] = ss;
    const int per_seg = W / 8;                                     // 16-byte pieces per stream segment
    for (int k = warp; k < MIX; k += HC_THREADS / 32) {
        const uint16_t *row = a.fn + (size_t)k * ME + d0;
        double acc = 0.0;
        for (int piece = lane; piece < M * per_seg; piece += 32) {
            const int i = piece / per_seg, off = (piece % per_seg) * 8;
            const uint4 wv = ld_stream16(row + (size_t)i * E + off);
            float w[8];
            bf16x2_to_f32(wv.x, w[0], w[1]); bf16x2_to_f32(wv.y, w[2], w[3]);
            bf16x2_to_f32(wv.z, w[4], w[5]); bf16x2_to_f32(wv.w, w[6], w[7]);
#pragma unroll
            for (int j = 0; j < 8; j++) acc = fma((double)w[j], (double)hs[i * W + off + j], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) mine[k] = acc;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(a.counters + t, 1);
        is_last = prev == HCF_SLICES - 1;
        if (is_last) a.counters[t] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    // ---- the token's last CTA: parts in slice order, factor, gates
    if (tid <= MIX) {
        double s = 0.0;
        for (int cc = 0; cc < HCF_SLICES; cc++) s += __ldcg(a.part + ((size_t)t * HCF_SLICES + cc) * (MIX + 1) + tid);
        dots[tid] = s;
    }
    __syncthreads();
    if (tid < MIX) {
        const float inv = (float)(1.0 / sqrt(dots[MIX] / (double)ME + (double)a.rms_eps));
        mx[tid] = (float)(dots[tid] * (double)inv);
    }
    __syncthreads();
    const double eps = (double)a.hc_eps;
    if (tid >= 32 && tid < 32 + M) {
        const int i = tid - 32;
        pre[i] = (double)sigmoid_host(mul_add_unfused(mx[i], a.scale[0], a.base[i])) + eps;
        a.post[(size_t)t * M + i] = __fmul_rn(2.0f, sigmoid_host(mul_add_unfused(mx[M + i], a.scale[1], a.base[M + i])));
    }
    __syncthreads();
    if (tid < 32) {
        // row softmax + eps, then column / row normalisations (src/core/glm53f_ops.c:577-598)
        const int MM = M * M;
        for (int e = tid; e < MM; e += 32) {
            const int i = e / M, j = e % M;
            double top = -INFINITY, z = 0.0, own = 0.0;
            for (int jj = 0; jj < M; jj++) {
                const int k = 2 * M + i * M + jj;
                const double l = (double)mul_add_unfused(mx[k], a.scale[2], a.base[k]);
                if (l > top) top = l;
            }
            for (int jj = 0; jj < M; jj++) {
                const int k = 2 * M + i * M + jj;
                const double l = (double)mul_add_unfused(mx[k], a.scale[2], a.base[k]);
                const double ex = exp(l - top);
                z += ex;
                if (jj == j) own = ex;
            }
            cm[e] = own / z + eps;
        }
        __syncwarp();
        if (MM <= 32) {
            // a lane per matrix element, sums gathered with shuffles in the reference's index order
            const int i = tid / M, j = tid % M;
            double v = tid < MM ? cm[tid] : 0.0;
            for (int pass = 0; pass < 2 * a.iters - 1; pass++) {
                const bool by_col = (pass & 1) == 0;
                double sum = 0.0;
                for (int b = 0; b < M; b++) {
                    const int src = by_col ? b * M + j : i * M + b;
                    sum += __shfl_sync(0xffffffffu, v, src < 32 ? src : 0);
                }
                if (tid < MM) v = v * recip_newton(sum + eps);
            }
            if (tid < MM) a.comb[(size_t)t * MM + tid] = (float)v;
        } else {
            for (int pass = 0; pass < 2 * a.iters - 1; pass++) {
                const bool by_col = (pass & 1) == 0;
                double nv[2];
                int n = 0;
                for (int e = tid; e < MM; e += 32, n++) {
                    const int i = e / M, j = e % M;
                    double s = 0.0;
                    for (int b = 0; b < M; b++) s += by_col ? cm[b * M + j] : cm[i * M + b];
                    nv[n] = cm[e] / (s + eps);
                }
                __syncwarp();
                n = 0;
                for (int e = tid; e < MM; e += 32, n++) cm[e] = nv[n];
                __syncwarp();
            }
            for (int e = tid; e < MM; e += 32) a.comb[(size_t)t * MM + e] = (float)cm[e];
        }
    } else {
        // x[d] = sum_i pre[i] * h[i][d] in FP64 (src/core/glm53f_ops.c:603-607), kept in shared memory.
        // Four columns per thread and all of a thread's loads issued before the sums: one CTA walks
        // the whole token here, so the loads must overlap (they hit L2: the slices were just read).
        for (int d0 = (tid - 32) * 4; d0 < E; d0 += (HC_THREADS - 32) * 4 * 2) {
            const int d1 = d0 + (HC_THREADS - 32) * 4;
            float4 va[G5B_MAX_HC], vb[G5B_MAX_HC];
#pragma unroll
            for (int i = 0; i < G5B_MAX_HC; i++)
                if (i < M) {
                    va[i] = *reinterpret_cast<const float4 *>(ht + (size_t)i * E + d0);
                    if (d1 < E) vb[i] = *reinterpret_cast<const float4 *>(ht + (size_t)i * E + d1);
                }
            double sa[4] = {0.0, 0.0, 0.0, 0.0}, sb[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
            for (int i = 0; i < G5B_MAX_HC; i++)
                if (i < M) {
                    const double p = pre[i];
                    sa[0] += p * (double)va[i].x; sa[1] += p * (double)va[i].y; sa[2] += p * (double)va[i].z; sa[3] += p * (double)va[i].w;
                    if (d1 < E) { sb[0] += p * (double)vb[i].x; sb[1] += p * (double)vb[i].y; sb[2] += p * (double)vb[i].z; sb[3] += p * (double)vb[i].w; }
                }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                xs[d0 + q] = (float)sa[q];
                if (d1 < E) xs[d1 + q] = (float)sb[q];
            }
        }
    }
    __syncthreads();
    // ---- the sub-block's input: RMSNorm(x) * w
    double s2 = 0.0;
    for (int d = tid; d < E; d += HC_THREADS) s2 += (double)xs[d] * (double)xs[d];
    s2 = block_sum(s2, red);
    __shared__ float inv2;
    if (tid == 0) inv2 = (float)(1.0 / sqrt(s2 / (double)E + (double)a.rms_eps));
    __syncthreads();
    const float f = inv2;
    for (int d = tid; d < E; d += HC_THREADS) a.xn[(size_t)t * E + d] = __fmul_rn(a.norm_w[d], __fmul_rn(xs[d], f));
}

// ---- the same site as one thread-block cluster per token.
// The kernel above hands a token to whichever CTA finishes last: a fence, an atomic, a reload of
// 32 x 25 partial sums and then ONE CTA walking the whole token for the collapse and the norm
// (about 21 us per site, two sites per layer: a quarter of a batch-1 decoder layer). Here the
// HCC_CTAS CTAs of a cluster each keep their columns of the streams in shared memory from the
// first load to the last store; the partial sums (mixer dots, then the collapsed vector's sum of
// squares) are exchanged through distributed shared memory at two cluster barriers, every CTA
// derives the gates for itself and collapses and normalises its own columns. The Sinkhorn chain
// (39 dependent normalisations, needed only for the NEXT stream expansion) runs in warp 0 of CTA 0
// beside all that: warp 0 arrives at the second barrier before it starts and waits after.
constexpr int HCC_CTAS = 8, HCC_THREADS = 512, HCC_WARPS = HCC_THREADS / 32, HCC_MAX_W = 1024, HCC_MAX_HS = 4096;
constexpr int HCC_ROWS = 3, HCC_ROW_WARPS = 8, HCC_SPLITS = HCC_WARPS / HCC_ROW_WARPS;

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the shared variable `p` of CTA `rank` of this cluster
__device__ __forceinline__ double ld_cluster_f64(const double *p, uint32_t rank)
{
    const uint32_t mine = (uint32_t)__cvta_generic_to_shared(p);
    uint32_t theirs;
    double v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(theirs) : "r"(mine), "r"(rank));
    asm volatile("ld.shared::cluster.f64 %0, [%1];" : "=d"(v) : "r"(theirs) : "memory");
    return v;
}

// v / d for d > 0 to a relative 2^-40: the hardware's reciprocal estimate r (20 bits), its error
// e = 1 - d r, and v r (1 + e). An FP64 instruction occupies its pipe for 32 cycles per warp here
// and a Sinkhorn pass is a chain of nothing else, so every instruction less is 0.6 us per site; the
// mixer is rounded to float (2^-24) after the last pass.
__device__ __forceinline__ double div_chain(double v, double d)
{
    double r;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(d));
    const double q = v * r;
    return fma(q, fma(-d, r, 1.0), q);
}

// The 2 iters - 1 alternating column / row normalisations v <- v / (sum + eps) of the mixer
// (src/core/glm53f_ops.c:583-598) for the lane that holds element (i, j); all 32 lanes call it. One
// warp runs this chain while the rest of the cluster waits for nothing else, so the M = 4 case is
// written without a loop or a branch inside a pass: four shuffles, the members' sum as a two-level
// tree (the reference keeps a running sum: a few ulps of FP64 apart), one division.
template <int MT>
__device__ __forceinline__ double sinkhorn_passes(double v, int M, int i, int j, int passes, double eps)
{
    if constexpr (MT == 4) {
        for (int pass = 0; pass < passes; pass++) {
            const bool by_col = (pass & 1) == 0;
            const int s0 = by_col ? j : i * 4, st = by_col ? 4 : 1;
            const double p0 = __shfl_sync(0xffffffffu, v, s0), p1 = __shfl_sync(0xffffffffu, v, s0 + st);
            const double p2 = __shfl_sync(0xffffffffu, v, s0 + 2 * st), p3 = __shfl_sync(0xffffffffu, v, s0 + 3 * st);
            v = div_chain(v, ((p0 + p1) + (p2 + p3)) + eps);
        }
    } else {
        for (int pass = 0; pass < passes; pass++) {
            const bool by_col = (pass & 1) == 0;
            double sum = 0.0;
            for (int m = 0; m < M; m++) sum += __shfl_sync(0xffffffffu, v, by_col ? m * M + j : i * M + m);
            v = div_chain(v, sum + eps);
        }
    }
    return v;
}

__global__ void __cluster_dims__(HCC_CTAS, 1, 1) __launch_bounds__(HCC_THREADS) hc_pre_cluster_kernel(const HcFused a)
{
    __shared__ __align__(16) float hs[HCC_MAX_HS];     // this CTA's columns of the M streams
    __shared__ float xs[HCC_MAX_W];                     // its columns of the collapsed vector
    __shared__ double red[32];
    __shared__ double mine[HCC_SPLITS][HCF_MAX_MIX + 1];   // this CTA's parts of the dots; [0][MIX] = sum h^2
    __shared__ double mine_s2;                          // its part of sum x^2
    __shared__ double dots[HCF_MAX_MIX + 1];
    __shared__ float mx[HCF_MAX_MIX];
    __shared__ double pre[G5B_MAX_HC];
    const int t = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_cta_rank();
    const int M = a.M, E = a.E, ME = M * E, MIX = (2 + M) * M, MM = M * M;
    const int W = E / HCC_CTAS, d0 = (int)rank * W;
    float *ht = a.h + (size_t)t * ME;
    const double eps = (double)a.hc_eps;

    // Warp (q, b) takes the mixer rows b, b + 8, ... HCC_ROWS at a time and every HCC_SPLITS-th group of
    // 32 16-byte pieces of each. The rows depend on nothing computed here: the first piece is
    // requested before anything else; after that the piece for the next turn of the loop is
    // requested before the current one is summed. (The loop is kept rolled on purpose: this kernel
    // runs once per site with a cold instruction cache, and with the twelve pieces of a warp
    // unrolled - 17 KB of straight-line code - it waited for instruction fetch more than for data.)
    const int per_seg = W / 8, n_pieces = M * per_seg;            // pieces per stream segment / per row
    const int q = warp / HCC_ROW_WARPS, b = warp % HCC_ROW_WARPS;
    const int p_first = lane + 32 * q, p_step = 32 * HCC_SPLITS;
    uint4 wnext[HCC_ROWS];
    auto load_piece = [&](int k0, int piece) {
#pragma unroll
        for (int r = 0; r < HCC_ROWS; r++) {
            const int k = k0 + r * HCC_ROW_WARPS;
            if (k < MIX && piece < n_pieces)
                wnext[r] = ld_stream16(a.fn + (size_t)k * ME + (size_t)(piece / per_seg) * E + d0 + (piece % per_seg) * 8);
        }
    };
    load_piece(b, p_first);
    pdl_wait();                  // the streams and y come from earlier kernels; the mixer rows do not

    for (int i = tid * 4; i < M * W; i += HCC_THREADS * 4)
        *reinterpret_cast<float4 *>(hs + i) = *reinterpret_cast<const float4 *>(ht + (size_t)(i / W) * E + d0 + (i % W));
    __syncthreads();
    if (a.y) {
        // the pending hc_post of the previous site: h'[j][d] = post[j] y[d] + sum_i comb[i][j] h[i][d]
        // (src/core/glm53f_ops.c:612-625, FP64 there, compensated FP32 here); a thread owns a column,
        // so no barrier inside
        const float *cb = a.comb + (size_t)t * MM, *po = a.post + (size_t)t * M;
        for (int d = tid; d < W; d += HCC_THREADS) {
            const float yv = a.y[(size_t)t * E + d0 + d];
            float hv[G5B_MAX_HC];
#pragma unroll
            for (int i = 0; i < G5B_MAX_HC; i++) hv[i] = i < M ? hs[i * W + d] : 0.f;
#pragma unroll 1
            for (int j = 0; j < M; j++) {                // rolled: cold instruction cache, see above
                Acc2 sj;
                acc2_fma(sj, po[j], yv);
#pragma unroll
                for (int i = 0; i < G5B_MAX_HC; i++)
                    if (i < M) acc2_fma(sj, cb[i * M + j], hv[i]);
                const float nv = acc2_f32(sj);
                hs[j * W + d] = nv;
                ht[(size_t)j * E + d0 + d] = nv;
            }
        }
        __syncthreads();
    }
    Acc2 sq;
    for (int i = tid; i < M * W; i += HCC_THREADS) acc2_fma(sq, hs[i], hs[i]);
    const double ss = block_sum(acc2_f64(sq), red);
    if (tid == 0) mine[0][MIX] = ss;

    // mixer rows (compensated FP32 sums; the reference's are FP64)
    for (int k0 = b; k0 < MIX; k0 += HCC_ROW_WARPS * HCC_ROWS) {
        Acc2 acc[HCC_ROWS];
        if (k0 != b) load_piece(k0, p_first);
#pragma unroll 1
        for (int piece = p_first; piece < n_pieces; piece += p_step) {
            uint4 wv[HCC_ROWS];
#pragma unroll
            for (int r = 0; r < HCC_ROWS; r++) wv[r] = wnext[r];
            load_piece(k0, piece + p_step);
            const float *hv = hs + (piece / per_seg) * W + (piece % per_seg) * 8;
            const float4 h0 = *reinterpret_cast<const float4 *>(hv), h1 = *reinterpret_cast<const float4 *>(hv + 4);
            const float hd[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
            for (int r = 0; r < HCC_ROWS; r++) {
                if (k0 + r * HCC_ROW_WARPS >= MIX) continue;
                const uint32_t wr[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc2_fma(acc[r], __uint_as_float(wr[j] << 16), hd[2 * j]);
                    acc2_fma(acc[r], __uint_as_float(wr[j] & 0xffff0000u), hd[2 * j + 1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < HCC_ROWS; r++) {
            const int k = k0 + r * HCC_ROW_WARPS;
            const double s = warp_sum(acc2_f64(acc[r]));
            if (lane == 0 && k < MIX) mine[q][k] = s;
        }
    }
    __syncthreads();
    cluster_arrive();
    cluster_wait();

    // ---- every CTA: the token's sums in CTA order, the norm factor, the gates
    if (tid <= MIX) {
        double s = 0.0;
        for (uint32_t r = 0; r < HCC_CTAS; r++) {
            double part = ld_cluster_f64(&mine[0][tid], r);
            if (tid < MIX)
                for (int qq = 1; qq < HCC_SPLITS; qq++) part += ld_cluster_f64(&mine[qq][tid], r);
            s += part;
        }
        dots[tid] = s;
    }
    __syncthreads();
    if (tid < MIX) {
        const float inv = (float)(1.0 / sqrt(dots[MIX] / (double)ME + (double)a.rms_eps));
        mx[tid] = (float)(dots[tid] * (double)inv);
    }
    __syncthreads();
    if (tid >= 32 && tid < 32 + M) {
        const int i = tid - 32;
        pre[i] = (double)sigmoid_host(mul_add_unfused(mx[i], a.scale[0], a.base[i])) + eps;
        if (rank == 0)
            a.post[(size_t)t * M + i] = __fmul_rn(2.0f, sigmoid_host(mul_add_unfused(mx[M + i], a.scale[1], a.base[M + i])));
    }
    if (warp == 0) {
        cluster_arrive();                                // nothing of this warp goes into sum x^2
        if (rank == 0) {
            // row softmax + eps, then column / row normalisations (src/core/glm53f_ops.c:577-598): a
            // lane per matrix element, the row's / column's members gathered with shuffles
            const int el = lane < MM ? lane : 0, i = el / M, j = el % M;
            const int k = 2 * M + el;
            const double l = (double)mul_add_unfused(mx[k], a.scale[2], a.base[k]);
            double top = -INFINITY;
            for (int jj = 0; jj < M; jj++) top = fmax(top, __shfl_sync(0xffffffffu, l, i * M + jj));
            const double ex = exp(l - top);
            double z = 0.0;
            for (int jj = 0; jj < M; jj++) z += __shfl_sync(0xffffffffu, ex, i * M + jj);
            double v = ex / z + eps;
            v = M == 4 ? sinkhorn_passes<4>(v, M, i, j, 2 * a.iters - 1, eps) : sinkhorn_passes<0>(v, M, i, j, 2 * a.iters - 1, eps);
            if (lane < MM) a.comb[(size_t)t * MM + lane] = (float)v;
            __syncwarp();
        }
        cluster_wait();
    } else {
        // x[d] = sum_i pre[i] * h[i][d] in FP64 (src/core/glm53f_ops.c:603-607) for this CTA's columns
        constexpr int NW = HCC_THREADS - 32;
        const int wt = tid - 32;
        asm volatile("bar.sync 1, %0;" ::"n"(NW) : "memory");     // `pre` comes from threads of these warps
        double s2 = 0.0;
        for (int d = wt; d < W; d += NW) {
            double s = 0.0;
            for (int i = 0; i < M; i++) s += pre[i] * (double)hs[i * W + d];
            const float xv = (float)s;
            xs[d] = xv;
            s2 += (double)xv * (double)xv;
        }
        s2 = warp_sum(s2);
        if (lane == 0) red[warp] = s2;
        asm volatile("bar.sync 1, %0;" ::"n"(NW) : "memory");
        if (wt == 0) {
            double s = 0.0;
            for (int w = 1; w < HCC_WARPS; w++) s += red[w];
            mine_s2 = s;
        }
        cluster_arrive();
        cluster_wait();
        // ---- the sub-block's input: RMSNorm(x) * w (glm53f_rmsnorm, src/core/glm53f_ops.c:473-480)
        double tot = 0.0;
        for (uint32_t r = 0; r < HCC_CTAS; r++) tot += ld_cluster_f64(&mine_s2, r);
        const float f = (float)(1.0 / sqrt(tot / (double)E + (double)a.rms_eps));
        for (int d = wt; d < W; d += NW)
            a.xn[(size_t)t * E + d0 + d] = __fmul_rn(a.norm_w[d0 + d], __fmul_rn(xs[d], f));
    }
    // no CTA leaves while another may still read its shared memory
    cluster_arrive();
    cluster_wait();
}

static bool hc_pre_cluster_takes(int M, int E)
{
    const int W = E / HCC_CTAS;
    return E % (HCC_CTAS * 8) == 0 && W <= HCC_MAX_W && M * W <= HCC_MAX_HS && M * M <= 32 && M <= G5B_MAX_HC;
}

bool hc_pre_fused_supported(const HcW &w, int M, int E)
{
    if (w.fn.dt != DT_BF16) return false;
    if (hc_pre_cluster_takes(M, E)) return true;
    return E <= HCF_MAX_E && E % (HCF_SLICES * 8) == 0 && M <= G5B_MAX_HC &&
           M * (E / HCF_SLICES) <= HCF_MAX_E * G5B_MAX_HC / HCF_SLICES && E / HCF_SLICES <= HC_THREADS;
}

void hc_pre_fused(cudaStream_t st, float *xn, float *post, float *comb, float *h, const float *y_pending,
                  const HcW &w, const float *norm_w, double *part, int *counters, int T, int M, int E, int iters,
                  float hc_eps, float rms_eps)
{
    HcFused a{xn, post, comb, h, y_pending, static_cast<const uint16_t *>(w.fn.w), w.base, w.scale, norm_w, part,
              counters, M, E, iters, hc_eps, rms_eps};
    if (hc_pre_cluster_takes(M, E)) G5B_LAUNCH_PDL(hc_pre_cluster_kernel, dim3(HCC_CTAS, T), dim3(HCC_THREADS), 0, st, a);
    else                            G5B_LAUNCH(hc_pre_fused_kernel, dim3(HCF_SLICES, T), HC_THREADS, 0, st, a);
}

// h'[j][d] = post[j]*y[d] + sum_i comb[i][j]*h[i][d] in FP64, in place: a thread owns column d of
// every stream (src/core/glm53f_ops.c:612-625; note comb is used transposed).
__global__ void hc_post_kernel(float *h, const float *y, const float *post, const float *comb, int M, int E)
{
    const int t = blockIdx.y;
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= E) return;
    float *ht = h + (size_t)t * M * E;
    double hv[G5B_MAX_HC];
    for (int i = 0; i < M; i++) hv[i] = (double)ht[(size_t)i * E + d];
    const double yv = (double)y[(size_t)t * E + d];
    const float *cb = comb + (size_t)t * M * M, *po = post + (size_t)t * M;
    for (int j = 0; j < M; j++) {
        double s = (double)po[j] * yv;
        for (int i = 0; i < M; i++) s += (double)cb[i * M + j] * hv[i];
        ht[(size_t)j * E + d] = (float)s;
    }
}

void hc_post(cudaStream_t st, float *h, const float *y, const float *post, const float *comb, int T,
             int M, int E)
{
    G5B_LAUNCH(hc_post_kernel, dim3((E + 127) / 128, T), 128, 0, st, h, y, post, comb, M, E);
}

}  // namespace g5b
