// mhc.cu - manifold-constrained hyper-connections: the 4-stream residual of the architecture.
//
// Reference: glm53f_hc_pre / glm53f_hc_post (src/core/glm53f_ops.c:560-625) and the device
// kernels k_hc_mix / k_hc_collapse / k_hc_post (src/gpu/glm53f_gpu_kernels.cu:455-535), where one
// thread per token ran the whole Sinkhorn normalisation and two more launches collapsed and
// expanded the streams. Here one launch per site does gates, Sinkhorn and the collapse: warp 0
// normalises the mixer while the other warps collapse the streams, which only need `pre`.
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
