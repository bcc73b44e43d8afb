// gemm_tokens.cu - BF16 projections for many tokens at once (prefill chunks, batches of sequences).
//
// y[t][r] = sum_c W[r][c] * x'[t][c] for T tokens is a plain GEMM, and it is given to cuBLAS (the
// one library call on a compute path in this engine; every kernel of the batch-1 decode path is
// hand written). What is done here around it keeps the reference's arithmetic: the activations
// are FP32 (after the optional RMSNorm prologue x' = w * (x * inv), rounded like the GEMV kernels
// round it), and BF16 x BF16 products would throw 16 of their 24 significant bits away, so every
// activation is split exactly into three BF16 terms (hi + mid + lo = x', 24 bits) that become
// three columns of the GEMM's B operand; products are exact in the tensor cores, accumulation is
// FP32, and the three partial results are added at the end (hi first). The GEMV kernel, four
// tokens per pass, re-read the weights sixteen times for 64 tokens.
//
// Reference: glm53f_mm_batch / matmul_bf16 (src/core/glm53f_ops.c:101-154, 378-444).
#include <cublas_v2.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.h"

namespace g5b {

// terms[term * T + t][c] = term of x'[t][c]; one CTA per token.
__global__ void __launch_bounds__(256) split_bf16_terms_kernel(__nv_bfloat16 *terms, const float *x, int ldx,
                                                               const float *xinv, const float *xw, int C, int T)
{
    const int t = blockIdx.x;
    const float *xt = x + (size_t)t * ldx;
    const float inv = xinv ? xinv[t] : 1.0f;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float v = xt[c];
        if (xinv) {
            v = __fmul_rn(v, inv);
            if (xw) v = __fmul_rn(xw[c], v);
        }
        const __nv_bfloat16 hi = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(hi);                  // exact
        const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
        const float r2 = r1 - __bfloat162float(mid);                // exact
        const __nv_bfloat16 lo = __float2bfloat16_rn(r2);
        terms[((size_t)0 * T + t) * C + c] = hi;
        terms[((size_t)1 * T + t) * C + c] = mid;
        terms[((size_t)2 * T + t) * C + c] = lo;
    }
}

// y[t][r0 + r] = (part[t][r] + part[T + t][r]) + part[2T + t][r]
__global__ void __launch_bounds__(256) sum_terms_kernel(float *y, int ldy, const float *part, int R, int T)
{
    const int r = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (r >= R) return;
    const float a = part[((size_t)0 * T + t) * R + r], b = part[((size_t)1 * T + t) * R + r], c = part[((size_t)2 * T + t) * R + r];
    y[(size_t)t * ldy + r] = __fadd_rn(__fadd_rn(a, b), c);
}

struct GemmTokens {
    cublasHandle_t h = nullptr;
    __nv_bfloat16 *terms = nullptr;     // [3 * max_t][max_c]
    float *part = nullptr;              // [3 * max_t][ROWS_PER_CALL]
    int max_t = 0, max_c = 0;
    // the activation the terms buffer currently holds (several matrices share one input)
    const float *x = nullptr, *xinv = nullptr, *xw = nullptr;
    int ldx = 0, C = 0, T = 0;
    unsigned long long stamp = 0;
};
constexpr int GEMM_ROWS_PER_CALL = 32768;

GemmTokens *gemm_tokens_create(cudaStream_t st, int max_t, int max_c)
{
    GemmTokens *g = new GemmTokens;
    if (cublasCreate(&g->h) != CUBLAS_STATUS_SUCCESS) { delete g; return nullptr; }
    cublasSetStream(g->h, st);
    g->max_t = max_t; g->max_c = max_c;
    if (cudaMalloc((void **)&g->terms, (size_t)3 * max_t * max_c * sizeof(__nv_bfloat16)) != cudaSuccess ||
        cudaMalloc((void **)&g->part, (size_t)3 * max_t * GEMM_ROWS_PER_CALL * sizeof(float)) != cudaSuccess) {
        gemm_tokens_free(g);
        return nullptr;
    }
    return g;
}

void gemm_tokens_free(GemmTokens *g)
{
    if (!g) return;
    if (g->terms) cudaFree(g->terms);
    if (g->part) cudaFree(g->part);
    if (g->h) cublasDestroy(g->h);
    delete g;
}

// The input buffers are reused by the caller with new contents: forget what the terms hold.
void gemm_tokens_new_input(GemmTokens *g) { if (g) g->x = nullptr; }

bool gemm_tokens_takes(const GemmTokens *g, const GemvSeg &s, int T)
{
    return g && T >= 8 && T <= g->max_t && s.dt == DT_BF16 && s.C <= g->max_c && s.C % 8 == 0 && s.R >= 16 &&
           (reinterpret_cast<uintptr_t>(s.W) & 15) == 0;
}

int gemm_tokens_run(GemmTokens *g, cudaStream_t st, const GemvSeg &s, int T)
{
    if (g->x != s.x || g->xinv != s.xinv || g->xw != s.xw || g->ldx != s.ldx || g->C != s.C || g->T != T) {
        G5B_LAUNCH(split_bf16_terms_kernel, T, 256, 0, st, g->terms, s.x, s.ldx, s.xinv, s.xw, s.C, T);
        g->x = s.x; g->xinv = s.xinv; g->xw = s.xw; g->ldx = s.ldx; g->C = s.C; g->T = T;
    }
    const float one = 1.0f, zero = 0.0f;
    for (int r0 = 0; r0 < s.R; r0 += GEMM_ROWS_PER_CALL) {
        const int rc = s.R - r0 < GEMM_ROWS_PER_CALL ? s.R - r0 : GEMM_ROWS_PER_CALL;
        // column-major view: W is C x R (lda = C), terms are C x 3T (ldb = C), part is rc x 3T (ldc = rc)
        const cublasStatus_t rcode = cublasGemmEx(
            g->h, CUBLAS_OP_T, CUBLAS_OP_N, rc, 3 * T, s.C, &one,
            static_cast<const __nv_bfloat16 *>(s.W) + (size_t)r0 * s.C, CUDA_R_16BF, s.C,
            g->terms, CUDA_R_16BF, s.C, &zero, g->part, CUDA_R_32F, rc, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
        if (rcode != CUBLAS_STATUS_SUCCESS) return -1;
        ++g_launches;
        G5B_LAUNCH(sum_terms_kernel, dim3((rc + 255) / 256, T), 256, 0, st, s.y + r0, s.ldy, g->part, rc, T);
    }
    return 0;
}

}  // namespace g5b
