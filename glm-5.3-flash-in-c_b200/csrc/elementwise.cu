// elementwise.cu - the small ops around the matrix products: RMSNorm, clamped SwiGLU, short
// convolution, embedding gather, head mean, argmax, and test-data generation.
#include "common.cuh"
#include "kernels.h"

namespace g5b {

unsigned long long g_launches = 0;

// ---------------------------------------------------------------- RMSNorm ----
// inv[row] = (float)(1 / sqrt(sum(x^2)/n + eps)), the sum in FP64 (reference glm53f_rmsnorm,
// src/core/glm53f_ops.c:473-480; device k_rmsnorm, src/gpu/glm53f_gpu_kernels.cu:142). The
// products with inv and the weight are applied by the consumer (gemv prologue or rms_apply).
__global__ void rms_factor_kernel(const float *x, int n, int ld, float eps, float *inv)
{
    __shared__ double red[32];
    const float *row = x + (size_t)blockIdx.x * ld;
    double ss = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += (double)row[i] * (double)row[i];
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) inv[blockIdx.x] = (float)(1.0 / sqrt(ss / (double)n + (double)eps));
}

void rms_factor(cudaStream_t st, const float *x, int n, int ld, int rows, float eps, float *inv)
{
    const int threads = n >= 4096 ? 512 : n >= 512 ? 256 : 64;
    G5B_LAUNCH(rms_factor_kernel, rows, threads, 0, st, x, n, ld, eps, inv);
}

__global__ void rms_apply_kernel(float *y, const float *x, const float *w, const float *inv, int n, int ld)
{
    const float f = inv[blockIdx.y];
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = __fmul_rn(x[(size_t)blockIdx.y * ld + i], f);
    y[(size_t)blockIdx.y * ld + i] = w ? __fmul_rn(w[i], v) : v;
}

void rms_apply(cudaStream_t st, float *y, const float *x, const float *w, const float *inv, int n,
               int ld, int rows)
{
    G5B_LAUNCH(rms_apply_kernel, dim3((n + 255) / 256, rows), 256, 0, st, y, x, w, inv, n, ld);
}

// x[i] += y[i], one FP32 rounding (the residual additions of the reference's MTP layer,
// src/model/glm53f_mtp.c:124,129).
__global__ void add_rows_kernel(float *x, const float *y, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __fadd_rn(x[i], y[i]);
}
void add_rows(cudaStream_t st, float *x, const float *y, size_t n)
{
    const size_t want = (n + 255) / 256;
    G5B_LAUNCH(add_rows_kernel, (int)(want < 1184 ? want : 1184), 256, 0, st, x, y, n);
}

// ----------------------------------------------------------------- SwiGLU ----
// glm53f_swiglu_clamp, src/core/glm53f_ops.c:486-494: gate clamped from above only.
__device__ __forceinline__ float swiglu_one(float g, float u, float lim)
{
    g = g > lim ? lim : g;
    u = u > lim ? lim : (u < -lim ? -lim : u);
    return __fmul_rn(__fmul_rn(g, sigmoid_host(g)), u);
}

__global__ void swiglu_kernel(float *y, const float *gu, int n, float lim)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float *row = gu + (size_t)blockIdx.y * 2 * n;
    y[(size_t)blockIdx.y * n + i] = swiglu_one(row[i], row[n + i], lim);
}

void swiglu(cudaStream_t st, float *y, const float *gu, int n, int rows, float limit)
{
    G5B_LAUNCH(swiglu_kernel, dim3((n + 255) / 256, rows), 256, 0, st, y, gu, n, limit);
}

// -------------------------------------------------------------- ShortConv ----
// glm53f_shortconv, src/core/glm53f_ops.c:517-542: one thread per channel walks the T positions;
// current-input term first, then history terms oldest first, each product and sum rounded.
__global__ void shortconv_kernel(float *y, const float *x, const float *w, float *state, int ch, int k, int T)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= ch) return;
    const int hist = k - 1;
    float past[16];
    for (int j = 0; j < hist; j++) past[j] = state ? state[(size_t)c * hist + j] : 0.f;
    for (int t = 0; t < T; t++) {
        const float cur = x[(size_t)t * ch + c];
        float acc = __fmul_rn(w[(size_t)c * k + hist], cur);
        for (int j = 0; j < hist; j++) acc = mul_add_unfused(w[(size_t)c * k + j], past[j], acc);
        for (int j = 0; j + 1 < hist; j++) past[j] = past[j + 1];
        if (hist > 0) past[hist - 1] = cur;
        y[(size_t)t * ch + c] = __fmul_rn(acc, sigmoid_host(acc));
    }
    if (state) for (int j = 0; j < hist; j++) state[(size_t)c * hist + j] = past[j];
}

void shortconv(cudaStream_t st, float *y, const float *x, const float *w, float *state, int channels,
               int k, int T)
{
    G5B_LAUNCH(shortconv_kernel, (channels + 127) / 128, 128, 0, st, y, x, w, state, channels, k, T);
}

// -------------------------------------------------------------- embedding ----
// Embedding row widened to FP32 and copied into every residual stream
// (src/core/glm53f_ops.c:460-468, src/model/glm53f_model.c:433-437).
__global__ void embed_kernel(float *h, const void *table, int dt, int E, const int *ids, int M)
{
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= E) return;
    const size_t row = (size_t)ids[t] * E;
    const float v = dt == DT_BF16 ? bf16_to_f32(static_cast<const uint16_t *>(table)[row + i])
                                  : static_cast<const float *>(table)[row + i];
    for (int m = 0; m < M; m++) h[((size_t)t * M + m) * E + i] = v;
}

void embed_rows(cudaStream_t st, float *h, const DMat &table, const int *ids, int T, int M)
{
    G5B_LAUNCH(embed_kernel, dim3((table.cols + 255) / 256, T), 256, 0, st, h, table.w, table.dt,
               table.cols, ids, M);
}

// Mean of the residual streams in FP64 (src/model/glm53f_model.c:463-467).
__global__ void head_mean_kernel(float *xm, const float *h, int M, int E)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= E) return;
    const float *ht = h + (size_t)blockIdx.y * M * E;
    double s = 0.0;
    for (int m = 0; m < M; m++) s += (double)ht[(size_t)m * E + i];
    xm[(size_t)blockIdx.y * E + i] = (float)(s / M);
}

void head_mean(cudaStream_t st, float *xm, const float *h, int T, int M, int E)
{
    G5B_LAUNCH(head_mean_kernel, dim3((E + 255) / 256, T), 256, 0, st, xm, h, M, E);
}

// ----------------------------------------------------------------- argmax ----
// First maximum (lowest index on ties, NaN never wins), like the reference's argmax_
// (src/model/glm53f_model.c:361-366). Two stages: 64 partials per row, then one block per row.
constexpr int AM_PARTS = 64;

__device__ __forceinline__ void am_better(float &bv, int &bi, float v, int i)
{
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__global__ void argmax_part_kernel(const float *logits, int n, float *pv, int *pi)
{
    __shared__ float sv[256];
    __shared__ int   si[256];
    const float *row = logits + (size_t)blockIdx.y * n;
    const int per = (n + AM_PARTS - 1) / AM_PARTS;
    const int lo = blockIdx.x * per, hi = min(n, lo + per);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) am_better(bv, bi, row[i], i);
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            float v = sv[threadIdx.x]; int i = si[threadIdx.x];
            am_better(v, i, sv[threadIdx.x + s], si[threadIdx.x + s]);
            sv[threadIdx.x] = v; si[threadIdx.x] = i;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        pv[blockIdx.y * AM_PARTS + blockIdx.x] = sv[0];
        pi[blockIdx.y * AM_PARTS + blockIdx.x] = si[0];
    }
}

__global__ void argmax_final_kernel(int *out, const float *pv, const int *pi)
{
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (threadIdx.x == 0) {
        for (int p = 0; p < AM_PARTS; p++) am_better(bv, bi, pv[blockIdx.x * AM_PARTS + p], pi[blockIdx.x * AM_PARTS + p]);
        out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

void argmax_rows(cudaStream_t st, int *out, const float *logits, int n, int rows, float *scratch_v,
                 int *scratch_i)
{
    G5B_LAUNCH(argmax_part_kernel, dim3(AM_PARTS, rows), 256, 0, st, logits, n, scratch_v, scratch_i);
    G5B_LAUNCH(argmax_final_kernel, rows, 32, 0, st, out, scratch_v, scratch_i);
}

// -------------------------------------------------------- synthetic experts ----
// Counter-based generator: a 64-bit mix of the stream key and the index of a group of four codes
// gives four 16-bit draws, each scaled to 0..253 and mapped past 0x7f: the 254 finite E4M3 codes,
// (near) equally likely, never NaN. The CPU checker has the same function, so any single expert
// can be regenerated on the host bit for bit.
__host__ __device__ inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__global__ void fill_codes_kernel(uint32_t *dst, uint64_t key, size_t groups)
{
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (size_t)gridDim.x * blockDim.x) {
        const uint64_t h = mix64(key + g);
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t v = (uint32_t)(((h >> (16 * j)) & 0xffffu) * 254u) >> 16;
            word |= (v + (v >= 127u)) << (8 * j);
        }
        dst[g] = word;
    }
}

void fill_codes(cudaStream_t st, uint8_t *dst, uint64_t seed, int layer, int expert, int which, size_t count)
{
    const uint64_t key = mix64(seed ^ mix64(((uint64_t)layer << 40) ^ ((uint64_t)expert << 8) ^ (uint64_t)which));
    const size_t groups = count / 4;               // count is a multiple of 4 for every expert matrix
    G5B_LAUNCH(fill_codes_kernel, 1184, 256, 0, st, reinterpret_cast<uint32_t *>(dst), key, groups);
}

// Synthetic matrices by tensor name: the key mixes the seed with an FNV-1a hash of the name, so that
// the CPU can regenerate any single tensor bit for bit (orc_synth_matrix_* in the checker).
uint64_t synth_key(uint64_t seed, const char *name)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for (const unsigned char *p = reinterpret_cast<const unsigned char *>(name); *p; p++) { h ^= *p; h *= 0x100000001b3ull; }
    return mix64(seed ^ mix64(h));
}

void fill_codes_key(cudaStream_t st, uint8_t *dst, uint64_t key, size_t count)
{
    G5B_LAUNCH(fill_codes_kernel, 1184, 256, 0, st, reinterpret_cast<uint32_t *>(dst), key, count / 4);
}

// BF16 values with a bell-shaped distribution made of integer arithmetic only: the sum of the four
// 16-bit fields of the element's hash, centred, times `mul` (one float rounding), rounded to BF16 -
// every step is exact or a single IEEE rounding, so host and device agree to the bit.
__global__ void fill_bf16_kernel(uint16_t *dst, uint64_t key, float mul, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t h = mix64(key + i);
        const int c = (int)((h & 0xffffu) + ((h >> 16) & 0xffffu) + ((h >> 32) & 0xffffu) + (h >> 48)) - 131070;
        dst[i] = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn((float)c, mul)));
    }
}
void fill_bf16_key(cudaStream_t st, uint16_t *dst, uint64_t key, float mul, size_t count)
{
    G5B_LAUNCH(fill_bf16_kernel, 1184, 256, 0, st, dst, key, mul, count);
}

// The same values as FP32 (each exactly representable in BF16): synthetic session state.
__global__ void fill_f32_kernel(float *dst, uint64_t key, float mul, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t h = mix64(key + i);
        const int c = (int)((h & 0xffffu) + ((h >> 16) & 0xffffu) + ((h >> 32) & 0xffffu) + (h >> 48)) - 131070;
        dst[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn((float)c, mul)));
    }
}
void fill_f32_key(cudaStream_t st, float *dst, uint64_t key, float mul, size_t count)
{
    G5B_LAUNCH(fill_f32_kernel, 1184, 256, 0, st, dst, key, mul, count);
}

__global__ void f32_to_bf16_kernel(uint16_t *dst, const float *src, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __bfloat16_as_ushort(__float2bfloat16_rn(src[i]));
}
void f32_to_bf16(cudaStream_t st, uint16_t *dst, const float *src, size_t n)
{
    G5B_LAUNCH(f32_to_bf16_kernel, 592, 256, 0, st, dst, src, n);
}

__global__ void bf16_to_f32_kernel(float *dst, const uint16_t *src, size_t n)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = bf16_to_f32(src[i]);
}
void bf16_to_f32(cudaStream_t st, float *dst, const uint16_t *src, size_t n)
{
    G5B_LAUNCH(bf16_to_f32_kernel, 592, 256, 0, st, dst, src, n);
}

// Flush L2 before a timed launch: overwrite the first half of a scratch buffer (each half larger
// than L2), then read the second half. The write evicts whatever the previous launch left; the
// read pass then pushes the dirty lines of the write out to HBM, so that the timed kernel starts
// with an L2 full of clean, unrelated lines and pays for no write-backs of the flush itself.
__global__ void flush_write_kernel(uint4 *buf, size_t n16)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        buf[i] = make_uint4((uint32_t)i, 0u, 0u, 0u);
}
__global__ void flush_read_kernel(const uint4 *buf, size_t n16, uint32_t *sink)
{
    uint32_t acc = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = ld_stream16(buf + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x9e3779b9u) *sink = acc;
}
void flush_l2(cudaStream_t st, void *buf, size_t bytes)
{
    const size_t half16 = bytes / 32;
    uint4 *p = static_cast<uint4 *>(buf);
    G5B_LAUNCH(flush_write_kernel, 1184, 256, 0, st, p, half16);
    G5B_LAUNCH(flush_read_kernel, 1184, 256, 0, st, p + half16, half16 - 1, reinterpret_cast<uint32_t *>(p + 2 * half16 - 1));
}

// ---------------------------------------------------------------- L2 prefetch ----
// Ask the memory system to bring [p, p + bytes) into L2 (no data reaches the SM, nothing waits):
// one bulk prefetch per 32 KB piece. Launched on a side stream while a latency-bound kernel runs,
// so that the weights of the product that follows it are already in L2.
__global__ void l2_prefetch_kernel(const uint8_t *p, size_t bytes)
{
    constexpr size_t PIECE = 32768;
    const size_t pieces = (bytes + PIECE - 1) / PIECE;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (size_t)gridDim.x * blockDim.x) {
        const size_t off = i * PIECE;
        const unsigned n = (unsigned)(((bytes - off < PIECE ? bytes - off : PIECE)) & ~(size_t)15);
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p + off), "r"(n) : "memory");
    }
}

void l2_prefetch(cudaStream_t st, const void *p, size_t bytes)
{
    if (!p || bytes < 16 || (reinterpret_cast<uintptr_t>(p) & 15)) return;
    const size_t pieces = (bytes + 32767) / 32768;
    const int blocks = (int)((pieces + 127) / 128);
    G5B_LAUNCH(l2_prefetch_kernel, blocks < 1 ? 1 : blocks, 128, 0, st, static_cast<const uint8_t *>(p), bytes);
}

}  // namespace g5b
