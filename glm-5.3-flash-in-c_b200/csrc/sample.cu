// sample.cu - the next token drawn from the logits on the device: temperature, then nucleus
// (top-p) truncation, then one draw from a counter-based generator.
//
// The reference decodes greedily only (src/cli/glm53f_run.c:492-494 takes the arg-max on the host);
// this is the sampled counterpart, kept on the GPU so that a decode loop never returns to the host
// between steps. The definition, which tests restate in numpy on the same logits:
//   p_i    = (float) exp((double) ((l_i - max l) / temperature))             (float subtract, divide)
//   Z      = sum_i p_i                                                       (FP64)
//   tau    = the largest probability value with  sum_{p_i >= tau} p_i >= top_p * Z
//            (the nucleus is every token at least that probable; top_p >= 1 keeps all of them)
//   u      = (mix64(seed ^ mix64(step + 1)) >> 11) * 2^-53                   (in [0, 1))
//   token  = the first index i, in index order, whose running nucleus mass exceeds u * (nucleus mass)
// FP64 sums are taken in a different association on the two sides, so a draw can differ only when
// a running sum falls within rounding (1e-16 relative) of a threshold.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace g5b {

constexpr int SMP_THREADS = 1024;

__device__ __forceinline__ uint64_t smp_mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

struct SampleArgs {
    const float *logits;   // [V]
    float *prob;           // [V] scratch
    int *out;              // [1]
    int V;
    float temperature, top_p;
    uint64_t seed, step;
};

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const SampleArgs a)
{
    __shared__ double red[32];
    __shared__ double hist_mass[256];
    __shared__ unsigned hist_cnt[256];
    __shared__ float s_max;
    __shared__ unsigned s_prefix, s_digit;
    __shared__ double s_above;              // mass of the tokens strictly above the current prefix range
    __shared__ double chunk_mass[SMP_THREADS];
    __shared__ int s_owner;
    __shared__ double s_before;
    const int tid = threadIdx.x, V = a.V;

    // ---- max logit
    float m = -INFINITY;
    for (int i = tid; i < V; i += SMP_THREADS) m = fmaxf(m, a.logits[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) red[tid >> 5] = (double)m;
    __syncthreads();
    if (tid == 0) {
        float mm = -INFINITY;
        for (int i = 0; i < SMP_THREADS / 32; i++) mm = fmaxf(mm, (float)red[i]);
        s_max = mm;
    }
    __syncthreads();
    const float mx = s_max;

    // ---- probabilities (unnormalised) and their sum
    double z = 0.0;
    for (int i = tid; i < V; i += SMP_THREADS) {
        const float p = expf_host(__fdiv_rn(__fsub_rn(a.logits[i], mx), a.temperature));
        a.prob[i] = p;
        z += (double)p;
    }
    const double Z = block_sum(z, red);
    __syncthreads();

    // ---- nucleus threshold: radix select on the bits of p (p >= 0, so the bits order like the values)
    unsigned tau_bits = 0u;                 // keep everything
    if (a.top_p < 1.0f) {
        const double target = (double)a.top_p * Z;
        if (tid == 0) { s_prefix = 0u; s_above = 0.0; }
        __syncthreads();
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) { hist_mass[tid] = 0.0; hist_cnt[tid] = 0u; }
            __syncthreads();
            const unsigned prefix = s_prefix, pmask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += SMP_THREADS) {
                const float p = a.prob[i];
                const unsigned b = __float_as_uint(p);
                if ((b & pmask) == prefix) {
                    atomicAdd(&hist_mass[(b >> shift) & 255u], (double)p);
                    atomicAdd(&hist_cnt[(b >> shift) & 255u], 1u);
                }
            }
            __syncthreads();
            if (tid == 0) {
                // walk the digits from the top: the digit where the running mass reaches the target
                double run = s_above;
                int d = 255;
                for (; d > 0; d--) {
                    if (hist_cnt[d] && run + hist_mass[d] >= target) break;
                    run += hist_mass[d];
                }
                s_above = run;
                s_digit = (unsigned)d;
                s_prefix = prefix | ((unsigned)d << shift);
            }
            __syncthreads();
        }
        tau_bits = s_prefix;
    }

    // ---- the draw: nucleus mass per contiguous chunk of indices, then the chunk that holds the target
    const int chunk = (V + SMP_THREADS - 1) / SMP_THREADS;
    const int i0 = tid * chunk, i1 = min(V, i0 + chunk);
    double cm = 0.0;
    for (int i = i0; i < i1; i++) {
        const float p = a.prob[i];
        if (__float_as_uint(p) >= tau_bits) cm += (double)p;
    }
    chunk_mass[tid] = cm;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int i = 0; i < SMP_THREADS; i++) total += chunk_mass[i];
        const double u = (double)(smp_mix64(a.seed ^ smp_mix64(a.step + 1)) >> 11) * (1.0 / 9007199254740992.0);
        const double want = u * total;
        double run = 0.0;
        int owner = SMP_THREADS - 1;
        for (int i = 0; i < SMP_THREADS; i++) {
            if (run + chunk_mass[i] > want) { owner = i; break; }
            run += chunk_mass[i];
        }
        s_owner = owner;
        s_before = run;
        red[0] = want;
    }
    __syncthreads();
    if (tid == s_owner) {
        const double want = red[0];
        double run = s_before;
        int pick = -1, last = -1;
        for (int i = i0; i < i1; i++) {
            const float p = a.prob[i];
            if (__float_as_uint(p) >= tau_bits) {
                last = i;
                run += (double)p;
                if (run > want) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last >= 0 ? last : 0;      // rounding left the target just past the last member
        *a.out = pick;
    }
}

void sample_token(cudaStream_t st, int *out, const float *logits, float *prob, int V, float temperature, float top_p,
                  uint64_t seed, uint64_t step)
{
    SampleArgs a{logits, prob, out, V, temperature, top_p, seed, step};
    G5B_LAUNCH(sample_kernel, 1, SMP_THREADS, 0, st, a);
}

}  // namespace g5b
