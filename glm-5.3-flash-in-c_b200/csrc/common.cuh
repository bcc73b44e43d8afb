// common.cuh - device helpers shared by every kernel file of libglm53f_b200 (sm_100a only).
//
// Number formats follow the reference engine (josesilva05/glm-5.3-flash-in-c):
//   E4M3FN decode  src/core/glm53f_ops.c:51-72   (bias 7, subnormals, s.1111.111 = NaN, no inf)
//   BF16 widen     include/glm53f/glm53f.h:150-155 (a 16-bit left shift)
//   sigmoid        src/core/glm53f_ops.c:46       (1.0f / (1.0f + expf(-x)), three float roundings)
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace g5b {

constexpr int DT_F32 = 0, DT_BF16 = 1, DT_FP8 = 2;
constexpr int WARP = 32;

// Host-side count of kernels launched by this library (reported by the benchmark).
extern unsigned long long g_launches;

#define G5B_LAUNCH(kernel, grid, block, smem, stream, ...)                     \
    do {                                                                       \
        kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);            \
        ++::g5b::g_launches;                                                   \
    } while (0)

// The same launch with programmatic stream serialization: the grid may be scheduled while the
// kernel before it in the stream is still draining (once all of that kernel's CTAs have passed
// pdl_trigger() or exited), so its launch latency and whatever it does before pdl_wait() overlap
// that kernel's tail. Only for kernels that call pdl_wait() before they read anything an earlier
// kernel wrote. (A kernel launched the ordinary way may call both: they do nothing then.)
#define G5B_LAUNCH_PDL(kernel, grid, block, smem, strm_, ...)                                      \
    do {                                                                                        \
        cudaLaunchConfig_t cfg_{};                                                              \
        cfg_.gridDim = (grid); cfg_.blockDim = (block);                                         \
        cfg_.dynamicSmemBytes = (smem); cfg_.stream = (strm_);                                  \
        cudaLaunchAttribute at_[1];                                                             \
        at_[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                         \
        at_[0].val.programmaticStreamSerializationAllowed = 1;                                  \
        cfg_.attrs = at_; cfg_.numAttrs = 1;                                                    \
        if (cudaLaunchKernelEx(&cfg_, kernel, __VA_ARGS__) != cudaSuccess) {                    \
            cudaGetLastError();                                                                 \
            kernel<<<(grid), (block), (smem), (strm_)>>>(__VA_ARGS__);                          \
        }                                                                                       \
        ++::g5b::g_launches;                                                                    \
    } while (0)

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 16-byte streaming load: weights are read once per token, so they bypass L1 allocation and
// leave it to the activations that every row re-reads.
__device__ __forceinline__ uint4 ld_stream16(const void *p)
{
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

// Four E4M3 codes (one 32-bit word, lowest byte first) to four floats, exactly: the hardware
// conversion to f16 is exact for every E4M3 value (f16 holds 2^-9 as a normal number) and
// f16 -> f32 is exact; NaN codes stay NaN.
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t w, float &a, float &b, float &c, float &d)
{
    uint32_t lo, hi;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((unsigned short)(w & 0xffffu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((unsigned short)(w >> 16)));
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&lo));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
    a = f0.x; b = f0.y; c = f1.x; d = f1.y;
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t code)
{
    float a, b, c, d;
    e4m3x4_to_f32((uint32_t)code, a, b, c, d);
    return a;
}

__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ void bf16x2_to_f32(uint32_t w, float &lo, float &hi)
{
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}

// expf as the host C library computes it: the double-precision exp rounded once to float agrees
// with a correctly rounded expf except on rare double-rounding cases.
__device__ __forceinline__ float expf_host(float x) { return (float)exp((double)x); }

// The reference's sigmoid: 1.0f / (1.0f + expf(-x)), each step rounded to float, never fused.
__device__ __forceinline__ float sigmoid_host(float x)
{
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_host(-x)));
}

// a*b + c with two float roundings, as C compiled without FMA contraction evaluates it.
__device__ __forceinline__ float mul_add_unfused(float a, float b, float c)
{
    return __fadd_rn(__fmul_rn(a, b), c);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a whole CTA (blockDim.x a multiple of 32, at most 1024). `red` holds 32 doubles of
// shared memory. Every thread receives the total; the order of the sum is fixed.
__device__ __forceinline__ double block_sum(double v, double *red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; i++) t += red[i];
    return t;
}

// System-scope acquire / release on 64-bit words that another GPU writes or reads.
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}


// One more on a 64-bit counter another GPU waits on, with release semantics at system scope.
__device__ __forceinline__ void red_release_sys_add(unsigned long long *p, unsigned long long v)
{
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Wait until the 64-bit word another GPU publishes reaches `want`. The limit is wall-clock time
// (the ranks are separate host processes: ordinary host skew must not look like a lost peer), with
// an iteration cap behind it in case the timer does not advance. False when the wait ran out.
__device__ __forceinline__ bool wait_word_sys(const unsigned long long *p, unsigned long long want,
                                              unsigned long long limit_ns)
{
    if (ld_acquire_sys(p) >= want) return true;
    const unsigned long long t0 = global_ns();
    for (long long i = 0; i < (1ll << 28); i++) {
        if (ld_acquire_sys(p) >= want) return true;
        if (global_ns() - t0 > limit_ns) return false;
        __nanosleep(100);
    }
    return false;
}

}  // namespace g5b
