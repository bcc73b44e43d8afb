// mma_stage.cuh - how a consumer warp multiplies one shared-memory stage of FP8 weights by the
// activation with the tensor cores. Shared by the batch-1 expert kernels.
//
// Stage: MM_ROWS rows of MM_CB codes, rows MM_PITCH bytes apart (the 64 spare bytes put the eight
// row groups of a warp in different banks). Warp = (M tile of 16 rows) x (quarter of the columns).
// Lane (g = lane / 4, t = lane % 4) loads 16 codes of rows g and g + 8; a pair of codes becomes an
// F16 pair with one conversion; mma.sync.m16n8k16 multiplies it with the activation, which sits in
// B columns 0 and 1 as two F16 terms (x = hi + mid / 2048, 22 significant bits) - the other six
// columns are zero. Which 16 physical columns stand for which logical k of an MMA does not matter
// as long as A and B agree, so each lane's 16-byte piece feeds four MMAs directly.
// Block scales are applied in FP32 whenever a scale block of bc columns ends.
#pragma once

#include "bulk.cuh"

namespace g5b {

constexpr int MM_ROWS = 32, MM_CB = 2048, MM_PITCH = MM_CB + 64, MM_NS = 3, MM_CONS = 8;
constexpr int MM_THREADS = (MM_CONS + 1) * 32;
constexpr int MM_MAX_SLOTS = 17;             // experts per token (top-k + shared) these kernels serve
constexpr int MM_MAX_ITEMS = 32;

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_codes)
{
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"((unsigned short)two_codes));
    return r;
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x = hi + mid / 2048 with hi, mid in F16: 22 significant bits of x (given |x| < 65504).
__device__ __forceinline__ void split_f16(float x, __half &hi, __half &mid)
{
    hi = __float2half_rn(x);
    mid = __float2half_rn((x - __half2float(hi)) * 2048.0f);
}

// The SwiGLU clamp bounds |silu(g) * u| by limit^2, so the activation terms of the down projection
// are stored times the largest power of two that keeps limit^2 below 2^15 (2^8 for a clamp at 10):
// small activations keep their bits in F16 and the factor comes off exactly in the down epilogue.
// Products below 2^-24 / factor still flush to zero - an absolute error far below the FP32 rounding
// of any output the layer produces from normalised activations.
__host__ __device__ __forceinline__ float act_term_scale(float limit)
{
    const float b = limit * limit;
    if (!(b > 0.f) || !(b < 32768.f)) return 1.0f;
    int ex;
    frexpf(32768.0f / b, &ex);                        // 32768 / b = m * 2^ex, 0.5 <= m < 1
    return ldexpf(1.0f, ex - 1 > 14 ? 14 : ex - 1);
}

// accf[0..1]: row g (hi, mid columns), accf[2..3]: row g + 8, meaningful in lanes with t == 0.
//   st     stage base (weights at offset 0)
//   sc     the scale row of this warp's M tile
//   xt     activation terms of this lane: term g (only g < 2 is read), element 0 = column 0 of the row
//   col0   first column (within the whole row) of the stage
__device__ __forceinline__ void mma_consume_stage(float (&accf)[4], const uint8_t *st, const float *sc,
                                                  const __half *xt, int col0, int bc, int mt, int kq, int g, int t)
{
    const uint8_t *w0p = st + (size_t)(mt * 16 + g) * MM_PITCH + kq * 512 + 16 * t;
    const uint8_t *w1p = w0p + 8 * MM_PITCH;
    const int c_lane = col0 + kq * 512 + 16 * t;
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
    // unrolled by four, not eight: as fast with a warm instruction cache and about 1 us faster when
    // the kernel runs after other kernels (cold code costs about 0.2 us per KB on the critical path)
#pragma unroll 4
    for (int step = 0; step < 8; step++) {
        const uint4 w0 = *reinterpret_cast<const uint4 *>(w0p + step * 64);
        const uint4 w1 = *reinterpret_cast<const uint4 *>(w1p + step * 64);
        uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
        if (g < 2) {
            xa = *reinterpret_cast<const uint4 *>(xt + c_lane + step * 64);
            xb = *reinterpret_cast<const uint4 *>(xt + c_lane + step * 64 + 8);
        }
        const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w}, wb[4] = {w1.x, w1.y, w1.z, w1.w};
        const uint32_t xr[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        // two accumulators: consecutive MMAs do not wait on each other
        mma_f16(c0, e4m3x2_to_f16x2(wa[0]), e4m3x2_to_f16x2(wb[0]), e4m3x2_to_f16x2(wa[0] >> 16), e4m3x2_to_f16x2(wb[0] >> 16), xr[0], xr[1]);
        mma_f16(c1, e4m3x2_to_f16x2(wa[1]), e4m3x2_to_f16x2(wb[1]), e4m3x2_to_f16x2(wa[1] >> 16), e4m3x2_to_f16x2(wb[1] >> 16), xr[2], xr[3]);
        mma_f16(c0, e4m3x2_to_f16x2(wa[2]), e4m3x2_to_f16x2(wb[2]), e4m3x2_to_f16x2(wa[2] >> 16), e4m3x2_to_f16x2(wb[2] >> 16), xr[4], xr[5]);
        mma_f16(c1, e4m3x2_to_f16x2(wa[3]), e4m3x2_to_f16x2(wb[3]), e4m3x2_to_f16x2(wa[3] >> 16), e4m3x2_to_f16x2(wb[3] >> 16), xr[6], xr[7]);
        if (((kq * 512 + (step + 1) * 64) % bc) == 0) {        // a scale block ends here
            const float sv = sc[(col0 + kq * 512 + step * 64) / bc];
#pragma unroll
            for (int i = 0; i < 4; i++) { accf[i] = fmaf(c0[i] + c1[i], sv, accf[i]); c0[i] = 0.f; c1[i] = 0.f; }
        }
    }
}

// The same stage against FOUR activation vectors: B column 2p is the hi term of vector p, column
// 2p + 1 its mid term, so all eight columns carry data and every lane loads a B fragment (row g of
// the activation tile; rows are XT_PITCH bytes apart: a lane reads two 16-byte pieces 32 bytes
// apart from its neighbour's, so the two rows of a quarter warp must sit 16 bytes off each other
// modulo 32 to use all banks once). The tile holds the columns of this stage only.
// accf[0..1]: row g, vector t (hi, mid); accf[2..3]: row g + 8 - meaningful in every lane.
constexpr int XT_PITCH = MM_CB * 2 + 16;
__device__ __forceinline__ void mma_consume_stage_x4(float (&accf)[4], const uint8_t *st, const float *sc,
                                                     const uint8_t *xtile, int col0, int bc, int mt, int kq, int g, int t)
{
    const uint8_t *w0p = st + (size_t)(mt * 16 + g) * MM_PITCH + kq * 512 + 16 * t;
    const uint8_t *w1p = w0p + 8 * MM_PITCH;
    const uint8_t *xp = xtile + (size_t)g * XT_PITCH + (size_t)(kq * 512 + 16 * t) * 2;
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int step = 0; step < 8; step++) {
        const uint4 w0 = *reinterpret_cast<const uint4 *>(w0p + step * 64);
        const uint4 w1 = *reinterpret_cast<const uint4 *>(w1p + step * 64);
        const uint4 xa = *reinterpret_cast<const uint4 *>(xp + step * 128);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xp + step * 128 + 16);
        const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w}, wb[4] = {w1.x, w1.y, w1.z, w1.w};
        const uint32_t xr[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        mma_f16(c0, e4m3x2_to_f16x2(wa[0]), e4m3x2_to_f16x2(wb[0]), e4m3x2_to_f16x2(wa[0] >> 16), e4m3x2_to_f16x2(wb[0] >> 16), xr[0], xr[1]);
        mma_f16(c1, e4m3x2_to_f16x2(wa[1]), e4m3x2_to_f16x2(wb[1]), e4m3x2_to_f16x2(wa[1] >> 16), e4m3x2_to_f16x2(wb[1] >> 16), xr[2], xr[3]);
        mma_f16(c0, e4m3x2_to_f16x2(wa[2]), e4m3x2_to_f16x2(wb[2]), e4m3x2_to_f16x2(wa[2] >> 16), e4m3x2_to_f16x2(wb[2] >> 16), xr[4], xr[5]);
        mma_f16(c1, e4m3x2_to_f16x2(wa[3]), e4m3x2_to_f16x2(wb[3]), e4m3x2_to_f16x2(wa[3] >> 16), e4m3x2_to_f16x2(wb[3] >> 16), xr[6], xr[7]);
        if (((kq * 512 + (step + 1) * 64) % bc) == 0) {        // a scale block ends here
            const float sv = sc[(col0 + kq * 512 + step * 64) / bc];
#pragma unroll
            for (int i = 0; i < 4; i++) { accf[i] = fmaf(c0[i] + c1[i], sv, accf[i]); c0[i] = 0.f; c1[i] = 0.f; }
        }
    }
}

}  // namespace g5b
