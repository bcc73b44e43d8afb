// dot_rows.cuh - the inner loop of every matrix-vector product in the engine.
//
// A warp multiplies RW weight rows by TT activation vectors at once. Each lane streams 16-byte
// pieces of every row (16 E4M3 codes, 8 BF16 or 4 FP32 values), so a warp covers 512 contiguous
// bytes of a row per step and keeps RW independent 16-byte loads in flight per lane; the
// activation piece is loaded once and reused by all RW rows. Sums are FP32 per lane and are
// folded across the warp at the end.
//
// FP8 matrices carry one FP32 scale per (br x bc) block (element = E4M3(code) * s[i/br][j/bc],
// reference include/glm53f/glm53f.h:113-114); a 16-column piece never straddles a column block
// because the fast path requires bc % 16 == 0, and its partial sum is scaled once, the same
// factoring as the reference's matmul_f8 (src/core/glm53f_ops.c:185-228).
#pragma once

#include "common.cuh"

namespace g5b {

constexpr int RW = 4;   // weight rows a warp multiplies together

// Optional transform of the activation on the way in: RMSNorm as the reference applies it,
// y = w * (x * inv) with both products rounded to float (src/core/glm53f_ops.c:473-480).
struct XForm {
    const float *inv;   // per activation row, or nullptr
    const float *w;     // per column, or nullptr
};

template <int N>
__device__ __forceinline__ void load_x(float (&xr)[N], const float *xp, int c, float inv, const float *xw,
                                       bool scaled)
{
#pragma unroll
    for (int j = 0; j < N; j += 4) {
        const float4 v = *reinterpret_cast<const float4 *>(xp + c + j);
        xr[j] = v.x; xr[j + 1] = v.y; xr[j + 2] = v.z; xr[j + 3] = v.w;
    }
    if (scaled) {
#pragma unroll
        for (int j = 0; j < N; j++) xr[j] = __fmul_rn(xr[j], inv);
        if (xw) {
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 wv = *reinterpret_cast<const float4 *>(xw + c + j);
                xr[j] = __fmul_rn(wv.x, xr[j]);         xr[j + 1] = __fmul_rn(wv.y, xr[j + 1]);
                xr[j + 2] = __fmul_rn(wv.z, xr[j + 2]); xr[j + 3] = __fmul_rn(wv.w, xr[j + 3]);
            }
        }
    }
}

// acc[r][t] += sum over this lane's pieces of row r times activation t.
//   wrow[r]  start of weight row r (16-byte aligned); srow[r] its row of block scales (FP8)
//   xp[t]    activation vectors (16-byte aligned); xinv[t] their RMSNorm factor when xf.inv
//   pieces [p0, p1) of the row are split over the 32 lanes
template <int TT>
__device__ __forceinline__ void dot_rows(float (&acc)[RW][TT], int dt, const void *const (&wrow)[RW],
                                         const float *const (&srow)[RW], int bc,
                                         const float *const (&xp)[TT], const float (&xinv)[TT],
                                         const float *xw, bool scaled, int p0, int p1, int lane)
{
    if (dt == DT_FP8) {
#pragma unroll 2
        for (int p = p0 + lane; p < p1; p += 32) {
            const int c = p << 4;
            uint4 wv[RW];
#pragma unroll
            for (int r = 0; r < RW; r++) wv[r] = ld_stream16(static_cast<const uint8_t *>(wrow[r]) + c);
            float xr[TT][16];
#pragma unroll
            for (int t = 0; t < TT; t++) load_x<16>(xr[t], xp[t], c, xinv[t], xw, scaled);
            const int cb = c / bc;
#pragma unroll
            for (int r = 0; r < RW; r++) {
                float w[16];
                e4m3x4_to_f32(wv[r].x, w[0], w[1], w[2], w[3]);
                e4m3x4_to_f32(wv[r].y, w[4], w[5], w[6], w[7]);
                e4m3x4_to_f32(wv[r].z, w[8], w[9], w[10], w[11]);
                e4m3x4_to_f32(wv[r].w, w[12], w[13], w[14], w[15]);
                const float sc = srow[r][cb];
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        s0 = fmaf(w[j], xr[t][j], s0);
                        s1 = fmaf(w[j + 1], xr[t][j + 1], s1);
                    }
                    acc[r][t] = fmaf(s0 + s1, sc, acc[r][t]);
                }
            }
        }
    } else if (dt == DT_BF16) {
#pragma unroll 2
        for (int p = p0 + lane; p < p1; p += 32) {
            const int c = p << 3;
            uint4 wv[RW];
#pragma unroll
            for (int r = 0; r < RW; r++) wv[r] = ld_stream16(static_cast<const uint16_t *>(wrow[r]) + c);
            float xr[TT][8];
#pragma unroll
            for (int t = 0; t < TT; t++) load_x<8>(xr[t], xp[t], c, xinv[t], xw, scaled);
#pragma unroll
            for (int r = 0; r < RW; r++) {
                float w[8];
                bf16x2_to_f32(wv[r].x, w[0], w[1]); bf16x2_to_f32(wv[r].y, w[2], w[3]);
                bf16x2_to_f32(wv[r].z, w[4], w[5]); bf16x2_to_f32(wv[r].w, w[6], w[7]);
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        s0 = fmaf(w[j], xr[t][j], s0);
                        s1 = fmaf(w[j + 1], xr[t][j + 1], s1);
                    }
                    acc[r][t] += s0 + s1;
                }
            }
        }
    } else {
#pragma unroll 2
        for (int p = p0 + lane; p < p1; p += 32) {
            const int c = p << 2;
            uint4 wv[RW];
#pragma unroll
            for (int r = 0; r < RW; r++) wv[r] = ld_stream16(static_cast<const float *>(wrow[r]) + c);
            float xr[TT][4];
#pragma unroll
            for (int t = 0; t < TT; t++) load_x<4>(xr[t], xp[t], c, xinv[t], xw, scaled);
#pragma unroll
            for (int r = 0; r < RW; r++) {
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    float s = fmaf(__uint_as_float(wv[r].x), xr[t][0], 0.f);
                    s = fmaf(__uint_as_float(wv[r].y), xr[t][1], s);
                    s = fmaf(__uint_as_float(wv[r].z), xr[t][2], s);
                    s = fmaf(__uint_as_float(wv[r].w), xr[t][3], s);
                    acc[r][t] += s;
                }
            }
        }
    }
}

// Values per 16-byte piece of a row.
__host__ __device__ inline int piece_elems(int dt) { return dt == DT_FP8 ? 16 : dt == DT_BF16 ? 8 : 4; }

}  // namespace g5b
