// gemv.cu - y[T][rows] = W x[T][cols] for FP32, BF16 and block-scaled FP8 matrices.
//
// Replaces the reference's glm53f_mm / glm53f_mm_batch (src/core/glm53f_ops.c:378-458) and its
// device kernels k_mv_f32 / k_mv_bf16 / k_mv_f8 (src/gpu/glm53f_gpu_kernels.cu:35-110), which
// used one thread per output and, outside "exact" mode, dequantised every matrix to FP32 for
// cuBLAS. Here the codes are multiplied where they lie: HBM traffic is the stored bytes, once.
//
// Several products that share nothing but the launch (q/k/v/b/f_a/g_a of a KDA layer, the five
// MLA input projections) go out as ONE grid: each segment owns a range of blocks.
#include "dot_rows.cuh"
#include "kernels.h"

namespace g5b {

struct GemvBatch {
    GemvSeg s[GEMV_MAX_SEG];
    int n, T;
};

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// Fast path: columns a multiple of the 16-byte piece, FP8 column blocks a multiple of 16.
template <int TT>
__global__ void __launch_bounds__(GEMV_THREADS, TT == 1 ? 3 : 2) gemv_fast_kernel(const GemvBatch b)
{
    pdl_trigger();      // a kernel launched early behind this one waits for this grid inside
    pdl_wait();         // and so does this one when it was launched early itself
    int si = 0;
#pragma unroll 1
    for (int i = 1; i < b.n; i++)
        if ((int)blockIdx.x >= b.s[i].block0) si = i;
    const GemvSeg &g = b.s[si];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x - g.block0;
    const int pieces = g.C / piece_elems(g.dt);
    const size_t row_bytes = (size_t)g.ldw * (g.dt == DT_FP8 ? 1 : g.dt == DT_BF16 ? 2 : 4);

    int r0, p0, p1;
    if (g.ksplit) {                               // the CTA's 8 warps split the columns of RW rows
        r0 = blk * RW;
        const int per = (pieces + GEMV_WARPS - 1) / GEMV_WARPS;
        p0 = warp * per;
        p1 = min(pieces, p0 + per);
    } else {                                      // every warp owns RW whole rows
        r0 = (blk * GEMV_WARPS + warp) * RW;
        p0 = 0;
        p1 = pieces;
    }
    if (!g.ksplit && r0 >= g.R) return;

    const void  *wrow[RW];
    const float *srow[RW];
#pragma unroll
    for (int r = 0; r < RW; r++) {
        const int row = min(r0 + r, g.R - 1);     // rows past the end repeat the last one, unwritten
        wrow[r] = static_cast<const uint8_t *>(g.W) + (size_t)row * row_bytes;
        srow[r] = g.dt == DT_FP8 ? g.S + (size_t)(row / g.br) * g.scols : nullptr;
    }

    __shared__ float red[GEMV_WARPS][RW * TT];
    for (int t0 = 0; t0 < b.T; t0 += TT) {
        const float *xp[TT];
        float xinv[TT];
#pragma unroll
        for (int t = 0; t < TT; t++) {
            const int tt = min(t0 + t, b.T - 1);
            xp[t] = g.x + (size_t)tt * g.ldx;
            xinv[t] = g.xinv ? g.xinv[tt] : 1.0f;
        }
        float acc[RW][TT];
#pragma unroll
        for (int r = 0; r < RW; r++)
#pragma unroll
            for (int t = 0; t < TT; t++) acc[r][t] = 0.f;
        dot_rows<TT>(acc, g.dt, wrow, srow, g.bc, xp, xinv, g.xw, g.xinv != nullptr, p0, p1, lane);
#pragma unroll
        for (int r = 0; r < RW; r++)
#pragma unroll
            for (int t = 0; t < TT; t++) acc[r][t] = warp_sum(acc[r][t]);

        if (g.ksplit) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < RW; r++)
#pragma unroll
                    for (int t = 0; t < TT; t++) red[warp][r * TT + t] = acc[r][t];
            }
            __syncthreads();
            if (threadIdx.x < RW * TT) {
                const int r = threadIdx.x / TT, t = threadIdx.x % TT;
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < GEMV_WARPS; w++) s += red[w][threadIdx.x];
                if (r0 + r < g.R && t0 + t < b.T) g.y[(size_t)(t0 + t) * g.ldy + r0 + r] = s;
            }
            __syncthreads();
        } else if (lane == 0) {
#pragma unroll
            for (int r = 0; r < RW; r++)
#pragma unroll
                for (int t = 0; t < TT; t++)
                    if (r0 + r < g.R && t0 + t < b.T) g.y[(size_t)(t0 + t) * g.ldy + r0 + r] = acc[r][t];
        }
    }
}

// Any shape, any block size (the reference's 4x4-block test fixture, ragged columns): a warp per
// row, lanes stride the columns, FP64 sums.
__global__ void __launch_bounds__(GEMV_THREADS) gemv_any_kernel(const GemvBatch b)
{
    int si = 0;
#pragma unroll 1
    for (int i = 1; i < b.n; i++)
        if ((int)blockIdx.x >= b.s[i].block0) si = i;
    const GemvSeg &g = b.s[si];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = (blockIdx.x - g.block0) * GEMV_WARPS + warp;
    if (row >= g.R) return;
    for (int t = 0; t < b.T; t++) {
        const float *x = g.x + (size_t)t * g.ldx;
        const float inv = g.xinv ? g.xinv[t] : 1.0f;
        double acc = 0.0;
        for (int c = lane; c < g.C; c += 32) {
            float xv = x[c];
            if (g.xinv) {
                xv = __fmul_rn(xv, inv);
                if (g.xw) xv = __fmul_rn(g.xw[c], xv);
            }
            double wv;
            if (g.dt == DT_FP8)
                wv = (double)e4m3_to_f32(static_cast<const uint8_t *>(g.W)[(size_t)row * g.ldw + c]) *
                     (double)g.S[(size_t)(row / g.br) * g.scols + c / g.bc];
            else if (g.dt == DT_BF16)
                wv = (double)bf16_to_f32(static_cast<const uint16_t *>(g.W)[(size_t)row * g.ldw + c]);
            else
                wv = (double)static_cast<const float *>(g.W)[(size_t)row * g.ldw + c];
            acc += wv * (double)xv;
        }
        acc = warp_sum(acc);
        if (lane == 0) g.y[(size_t)t * g.ldy + row] = (float)acc;
    }
}

GemvSeg make_seg(const DMat &m, const float *x, int ldx, float *y, int ldy, const float *xinv,
                 const float *xw)
{
    GemvSeg s;
    s.W = m.w; s.S = m.s; s.x = x; s.xinv = xinv; s.xw = xw; s.y = y;
    s.dt = m.dt; s.R = m.rows; s.C = m.cols; s.br = m.br; s.bc = m.bc; s.scols = m.scols;
    s.ldx = ldx; s.ldy = ldy;
    s.ldw = m.ld ? m.ld : m.cols;
    s.ksplit = 0; s.block0 = 0;
    return s;
}

DMat row_slice(const DMat &m, int r0, int n)
{
    DMat s = m;
    s.rows = n;
    const size_t eb = m.dt == DT_FP8 ? 1 : m.dt == DT_BF16 ? 2 : 4;
    s.w = static_cast<uint8_t *>(m.w) + (size_t)r0 * (m.ld ? m.ld : m.cols) * eb;
    if (m.dt == DT_FP8) s.s = m.s + (size_t)(r0 / m.br) * m.scols;
    return s;
}

DMat col_slice(const DMat &m, int c0, int n)
{
    DMat s = m;
    s.cols = n;
    s.ld = m.ld ? m.ld : m.cols;
    const size_t eb = m.dt == DT_FP8 ? 1 : m.dt == DT_BF16 ? 2 : 4;
    s.w = static_cast<uint8_t *>(m.w) + (size_t)c0 * eb;
    if (m.dt == DT_FP8) s.s = m.s + c0 / m.bc;          // same scale-row pitch (scols) as the parent
    return s;
}

static bool seg_is_fast(const GemvSeg &s)
{
    const int pe = piece_elems(s.dt);
    if (s.C % pe || s.ldw % pe) return false;
    if (s.dt == DT_FP8 && (s.bc % 16 || s.br < 1)) return false;
    if ((reinterpret_cast<uintptr_t>(s.W) & 15) || (reinterpret_cast<uintptr_t>(s.x) & 15) || (s.ldx & 3))
        return false;
    if (s.xw && (reinterpret_cast<uintptr_t>(s.xw) & 15)) return false;
    return true;
}

void gemv_batch(cudaStream_t st, const GemvSeg *segs, int n, int T, bool early)
{
    GemvBatch fast, any;
    fast.n = any.n = 0;
    fast.T = any.T = T;
    int fb = 0, ab = 0;
    for (int i = 0; i < n; i++) {
        GemvSeg s = segs[i];
        if (seg_is_fast(s)) {
            // Matrices whose whole-row grid would not even give every SM a CTA take one CTA per RW
            // rows, the eight warps splitting the columns, provided a row gives every lane a piece
            // (measured: with 256 whole-row CTAs available the split is the slower of the two).
            const long bytes = (long)s.R * s.C;
            const int pieces = s.C / piece_elems(s.dt);
            const int whole_row_blocks = (s.R + RW * GEMV_WARPS - 1) / (RW * GEMV_WARPS);
            s.ksplit = (bytes >= 32768 && pieces >= 64 &&
                        (s.R <= 1024 || (pieces >= GEMV_THREADS && whole_row_blocks < 148))) ? 1 : 0;
            s.block0 = fb;
            fb += s.ksplit ? (s.R + RW - 1) / RW : (s.R + RW * GEMV_WARPS - 1) / (RW * GEMV_WARPS);
            fast.s[fast.n++] = s;
        } else {
            s.block0 = ab;
            ab += (s.R + GEMV_WARPS - 1) / GEMV_WARPS;
            any.s[any.n++] = s;
        }
    }
    if (fast.n) {
        if (T == 1 && early) G5B_LAUNCH_PDL(gemv_fast_kernel<1>, fb, GEMV_THREADS, 0, st, fast);
        else if (T == 1) G5B_LAUNCH(gemv_fast_kernel<1>, fb, GEMV_THREADS, 0, st, fast);
        else if (T == 2) G5B_LAUNCH(gemv_fast_kernel<2>, fb, GEMV_THREADS, 0, st, fast);
        else             G5B_LAUNCH(gemv_fast_kernel<4>, fb, GEMV_THREADS, 0, st, fast);
    }
    if (any.n) G5B_LAUNCH(gemv_any_kernel, ab, GEMV_THREADS, 0, st, any);
}

}  // namespace g5b
