// kda.cu - the gated delta-rule linear attention step (KDA), everything between the input
// projections and the output projection in one kernel.
//
// Reference: glm53f_kda_layer and kda_step (src/core/glm53f_ops.c:630-755). Its device form was
// nine launches per layer and token (three k_shortconv, k_kda_prep, k_kda_decay, k_kda_read,
// k_kda_write, k_kda_out, k_onorm_gate; src/gpu/glm53f_gpu_kernels.cu:243-450) that passed over
// the 64 KB per-head state four times. Here one CTA per head does: short convolution + SiLU of
// q/k/v with the carried history, L2 norm of q and k, beta and the per-channel decay, the
// recurrence, and the gated per-head RMSNorm of the output. A thread owns one value column of
// the state and keeps it in registers, so the state is read once and written once per call
// however many tokens the call carries.
//
// The recurrence keeps the reference's order of FP32 operations (decay row i, u_j += S_ij k_i,
// S_ij += k_i u_j, o_j += S_ij q_i, ascending i, products and sums rounded separately).
#include "common.cuh"
#include "kernels.h"

namespace g5b {

struct KdaArgs {
    float *o;
    const float *q, *k, *v, *z, *braw, *gb;
    const float *q_conv, *k_conv, *v_conv, *A_log, *dt_bias, *o_norm;
    float *state;
    int T, H, D, K;
    int head0;                    // the grid covers heads head0 .. head0 + gridDim.x - 1 of the H heads
    float gate_lb, rms_eps;
    size_t seq_stride;            // floats between the states of consecutive sequences (grid.y > 1:
                                  // CTA (h, s) advances sequence s by the T positions at rows s*T ...)
    const uint16_t *f_b, *g_b;    // optional (T == 1): z and gb are computed here from lrf / lrg
    const float *lrf, *lrg;
    float *snap;                  // optional: a second state buffer (same layout) that receives the state as it
    int snap_after;               // is after position snap_after of the call (speculative decode keeps it to fall back on)
};

// conv + SiLU of one channel at one position; `past` holds K-1 previous inputs, oldest first.
__device__ __forceinline__ float conv_step(float cur, const float *w, float *past, int K)
{
    const int hist = K - 1;
    float acc = __fmul_rn(w[hist], cur);
    for (int j = 0; j < hist; j++) acc = mul_add_unfused(w[j], past[j], acc);
    for (int j = 0; j + 1 < hist; j++) past[j] = past[j + 1];
    if (hist > 0) past[hist - 1] = cur;
    return __fmul_rn(acc, sigmoid_host(acc));
}

// DS > 0: head_dim known at compile time, the state column lives in registers.
// DS == 0: any head_dim up to 512, the state column is re-read from memory.
template <int DS>
__global__ void __launch_bounds__(DS > 0 ? DS : 512) kda_core_kernel(const KdaArgs a)
{
    __shared__ float sq[512], sk[512], sal[512];
    __shared__ double red[32];
    const int h = a.head0 + blockIdx.x, d = threadIdx.x;
    const int D = DS > 0 ? DS : a.D, P = a.H * D, K = a.K, hist = K - 1;
    const bool live = d < D;
    const int ch = h * D + (live ? d : 0);
    float *state = a.state + (size_t)blockIdx.y * a.seq_stride;
    float *S = state + (size_t)h * D * D;
    float *cs = state + (size_t)a.H * D * D;
    const int row0 = blockIdx.y * a.T;                       // first activation row of this sequence

    // One new token: the two low-rank up-projections z = f_b lrf, gb = g_b lrg of this head's channels
    // are taken here. Their 2 x D rows of D BF16 are copied to shared memory asynchronously first
    // thing (16-byte pieces, a warp reads consecutive pieces of consecutive rows), so they travel
    // beside the state; each thread later multiplies the two rows of its own channel.
    extern __shared__ __align__(16) uint8_t lrw[];               // [2 D][pitch]: f_b rows, then g_b rows
    const int pitch = 2 * D + 16;                                // 16 bytes of padding: rows fall on different banks
    if (a.f_b) {
        const int per_row = D / 8;
        for (int i = d; i < 2 * D * per_row; i += (int)blockDim.x) {
            const int row = i / per_row, piece = i % per_row;
            const uint16_t *src = (row < D ? a.f_b : a.g_b) + ((size_t)h * D + (row < D ? row : row - D)) * D + piece * 8;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(lrw + (size_t)row * pitch + piece * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    float pq[16], pk[16], pv[16], wq[17], wk[17], wv[17];
    for (int j = 0; j < hist; j++) {
        pq[j] = cs[(size_t)ch * hist + j];
        pk[j] = cs[(size_t)P * hist + (size_t)ch * hist + j];
        pv[j] = cs[(size_t)2 * P * hist + (size_t)ch * hist + j];
    }
    for (int j = 0; j < K; j++) {
        wq[j] = a.q_conv[(size_t)ch * K + j];
        wk[j] = a.k_conv[(size_t)ch * K + j];
        wv[j] = a.v_conv[(size_t)ch * K + j];
    }
    float sreg[DS > 0 ? DS : 1];
    if (DS > 0) {
#pragma unroll
        for (int i = 0; i < DS; i++) sreg[i] = S[(size_t)i * DS + d];
    }
    // Everything above reads weights and this layer's own state. From here on the projections of the
    // kernel before this one are read: when this grid was launched early (programmatic stream
    // serialization), wait until that grid has completed and its results are visible.
    pdl_wait();
    // (the low-rank rows requested above have landed by now, under the state's and the histories' loads)
    float z_own = 0.f, gb_own = 0.f;
    if (a.f_b) {
        if (live) { sq[d] = a.lrf[d]; sk[d] = a.lrg[d]; }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        if (live) {
            const uint8_t *fr = lrw + (size_t)d * pitch, *gr = lrw + (size_t)(D + d) * pitch;
            float z0 = 0.f, z1 = 0.f, g0 = 0.f, g1 = 0.f;
#pragma unroll 4
            for (int c = 0; c < D; c += 8) {
                const uint4 fw = *reinterpret_cast<const uint4 *>(fr + 2 * c), gw = *reinterpret_cast<const uint4 *>(gr + 2 * c);
                const uint32_t fu[4] = {fw.x, fw.y, fw.z, fw.w}, gu[4] = {gw.x, gw.y, gw.z, gw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float lo, hi;
                    bf16x2_to_f32(fu[j], lo, hi);
                    z0 = fmaf(lo, sq[c + 2 * j], z0); z1 = fmaf(hi, sq[c + 2 * j + 1], z1);
                    bf16x2_to_f32(gu[j], lo, hi);
                    g0 = fmaf(lo, sk[c + 2 * j], g0); g1 = fmaf(hi, sk[c + 2 * j + 1], g1);
                }
            }
            z_own = z0 + z1; gb_own = g0 + g1;
        }
        __syncthreads();
    }
    const float ea = expf_host(a.A_log[h]);
    const float dtb = a.dt_bias[ch], onw = a.o_norm[live ? d : 0];
    const float qscale = 1.0f / sqrtf((float)D);

    for (int t = 0; t < a.T; t++) {
        const size_t off = (size_t)(row0 + t) * P + ch;
        float qv = 0.f, kv = 0.f, vv = 0.f;
        if (live) {
            qv = conv_step(a.q[off], wq, pq, K);
            kv = conv_step(a.k[off], wk, pk, K);
            vv = conv_step(a.v[off], wv, pv, K);
        }
        // l2norm: divide by sqrt(sum of squares + 1e-6), sums in FP64 (glm53f_ops.c:661-667)
        const double qq = block_sum(live ? (double)qv * (double)qv : 0.0, red);
        const double kk = block_sum(live ? (double)kv * (double)kv : 0.0, red);
        const float qinv = (float)(1.0 / sqrt(qq + (double)1e-6f));
        const float kinv = (float)(1.0 / sqrt(kk + (double)1e-6f));
        const float beta = sigmoid_host(a.braw[(size_t)(row0 + t) * a.H + h]);
        __syncthreads();
        if (live) {
            sq[d] = __fmul_rn(__fmul_rn(qv, qinv), qscale);
            sk[d] = __fmul_rn(kv, kinv);
            const float g = __fmul_rn(a.gate_lb, sigmoid_host(__fmul_rn(ea, __fadd_rn(a.f_b ? z_own : a.z[off], dtb))));
            sal[d] = expf_host(g);
        }
        __syncthreads();

        float ov = 0.f;
        if (live) {
            float u = 0.f;
            if (DS > 0) {
#pragma unroll
                for (int i = 0; i < DS; i++) {
                    sreg[i] = __fmul_rn(sreg[i], sal[i]);
                    u = __fadd_rn(u, __fmul_rn(sreg[i], sk[i]));
                }
                u = __fmul_rn(__fsub_rn(vv, u), beta);
#pragma unroll
                for (int i = 0; i < DS; i++) {
                    sreg[i] = __fadd_rn(sreg[i], __fmul_rn(sk[i], u));
                    ov = __fadd_rn(ov, __fmul_rn(sreg[i], sq[i]));
                }
            } else {
                for (int i = 0; i < D; i++) {
                    const float s = __fmul_rn(S[(size_t)i * D + d], sal[i]);
                    S[(size_t)i * D + d] = s;
                    u = __fadd_rn(u, __fmul_rn(s, sk[i]));
                }
                u = __fmul_rn(__fsub_rn(vv, u), beta);
                for (int i = 0; i < D; i++) {
                    const float s = __fadd_rn(S[(size_t)i * D + d], __fmul_rn(sk[i], u));
                    S[(size_t)i * D + d] = s;
                    ov = __fadd_rn(ov, __fmul_rn(s, sq[i]));
                }
            }
        }
        // per-head RMSNorm with weight, then the sigmoid output gate (glm53f_ops.c:748-752)
        const double oo = block_sum(live ? (double)ov * (double)ov : 0.0, red);
        if (live) {
            const float inv = (float)(1.0 / sqrt(oo / (double)D + (double)a.rms_eps));
            const float n = __fmul_rn(onw, __fmul_rn(ov, inv));
            a.o[off] = __fmul_rn(n, sigmoid_host(a.f_b ? gb_own : a.gb[off]));
        }
        if (a.snap && t == a.snap_after && live) {
            float *sn = a.snap + (size_t)blockIdx.y * a.seq_stride;
            float *Sn = sn + (size_t)h * D * D, *cn = sn + (size_t)a.H * D * D;
            if (DS > 0) {
#pragma unroll
                for (int i = 0; i < DS; i++) Sn[(size_t)i * DS + d] = sreg[i];
            } else {
                for (int i = 0; i < D; i++) Sn[(size_t)i * D + d] = S[(size_t)i * D + d];
            }
            for (int j = 0; j < hist; j++) {
                cn[(size_t)ch * hist + j] = pq[j];
                cn[(size_t)P * hist + (size_t)ch * hist + j] = pk[j];
                cn[(size_t)2 * P * hist + (size_t)ch * hist + j] = pv[j];
            }
        }
    }

    if (live) {
        if (DS > 0) {
#pragma unroll
            for (int i = 0; i < DS; i++) S[(size_t)i * DS + d] = sreg[i];
        }
        for (int j = 0; j < hist; j++) {
            cs[(size_t)ch * hist + j] = pq[j];
            cs[(size_t)P * hist + (size_t)ch * hist + j] = pk[j];
            cs[(size_t)2 * P * hist + (size_t)ch * hist + j] = pv[j];
        }
    }
}

// Several positions of one sequence (prefill chunks, the two-position pass of speculative decode).
// Run position by position, the kernel above spends its time in what does NOT depend on the
// previous position: three convolutions with an exactly rounded SiLU, the gate's exactly rounded
// sigmoid and exponential, the l2norm sums in FP64 - about 8 us per position for a head, 0.5 ms for a
// chunk of 64. Here that part runs for all positions at once (kda_prep_kernel: one CTA per head and
// position) into scratch rows, and only the state update walks the positions (kda_scan_kernel: one
// CTA per head, the state column in registers, eight positions' vectors in shared memory at a time,
// their output norms reduced together). Every value is computed by the same operations in the
// same order as in kda_core_kernel, so the results are bit-identical.
struct KdaPrep {
    KdaArgs a;
    float *qn, *kn, *vn, *al, *beta;        // [T][P] normalised q (scaled), normalised k, v, exp(gate); [T][H] beta
};

template <int DS>
__global__ void __launch_bounds__(DS) kda_prep_kernel(const KdaPrep p)
{
    __shared__ double red[32];
    const KdaArgs &a = p.a;
    constexpr int D = DS;
    const int h = a.head0 + blockIdx.x, t = blockIdx.y, d = threadIdx.x;
    const int P = a.H * D, K = a.K, hist = K - 1;
    const int ch = h * D + d;
    const float *cs = a.state + (size_t)a.H * D * D;
    pdl_wait();
    // the K - 1 inputs before position t: earlier rows of this call, or the carried history (oldest first)
    auto conv = [&](const float *x, const float *w, const float *past) {
        float acc = __fmul_rn(w[(size_t)ch * K + hist], x[(size_t)t * P + ch]);
        for (int j = 0; j < hist; j++) {
            const int tt = t - hist + j;
            const float v = tt >= 0 ? x[(size_t)tt * P + ch] : past[(size_t)ch * hist + (hist + tt)];
            acc = mul_add_unfused(w[(size_t)ch * K + j], v, acc);
        }
        return __fmul_rn(acc, sigmoid_host(acc));
    };
    const float qv = conv(a.q, a.q_conv, cs);
    const float kv = conv(a.k, a.k_conv, cs + (size_t)P * hist);
    const float vv = conv(a.v, a.v_conv, cs + (size_t)2 * P * hist);
    const double qq = block_sum((double)qv * (double)qv, red);
    const double kk = block_sum((double)kv * (double)kv, red);
    const float qinv = (float)(1.0 / sqrt(qq + (double)1e-6f));
    const float kinv = (float)(1.0 / sqrt(kk + (double)1e-6f));
    const size_t off = (size_t)t * P + ch;
    p.qn[off] = __fmul_rn(__fmul_rn(qv, qinv), 1.0f / sqrtf((float)D));
    p.kn[off] = __fmul_rn(kv, kinv);
    p.vn[off] = vv;
    const float ea = expf_host(a.A_log[h]);
    const float g = __fmul_rn(a.gate_lb, sigmoid_host(__fmul_rn(ea, __fadd_rn(a.z[off], a.dt_bias[ch]))));
    p.al[off] = expf_host(g);
    if (d == 0) p.beta[(size_t)t * a.H + h] = sigmoid_host(a.braw[(size_t)t * a.H + h]);
}

constexpr int KDA_TB = 8;
template <int DS>
__global__ void __launch_bounds__(DS) kda_scan_kernel(const KdaPrep p)
{
    constexpr int NW = DS / 32, D = DS;
    __shared__ __align__(16) float sQ[KDA_TB][DS], sK[KDA_TB][DS], sAl[KDA_TB][DS];
    __shared__ float sV[KDA_TB][DS], sO[KDA_TB][DS], sBeta[KDA_TB];
    __shared__ double redo[KDA_TB][NW];
    const KdaArgs &a = p.a;
    const int h = a.head0 + blockIdx.x, d = threadIdx.x, lane = d & 31, wid = d >> 5;
    const int P = a.H * D, K = a.K, hist = K - 1;
    const int ch = h * D + d;
    float *S = a.state + (size_t)h * D * D;
    float *cs = a.state + (size_t)a.H * D * D;
    float sreg[DS];
#pragma unroll
    for (int i = 0; i < DS; i++) sreg[i] = S[(size_t)i * DS + d];
    const float onw = a.o_norm[d];
    pdl_wait();
    for (int t0 = 0; t0 < a.T; t0 += KDA_TB) {
        const int nt = a.T - t0 < KDA_TB ? a.T - t0 : KDA_TB;
#pragma unroll
        for (int j = 0; j < KDA_TB; j++) {
            if (j < nt) {
                const size_t off = (size_t)(t0 + j) * P + ch;
                sQ[j][d] = p.qn[off]; sK[j][d] = p.kn[off]; sAl[j][d] = p.al[off];
                sV[j][d] = p.vn[off];
                if (d == 0) sBeta[j] = p.beta[(size_t)(t0 + j) * a.H + h];
            }
        }
        __syncthreads();
        // the recurrence: this thread's column of the state through nt positions, no barrier inside
#pragma unroll 1
        for (int j = 0; j < nt; j++) {
            {
                float u = 0.f, o1 = 0.f;
                // (the vectors are read four elements at a time: every lane reads the same address, a broadcast)
                const float4 *al4 = reinterpret_cast<const float4 *>(sAl[j]), *k4 = reinterpret_cast<const float4 *>(sK[j]),
                             *q4 = reinterpret_cast<const float4 *>(sQ[j]);
#pragma unroll
                for (int i = 0; i < DS; i += 4) {
                    const float4 al = al4[i / 4], kk = k4[i / 4];
                    sreg[i] = __fmul_rn(sreg[i], al.x);         u = __fadd_rn(u, __fmul_rn(sreg[i], kk.x));
                    sreg[i + 1] = __fmul_rn(sreg[i + 1], al.y); u = __fadd_rn(u, __fmul_rn(sreg[i + 1], kk.y));
                    sreg[i + 2] = __fmul_rn(sreg[i + 2], al.z); u = __fadd_rn(u, __fmul_rn(sreg[i + 2], kk.z));
                    sreg[i + 3] = __fmul_rn(sreg[i + 3], al.w); u = __fadd_rn(u, __fmul_rn(sreg[i + 3], kk.w));
                }
                u = __fmul_rn(__fsub_rn(sV[j][d], u), sBeta[j]);
#pragma unroll
                for (int i = 0; i < DS; i += 4) {
                    const float4 kk = k4[i / 4], qq = q4[i / 4];
                    sreg[i] = __fadd_rn(sreg[i], __fmul_rn(kk.x, u));         o1 = __fadd_rn(o1, __fmul_rn(sreg[i], qq.x));
                    sreg[i + 1] = __fadd_rn(sreg[i + 1], __fmul_rn(kk.y, u)); o1 = __fadd_rn(o1, __fmul_rn(sreg[i + 1], qq.y));
                    sreg[i + 2] = __fadd_rn(sreg[i + 2], __fmul_rn(kk.z, u)); o1 = __fadd_rn(o1, __fmul_rn(sreg[i + 2], qq.z));
                    sreg[i + 3] = __fadd_rn(sreg[i + 3], __fmul_rn(kk.w, u)); o1 = __fadd_rn(o1, __fmul_rn(sreg[i + 3], qq.w));
                }
                sO[j][d] = o1;
                if (a.snap && t0 + j == a.snap_after) {
                    float *Sn = a.snap + (size_t)h * D * D;
#pragma unroll
                    for (int i = 0; i < DS; i++) Sn[(size_t)i * DS + d] = sreg[i];
                }
            }
        }
        // per-head RMSNorm with weight and the output gate of the nt positions, their sums reduced together
        // (the warp tree and warp order of block_sum)
#pragma unroll
        for (int j = 0; j < KDA_TB; j++) {
            const double woo = warp_sum(j < nt ? (double)sO[j][d] * (double)sO[j][d] : 0.0);
            if (lane == 0) redo[j][wid] = woo;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < KDA_TB; j++) {
            if (j < nt) {
                double oo = 0.0;
#pragma unroll
                for (int w = 0; w < NW; w++) oo += redo[j][w];
                const size_t off = (size_t)(t0 + j) * P + ch;
                const float inv = (float)(1.0 / sqrt(oo / (double)D + (double)a.rms_eps));
                const float n = __fmul_rn(onw, __fmul_rn(sO[j][d], inv));
                a.o[off] = __fmul_rn(n, sigmoid_host(a.gb[off]));
            }
        }
        __syncthreads();                                          // the vectors are rewritten by the next group
    }
#pragma unroll
    for (int i = 0; i < DS; i++) S[(size_t)i * DS + d] = sreg[i];
    // the convolution histories: the K - 1 inputs before position `upto` (the call's rows, older ones from the old history)
    auto histories = [&](float *dst, int upto) {
        const float *src[3] = {a.q, a.k, a.v};
        for (int part = 0; part < 3; part++) {
            float nv[16];
            for (int j = 0; j < hist; j++) {
                const int tt = upto - hist + j;
                nv[j] = tt >= 0 ? src[part][(size_t)tt * P + ch] : cs[(size_t)part * P * hist + (size_t)ch * hist + (hist + tt)];
            }
            for (int j = 0; j < hist; j++) dst[(size_t)part * P * hist + (size_t)ch * hist + j] = nv[j];
        }
    };
    if (a.snap && a.snap_after + 1 <= a.T) histories(a.snap + (size_t)a.H * D * D, a.snap_after + 1);   // before cs changes
    histories(cs, a.T);
}

void kda_core(cudaStream_t st, float *o, const float *q, const float *k, const float *v, const float *z,
              const float *braw, const float *gb, const float *q_conv, const float *k_conv,
              const float *v_conv, const float *A_log, const float *dt_bias, const float *o_norm,
              float *state, int T, const KdaShape &s, int n_seq, size_t seq_stride, const KdaLowRank *lr, int head0, int heads,
              float *snap, int snap_after, const KdaScratch *scratch)
{
    const bool fused = lr && T == 1 && n_seq <= 1 && (s.D == 64 || s.D == 128);
    KdaArgs a{o, q, k, v, z, braw, gb, q_conv, k_conv, v_conv, A_log, dt_bias, o_norm, state,
              T, s.H, s.D, s.K, head0, s.gate_lb, s.rms_eps, seq_stride,
              fused ? static_cast<const uint16_t *>(lr->f_b) : nullptr, fused ? static_cast<const uint16_t *>(lr->g_b) : nullptr,
              fused ? lr->lrf : nullptr, fused ? lr->lrg : nullptr, snap, snap_after};
    const dim3 grid(heads > 0 ? heads : s.H, n_seq < 1 ? 1 : n_seq);
    const size_t smem = fused ? (size_t)2 * s.D * (2 * s.D + 16) : 0;
    if (T > 1 && n_seq <= 1 && scratch && s.K <= 17 && (s.D == 128 || s.D == 64)) {
        // several positions: everything that does not depend on the previous position first, in parallel
        KdaPrep p{a, scratch->qn, scratch->kn, scratch->vn, scratch->al, scratch->beta};
        const dim3 pgrid(grid.x, T);
        if (s.D == 128) {
            G5B_LAUNCH_PDL(kda_prep_kernel<128>, pgrid, dim3(128), 0, st, p);
            G5B_LAUNCH(kda_scan_kernel<128>, dim3(grid.x), dim3(128), 0, st, p);
        } else {
            G5B_LAUNCH(kda_prep_kernel<64>, pgrid, dim3(64), 0, st, p);
            G5B_LAUNCH(kda_scan_kernel<64>, dim3(grid.x), dim3(64), 0, st, p);
        }
        return;
    }
    if (s.D == 128) {
        static SmemGrant grant;
        if (!dev_opt_in_smem((const void *)kda_core_kernel<128>, 2 * 128 * (2 * 128 + 16), grant)) return;
        // launched early: its CTAs load the 64 KB state and the histories while the projection kernel
        // before it drains, and wait for that kernel inside (griddepcontrol.wait above)
        G5B_LAUNCH_PDL(kda_core_kernel<128>, grid, dim3(128), smem, st, a);
    }
    else if (s.D == 64) G5B_LAUNCH(kda_core_kernel<64>, grid, 64, smem, st, a);
    else                G5B_LAUNCH(kda_core_kernel<0>, grid, ((s.D + 31) / 32) * 32, 0, st, a);
}

}  // namespace g5b
