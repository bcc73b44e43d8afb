// mla.cu - multi-head latent attention over the compressed KV cache, and the DSA indexer that
// chooses which positions a query attends to.
//
// Reference: glm53f_mla, compressed-latent branch (src/core/glm53f_ops.c:828-911) and
// glm53f_dsa_append / glm53f_dsa_select (src/core/glm53f_dsa.c:74-171). The reference's GPU
// backend had neither: it expanded keys and values on the device, attended densely and refused
// sessions past 2051 positions (src/model/glm53f_model.c:337-349). Here the cache holds only the
// kv_lora latent per position (FP32, or BF16 when the engine is told so), kv_b is folded into
// the query (W_k^T q) and into the output (W_v applied once to the weighted latent sum), and the
// indexer runs on the device: pool scoring, an exact top-k by radix selection, and an ascending
// position list that the attention kernels gather through.
//
// Sums that decide indices (pool scores) repeat the reference's order in FP64, so equal inputs
// give bit-equal scores and therefore the same selection, ties included (lower pool wins).
#include "dot_rows.cuh"
#include "kernels.h"

namespace g5b {

// Indexer state, three consecutive arrays (src/core/glm53f_dsa.c:44-53).
__device__ __forceinline__ float *st_key(float *s, int ID, int pos) { return s + (size_t)pos * ID; }
__device__ __forceinline__ float *st_gate(float *s, int ID, int cap, int pos) { return s + ((size_t)cap + pos) * ID; }
__device__ __forceinline__ float *st_pool(float *s, int ID, int cap, int pool) { return s + ((size_t)2 * cap + pool) * ID; }

__device__ __forceinline__ float latent_at(const void *latent, int bf16, size_t i)
{
    return bf16 ? bf16_to_f32(static_cast<const uint16_t *>(latent)[i]) : static_cast<const float *>(latent)[i];
}

// Batch of sequences (MlaShape::batch): token t works on sequence t's caches, at position `cached`.
__device__ __forceinline__ int pos_of(const MlaShape &s, int cached, int t) { return s.batch ? cached : cached + t; }
__device__ __forceinline__ const void *seq_latent(const void *latent, const MlaShape &s, int t)
{
    if (!s.batch) return latent;
    return s.latent_bf16 ? static_cast<const void *>(static_cast<const uint16_t *>(latent) + (size_t)t * s.lat_seq)
                         : static_cast<const void *>(static_cast<const float *>(latent) + (size_t)t * s.lat_seq);
}
__device__ __forceinline__ float *seq_idx(float *idx_state, const MlaShape &s, int t)
{
    return s.batch ? idx_state + (size_t)t * s.idx_seq : idx_state;
}

// ------------------------------------------------------------------- append ----
// Per new position: latent = RMSNorm(kv_a x) into the cache; indexer key = LayerNorm(wk x)
// (biased variance, eps 1e-6, FP64) and gate = gate x into the indexer state.
__device__ void dsa_pool_one(float *idx_state, const float *ape, int pool, int i, const MlaShape &s);

// Blocks [0, T) do the above; blocks [T, 2T) compute the RMSNorm factor of q_a's output for the same
// positions (it used to be a launch of its own). With one new position, the block also closes the
// pool that position completes (otherwise dsa_pool_kernel follows).
__global__ void __launch_bounds__(256) mla_store_kernel(
    void *latent, float *idx_state, const float *ct_raw, const float *kv_norm_w, const float *wk_raw,
    const float *gate_raw, const float *k_norm_w, const float *k_norm_b, int cached, MlaShape s,
    const float *q_raw, float *q_inv, int T, const float *ape, int pool_here)
{
    pdl_trigger();
    pdl_wait();
    __shared__ double red[32];
    if ((int)blockIdx.x >= T) {
        const int tq = blockIdx.x - T;
        const float *row = q_raw + (size_t)tq * s.q_lora;
        double ssq = 0.0;
        for (int i = threadIdx.x; i < s.q_lora; i += blockDim.x) ssq += (double)row[i] * (double)row[i];
        ssq = block_sum(ssq, red);
        if (threadIdx.x == 0) q_inv[tq] = (float)(1.0 / sqrt(ssq / (double)s.q_lora + (double)s.rms_eps));
        return;
    }
    const int t = blockIdx.x, pos = pos_of(s, cached, t);
    latent = const_cast<void *>(seq_latent(latent, s, t));
    idx_state = seq_idx(idx_state, s, t);
    const float *ct = ct_raw + (size_t)t * s.KL;
    double ss = 0.0;
    for (int i = threadIdx.x; i < s.KL; i += blockDim.x) ss += (double)ct[i] * (double)ct[i];
    ss = block_sum(ss, red);
    const float inv = (float)(1.0 / sqrt(ss / (double)s.KL + (double)s.rms_eps));
    for (int i = threadIdx.x; i < s.KL; i += blockDim.x) {
        const float v = __fmul_rn(kv_norm_w[i], __fmul_rn(ct[i], inv));
        if (s.latent_bf16) static_cast<uint16_t *>(latent)[(size_t)pos * s.KL + i] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        else               static_cast<float *>(latent)[(size_t)pos * s.KL + i] = v;
    }
    const float *raw = wk_raw + (size_t)t * s.ID;
    double sum = 0.0;
    for (int i = threadIdx.x; i < s.ID; i += blockDim.x) sum += (double)raw[i];
    const double mean = block_sum(sum, red) / (double)s.ID;
    double var = 0.0;
    for (int i = threadIdx.x; i < s.ID; i += blockDim.x) { const double d = (double)raw[i] - mean; var += d * d; }
    var = block_sum(var, red) / (double)s.ID;
    const double linv = 1.0 / sqrt(var + 1e-6);
    float *kp = st_key(idx_state, s.ID, pos), *gp = st_gate(idx_state, s.ID, s.cap, pos);
    for (int i = threadIdx.x; i < s.ID; i += blockDim.x) {
        kp[i] = mul_add_unfused((float)(((double)raw[i] - mean) * linv), k_norm_w[i], k_norm_b[i]);
        gp[i] = gate_raw[(size_t)t * s.ID + i];
    }
    if (pool_here >= 0) {                                     // this position completes a pool
        __syncthreads();                                      // its key and gate are written (same block)
        for (int i = threadIdx.x; i < s.ID; i += blockDim.x) dsa_pool_one(idx_state, ape, pool_here, i, s);
    }
}

// Pools closed by this call: per channel, softmax over the pool's (gate + ape) weights its keys.
__device__ void dsa_pool_one(float *idx_state, const float *ape, int pool, int i, const MlaShape &s)
{
    const int KP = s.KP;
    double top = -INFINITY, z = 0.0, acc = 0.0;
    for (int j = 0; j < KP; j++) {
        const double l = (double)st_gate(idx_state, s.ID, s.cap, pool * KP + j)[i] + (double)ape[j * s.ID + i];
        if (l > top) top = l;
    }
    for (int j = 0; j < KP; j++)
        z += exp((double)st_gate(idx_state, s.ID, s.cap, pool * KP + j)[i] + (double)ape[j * s.ID + i] - top);
    for (int j = 0; j < KP; j++) {
        const double p = exp((double)st_gate(idx_state, s.ID, s.cap, pool * KP + j)[i] + (double)ape[j * s.ID + i] - top) / z;
        acc = __dadd_rn(acc, __dmul_rn(p, (double)st_key(idx_state, s.ID, pool * KP + j)[i]));
    }
    st_pool(idx_state, s.ID, s.cap, pool)[i] = (float)acc;
}

__global__ void dsa_pool_kernel(float *idx_state, const float *ape, int pool0, MlaShape s)
{
    const int pool = pool0 + blockIdx.x, i = threadIdx.x;
    if (i >= s.ID) return;
    dsa_pool_one(idx_state, ape, pool, i, s);
}

void mla_store(cudaStream_t st, void *latent, float *idx_state, const float *ct_raw,
               const float *kv_norm_w, const float *wk_raw, const float *gate_raw,
               const float *k_norm_w, const float *k_norm_b, const float *ape, const float *q_raw, float *q_inv,
               int T, int cached, const MlaShape &s)
{
    const int pool0 = cached / s.KP;                                         // pools closed before this call
    const int pool1 = (cached + (s.batch ? 1 : T)) / s.KP;                   // pools closed after this call
    const int pool_here = ((T == 1 || s.batch) && pool1 > pool0) ? pool0 : -1;
    G5B_LAUNCH_PDL(mla_store_kernel, 2 * T, 256, 0, st, latent, idx_state, ct_raw, kv_norm_w, wk_raw, gate_raw,
               k_norm_w, k_norm_b, cached, s, q_raw, q_inv, T, ape, pool_here);
    if (pool1 > pool0 && pool_here < 0)
        G5B_LAUNCH(dsa_pool_kernel, pool1 - pool0, ((s.ID + 31) / 32) * 32, 0, st, idx_state, ape, pool0, s);
}

// ------------------------------------------------------------------- select ----
// score[pool] = (float) sum_h w[h]/sqrt(heads) * relu((q_h . P_pool)/sqrt(dim)), FP64, heads and
// dimensions in ascending order as the reference sums them (glm53f_dsa.c:141-157). A lane owns a
// head's dot product; lane 0 then adds the heads in order.
constexpr int DSA_WARPS = 8;
__global__ void __launch_bounds__(DSA_WARPS * 32) dsa_score_kernel(
    float *score, const float *idx_state, const float *qidx, const float *wproj, int cached, MlaShape s)
{
    extern __shared__ float dsa_smem[];
    float  *qT = dsa_smem;                                   // [ID][IH]
    double *dh = reinterpret_cast<double *>(dsa_smem + (size_t)s.ID * s.IH);   // [warps][IH]
    const int t = blockIdx.y, p = pos_of(s, cached, t);
    idx_state = seq_idx(const_cast<float *>(idx_state), s, t);
    const int np = (p + 1) / s.KP;
    if (np <= s.topk / s.KP) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *q = qidx + (size_t)t * s.IH * s.ID, *wt = wproj + (size_t)t * s.IH;
    for (int e = threadIdx.x; e < s.IH * s.ID; e += blockDim.x) qT[(e % s.ID) * s.IH + e / s.ID] = q[e];
    __syncthreads();
    const float hscale = 1.0f / sqrtf((float)s.IH), dscale = 1.0f / sqrtf((float)s.ID);
    double *mine = dh + (size_t)warp * s.IH;
    float *pks = reinterpret_cast<float *>(dh + (size_t)DSA_WARPS * s.IH) + (size_t)warp * s.ID;   // this warp's pooled key
    for (int pp = blockIdx.x * DSA_WARPS + warp; pp < np; pp += gridDim.x * DSA_WARPS) {
        const float *pk = idx_state + ((size_t)2 * s.cap + pp) * s.ID;
        // the key goes to shared memory in one coalesced load: read from global inside the dot
        // product, every one of its ID dependent steps waited for a load
        for (int i = lane; i < s.ID; i += 32) pks[i] = pk[i];
        __syncwarp();
        for (int h = lane; h < s.IH; h += 32) {
            double d = 0.0;
#pragma unroll 8
            for (int i = 0; i < s.ID; i++) d = fma((double)qT[i * s.IH + h], (double)pks[i], d);
            mine[h] = __dmul_rn(d, (double)dscale);
        }
        __syncwarp();
        if (lane == 0) {
            double acc = 0.0;
            for (int h = 0; h < s.IH; h++) {
                const double d = mine[h];
                if (d > 0.0) acc = __dadd_rn(acc, __dmul_rn(__dmul_rn((double)wt[h], (double)hscale), d));
            }
            score[(size_t)t * (s.cap / s.KP + 1) + pp] = (float)acc;
        }
        __syncwarp();
    }
}

// Exact top-k of the pool scores (score descending, pool index ascending on ties, the order of
// the reference's qsort comparator, glm53f_dsa.c:111-116), by radix selection on a 64-bit key,
// then an order-preserving compaction: kept pools ascending, each expanded to its positions, then
// the incomplete tail pool.
constexpr int TOPK_THREADS = 1024;
__device__ __forceinline__ unsigned long long rank_key(float sc, int pool)
{
    if (sc == 0.0f) sc = 0.0f;                                    // -0 and +0 compare equal
    uint32_t b = __float_as_uint(sc);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);               // ascending float order
    return ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (uint32_t)pool);
}

__global__ void __launch_bounds__(TOPK_THREADS) dsa_topk_kernel(int *sel, int *nsel, const float *score,
                                                                int cached, MlaShape s)
{
    pdl_trigger();
    pdl_wait();
    __shared__ int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int want_s;
    __shared__ int scan[TOPK_THREADS];
    const int t = blockIdx.x, p = pos_of(s, cached, t), tid = threadIdx.x;
    const int np = (p + 1) / s.KP, keep = s.topk / s.KP;
    int *out = sel + (size_t)t * (s.topk + s.KP);
    if (np <= keep) { if (tid == 0) nsel[t] = -1; return; }
    const float *sc = score + (size_t)t * (s.cap / s.KP + 1);

    // the keep-th largest key, one byte at a time from the top
    if (tid == 0) { prefix_s = 0ull; want_s = keep; }
    __syncthreads();
    for (int shift = 56; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned long long prefix = prefix_s;
        const unsigned long long mask = shift == 56 ? 0ull : (~0ull << (shift + 8));
        for (int i = tid; i < np; i += TOPK_THREADS) {
            const unsigned long long k = rank_key(sc[i], i);
            if ((k & mask) == prefix) atomicAdd(&hist[(int)((k >> shift) & 0xff)], 1);
        }
        __syncthreads();
        if (tid < 32) {
            // the digit holding the want-th largest key: lane l owns digits 255 - 8l .. 248 - 8l; a warp
            // scan over the lanes' totals, then a walk over the owning lane's eight bins
            int c[8], tot = 0;
#pragma unroll
            for (int k = 0; k < 8; k++) { c[k] = hist[255 - (8 * tid + k)]; tot += c[k]; }
            int incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += v;
            }
            const int excl = incl - tot, want = want_s;
            __syncwarp();
            if (excl < want && want <= incl) {
                int w = want - excl, dgt = 255 - 8 * tid;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    if (c[k] >= w) { dgt = 255 - (8 * tid + k); break; }
                    w -= c[k];
                    dgt = 255 - (8 * tid + k) - 1;
                }
                if (dgt < 0) dgt = 0;
                prefix_s = prefix | ((unsigned long long)dgt << shift);
                want_s = w;
            }
        }
        __syncthreads();
    }
    const unsigned long long threshold = prefix_s;     // keys are distinct: exactly `keep` are >= it

    // order-preserving compaction over pool index
    const int per = (np + TOPK_THREADS - 1) / TOPK_THREADS;
    const int lo = min(np, tid * per), hi = min(np, lo + per);
    int mine = 0;
    for (int i = lo; i < hi; i++) mine += rank_key(sc[i], i) >= threshold;
    scan[tid] = mine;
    __syncthreads();
    for (int o = 1; o < TOPK_THREADS; o <<= 1) {
        const int v = tid >= o ? scan[tid - o] : 0;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    int at = scan[tid] - mine;
    for (int i = lo; i < hi; i++)
        if (rank_key(sc[i], i) >= threshold) {
            for (int j = 0; j < s.KP; j++) out[at * s.KP + j] = i * s.KP + j;
            at++;
        }
    const int base = keep * s.KP;
    for (int j = np * s.KP + tid; j <= p; j += TOPK_THREADS) out[base + (j - np * s.KP)] = j;
    if (tid == 0) nsel[t] = base + (p - np * s.KP + 1);
}

void dsa_select(cudaStream_t st, int *sel, int *nsel, const float *idx_state, const float *qidx,
                const float *wproj, float *score, int T, int cached, const MlaShape &s)
{
    const int np_max = (cached + (s.batch ? 1 : T)) / s.KP;
    if (np_max > s.topk / s.KP) {
        const size_t smem = (size_t)s.ID * s.IH * sizeof(float) + (size_t)DSA_WARPS * s.IH * sizeof(double) +
                            (size_t)DSA_WARPS * s.ID * sizeof(float);
        int blocks = (np_max + DSA_WARPS - 1) / DSA_WARPS;
        if (blocks > 296) blocks = 296;
        G5B_LAUNCH(dsa_score_kernel, dim3(blocks, T), DSA_WARPS * 32, smem, st, score, idx_state, qidx, wproj, cached, s);
    }
    G5B_LAUNCH_PDL(dsa_topk_kernel, T, TOPK_THREADS, 0, st, sel, nsel, score, cached, s);
}

// ---------------------------------------------------------------- attention ----
__device__ __forceinline__ double mat_elem(const DMat &m, int r, int c)
{
    if (m.dt == DT_BF16) return (double)bf16_to_f32(static_cast<const uint16_t *>(m.w)[(size_t)r * m.cols + c]);
    if (m.dt == DT_FP8)
        return __dmul_rn((double)e4m3_to_f32(static_cast<const uint8_t *>(m.w)[(size_t)r * m.cols + c]),
                         (double)m.s[(size_t)(r / m.br) * m.scols + c / m.bc]);
    return (double)static_cast<const float *>(m.w)[(size_t)r * m.cols + c];
}

// qa[t][h][c] = sum_i q[t][h][i] * W_k[h][i][c] in FP64, ascending i (matmul_transposed,
// glm53f_ops.c:793-814). A thread owns a latent column.
__global__ void mla_absorb_kernel(double *qa, const float *q, const DMat kv_b, MlaShape s)
{
    const int h = blockIdx.x, t = blockIdx.y;
    const int kvd = s.qn + s.vh;
    const float *qt = q + ((size_t)t * s.H + h) * s.qn;
    for (int c = threadIdx.x; c < s.KL; c += blockDim.x) {
        double acc = 0.0;
        if (kv_b.dt == DT_BF16) {
            const uint16_t *w = static_cast<const uint16_t *>(kv_b.w) + (size_t)h * kvd * s.KL + c;
#pragma unroll 8
            for (int i = 0; i < s.qn; i++) acc = fma((double)qt[i], (double)bf16_to_f32(w[(size_t)i * s.KL]), acc);
        } else {
            for (int i = 0; i < s.qn; i++) acc = __dadd_rn(acc, __dmul_rn((double)qt[i], mat_elem(kv_b, h * kvd + i, c)));
        }
        qa[((size_t)t * s.H + h) * s.KL + c] = acc;
    }
}

// The same sums with the GPU filled: a CTA takes 128 latent columns of one head, its eight row
// groups (32 rows each at qk_nope = 256) accumulate in FP64 and are added in ascending order.
constexpr int AB_COLS = 128, AB_GROUPS = 8;
// TT queries per block (blockIdx.y = group of TT): a weight is read once for all of them; every query's
// sum is taken in the same order as alone.
template <int TT>
__global__ void __launch_bounds__(AB_COLS * AB_GROUPS) mla_absorb_split_kernel(double *qa, const float *q, const DMat kv_b,
                                                                              MlaShape s, int T)
{
    __shared__ double part[TT][AB_GROUPS][AB_COLS];
    const int h = blockIdx.x, t0 = blockIdx.y * TT, c = blockIdx.z * AB_COLS + (threadIdx.x % AB_COLS), grp = threadIdx.x / AB_COLS;
    const int kvd = s.qn + s.vh, per = s.qn / AB_GROUPS;
    const float *qt[TT];
#pragma unroll
    for (int k = 0; k < TT; k++) qt[k] = q + ((size_t)min(t0 + k, T - 1) * s.H + h) * s.qn + grp * per;   // past the last query: repeated, unused
    const uint16_t *w = static_cast<const uint16_t *>(kv_b.w) + ((size_t)h * kvd + (size_t)grp * per) * s.KL + c;
    double acc[TT];
#pragma unroll
    for (int k = 0; k < TT; k++) acc[k] = 0.0;
#pragma unroll 8
    for (int i = 0; i < per; i++) {
        const double wv = (double)bf16_to_f32(w[(size_t)i * s.KL]);
#pragma unroll
        for (int k = 0; k < TT; k++) acc[k] = fma((double)qt[k][i], wv, acc[k]);
    }
#pragma unroll
    for (int k = 0; k < TT; k++) part[k][grp][threadIdx.x % AB_COLS] = acc[k];
    __syncthreads();
    if (grp == 0) {
#pragma unroll
        for (int k = 0; k < TT; k++) {
            double sum = part[k][0][threadIdx.x];
#pragma unroll
            for (int g = 1; g < AB_GROUPS; g++) sum += part[k][g][threadIdx.x];
            if (t0 + k < T) qa[((size_t)(t0 + k) * s.H + h) * s.KL + c] = sum;
        }
    }
}

void mla_absorb(cudaStream_t st, double *qa, const float *q, const DMat &kv_b, int T, const MlaShape &s)
{
    if (kv_b.dt == DT_BF16 && s.KL % AB_COLS == 0 && s.qn % (AB_GROUPS * 8) == 0) {
        if (T >= 4) G5B_LAUNCH(mla_absorb_split_kernel<4>, dim3(s.H, (T + 3) / 4, s.KL / AB_COLS), AB_COLS * AB_GROUPS, 0, st, qa, q, kv_b, s, T);
        else        G5B_LAUNCH(mla_absorb_split_kernel<1>, dim3(s.H, T, s.KL / AB_COLS), AB_COLS * AB_GROUPS, 0, st, qa, q, kv_b, s, T);
        return;
    }
    G5B_LAUNCH(mla_absorb_kernel, dim3(s.H, T), s.KL >= 512 ? 512 : 128, 0, st, qa, q, kv_b, s);
}

// d[t][h][jj] = (qa . c_j) * scale in FP64 for the visible positions (all, or the selection).
constexpr int ATT_WARPS = 8;
__global__ void __launch_bounds__(ATT_WARPS * 32) mla_score_kernel(
    double *dsc, const double *qa, const void *latent, const int *sel, const int *nsel, int cached,
    int stride, MlaShape s)
{
    extern __shared__ double qs[];                            // [KL]
    const int h = blockIdx.y, t = blockIdx.z, p = pos_of(s, cached, t);
    latent = seq_latent(latent, s, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (blockIdx.x * ATT_WARPS >= nvis) return;
    for (int i = threadIdx.x; i < s.KL; i += blockDim.x) qs[i] = qa[((size_t)t * s.H + h) * s.KL + i];
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)s.qn);
    const int *sl = sel ? sel + (size_t)t * (s.topk + s.KP) : nullptr;
    for (int jj = blockIdx.x * ATT_WARPS + warp; jj < nvis; jj += gridDim.x * ATT_WARPS) {
        const int j = ns < 0 ? jj : sl[jj];
        double d = 0.0;
        for (int i = lane; i < s.KL; i += 32) d = fma(qs[i], (double)latent_at(latent, s.latent_bf16, (size_t)j * s.KL + i), d);
        d = warp_sum(d);
        if (lane == 0) dsc[((size_t)t * s.H + h) * stride + jj] = d * (double)scale;
    }
}

// The same scores for kv_lora = 512 with four heads per CTA: the absorbed queries of the four
// heads stay in registers (lane l holds elements 2l, 2l+1 of every 64), a latent row is loaded
// once for the four of them, and the four sums cross the warp in six exchanges instead of twenty.
constexpr int SC_HEADS = 4, SC_CHUNK = 64;
// The chunk CTA that finishes a (token, head group) last - a counter, no spinning - also takes the
// softmax statistics of its four heads (max of the unrounded scores, z of the float-rounded ones:
// src/core/glm53f_ops.c:890-903), which saves the launch that did only that.
__global__ void __launch_bounds__(256) mla_score4_kernel(double *dsc, const double *qa, const void *latent, const int *sel,
                                                         const int *nsel, int cached, int stride, MlaShape s,
                                                         double *stats, int *counters, int chunk)
{
    pdl_trigger();
    pdl_wait();
    __shared__ double ptop[8], pz[8];
    __shared__ int is_last;
    const int h0 = blockIdx.y * SC_HEADS, t = blockIdx.z, p = pos_of(s, cached, t);
    latent = seq_latent(latent, s, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const int j0 = blockIdx.x * chunk;                         // chunk = 64 or 256 positions (<= 32 per warp)
    if (j0 >= nvis) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double q[SC_HEADS][16];
#pragma unroll
    for (int hh = 0; hh < SC_HEADS; hh++)
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const double2 v = *reinterpret_cast<const double2 *>(qa + ((size_t)t * s.H + h0 + hh) * s.KL + 64 * k + 2 * lane);
            q[hh][2 * k] = v.x;
            q[hh][2 * k + 1] = v.y;
        }
    const double scale = (double)(1.0f / sqrtf((float)s.qn));
    const int *sl = sel ? sel + (size_t)t * (s.topk + s.KP) : nullptr;
    const int jend = min(j0 + chunk, nvis);
    // this warp's positions are j0 + warp + 8k; their cache rows are looked up first (lane k holds
    // row k), and four positions' latent rows are in flight at a time
    int myrow = 0;
    {
        const int jj = j0 + warp + 8 * lane;
        if (lane < chunk / 8 && jj < jend) myrow = ns < 0 ? jj : sl[jj];
    }
    auto load_row = [&](float (&c)[16], int j) {
        if (s.latent_bf16) {
            const uint32_t *row = reinterpret_cast<const uint32_t *>(static_cast<const uint16_t *>(latent) + (size_t)j * s.KL);
#pragma unroll
            for (int k = 0; k < 8; k++) bf16x2_to_f32(row[32 * k + lane], c[2 * k], c[2 * k + 1]);
        } else {
            const float2 *row = reinterpret_cast<const float2 *>(static_cast<const float *>(latent) + (size_t)j * s.KL);
#pragma unroll
            for (int k = 0; k < 8; k++) { const float2 v = row[32 * k + lane]; c[2 * k] = v.x; c[2 * k + 1] = v.y; }
        }
    };
    auto finish = [&](const float (&c)[16], int jj) {
        double a[SC_HEADS] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
        for (int k = 0; k < 16; k++) {
            const double cd = (double)c[k];
#pragma unroll
            for (int hh = 0; hh < SC_HEADS; hh++) a[hh] = fma(q[hh][k], cd, a[hh]);
        }
        // four sums across 32 lanes: halve the values a lane carries, twice, then a plain butterfly
        const bool up16 = lane & 16, up8 = lane & 8;
        const double r0 = (up16 ? a[2] : a[0]) + __shfl_xor_sync(0xffffffffu, up16 ? a[0] : a[2], 16);
        const double r1 = (up16 ? a[3] : a[1]) + __shfl_xor_sync(0xffffffffu, up16 ? a[1] : a[3], 16);
        double v = (up8 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, up8 ? r0 : r1, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 7) == 0) {
            const int hh = ((lane >> 4) << 1) | ((lane >> 3) & 1);
            dsc[((size_t)t * s.H + h0 + hh) * stride + jj] = v * scale;
        }
    };
    for (int k = 0; k < chunk / 8; k += 4) {                     // four latent rows in flight per warp
        const int jj0 = j0 + warp + 8 * k, jj1 = jj0 + 8, jj2 = jj0 + 16, jj3 = jj0 + 24;
        if (jj0 >= jend) break;
        const int row0 = __shfl_sync(0xffffffffu, myrow, k), row1 = __shfl_sync(0xffffffffu, myrow, k + 1);
        const int row2 = __shfl_sync(0xffffffffu, myrow, k + 2), row3 = __shfl_sync(0xffffffffu, myrow, k + 3);
        float c0[16], c1[16], c2[16], c3[16];
        load_row(c0, row0);
        if (jj1 < jend) load_row(c1, row1);
        if (jj2 < jend) load_row(c2, row2);
        if (jj3 < jend) load_row(c3, row3);
        finish(c0, jj0);
        if (jj1 < jend) finish(c1, jj1);
        if (jj2 < jend) finish(c2, jj2);
        if (jj3 < jend) finish(c3, jj3);
    }
    // ---- statistics by the last chunk of this (token, head group)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int *cnt = counters + (size_t)t * gridDim.y + blockIdx.y;
        const int active = (nvis + chunk - 1) / chunk;
        const int prev = atomicAdd(cnt, 1);
        is_last = prev == active - 1;
        if (is_last) *cnt = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int hh = warp >> 1, half = warp & 1;                 // two warps per head
    const double *d = dsc + ((size_t)t * s.H + h0 + hh) * stride;
    double top = -INFINITY;
    for (int jj = half * 32 + lane; jj < nvis; jj += 64) top = fmax(top, __ldcg(d + jj));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmax(top, __shfl_xor_sync(0xffffffffu, top, o));
    if (lane == 0) ptop[warp] = top;
    __syncthreads();
    top = fmax(ptop[2 * hh], ptop[2 * hh + 1]);
    double z = 0.0;
    for (int jj = half * 32 + lane; jj < nvis; jj += 64) z += exp((double)(float)__ldcg(d + jj) - top);
    z = warp_sum(z);
    if (lane == 0) pz[warp] = z;
    __syncthreads();
    if (half == 0 && lane == 0) {
        stats[((size_t)t * s.H + h0 + hh) * 2] = top;
        stats[((size_t)t * s.H + h0 + hh) * 2 + 1] = pz[2 * hh] + pz[2 * hh + 1];
    }
}

// Softmax as the reference takes it (glm53f_ops.c:890-903): max over the unrounded scores, the
// exponent of the score rounded to float, probabilities in FP64; then cb = sum_j p_j c_j with a
// thread per latent column walking the positions in ascending order.
__global__ void __launch_bounds__(512) mla_wsum_kernel(
    float *cb, double *dsc, const void *latent, const int *sel, const int *nsel, int cached,
    int stride, MlaShape s)
{
    __shared__ double red[32];
    __shared__ double zs;
    const int h = blockIdx.x, t = blockIdx.y, p = pos_of(s, cached, t);
    latent = seq_latent(latent, s, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    double *d = dsc + ((size_t)t * s.H + h) * stride;
    const int *sl = sel ? sel + (size_t)t * (s.topk + s.KP) : nullptr;

    double top = -INFINITY;
    for (int jj = threadIdx.x; jj < nvis; jj += blockDim.x) top = fmax(top, d[jj]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmax(top, __shfl_xor_sync(0xffffffffu, top, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = top;
    __syncthreads();
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) top = fmax(top, red[w]);
    __syncthreads();

    double z = 0.0;
    for (int jj = threadIdx.x; jj < nvis; jj += blockDim.x) {
        const double e = exp((double)(float)d[jj] - top);
        d[jj] = e;                                         // keep the numerator
        z += e;
    }
    z = block_sum(z, red);
    if (threadIdx.x == 0) zs = z;
    __syncthreads();
    z = zs;
    for (int jj = threadIdx.x; jj < nvis; jj += blockDim.x) d[jj] = d[jj] / z;
    __syncthreads();
    for (int i = threadIdx.x; i < s.KL; i += blockDim.x) {
        double acc = 0.0;
        for (int jj = 0; jj < nvis; jj++) {
            const int j = ns < 0 ? jj : sl[jj];
            acc = fma(d[jj], (double)latent_at(latent, s.latent_bf16, (size_t)j * s.KL + i), acc);
        }
        cb[((size_t)t * s.H + h) * s.KL + i] = (float)acc;
    }
}

// The same softmax and weighted sum spread over the whole GPU (the kernel above walks all positions
// with one CTA per head: 0.44 ms at 2051 positions). Three small launches:
//   stats   per (head, token): max of the unrounded scores and z = sum exp((double)(float)s - max)
//   chunk   per (32 positions, 8 heads, token): p_j = exp(.) / z, partial sums of p_j c_j in FP64,
//           positions ascending; the eight heads share every latent row they load
//   reduce  per (head, token, column): the chunks' partial sums added in ascending order
// The association of the FP64 sum differs from the reference's single ascending walk by the chunk
// boundaries only; the result is rounded to float once, at the end, like the reference's.
constexpr int WS_CHUNK = 32, WS_HEADS = 8, WS_THREADS = 256;

__global__ void __launch_bounds__(256) mla_softmax_stats_kernel(double *stats, const double *dsc, const int *nsel,
                                                                int cached, int stride, MlaShape s)
{
    __shared__ double red[32];
    const int h = blockIdx.x, t = blockIdx.y, p = pos_of(s, cached, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const double *d = dsc + ((size_t)t * s.H + h) * stride;
    double top = -INFINITY;
    for (int jj = threadIdx.x; jj < nvis; jj += blockDim.x) top = fmax(top, d[jj]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) top = fmax(top, __shfl_xor_sync(0xffffffffu, top, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = top;
    __syncthreads();
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) top = fmax(top, red[w]);
    __syncthreads();
    double z = 0.0;
    for (int jj = threadIdx.x; jj < nvis; jj += blockDim.x) z += exp((double)(float)d[jj] - top);
    z = block_sum(z, red);
    if (threadIdx.x == 0) {
        stats[((size_t)t * s.H + h) * 2] = top;
        stats[((size_t)t * s.H + h) * 2 + 1] = z;
    }
}

__global__ void __launch_bounds__(WS_THREADS) mla_wsum_chunk_kernel(
    double *part, const double *dsc, const double *stats, const void *latent, const int *sel, const int *nsel,
    int cached, int stride, int nchunks, MlaShape s)
{
    pdl_trigger();
    pdl_wait();
    __shared__ double pj[WS_HEADS][WS_CHUNK];
    __shared__ int idx[WS_CHUNK];
    const int chunk = blockIdx.x, h0 = blockIdx.y * WS_HEADS, t = blockIdx.z, p = pos_of(s, cached, t);
    latent = seq_latent(latent, s, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const int j0 = chunk * WS_CHUNK;
    const int cnt = min(WS_CHUNK, nvis - j0);
    const int i0 = threadIdx.x, i1 = threadIdx.x + WS_THREADS;         // this thread's two latent columns
    double acc0[WS_HEADS], acc1[WS_HEADS];
#pragma unroll
    for (int q = 0; q < WS_HEADS; q++) { acc0[q] = 0.0; acc1[q] = 0.0; }
    if (cnt > 0) {
        const int *sl = sel ? sel + (size_t)t * (s.topk + s.KP) : nullptr;
        for (int k = threadIdx.x; k < WS_HEADS * WS_CHUNK; k += WS_THREADS) {
            const int q = k / WS_CHUNK, jj = k % WS_CHUNK;
            double v = 0.0;
            if (jj < cnt) {
                const size_t hs = (size_t)t * s.H + h0 + q;
                v = exp((double)(float)dsc[hs * stride + j0 + jj] - stats[hs * 2]) / stats[hs * 2 + 1];
            }
            pj[q][jj] = v;
        }
        for (int jj = threadIdx.x; jj < WS_CHUNK; jj += WS_THREADS) idx[jj] = jj < cnt ? (ns < 0 ? j0 + jj : sl[j0 + jj]) : 0;
        __syncthreads();
#pragma unroll 8
        for (int jj = 0; jj < cnt; jj++) {
            const size_t row = (size_t)idx[jj] * s.KL;
            const double c0 = (double)latent_at(latent, s.latent_bf16, row + i0);
            const double c1 = (double)latent_at(latent, s.latent_bf16, row + i1);
#pragma unroll
            for (int q = 0; q < WS_HEADS; q++) {
                const double pv = pj[q][jj];
                acc0[q] = fma(pv, c0, acc0[q]);
                acc1[q] = fma(pv, c1, acc1[q]);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < WS_HEADS; q++) {
        double *dst = part + (((size_t)t * s.H + h0 + q) * nchunks + chunk) * s.KL;
        dst[i0] = acc0[q];
        dst[i1] = acc1[q];
    }
}

__global__ void __launch_bounds__(256) mla_wsum_reduce_kernel(float *cb, const double *part, int nchunks, int used,
                                                              int n, int KL)
{
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;                // (t, h, column)
    if (i >= n) return;
    const int th = i / KL, col = i % KL;
    const double *src = part + (size_t)th * nchunks * KL + col;
    double acc = 0.0;
    for (int c = 0; c < used; c++) acc += src[(size_t)c * KL];
    cb[i] = (float)acc;
}

void mla_attend(cudaStream_t st, float *cb, const double *qa, const void *latent, const int *sel,
                const int *nsel, double *dsc, double *part, double *stats, int *counters, int part_tokens, int T,
                int cached, const MlaShape &s)
{
    const int span = s.batch ? 1 : T;                                      // positions this call adds to a sequence
    const int nvis_max = cached + span < s.topk + s.KP ? cached + span : s.topk + s.KP;
    const int stride = s.topk + s.KP;
    int blocks = (nvis_max + ATT_WARPS - 1) / ATT_WARPS;
    if (blocks > 32) blocks = 32;
    const bool fast_score = s.KL == 512 && s.H % SC_HEADS == 0 && stats && counters;
    if (fast_score) {
        // many tokens: fewer, longer CTAs, so that loading the four absorbed queries (16 KB) is a small
        // part of a CTA's work; one token: many short CTAs, for the latency
        const int chunk = T >= 8 ? 4 * SC_CHUNK : SC_CHUNK;
        G5B_LAUNCH_PDL(mla_score4_kernel, dim3((nvis_max + chunk - 1) / chunk, s.H / SC_HEADS, T), 256, 0, st, dsc, qa,
                   latent, sel, nsel, cached, stride, s, stats, counters, chunk);
    }
    else
        G5B_LAUNCH(mla_score_kernel, dim3(blocks, s.H, T), ATT_WARPS * 32, (size_t)s.KL * sizeof(double), st, dsc, qa,
                   latent, sel, nsel, cached, stride, s);
    if (s.KL != 2 * WS_THREADS || s.H % WS_HEADS != 0 || !part || part_tokens < 1) {
        G5B_LAUNCH(mla_wsum_kernel, dim3(s.H, T), s.KL >= 512 ? 512 : 128, 0, st, cb, dsc, latent, sel, nsel, cached,
                   stride, s);
        return;
    }
    const int nchunks = (stride + WS_CHUNK - 1) / WS_CHUNK;             // the partial buffer is laid out for this many
    if (!fast_score) G5B_LAUNCH(mla_softmax_stats_kernel, dim3(s.H, T), 256, 0, st, stats, dsc, nsel, cached, stride, s);
    for (int t0 = 0; t0 < T; t0 += part_tokens) {
        const int n = T - t0 < part_tokens ? T - t0 : part_tokens;
        const int reach = s.batch ? cached + 1 : cached + t0 + n;
        const void *lat0 = latent;                                 // the kernel's token 0 is sequence t0 of a batch
        if (s.batch)
            lat0 = s.latent_bf16 ? static_cast<const void *>(static_cast<const uint16_t *>(latent) + (size_t)t0 * s.lat_seq)
                                 : static_cast<const void *>(static_cast<const float *>(latent) + (size_t)t0 * s.lat_seq);
        const int used = (((reach < stride) ? reach : stride) + WS_CHUNK - 1) / WS_CHUNK;
        G5B_LAUNCH_PDL(mla_wsum_chunk_kernel, dim3(used, s.H / WS_HEADS, n), WS_THREADS, 0, st, part,
                   dsc + (size_t)t0 * s.H * stride, stats + (size_t)t0 * s.H * 2, lat0,
                   sel ? sel + (size_t)t0 * stride : nullptr, nsel ? nsel + t0 : nullptr, s.batch ? cached : cached + t0, stride, nchunks,
                   s);
        // chunks beyond `used` were not written: reduce over the used ones only
        G5B_LAUNCH_PDL(mla_wsum_reduce_kernel, dim3((n * s.H * s.KL + 255) / 256), 256, 0, st,
                   cb + (size_t)t0 * s.H * s.KL, part, nchunks, used, n * s.H * s.KL, s.KL);
    }
}

// ------------------------------------------------- attention core on the tensor cores ----
// With the latent cache in BF16 the two contractions of the attention core - scores q~ . c_j over
// the 512 latent columns, and the weighted sum of the latent rows - are small GEMMs whose one
// operand (the cache) is already exact in BF16. The other operand is split into three BF16 terms
// (24 significant bits: the absorbed query after the 1/sqrt(d) scaling, the probabilities), so the
// products are exact and only the FP32 accumulation of mma.sync rounds (about 1e-6 relative; the
// reference, src/core/glm53f_ops.c:879-911, accumulates in FP64 and rounds the score to float).
// A CTA takes FL_POS visible positions and FL_HEADS heads of one query: it gathers the latent rows
// into shared memory once (the DSA selection is a list of row numbers), multiplies scores, takes the
// chunk's own maximum and exponentials, multiplies the weighted sum and leaves (max, sum, partial
// rows) for the reduction kernel, which rescales the chunks to the common maximum the way a
// two-pass softmax would have (the reference's max over all scores first, then the exponentials).
constexpr int FL_POS = 64, FL_HEADS = 16, FL_KL = 512, FL_PITCH = FL_KL + 8, FL_PPITCH = FL_POS + 8;
constexpr int FL_THREADS = 256;
constexpr size_t FL_SMEM = (size_t)3 * FL_HEADS * FL_PITCH * 2 + (size_t)FL_POS * FL_PITCH * 2 +
                           (size_t)FL_HEADS * FL_POS * 4 + (size_t)3 * FL_HEADS * FL_PPITCH * 2;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void *p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// v = hi + mid + lo exactly enough (24 bits), each a BF16
__device__ __forceinline__ void split3_bf16(float v, __nv_bfloat16 &hi, __nv_bfloat16 &mid, __nv_bfloat16 &lo)
{
    hi = __float2bfloat16_rn(v);
    const float e1 = v - __bfloat162float(hi);
    mid = __float2bfloat16_rn(e1);
    lo = __float2bfloat16_rn(e1 - __bfloat162float(mid));
}

// part: [T][H][nchunks][KL] floats (unnormalised partial rows); cstat: [T][H][nchunks][2] doubles
// (chunk maximum, sum of exponentials).
__global__ void __launch_bounds__(FL_THREADS) mla_flash_kernel(float *part, double *cstat, const double *qa, const void *latent,
                                                               const int *sel, const int *nsel, int cached, int nchunks, MlaShape s)
{
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t fl_smem[];
    __nv_bfloat16 *qs = reinterpret_cast<__nv_bfloat16 *>(fl_smem);                          // [3][16][FL_PITCH]
    __nv_bfloat16 *cs = qs + 3 * FL_HEADS * FL_PITCH;                                       // [64][FL_PITCH]
    float *ss = reinterpret_cast<float *>(cs + FL_POS * FL_PITCH);                          // [16][64]
    __nv_bfloat16 *ps = reinterpret_cast<__nv_bfloat16 *>(ss + FL_HEADS * FL_POS);          // [3][16][FL_PPITCH]
    const int chunk = blockIdx.x, h0 = blockIdx.y * FL_HEADS, t = blockIdx.z, p = pos_of(s, cached, t);
    const uint16_t *lat = static_cast<const uint16_t *>(seq_latent(latent, s, t));
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const int j0 = chunk * FL_POS;
    if (j0 >= nvis) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int *sl = sel ? sel + (size_t)t * (s.topk + s.KP) : nullptr;

    // ---- the chunk's latent rows (16-byte pieces, four threads per row); rows past the last visible
    // position are zero so that nothing undefined enters a product
    // (all of a thread's row numbers are requested first, then all of its pieces: one round trip for the
    // selection list and one for the rows, instead of a dependent pair per piece)
    {
        constexpr int PER = FL_POS * (FL_KL / 8) / FL_THREADS;
        static_assert(FL_POS * (FL_KL / 8) % FL_THREADS == 0, "pieces per thread");
        int jrow[PER];
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int jj = j0 + (tid + k * FL_THREADS) / (FL_KL / 8);
            jrow[k] = jj < nvis ? (ns < 0 ? jj : sl[jj]) : -1;
        }
        uint4 v[PER];
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int c8 = (tid + k * FL_THREADS) % (FL_KL / 8);
            v[k] = jrow[k] >= 0 ? *reinterpret_cast<const uint4 *>(lat + (size_t)jrow[k] * FL_KL + c8 * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int k = 0; k < PER; k++) {
            const int i = tid + k * FL_THREADS;
            *reinterpret_cast<uint4 *>(cs + (size_t)(i / (FL_KL / 8)) * FL_PITCH + (i % (FL_KL / 8)) * 8) = v[k];
        }
    }
    // ---- the absorbed queries of the 16 heads, scaled, as three BF16 terms
    const double scale = (double)(1.0f / sqrtf((float)s.qn));
#pragma unroll 8
    for (int i = tid; i < FL_HEADS * FL_KL; i += FL_THREADS) {
        const int hh = i / FL_KL, c = i % FL_KL;
        const float v = (float)(qa[((size_t)t * s.H + h0 + hh) * FL_KL + c] * scale);
        __nv_bfloat16 a, b, d;
        split3_bf16(v, a, b, d);
        qs[(0 * FL_HEADS + hh) * FL_PITCH + c] = a;
        qs[(1 * FL_HEADS + hh) * FL_PITCH + c] = b;
        qs[(2 * FL_HEADS + hh) * FL_PITCH + c] = d;
    }
    __syncthreads();

    // ---- scores: warp w takes positions 8w..8w+7 of the chunk, all 16 heads, all 512 columns
    {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        const __nv_bfloat16 *brow = cs + (size_t)(warp * 8 + (lane & 7)) * FL_PITCH + 8 * ((lane >> 3) & 1);
        const __nv_bfloat16 *arow = qs + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * FL_PITCH + 8 * (lane >> 4);
#pragma unroll 4
        for (int k0 = 0; k0 < FL_KL; k0 += 16) {
            uint32_t b[2];
            ldsm_x2(b, brow + k0);
#pragma unroll
            for (int term = 0; term < 3; term++) {
                uint32_t a[4];
                ldsm_x4(a, arow + (size_t)term * FL_HEADS * FL_PITCH + k0);
                mma_bf16(c, a, b);
            }
        }
        const int r = lane >> 2, col = warp * 8 + 2 * (lane & 3);
        ss[r * FL_POS + col] = c[0]; ss[r * FL_POS + col + 1] = c[1];
        ss[(r + 8) * FL_POS + col] = c[2]; ss[(r + 8) * FL_POS + col + 1] = c[3];
    }
    __syncthreads();

    // ---- the chunk's maximum and exponentials: a warp takes two heads, a lane two positions
    for (int hh = warp * 2; hh < warp * 2 + 2; hh++) {
        const int ja = lane, jb = lane + 32;
        const float sa = j0 + ja < nvis ? ss[hh * FL_POS + ja] : -INFINITY;
        const float sb = j0 + jb < nvis ? ss[hh * FL_POS + jb] : -INFINITY;
        float m = fmaxf(sa, sb);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const double ea = j0 + ja < nvis ? exp((double)sa - (double)m) : 0.0;
        const double eb = j0 + jb < nvis ? exp((double)sb - (double)m) : 0.0;
        const double z = warp_sum(ea + eb);
        __nv_bfloat16 a, b, d;
        split3_bf16((float)ea, a, b, d);
        ps[(0 * FL_HEADS + hh) * FL_PPITCH + ja] = a; ps[(1 * FL_HEADS + hh) * FL_PPITCH + ja] = b; ps[(2 * FL_HEADS + hh) * FL_PPITCH + ja] = d;
        split3_bf16((float)eb, a, b, d);
        ps[(0 * FL_HEADS + hh) * FL_PPITCH + jb] = a; ps[(1 * FL_HEADS + hh) * FL_PPITCH + jb] = b; ps[(2 * FL_HEADS + hh) * FL_PPITCH + jb] = d;
        if (lane == 0) {
            double *st = cstat + (((size_t)t * s.H + h0 + hh) * nchunks + chunk) * 2;
            st[0] = (double)m;
            st[1] = z;
        }
    }
    __syncthreads();

    // ---- weighted sum of the rows: warp w takes latent columns 64w..64w+63 for the 16 heads
    {
        float acc[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
        const __nv_bfloat16 *arow = ps + (size_t)((lane & 7) + 8 * ((lane >> 3) & 1)) * FL_PPITCH + 8 * (lane >> 4);
#pragma unroll
        for (int k0 = 0; k0 < FL_POS; k0 += 16) {
            uint32_t a[3][4];
#pragma unroll
            for (int term = 0; term < 3; term++) ldsm_x4(a[term], arow + (size_t)term * FL_HEADS * FL_PPITCH + k0);
            const __nv_bfloat16 *brow = cs + (size_t)(k0 + (lane & 15)) * FL_PITCH + warp * 64;
#pragma unroll
            for (int n = 0; n < 8; n++) {
                uint32_t b[2];
                ldsm_x2_trans(b, brow + n * 8);
#pragma unroll
                for (int term = 0; term < 3; term++) mma_bf16(acc[n], a[term], b);
            }
        }
        const int r = lane >> 2;
        float *o0 = part + (((size_t)t * s.H + h0 + r) * nchunks + chunk) * FL_KL + warp * 64 + 2 * (lane & 3);
        float *o1 = part + (((size_t)t * s.H + h0 + r + 8) * nchunks + chunk) * FL_KL + warp * 64 + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < 8; n++) {
            *reinterpret_cast<float2 *>(o0 + n * 8) = make_float2(acc[n][0], acc[n][1]);
            *reinterpret_cast<float2 *>(o1 + n * 8) = make_float2(acc[n][2], acc[n][3]);
        }
    }
}

// cb[t][h][c] = sum_chunks e^(m_c - M) part_c[c] / sum_chunks e^(m_c - M) z_c, chunks ascending, FP64.
// The chunk weights are computed once per (query, head) - one exponential per chunk, by as many
// threads - and shared; a thread then owns latent columns.
constexpr int FL_MAX_CHUNKS = 64;
__global__ void __launch_bounds__(FL_KL) mla_flash_reduce_kernel(float *cb, const float *part, const double *cstat, const int *nsel,
                                                               int cached, int nchunks, MlaShape s)
{
    pdl_trigger();
    pdl_wait();
    __shared__ double s_m[FL_MAX_CHUNKS], s_w[FL_MAX_CHUNKS];
    __shared__ double s_z;
    const int h = blockIdx.x, t = blockIdx.y, p = pos_of(s, cached, t);
    const int ns = nsel ? nsel[t] : -1;
    const int nvis = ns < 0 ? p + 1 : ns;
    const int used = (nvis + FL_POS - 1) / FL_POS;
    const double *st = cstat + ((size_t)t * s.H + h) * nchunks * 2;
    double zc = 0.0;
    if ((int)threadIdx.x < used) { s_m[threadIdx.x] = st[2 * threadIdx.x]; zc = st[2 * threadIdx.x + 1]; }
    __syncthreads();
    double M = -INFINITY;
    for (int c = 0; c < used; c++) M = fmax(M, s_m[c]);
    if ((int)threadIdx.x < used) s_w[threadIdx.x] = exp(s_m[threadIdx.x] - M);
    __syncthreads();
    if ((int)threadIdx.x < used) s_m[threadIdx.x] = s_w[threadIdx.x] * zc;       // reuse: the chunk's share of the denominator
    __syncthreads();
    if (threadIdx.x == 0) {
        double Z = 0.0;
        for (int c = 0; c < used; c++) Z += s_m[c];
        s_z = Z;
    }
    __syncthreads();
    const double Z = s_z;
    const float *pr = part + ((size_t)t * s.H + h) * nchunks * FL_KL;
    for (int col = threadIdx.x; col < FL_KL; col += blockDim.x) {
        double acc = 0.0;
        for (int c0 = 0; c0 < used; c0 += 8) {                 // eight chunks' rows requested before the first is used
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = c0 + i < used ? __ldcg(pr + (size_t)(c0 + i) * FL_KL + col) : 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) if (c0 + i < used) acc = fma(s_w[c0 + i], (double)v[i], acc);
        }
        cb[((size_t)t * s.H + h) * FL_KL + col] = (float)(acc / Z);
    }
}

bool mla_flash_takes(const MlaShape &s)
{
    return s.latent_bf16 && s.KL == FL_KL && s.H % FL_HEADS == 0 && (s.topk + s.KP + FL_POS - 1) / FL_POS <= FL_MAX_CHUNKS;
}

// scratch: `part_bytes` bytes for the partial rows; `cstat` room for [T][H][nchunks][2] doubles.
void mla_attend_flash(cudaStream_t st, float *cb, const double *qa, const void *latent, const int *sel, const int *nsel,
                      void *part, size_t part_bytes, double *cstat, int T, int cached, const MlaShape &s)
{
    static SmemGrant grant;
    if (!dev_opt_in_smem((const void *)mla_flash_kernel, FL_SMEM, grant)) return;
    const int stride = s.topk + s.KP;
    const int nchunks = (stride + FL_POS - 1) / FL_POS;
    const size_t per_token = (size_t)s.H * nchunks * FL_KL * sizeof(float);
    int group = (int)(part_bytes / per_token);
    if (group < 1) group = 1;
    for (int t0 = 0; t0 < T; t0 += group) {
        const int n = T - t0 < group ? T - t0 : group;
        const int reach = s.batch ? cached + 1 : cached + t0 + n;
        const int used = (((reach < stride) ? reach : stride) + FL_POS - 1) / FL_POS;
        const void *lat0 = latent;                                 // the kernel's token 0 is sequence t0 of a batch
        if (s.batch) lat0 = static_cast<const void *>(static_cast<const uint16_t *>(latent) + (size_t)t0 * s.lat_seq);
        G5B_LAUNCH_PDL(mla_flash_kernel, dim3(used, s.H / FL_HEADS, n), FL_THREADS, FL_SMEM, st, static_cast<float *>(part), cstat,
                       qa + (size_t)t0 * s.H * s.KL, lat0, sel ? sel + (size_t)t0 * stride : nullptr, nsel ? nsel + t0 : nullptr,
                       s.batch ? cached : cached + t0, nchunks, s);
        G5B_LAUNCH_PDL(mla_flash_reduce_kernel, dim3(s.H, n), FL_KL, 0, st, cb + (size_t)t0 * s.H * s.KL, static_cast<const float *>(part),
                       cstat, nsel ? nsel + t0 : nullptr, s.batch ? cached : cached + t0, nchunks, s);
    }
}


// o[t][h][r] = W_v[h][r] . cb[t][h]: the value half of kv_b applied once per query and head
// (glm53f_ops.c:904-909). A warp takes RW rows of one head.
// TT queries per block (blockIdx.z = group of TT): the head's rows are read once for all of them.
template <int TT>
__global__ void __launch_bounds__(256) mla_vout_kernel(float *acc_out, const float *cb, const DMat kv_b, MlaShape s, int T)
{
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.y, t0 = blockIdx.z * TT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (blockIdx.x * 8 + warp) * RW;
    if (r >= s.vh) return;
    const int kvd = s.qn + s.vh;
    const size_t rb = (size_t)s.KL * (kv_b.dt == DT_FP8 ? 1 : kv_b.dt == DT_BF16 ? 2 : 4);
    const void *wrow[RW];
    const float *srow[RW];
#pragma unroll
    for (int q = 0; q < RW; q++) {
        const int row = h * kvd + s.qn + min(r + q, s.vh - 1);
        wrow[q] = static_cast<const uint8_t *>(kv_b.w) + (size_t)row * rb;
        srow[q] = kv_b.dt == DT_FP8 ? kv_b.s + (size_t)(row / kv_b.br) * kv_b.scols : nullptr;
    }
    const float *xp[TT];
    float xinv[TT];
#pragma unroll
    for (int i = 0; i < TT; i++) {
        xp[i] = cb + ((size_t)min(t0 + i, T - 1) * s.H + h) * s.KL;       // queries past the last one repeat it, unused
        xinv[i] = 1.f;
    }
    float acc[RW][TT];
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
        for (int i = 0; i < TT; i++) acc[q][i] = 0.f;
    dot_rows<TT>(acc, kv_b.dt, wrow, srow, kv_b.bc, xp, xinv, nullptr, false, 0, s.KL / piece_elems(kv_b.dt), lane);
#pragma unroll
    for (int q = 0; q < RW; q++)
#pragma unroll
        for (int i = 0; i < TT; i++) {
            const float v = warp_sum(acc[q][i]);
            if (lane == 0 && r + q < s.vh && t0 + i < T) acc_out[((size_t)(t0 + i) * s.H + h) * s.vh + r + q] = v;
        }
}

// Same product for shapes the streaming loop cannot take (ragged columns, tiny FP8 blocks).
__global__ void mla_vout_any_kernel(float *acc_out, const float *cb, const DMat kv_b, MlaShape s)
{
    const int h = blockIdx.y, t = blockIdx.z;
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= s.vh) return;
    const int row = h * (s.qn + s.vh) + s.qn + r;
    const float *x = cb + ((size_t)t * s.H + h) * s.KL;
    double acc = 0.0;
    for (int c = 0; c < s.KL; c++) acc += mat_elem(kv_b, row, c) * (double)x[c];
    acc_out[((size_t)t * s.H + h) * s.vh + r] = (float)acc;
}

void mla_vout(cudaStream_t st, float *acc_out, const float *cb, const DMat &kv_b, int T, const MlaShape &s)
{
    const bool fast = s.KL % piece_elems(kv_b.dt) == 0 && (kv_b.dt != DT_FP8 || kv_b.bc % 16 == 0);
    if (fast && T >= 4) G5B_LAUNCH_PDL(mla_vout_kernel<4>, dim3((s.vh + 8 * RW - 1) / (8 * RW), s.H, (T + 3) / 4), 256, 0, st, acc_out, cb, kv_b, s, T);
    else if (fast)      G5B_LAUNCH_PDL(mla_vout_kernel<1>, dim3((s.vh + 8 * RW - 1) / (8 * RW), s.H, T), 256, 0, st, acc_out, cb, kv_b, s, T);
    else      G5B_LAUNCH(mla_vout_any_kernel, dim3((s.vh + 63) / 64, s.H, T), 64, 0, st, acc_out, cb, kv_b, s);
}

}  // namespace g5b
