// kernels.h - launchers of the engine's CUDA kernels (internal to libglm53f_b200).
// Every launcher enqueues on the given stream and returns without waiting.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/glm53f_b200.h"

namespace g5b {

// A weight matrix resident in HBM, row-major, in its checkpoint format.
struct DMat {
    void  *w = nullptr;
    float *s = nullptr;        // FP8 block scales [ceil(rows/br)][scols]
    int    dt = 0, rows = 0, cols = 0, br = 0, bc = 0, scols = 0;
    int    ld = 0;             // elements between consecutive rows; 0 = cols (a column slice keeps its parent's)
    bool   loaded() const { return w != nullptr; }
    size_t bytes() const { return (size_t)rows * cols * (dt == 0 ? 4 : dt == 1 ? 2 : 1); }
};

// ---- device_info.cu -----------------------------------------------------------------------
// Facts about, and one-time kernel set-up on, the device that is current at the call. Nothing is
// cached across devices: a process may hold engines on several GPUs.
constexpr int G5B_MAX_DEVICES = 64;
struct SmemGrant { size_t bytes[G5B_MAX_DEVICES] = {}; };   // per kernel: what each device has granted
int  dev_now();
int  dev_sms();
bool dev_cooperative();
// Opt `kernel` into `bytes` of dynamic shared memory on the current device (again if a later call
// asks for more). False, with the message kept for g5b_last_error, when the device refuses.
bool dev_opt_in_smem(const void *kernel, size_t bytes, SmemGrant &grant);
void set_last_error(const char *msg);

// ---- gemv.cu ------------------------------------------------------------------------------
// One product y[T][rows] = W (xform(x))[T][cols] of a batch launched as a single grid.
struct GemvSeg {
    const void  *W;
    const float *S;
    const float *x;       // [T][ldx]
    const float *xinv;    // optional RMSNorm factor per activation row
    const float *xw;      // optional RMSNorm weight per column
    float       *y;       // [T][ldy]
    int dt, R, C, br, bc, scols, ldx, ldy;
    int ldw;              // elements between consecutive rows of W (C unless W is a column slice)
    int ksplit;           // 1: a whole CTA shares each group of rows (few-row matrices)
    int block0;           // first block of this segment in the grid (filled by the launcher)
};
constexpr int GEMV_MAX_SEG = 8;

GemvSeg make_seg(const DMat &m, const float *x, int ldx, float *y, int ldy,
                 const float *xinv = nullptr, const float *xw = nullptr);
// Matrix restricted to rows [r0, r0+n) (FP8: r0 must lie on a scale-block row).
DMat row_slice(const DMat &m, int r0, int n);
// Matrix restricted to columns [c0, c0+n) (FP8: c0 must lie on a scale-block column).
DMat col_slice(const DMat &m, int c0, int n);
// early: one token, launched with programmatic stream serialization (the grid may be scheduled while
// the kernel before it drains; it waits for that kernel before it reads anything)
void gemv_batch(cudaStream_t st, const GemvSeg *segs, int n, int T, bool early = false);
inline void gemv(cudaStream_t st, const DMat &m, const float *x, int ldx, float *y, int ldy, int T,
                 const float *xinv = nullptr, const float *xw = nullptr)
{
    GemvSeg s = make_seg(m, x, ldx, y, ldy, xinv, xw);
    gemv_batch(st, &s, 1, T);
}

// ---- tc_gemm.cu ---------------------------------------------------------------------------
// FP8 block-scaled (128 x 128 blocks) and BF16 matrices times 8..64 positions on tcgen05 tensor
// cores, weights streamed once by TMA; activations as exact 16-bit term sums. Segments that share
// an input reuse its terms within one burst of calls; tc_gemm_new_input forgets them (call it
// whenever the input buffers get new contents). err: where a bounded wait that ran out is recorded.
struct TcGemm;
TcGemm *tc_gemm_create(int max_c, int *err);
void tc_gemm_free(TcGemm *g);
void tc_gemm_new_input(TcGemm *g);
bool tc_gemm_takes(const TcGemm *g, const GemvSeg &s, int T);
int  tc_gemm_run(TcGemm *g, cudaStream_t st, const GemvSeg &s, int T);

// ---- elementwise.cu -----------------------------------------------------------------------
void rms_factor(cudaStream_t st, const float *x, int n, int ld, int rows, float eps, float *inv);
void rms_apply(cudaStream_t st, float *y, const float *x, const float *w, const float *inv, int n,
               int ld, int rows);
void swiglu(cudaStream_t st, float *y, const float *gu, int n, int rows, float limit);
void shortconv(cudaStream_t st, float *y, const float *x, const float *w, float *state, int channels,
               int k, int T);
void embed_rows(cudaStream_t st, float *h, const DMat &table, const int *ids, int T, int M);
void add_rows(cudaStream_t st, float *x, const float *y, size_t n);
void head_mean(cudaStream_t st, float *xm, const float *h, int T, int M, int E);
void argmax_rows(cudaStream_t st, int *out, const float *logits, int n, int rows, float *scratch_v,
                 int *scratch_i);
void fill_codes(cudaStream_t st, uint8_t *dst, uint64_t seed, int layer, int expert, int which,
                size_t count);
uint64_t synth_key(uint64_t seed, const char *name);
void fill_codes_key(cudaStream_t st, uint8_t *dst, uint64_t key, size_t count);      // count a multiple of 4
void fill_bf16_key(cudaStream_t st, uint16_t *dst, uint64_t key, float mul, size_t count);
void fill_f32_key(cudaStream_t st, float *dst, uint64_t key, float mul, size_t count);
void f32_to_bf16(cudaStream_t st, uint16_t *dst, const float *src, size_t n);
void bf16_to_f32(cudaStream_t st, float *dst, const uint16_t *src, size_t n);
void flush_l2(cudaStream_t st, void *buf, size_t bytes);
// Hint: bring [p, p + bytes) into L2 (16-byte aligned p; nothing waits for it).
void l2_prefetch(cudaStream_t st, const void *p, size_t bytes);

// ---- sample.cu ----------------------------------------------------------------------------
// One token drawn from logits[V] (temperature, nucleus truncation, counter-based draw); prob: V floats of scratch.
void sample_token(cudaStream_t st, int *out, const float *logits, float *prob, int V, float temperature, float top_p,
                  uint64_t seed, uint64_t step);

// ---- mhc.cu -------------------------------------------------------------------------------
struct HcW {
    DMat   fn;
    float *base = nullptr, *scale = nullptr;
};
// mix [T][(2+M)*M] must already hold fn . RMSNorm0(h). Writes x, post, comb.
void hc_finish(cudaStream_t st, float *x, float *post, float *comb, const float *h, const float *mix,
               const HcW &w, int T, int M, int E, int iters, float eps);
// The whole pre side of a site in one launch, ending in the sub-block's normalised input xn
// (RMSNorm with norm_w). part: [T][32][(2+M)M + 1] doubles, counters: [T] zeroed ints.
bool hc_pre_fused_supported(const HcW &w, int M, int E);
// y_pending != nullptr: the previous site's hc_post (y_pending with the post / comb still in the
// arrays) is applied to h first, in the same launch.
void hc_pre_fused(cudaStream_t st, float *xn, float *post, float *comb, float *h, const float *y_pending,
                  const HcW &w, const float *norm_w, double *part, int *counters, int T, int M, int E, int iters,
                  float hc_eps, float rms_eps);
void hc_post(cudaStream_t st, float *h, const float *y, const float *post, const float *comb, int T,
             int M, int E);

// ---- moe.cu -------------------------------------------------------------------------------
struct ExpertW {          // one expert's three matrices, device pointers
    const uint8_t *gate, *up, *down;
    const float   *gate_s, *up_s, *down_s;
};
struct MoePlan {          // device arrays describing which expert multiplies which tokens
    int *n_slots;         // [1] experts with work this call (shared expert included)
    int *slot_expert;     // [max_slots] index into the ExpertW table
    int *slot_off;        // [max_slots] first pair of the slot
    int *slot_cnt;        // [max_slots] pairs of the slot
    int *pair_tok;        // [max_pairs] activation row of the pair
    int *pair_dst;        // [max_pairs] row of the contribution buffer the pair writes
    int  max_slots, max_pairs;
};
struct MoeShape {
    int E, I, NE, K, br, bc, dt;       // dt of expert matrices
    int n_local0, n_local;             // experts [n_local0, n_local0+n_local) live on this GPU
    float limit, routed_scale;
    int norm_topk;
};
// Router scores, top-k and the expert-major plan in one launch. p.n_slots == nullptr: routing only.
void router_plan(cudaStream_t st, int *idx, float *w, float *score, const float *x, int ldx, const void *gate,
                 int gate_dt, const float *bias, int T, const MoeShape &s, const MoePlan &p, int with_shared,
                 int *counter, int shared_t0 = 0, int shared_n = -1);
// Batch-1 experts multiplied by the tensor cores from their FP8 codes (moe_mma.cu); act_terms holds
// the SwiGLU output split into two F16 terms per element, [pairs][2][I].
bool moe_mma_supported(const MoeShape &s, int T);
void moe_mma_gateup(cudaStream_t st, void *act_terms, const float *x, const ExpertW *experts, const MoePlan &p,
                    const MoeShape &s, int *err);
void moe_mma_down(cudaStream_t st, float *out, float *contrib, const void *act_terms, const float *w,
                  const ExpertW *experts, const MoePlan &p, const MoeShape &s, int with_shared, int *tile_done,
                  int *err);
// Batches of 2..64 tokens on the same pipeline, four tokens per weight stage (moe_mma_batch.cu).
// xterms: scratch for [T][2][E] F16, xinv: [T] floats. Contributions only; the caller combines.
bool moe_mma_batch_supported(const MoeShape &s, int T);
void moe_mma_batch_gateup(cudaStream_t st, void *act_terms, void *xterms, float *xinv, const float *x, int ldx,
                          const ExpertW *experts, const MoePlan &p, int T, const MoeShape &s, int *err);
void moe_mma_batch_down(cudaStream_t st, float *contrib, const void *act_terms, const ExpertW *experts,
                        const MoePlan &p, int T, const MoeShape &s, int *err);
// The whole batch-1 layer (router, top-k, experts, combine) as one cooperative kernel
// (moe_decode.cu). `sync` holds two device counters that only grow; `launches` is the host's count of
// launches so far on them. Returns -1 when the cooperative launch is refused.
bool moe_decode_supported(const MoeShape &s, int T);
// ep != nullptr: expert parallel - this rank computes the picks it owns (and the shared expert),
// stores their rows into every rank's exchange region from the down epilogue and combines after
// every rank's step word has arrived (see ep_exchange.cu for the region's layout).
struct DecodeEp {
    int rank, size;
    void *const *peers;
    size_t rows_off;
    unsigned long long launch;     // expert-parallel launches of the decode kernel so far, this one included
    unsigned long long wait_ns;    // wall-clock limit of the wait for the other ranks' arrival counters
};
int moe_decode(cudaStream_t st, float *out, const float *x, const void *gate, int gate_dt, const float *bias,
               const ExpertW *experts, float *score, int *idx, float *w, void *act, float *contrib,
               const MoeShape &s, int with_shared, unsigned long long *sync, unsigned long long *launches,
               int *tile_done, int *err, const DecodeEp *ep = nullptr);
void moe_gateup(cudaStream_t st, float *act, const float *x, int ldx, const ExpertW *experts,
                const MoePlan &p, int T, const MoeShape &s);
void moe_down(cudaStream_t st, float *contrib, const float *act, const ExpertW *experts,
              const MoePlan &p, int T, const MoeShape &s);
void moe_combine(cudaStream_t st, float *out, int ldo, const float *contrib, const float *w, int T,
                 const MoeShape &s, int with_shared);

// ---- ep_exchange.cu ------------------------------------------------------------------------
// Expert-parallel exchange + combine. peers[r] is rank r's exchange region as mapped in this
// process: ep_size 64-bit words (word q = last step rank q delivered), then at rows_off the
// buffer of this step's parity, [T*K][E] floats.
struct EpExchange {
    const float *contrib;          // local contribution rows [T*K + T][E] (shared expert's rows last)
    MoePlan plan;                  // local slots; pair_dst < T*K are the rows to deliver
    void *const *peers;            // device array [size]
    int rank, size, T, K, E, with_shared;
    size_t rows_off;
    unsigned long long step;       // this call's number, the same on every rank, starting at 1
    int *arrive;                   // local counter, zero between launches
    const float *w;                // router weights [T][K]
    float *out; int ldo;
    int *err;
    unsigned long long wait_ns;    // wall-clock limit of the wait for the other ranks' step words
};
void ep_exchange_combine(cudaStream_t st, const EpExchange &a, int ctas);

// All-reduce (sum, in rank order) of one partial vector per rank and position over peer mappings,
// for a trunk product whose columns are split over the expert-parallel ranks: every rank stores its
// partial rows [T][E] into slot `rank` of every rank's buffer, counts itself done there with one
// release-add per CTA, waits (wall-clock limited) for all ranks' counters and adds the slots in rank
// order, so every rank gets the same bits. peers[r] + area_off = rank r's [size][max_t][E] buffer of
// this launch's parity; counters at word cnt0 + q of each region.
struct TsReduce {
    const float *partial;     // [T][E]
    float *out; int ldo;      // [T][ldo]
    void *const *peers;
    int rank, size, T, E, max_t;
    size_t area_off;
    int cnt0;
    unsigned long long launch;  // launches of this exchange so far, this one included
    unsigned long long wait_ns;
    int *err;
    int gather_only;            // 1: stop after the wait - the slots (max_t = T makes them one dense
                                // [size * T][E] block in rank order) are the result, nothing is summed
};
void ts_allreduce(cudaStream_t st, const TsReduce &a);

// The arg-max of a head whose vocabulary rows are split over the ranks: this rank's best row is
// local_idx[0] (an index into its own slice, whose logits start at `logits`), its first row is row0 of
// the whole vocabulary. Every rank stores (value, global index) into its slot on every rank, counts
// itself done there, waits (wall-clock limited) for all ranks and keeps the first maximum in index
// order in local_idx[0]. Words of the flag region from word0: [parity][rank] pairs (2 words each),
// then the arrival counters; at most 8 ranks.
struct HeadPick {
    const float *logits; int *local_idx; int row0;
    void *const *peers;
    int rank, size, word0;
    unsigned long long launch, wait_ns;
    int *err;
};
void head_pick_exchange(cudaStream_t st, const HeadPick &a);

// The exchange of a MoE layer whose sequences are split over the ranks (each rank runs attention and
// every other per-token kernel for its own sequences only). The tokens of all ranks were gathered
// first (TsReduce with gather_only); this rank routed a group of them - `m` consecutive tokens of
// the gathered block starting at global token g0, `n` tokens per rank - and computed the rows of
// the picks it owns. The kernel stores each row into the exchange buffer of the token's home rank
// (global token / n) at row (token % n) * K + pick. With `finish` (the last group of the call,
// the one that holds this rank's own tokens) it then publishes the step word on every rank, waits
// (wall-clock limited) for every rank's word and combines its own n tokens in top-k order, adding
// the shared expert's rows, which the plan computed for the own tokens only.
struct SeqExchange {
    const float *contrib;          // [m*K + m][E]
    MoePlan plan;
    void *const *peers;
    int rank, size, n, m, g0, K, E, with_shared, finish;
    size_t rows_off;
    unsigned long long step;
    int *arrive;
    const float *w;                // router weights of the group [m][K]
    float *out; int ldo;           // own tokens [n][ldo]
    int *err;
    unsigned long long wait_ns;
};
void seq_exchange(cudaStream_t st, const SeqExchange &a, int ctas);

// ---- kda.cu -------------------------------------------------------------------------------
struct KdaShape { int H, D, K; float gate_lb, rms_eps; };
// One new token only: the two low-rank up-projections z = f_b lrf and gb = g_b lrg (BF16 [H*D][D],
// inputs of D floats) are taken inside the kernel, each thread the two rows of its own channel,
// instead of by a launch of their own between the input projections and this kernel.
struct KdaLowRank {
    const void *f_b, *g_b;
    const float *lrf, *lrg;
};

// q,k,v,z,gb: [T][H*D] projections (q,k,v before the short convolution); braw [T][H]; state as
// the reference lays it out (S [H][D][D] then conv histories q|k|v, glm53f.h:363-367).
// Rows for calls with several positions: [T][H * D] normalised q, normalised k, v, exp(gate) and [T][H] beta.
struct KdaScratch { float *qn, *kn, *vn, *al, *beta; };
void kda_core(cudaStream_t st, float *o, const float *q, const float *k, const float *v, const float *z,
              const float *braw, const float *gb, const float *q_conv, const float *k_conv,
              const float *v_conv, const float *A_log, const float *dt_bias, const float *o_norm,
              float *state, int T, const KdaShape &s, int n_seq = 1, size_t seq_stride = 0,
              const KdaLowRank *lr = nullptr, int head0 = 0, int heads = -1, float *snap = nullptr, int snap_after = 0,
              const struct KdaScratch *scratch = nullptr);   // heads [head0, head0 + heads) only

// ---- mla.cu -------------------------------------------------------------------------------
struct MlaShape {
    int H, qn, vh, KL, q_lora, E, cap;
    int ID, IH, KP, topk;              // indexer dim, heads, pool size, index_topk
    float rms_eps;
    int latent_bf16;
    // batch of sequences: token t of a call belongs to sequence t, all at the same position; the
    // caches of consecutive sequences lie lat_seq / idx_seq elements apart (0 = one sequence, token
    // t at position cached + t)
    int batch = 0;
    size_t lat_seq = 0, idx_seq = 0;
};
// Also writes q_inv[t] = RMSNorm factor of q_raw[t][q_lora] (the q_a output of the same positions).
void mla_store(cudaStream_t st, void *latent, float *idx_state, const float *ct_raw,
               const float *kv_norm_w, const float *wk_raw, const float *gate_raw,
               const float *k_norm_w, const float *k_norm_b, const float *ape, const float *q_raw, float *q_inv,
               int T, int cached, const MlaShape &s);
void dsa_select(cudaStream_t st, int *sel, int *nsel, const float *idx_state, const float *qidx,
                const float *wproj, float *score, int T, int cached, const MlaShape &s);
void mla_absorb(cudaStream_t st, double *qa, const float *q, const DMat &kv_b, int T, const MlaShape &s);
// part: FP64 partial sums [part_tokens][H][ceil((topk+KP)/32)][KL], stats [T][H][2]; part == nullptr
// falls back to one CTA per head.
// counters: [T][H / 4] zeroed ints (the score kernel's per head-group arrival counts).
void mla_attend(cudaStream_t st, float *cb, const double *qa, const void *latent, const int *sel,
                const int *nsel, double *dsc, double *part, double *stats, int *counters, int part_tokens, int T,
                int cached, const MlaShape &s);
// The same attention core on the tensor cores (BF16 latent cache, kv_lora 512): scores and weighted
// sums as mma.sync products on exact BF16 term splits, softmax per chunk of 64 positions and a
// rescaling reduction. part / part_bytes: scratch for the chunks' partial rows; cstat: room for
// [T][H][ceil((topk + KP) / 64)][2] doubles.
bool mla_flash_takes(const MlaShape &s);
void mla_attend_flash(cudaStream_t st, float *cb, const double *qa, const void *latent, const int *sel, const int *nsel,
                      void *part, size_t part_bytes, double *cstat, int T, int cached, const MlaShape &s);
void mla_vout(cudaStream_t st, float *acc_out, const float *cb, const DMat &kv_b, int T, const MlaShape &s);

}  // namespace g5b
