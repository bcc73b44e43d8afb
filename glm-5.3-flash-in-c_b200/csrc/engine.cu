// engine.cu - the engine object behind include/glm53f_b200.h: HBM-resident weights loaded by
// checkpoint name, per-session state, and the sequencing of kernels for one forward pass.
//
// Replaces the host side of the reference's CUDA backend (src/gpu/glm53f_gpu.c): its placement of
// whole layers on devices, the FP32 widening copies for cuBLAS, the per-MoE-layer round trip of
// activations to the CPU for the routed experts (:1024-1040), and the blocking copies between
// every step. Here nothing leaves the GPU between the token ids going in and the logits (or the
// arg-max) coming out: router, expert selection, DSA selection, embedding gather and arg-max all
// run on the device, and every routed expert of this engine's expert-parallel range is resident.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "kernels.h"

namespace g5b {
extern unsigned long long g_launches;

static thread_local char g_err[512] = "";
static int fail(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    fprintf(stderr, "glm53f_b200: %s\n", g_err);
    return -1;
}
void set_last_error(const char *msg) { snprintf(g_err, sizeof g_err, "%s", msg); }
#define CU(call)                                                                           \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess) return fail("%s: %s", #call, cudaGetErrorString(e_));       \
    } while (0)

constexpr size_t EP_FLAG_BYTES = 1024;   // exchange region: the ranks' step words, then the row buffers
constexpr int EP_HEAD_WORD0 = 64;        // words [64, 64 + 5 x 8): the vocabulary-split head's (value, index) slots of two parities and its arrival counters (up to 8 ranks)
constexpr int MLA_PART_TOKENS = 4;     // tokens whose attention partial sums are held at once
constexpr int CHUNK = 64;       // positions one pass of a layer works on (the reference's MoE chunk, glm53f_ops.c:988)
constexpr int PROF_SLOTS = 8;

struct Layer {
    HcW    hc[2];
    float *in_norm = nullptr, *post_norm = nullptr;
    bool   is_mla = false, is_dense = false;
    // KDA
    DMat   kq, kk, kv, f_a, f_b, kb, g_a, g_b, ko;
    float *q_conv = nullptr, *k_conv = nullptr, *v_conv = nullptr, *A_log = nullptr, *dt_bias = nullptr,
          *o_norm = nullptr;
    // MLA + indexer
    DMat   q_a, q_b, kv_a, kv_b, mo, wq_b, wk, wproj, igate;
    float *q_a_norm = nullptr, *kv_a_norm = nullptr, *k_norm_w = nullptr, *k_norm_b = nullptr, *ape = nullptr;
    // feed-forward
    DMat   d_gate, d_up, d_down, sh_gate, sh_up, sh_down;
    DMat   router;
    float *bias = nullptr;
    uint8_t *expert_slab = nullptr;
    size_t   expert_stride = 0;
    int      expert_dt = -1;
    std::vector<ExpertW> table;          // n_local routed + 1 shared (host mirror)
    std::vector<uint8_t> have;           // [n_local][3]
    ExpertW *table_dev = nullptr;
    // session state
    float *kda_state = nullptr;
    void  *latent = nullptr;
    float *idx_state = nullptr;
};

struct Target { int kind; DMat *mat; float **vec; int rows, cols; };   // kind 0 matrix, 1 vector

}  // namespace g5b

using namespace g5b;

struct g5b_engine {
    g5b_config c;
    int cap = 0, cached = 0, device = 0, ep_rank = 0, ep_size = 1, n_local0 = 0, n_local = 0;
    bool finalized = false, ep_connected = false;
    // independent sequences (option "sequences", default 1): every layer's session state exists once
    // per sequence; single-sequence calls address sequence `cur_seq`
    int n_seq = 1, cur_seq = 0;
    std::vector<int> cached_seq;
    size_t kda_seq = 0, lat_seq = 0, idx_seq = 0;          // elements between consecutive sequences' states
    // expert-parallel exchange region of this rank: ep_size 64-bit words, then two row buffers
    uint8_t *ep_region = nullptr;
    size_t ep_rows_bytes = 0;
    void **ep_peers_dev = nullptr;
    std::vector<void *> ep_opened;               // peer mappings to close
    std::vector<void *> ep_standins;             // local stand-ins for peers (option ep_loopback)
    unsigned long long ep_step = 0;              // exchanges so far (both kernels): picks the row buffer
    unsigned long long ep_decode_launches = 0;
    unsigned long long head_launches = 0;        // arg-max exchanges of the vocabulary-split head so far
    unsigned long long ts_launches = 0;          // all-reduces of column-split trunk products so far
    size_t ts_area_bytes = 0;                    // one parity's [ep_size][CHUNK][hidden] floats
    float *ts_part = nullptr;                    // this rank's partial rows [CHUNK][hidden]
    int tensor_split = 1;                        // option "tensor_split": KDA heads and their state split over the ranks   // of them, by the one-token kernel (its arrival counters count CTAs)
    // the multi-token-prediction layer (checkpoint layer n_layers; g5b_engine_enable_mtp): one more
    // Layer slot (MLA + MoE, no mHC tensors), its norms and input projection, its own position count
    bool mtp = false;
    int mtp_cached = 0;
    int last_T = 0;                              // positions of the last forward call (rows of mtp_h in use)
    float *enorm = nullptr, *hnorm = nullptr, *head_norm = nullptr;
    DMat eh;
    float *mtp_h = nullptr;                      // [cap + CHUNK][hidden]: stream means of the positions of the last forward call
    float *mtp_cat = nullptr, *mtp_x = nullptr;  // [CHUNK][2 hidden], [CHUNK][hidden]
    std::vector<float *> kda_snap;               // speculative decode: per layer, the current sequence's KDA state as it was
    bool snap_first = false;                     // after the first position of the two-position pass in flight
    int seq_split = 0;                           // option "sequence_split": every rank runs its own sequences, MoE layers
                                                 // gather the ranks' tokens and send contribution rows home
    int *ep_arrive = nullptr;
    int ep_wait_ms = 5000;                       // wall-clock limit of a wait for the other ranks (option "ep_wait_ms")
    bool dirty = false;                          // a call failed half-way: session state is undefined until reset
    int latent_bf16 = 0, profile = 0, partial = 0, expert_path = 2;
    unsigned long long *grid_sync = nullptr, grid_launches = 0;
    int *counter = nullptr, *tile_done = nullptr, *err_dev = nullptr;
    volatile int *err_host = nullptr;   // mapped host memory: kernels record a timed-out wait here
    cudaStream_t st = nullptr;
    cudaStream_t side = nullptr;                         // L2 prefetches that run beside latency-bound kernels
    cudaEvent_t side_ev = nullptr, side_done = nullptr;  // fork from / join into the main stream
    std::vector<Layer> L;
    std::vector<std::unordered_map<std::string, Target>> names;   // per layer
    DMat embed, lm_head;
    float *norm = nullptr;
    std::vector<void *> owned;

    // work buffers (CHUNK positions)
    float *h = nullptr; size_t h_tokens = 0;
    int   *ids_dev = nullptr; size_t ids_cap = 0;
    float *inv0, *inv1, *mix, *xc, *xn, *y, *post, *comb;
    float *kq, *kk, *kv, *kz, *kgb, *ko, *kbraw, *klr;
    KdaScratch kscr{};                           // rows of the position-parallel part of the KDA layer for calls with several positions
    float *mq_raw, *mct, *mwk, *mgate, *mwp, *mq, *mqidx, *mcb, *macc, *mscore, *minvq;
    double *mqa, *mdsc, *mpart = nullptr, *mstats = nullptr;
    int *mcount = nullptr;
    TcGemm *tc = nullptr;                                // FP8 / BF16 projections of 8+ positions on tcgen05
    int mla_tensor = 1;                                  // option "mla_tensor": 0 keeps the attention core on the FP64 kernels
    size_t mpart_bytes = 0;
    int tensor_gemm = 1;                                 // option "tensor_gemm": 0 keeps 8+ positions on the one-token kernels
    float *post_h = nullptr; int post_n = 0;             // positions whose hc_post is still owed (run_layer)
    double *hc_part = nullptr; int *hc_count = nullptr;  // fused mHC site: partial sums and per-token counters
    void *xterms = nullptr; float *xinv = nullptr;      // batched expert kernels: F16 terms of the activations
    int   *msel, *mnsel;
    float *rscore, *rw, *act, *contrib, *gu, *dact;
    int   *ridx;
    MoePlan plan;
    float *xm, *inv_head, *logits, *am_v;
    int   *am_i, *am_out;
    void  *flush_buf = nullptr; size_t flush_bytes = 0;
    cudaEvent_t prof_ev[PROF_SLOTS + 1];
    float prof_ms[PROF_SLOTS];
    long  prof_n = 0;

    int dalloc(void **p, size_t bytes)
    {
        if (bytes == 0) bytes = 16;
        CU(cudaMalloc(p, bytes));
        CU(cudaMemsetAsync(*p, 0, bytes, st));
        owned.push_back(*p);
        return 0;
    }
};

// ------------------------------------------------------------------ creation ----
extern "C" const char *g5b_last_error(void) { return g_err; }

extern "C" int g5b_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}

extern "C" uint64_t g5b_launch_count(void) { return g_launches; }

static void add_mat(g5b_engine *e, int l, const char *nm, DMat *m, int rows, int cols)
{
    e->names[l][nm] = Target{0, m, nullptr, rows, cols};
}
static void add_vec(g5b_engine *e, int l, const char *nm, float **v, int n)
{
    e->names[l][nm] = Target{1, nullptr, v, n, 1};
}

// The tensors a layer consists of: names, shapes as the reference binds them
// (src/model/glm53f_bind.c:139-206).
static void plan_layer(g5b_engine *e, int l)
{
    const g5b_config &c = e->c;
    Layer &w = e->L[l];
    const int E = c.hidden, M = c.hc_mult, MIX = (2 + M) * M;
    add_vec(e, l, "input_layernorm.weight", &w.in_norm, E);
    add_vec(e, l, "post_attention_layernorm.weight", &w.post_norm, E);
    if (l == c.n_layers) {
        // the MTP layer carries no mHC mixers (src/model/glm53f_bind.c:208-222)
        add_vec(e, l, "enorm.weight", &e->enorm, E);
        add_vec(e, l, "hnorm.weight", &e->hnorm, E);
        add_vec(e, l, "shared_head.norm.weight", &e->head_norm, E);
        add_mat(e, l, "eh_proj.weight", &e->eh, E, 2 * E);
    } else {
        add_mat(e, l, "hc_attn_fn", &w.hc[0].fn, MIX, M * E);
        add_vec(e, l, "hc_attn_base", &w.hc[0].base, MIX);
        add_vec(e, l, "hc_attn_scale", &w.hc[0].scale, 3);
        add_mat(e, l, "hc_ffn_fn", &w.hc[1].fn, MIX, M * E);
        add_vec(e, l, "hc_ffn_base", &w.hc[1].base, MIX);
        add_vec(e, l, "hc_ffn_scale", &w.hc[1].scale, 3);
    }
    if (w.is_mla) {
        const int H = c.mla_heads, IH = c.index_heads, ID = c.index_dim;
        add_mat(e, l, "self_attn.q_a_proj.weight", &w.q_a, c.q_lora, E);
        add_vec(e, l, "self_attn.q_a_layernorm.weight", &w.q_a_norm, c.q_lora);
        add_mat(e, l, "self_attn.q_b_proj.weight", &w.q_b, H * c.qk_nope, c.q_lora);
        add_mat(e, l, "self_attn.kv_a_proj_with_mqa.weight", &w.kv_a, c.kv_lora, E);
        add_vec(e, l, "self_attn.kv_a_layernorm.weight", &w.kv_a_norm, c.kv_lora);
        add_mat(e, l, "self_attn.kv_b_proj.weight", &w.kv_b, H * (c.qk_nope + c.v_head), c.kv_lora);
        add_mat(e, l, "self_attn.o_proj.weight", &w.mo, E, H * c.v_head);
        add_mat(e, l, "self_attn.indexer.wq_b.weight", &w.wq_b, IH * ID, c.q_lora);
        add_mat(e, l, "self_attn.indexer.wk.weight", &w.wk, ID, E);
        add_vec(e, l, "self_attn.indexer.k_norm.weight", &w.k_norm_w, ID);
        add_vec(e, l, "self_attn.indexer.k_norm.bias", &w.k_norm_b, ID);
        add_mat(e, l, "self_attn.indexer.weights_proj.weight", &w.wproj, IH, E);
        add_mat(e, l, "self_attn.indexer.index_kpool_compress_gate", &w.igate, ID, E);
        add_vec(e, l, "self_attn.indexer.index_kpool_compress_ape", &w.ape, c.index_kpool * ID);
    } else {
        const int H = c.kda_heads, D = c.kda_head_dim, P = H * D;
        add_mat(e, l, "self_attn.q_proj.weight", &w.kq, P, E);
        add_mat(e, l, "self_attn.k_proj.weight", &w.kk, P, E);
        add_mat(e, l, "self_attn.v_proj.weight", &w.kv, P, E);
        add_vec(e, l, "self_attn.q_conv1d.weight", &w.q_conv, P * c.conv_k);
        add_vec(e, l, "self_attn.k_conv1d.weight", &w.k_conv, P * c.conv_k);
        add_vec(e, l, "self_attn.v_conv1d.weight", &w.v_conv, P * c.conv_k);
        add_mat(e, l, "self_attn.f_a_proj.weight", &w.f_a, D, E);
        add_mat(e, l, "self_attn.f_b_proj.weight", &w.f_b, P, D);
        add_vec(e, l, "self_attn.A_log", &w.A_log, H);
        add_vec(e, l, "self_attn.dt_bias", &w.dt_bias, P);
        add_mat(e, l, "self_attn.b_proj.weight", &w.kb, H, E);
        add_mat(e, l, "self_attn.g_a_proj.weight", &w.g_a, D, E);
        add_mat(e, l, "self_attn.g_b_proj.weight", &w.g_b, P, D);
        add_vec(e, l, "self_attn.o_norm.weight", &w.o_norm, D);
        add_mat(e, l, "self_attn.o_proj.weight", &w.ko, E, P);
    }
    if (w.is_dense) {
        add_mat(e, l, "mlp.gate_proj.weight", &w.d_gate, c.dense_inter, E);
        add_mat(e, l, "mlp.up_proj.weight", &w.d_up, c.dense_inter, E);
        add_mat(e, l, "mlp.down_proj.weight", &w.d_down, E, c.dense_inter);
    } else {
        const int SI = c.moe_inter * c.n_shared;
        add_mat(e, l, "mlp.gate.weight", &w.router, c.n_experts, E);
        add_vec(e, l, "mlp.gate.e_score_correction_bias", &w.bias, c.n_experts);
        add_mat(e, l, "mlp.shared_experts.gate_proj.weight", &w.sh_gate, SI, E);
        add_mat(e, l, "mlp.shared_experts.up_proj.weight", &w.sh_up, SI, E);
        add_mat(e, l, "mlp.shared_experts.down_proj.weight", &w.sh_down, E, SI);
    }
}

extern "C" g5b_engine *g5b_engine_create(const g5b_config *cfg, const uint8_t *is_mla,
                                         const uint8_t *is_dense, int cap, int device, int ep_rank,
                                         int ep_size)
{
    g_err[0] = 0;
    const g5b_config &c = *cfg;
    if (c.n_layers < 1 || c.n_layers > G5B_MAX_LAYERS || c.topk < 1 || c.topk > G5B_MAX_TOPK ||
        c.hc_mult < 1 || c.hc_mult > G5B_MAX_HC || c.n_experts > G5B_MAX_EXPERTS || c.conv_k > 17 ||
        c.kda_head_dim > 512 || c.kv_lora > 1024 || c.index_heads > 256 || c.index_dim > 512 ||
        cap > G5B_MAX_POSITIONS || c.index_kpool < 1) {
        fail("config outside the engine limits");
        return nullptr;
    }
    if (ep_size < 1 || ep_rank < 0 || ep_rank >= ep_size || (c.n_experts % ep_size) != 0) {
        fail("expert-parallel rank %d of %d does not divide %d experts", ep_rank, ep_size, c.n_experts);
        return nullptr;
    }
    if (device < 0 || device >= g5b_device_count()) {
        fail("CUDA device %d is not available (this library has no CPU path)", device);
        return nullptr;
    }
    if (cudaSetDevice(device) != cudaSuccess) { fail("cudaSetDevice(%d) failed", device); return nullptr; }
    g5b_engine *e = new g5b_engine();
    e->c = c;
    e->cap = cap < 1 ? 1 : cap;
    e->device = device;
    e->ep_rank = ep_rank; e->ep_size = ep_size;
    e->n_local = c.n_experts / ep_size;
    e->n_local0 = ep_rank * e->n_local;
    cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking);
    cudaEventCreateWithFlags(&e->side_ev, cudaEventDisableTiming);
    cudaEventCreateWithFlags(&e->side_done, cudaEventDisableTiming);
    if (cudaStreamCreateWithFlags(&e->st, cudaStreamNonBlocking) != cudaSuccess) {
        fail("cannot create a stream"); delete e; return nullptr;
    }
    for (int i = 0; i <= PROF_SLOTS; i++) cudaEventCreate(&e->prof_ev[i]);
    memset(e->prof_ms, 0, sizeof e->prof_ms);
    e->L.reserve((size_t)c.n_layers + 1);           // the name table points into L: enabling the MTP layer must not move it
    e->L.resize(c.n_layers);
    e->names.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        e->L[l].is_mla = is_mla[l] != 0;
        e->L[l].is_dense = is_dense[l] != 0;
        plan_layer(e, l);
    }
    return e;
}

// Checkpoint layer n_layers, the multi-token-prediction layer (src/model/glm53f_mtp.h): call before
// loading; the engine then expects "layers.<n_layers>.*" (an MLA + MoE layer without mHC tensors,
// enorm, hnorm, shared_head.norm, eh_proj) and keeps every position's stream mean for g5b_mtp_feed.
extern "C" int g5b_engine_enable_mtp(g5b_engine *e)
{
    if (!e || e->finalized) return fail("enable_mtp after finalize");
    if (e->mtp) return 0;
    if (e->c.n_layers + 1 > G5B_MAX_LAYERS) return fail("no room for the MTP layer");
    const int l = e->c.n_layers;
    if (e->L.capacity() < (size_t)l + 1) return fail("no room for the MTP layer");
    e->L.resize((size_t)l + 1);
    e->names.resize((size_t)l + 1);
    e->L[l].is_mla = true;
    e->L[l].is_dense = false;
    e->mtp = true;
    plan_layer(e, l);
    return 0;
}

static int ep_loopback(g5b_engine *e);
extern "C" int g5b_engine_set_option(g5b_engine *e, const char *name, int value)
{
    if (!strcmp(name, "latent_bf16")) {
        if (e->finalized) return fail("latent_bf16 must be set before finalize");
        e->latent_bf16 = value != 0;
        return 0;
    }
    if (!strcmp(name, "profile")) { e->profile = value; return 0; }
    if (!strcmp(name, "allow_partial")) { e->partial = value != 0; return 0; }
    if (!strcmp(name, "sequences")) {
        if (e->finalized) return fail("set the number of sequences before finalize");
        if (value < 1 || value > CHUNK) return fail("sequences is 1..%d", CHUNK);
        e->n_seq = value;
        return 0;
    }
    if (!strcmp(name, "tensor_gemm")) { e->tensor_gemm = value; return 0; }
    if (!strcmp(name, "mla_tensor")) { e->mla_tensor = value; return 0; }
    if (!strcmp(name, "tensor_split")) {
        if (e->ts_launches) return fail("tensor_split cannot change once a split layer has run (each rank holds only its heads' state)");
        e->tensor_split = value != 0;
        return 0;
    }
    if (!strcmp(name, "sequence_split")) {
        if (e->ts_launches || e->ep_step) return fail("sequence_split cannot change once the ranks have exchanged anything");
        if (value && e->ep_size < 2) return fail("sequence_split needs an expert-parallel engine (ep_size > 1)");
        e->seq_split = value != 0;
        return 0;
    }
    if (!strcmp(name, "ep_loopback")) return value ? ep_loopback(e) : 0;
    if (!strcmp(name, "ep_wait_ms")) {
        if (value < 1 || value > 600000) return fail("ep_wait_ms is 1..600000");
        e->ep_wait_ms = value;
        return 0;
    }
    if (!strcmp(name, "expert_path")) {          // batch-1 experts: 0 register kernels, 1 tensor-core kernels (router,
                                                 // gate/up, down as three launches), 2 the whole layer as one kernel
        if (value < 0 || value > 2) return fail("expert_path is 0, 1 or 2");
        e->expert_path = value;
        return 0;
    }
    return fail("unknown option %s", name);
}

// ------------------------------------------------------------------- loading ----
static size_t elt(int dt) { return dt == G5B_DT_F32 ? 4 : dt == G5B_DT_BF16 ? 2 : 1; }

static int copy_in(g5b_engine *e, void *dst, const void *src, size_t bytes, int on_device)
{
    CU(cudaMemcpyAsync(dst, src, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, e->st));
    CU(cudaStreamSynchronize(e->st));
    return 0;
}

static int upload_mat(g5b_engine *e, DMat *m, const g5b_tensor *t, int rows, int cols, const char *name)
{
    if (t->rows != rows || t->cols != cols)
        return fail("%s is %d x %d, the config implies %d x %d", name, t->rows, t->cols, rows, cols);
    if (t->dtype < 0 || t->dtype > 2) return fail("%s has a dtype this engine cannot multiply", name);
    m->dt = t->dtype; m->rows = rows; m->cols = cols;
    if (e->dalloc(&m->w, (size_t)rows * cols * elt(t->dtype))) return -1;
    if (copy_in(e, m->w, t->data, (size_t)rows * cols * elt(t->dtype), t->on_device)) return -1;
    if (t->dtype == G5B_DT_FP8) {
        if (!t->scale_inv || e->c.fp8_block_r < 1 || e->c.fp8_block_c < 1)
            return fail("%s is FP8 but has no scale grid / the config has no block size", name);
        m->br = e->c.fp8_block_r; m->bc = e->c.fp8_block_c;
        m->scols = (cols + m->bc - 1) / m->bc;
        const size_t ns = (size_t)((rows + m->br - 1) / m->br) * m->scols;
        if (e->dalloc((void **)&m->s, ns * 4)) return -1;
        if (copy_in(e, m->s, t->scale_inv, ns * 4, t->on_device)) return -1;
    }
    return 0;
}

// Vectors are widened to FP32 on the way in (reference: src/model/glm53f_bind.c:130-133).
static int upload_vec(g5b_engine *e, float **v, const g5b_tensor *t, size_t n, const char *name)
{
    if ((size_t)t->rows * (size_t)t->cols != n)
        return fail("%s has %zu values, the config implies %zu", name, (size_t)t->rows * (size_t)t->cols, n);
    if (t->on_device) return fail("%s: vectors are loaded from host memory", name);
    std::vector<float> tmp(n);
    if (t->dtype == G5B_DT_F32) memcpy(tmp.data(), t->data, n * 4);
    else if (t->dtype == G5B_DT_BF16) {
        const uint16_t *s = (const uint16_t *)t->data;
        for (size_t i = 0; i < n; i++) { uint32_t u = (uint32_t)s[i] << 16; memcpy(&tmp[i], &u, 4); }
    } else return fail("%s must be a float vector", name);
    if (e->dalloc((void **)v, n * 4)) return -1;
    return copy_in(e, *v, tmp.data(), n * 4, 0);
}

// Per layer, every local expert in one slab: [gate | up | down codes][gate | up | down scales],
// each part 256-byte aligned, so an expert is one contiguous ~25 MB range of HBM.
static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

static int ensure_expert_slab(g5b_engine *e, Layer &w, int dt)
{
    if (w.expert_slab) {
        if (w.expert_dt != dt) return fail("routed experts of one layer must share a dtype");
        return 0;
    }
    const g5b_config &c = e->c;
    const size_t mat = up256((size_t)c.moe_inter * c.hidden * elt(dt));
    size_t sc = 0;
    if (dt == G5B_DT_FP8) {
        const int br = c.fp8_block_r, bc = c.fp8_block_c;
        if (br < 1 || bc < 1) return fail("FP8 experts need the config's block size");
        sc = up256((size_t)((c.moe_inter + br - 1) / br) * ((c.hidden + bc - 1) / bc) * 4) * 2 +
             up256((size_t)((c.hidden + br - 1) / br) * ((c.moe_inter + bc - 1) / bc) * 4);
    }
    w.expert_stride = 3 * mat + sc;
    w.expert_dt = dt;
    if (e->dalloc((void **)&w.expert_slab, w.expert_stride * (size_t)e->n_local)) return -1;
    w.table.assign((size_t)e->n_local + 1, ExpertW{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr});
    w.have.assign((size_t)e->n_local * 3, 0);
    for (int i = 0; i < e->n_local; i++) {
        uint8_t *base = w.expert_slab + (size_t)i * w.expert_stride;
        ExpertW &x = w.table[i];
        x.gate = base; x.up = base + mat; x.down = base + 2 * mat;
        if (dt == G5B_DT_FP8) {
            const int br = c.fp8_block_r, bc = c.fp8_block_c;
            const size_t gs = up256((size_t)((c.moe_inter + br - 1) / br) * ((c.hidden + bc - 1) / bc) * 4);
            x.gate_s = (const float *)(base + 3 * mat);
            x.up_s   = (const float *)(base + 3 * mat + gs);
            x.down_s = (const float *)(base + 3 * mat + 2 * gs);
        }
    }
    return 0;
}

static int load_expert_part(g5b_engine *e, int l, int ex, int which, const g5b_tensor *t, const char *name)
{
    const g5b_config &c = e->c;
    Layer &w = e->L[l];
    if (ex < e->n_local0 || ex >= e->n_local0 + e->n_local) return 0;   // another rank's expert
    const int rows = which == 2 ? c.hidden : c.moe_inter, cols = which == 2 ? c.moe_inter : c.hidden;
    if (t->rows != rows || t->cols != cols)
        return fail("%s is %d x %d, the config implies %d x %d", name, t->rows, t->cols, rows, cols);
    if (ensure_expert_slab(e, w, t->dtype)) return -1;
    ExpertW &x = w.table[ex - e->n_local0];
    const uint8_t *dstw = which == 0 ? x.gate : which == 1 ? x.up : x.down;
    const float *dsts = which == 0 ? x.gate_s : which == 1 ? x.up_s : x.down_s;
    if (copy_in(e, (void *)dstw, t->data, (size_t)rows * cols * elt(t->dtype), t->on_device)) return -1;
    if (t->dtype == G5B_DT_FP8) {
        if (!t->scale_inv) return fail("%s is FP8 but has no scale grid", name);
        const size_t ns = (size_t)((rows + c.fp8_block_r - 1) / c.fp8_block_r) * ((cols + c.fp8_block_c - 1) / c.fp8_block_c);
        if (copy_in(e, (void *)dsts, t->scale_inv, ns * 4, t->on_device)) return -1;
    }
    w.have[(size_t)(ex - e->n_local0) * 3 + which] = 1;
    return 0;
}

extern "C" int g5b_engine_load(g5b_engine *e, const char *name, const g5b_tensor *t)
{
    if (e->finalized) return fail("load after finalize");
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    if (!strcmp(name, "embed_tokens.weight")) {
        if (t->dtype == G5B_DT_FP8) return fail("an FP8 embedding table is not supported");
        return upload_mat(e, &e->embed, t, c.vocab, c.hidden, name);
    }
    if (!strcmp(name, "lm_head.weight")) return upload_mat(e, &e->lm_head, t, c.vocab, c.hidden, name);
    if (!strcmp(name, "norm.weight")) return upload_vec(e, &e->norm, t, (size_t)c.hidden, name);
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= (int)e->L.size())
        return fail("unknown tensor %s", name);
    const char *rest = name + used;
    int ex = -1, n2 = 0;
    if (!e->L[l].is_dense && sscanf(rest, "mlp.experts.%d.%n", &ex, &n2) == 1) {
        if (ex < 0 || ex >= c.n_experts) return fail("%s: expert out of range", name);
        const char *p = rest + n2;
        const int which = !strcmp(p, "gate_proj.weight") ? 0 : !strcmp(p, "up_proj.weight") ? 1
                        : !strcmp(p, "down_proj.weight") ? 2 : -1;
        if (which < 0) return fail("unknown tensor %s", name);
        return load_expert_part(e, l, ex, which, t, name);
    }
    auto it = e->names[l].find(rest);
    if (it == e->names[l].end()) return fail("tensor %s does not belong to layer %d of this config", name, l);
    const Target &tg = it->second;
    if (tg.kind == 0) return upload_mat(e, tg.mat, t, tg.rows, tg.cols, name);
    return upload_vec(e, tg.vec, t, (size_t)tg.rows, name);
}

// Reserve a named tensor's place in HBM and hand its device addresses to a caller that will write the
// bytes itself (the streaming checkpoint loader, loader.cu): same names, shapes and dtypes as
// g5b_engine_load; the tensor counts as loaded. A routed expert of another rank returns NULL
// addresses and success. Vectors are not served here (they are widened on the host: g5b_engine_load).
extern "C" int g5b_engine_reserve(g5b_engine *e, const char *name, int dtype, int rows, int cols, void **data_dev,
                                  float **scale_dev)
{
    if (e->finalized) return fail("load after finalize");
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    *data_dev = nullptr; *scale_dev = nullptr;
    if (dtype < 0 || dtype > 2) return fail("%s has a dtype this engine cannot multiply", name);
    DMat *m = nullptr;
    int want_r = 0, want_c = 0;
    if (!strcmp(name, "embed_tokens.weight")) {
        if (dtype == G5B_DT_FP8) return fail("an FP8 embedding table is not supported");
        m = &e->embed; want_r = c.vocab; want_c = c.hidden;
    } else if (!strcmp(name, "lm_head.weight")) { m = &e->lm_head; want_r = c.vocab; want_c = c.hidden; }
    else {
        int l = -1, used = 0;
        if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= (int)e->L.size()) return fail("unknown tensor %s", name);
        const char *rest = name + used;
        int ex = -1, n2 = 0;
        if (!e->L[l].is_dense && sscanf(rest, "mlp.experts.%d.%n", &ex, &n2) == 1) {
            if (ex < 0 || ex >= c.n_experts) return fail("%s: expert out of range", name);
            const char *p = rest + n2;
            const int which = !strcmp(p, "gate_proj.weight") ? 0 : !strcmp(p, "up_proj.weight") ? 1 : !strcmp(p, "down_proj.weight") ? 2 : -1;
            if (which < 0) return fail("unknown tensor %s", name);
            if (ex < e->n_local0 || ex >= e->n_local0 + e->n_local) return 0;      // another rank's expert
            const int er = which == 2 ? c.hidden : c.moe_inter, ec = which == 2 ? c.moe_inter : c.hidden;
            if (rows != er || cols != ec) return fail("%s is %d x %d, the config implies %d x %d", name, rows, cols, er, ec);
            Layer &w = e->L[l];
            if (ensure_expert_slab(e, w, dtype)) return -1;
            ExpertW &x = w.table[ex - e->n_local0];
            *data_dev = (void *)(which == 0 ? x.gate : which == 1 ? x.up : x.down);
            *scale_dev = (float *)(which == 0 ? x.gate_s : which == 1 ? x.up_s : x.down_s);
            w.have[(size_t)(ex - e->n_local0) * 3 + which] = 1;
            return 0;
        }
        auto it = e->names[l].find(rest);
        if (it == e->names[l].end()) return fail("tensor %s does not belong to layer %d of this config", name, l);
        if (it->second.kind != 0) return fail("%s is a vector: load it with g5b_engine_load", name);
        m = it->second.mat; want_r = it->second.rows; want_c = it->second.cols;
    }
    if (rows != want_r || cols != want_c) return fail("%s is %d x %d, the config implies %d x %d", name, rows, cols, want_r, want_c);
    if (m->loaded()) return fail("%s is already loaded", name);
    m->dt = dtype; m->rows = rows; m->cols = cols;
    if (e->dalloc(&m->w, (size_t)rows * cols * elt(dtype))) return -1;
    if (dtype == G5B_DT_FP8) {
        if (c.fp8_block_r < 1 || c.fp8_block_c < 1) return fail("%s is FP8 but the config has no block size", name);
        m->br = c.fp8_block_r; m->bc = c.fp8_block_c; m->scols = (cols + m->bc - 1) / m->bc;
        if (e->dalloc((void **)&m->s, (size_t)((rows + m->br - 1) / m->br) * m->scols * 4)) return -1;
    }
    CU(cudaStreamSynchronize(e->st));                // the allocation's zero fill must not overtake the loader's copies
    *data_dev = m->w; *scale_dev = m->s;
    return 0;
}

// Does this engine take the named vector (so that the loader reads it at all)?
extern "C" int g5b_engine_wants_vector(g5b_engine *e, const char *name)
{
    if (!strcmp(name, "norm.weight")) return 1;
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= (int)e->L.size()) return 0;
    auto it = e->names[l].find(name + used);
    return it != e->names[l].end() && it->second.kind == 1;
}

extern "C" int g5b_engine_device(const g5b_engine *e) { return e->device; }
extern "C" int g5b_engine_layers(const g5b_engine *e) { return (int)e->L.size(); }   // the MTP layer included once enabled

extern "C" int g5b_engine_fill_expert(g5b_engine *e, int layer, int expert, uint64_t seed,
                                      const float *gate_s, const float *up_s, const float *down_s)
{
    if (e->finalized) return fail("fill after finalize");
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    if (layer < 0 || layer >= (int)e->L.size() || e->L[layer].is_dense) return fail("layer %d is not a MoE layer", layer);
    if (expert < e->n_local0 || expert >= e->n_local0 + e->n_local) return 0;
    Layer &w = e->L[layer];
    if (ensure_expert_slab(e, w, G5B_DT_FP8)) return -1;
    ExpertW &x = w.table[expert - e->n_local0];
    const size_t n = (size_t)c.moe_inter * c.hidden;
    if (n % 4) return fail("synthetic experts need moe_inter * hidden to be a multiple of 4");
    fill_codes(e->st, (uint8_t *)x.gate, seed, layer, expert, 0, n);
    fill_codes(e->st, (uint8_t *)x.up, seed, layer, expert, 1, n);
    fill_codes(e->st, (uint8_t *)x.down, seed, layer, expert, 2, n);
    const int br = c.fp8_block_r, bc = c.fp8_block_c;
    const size_t gs = (size_t)((c.moe_inter + br - 1) / br) * ((c.hidden + bc - 1) / bc);
    const size_t ds = (size_t)((c.hidden + br - 1) / br) * ((c.moe_inter + bc - 1) / bc);
    if (copy_in(e, (void *)x.gate_s, gate_s, gs * 4, 0) || copy_in(e, (void *)x.up_s, up_s, gs * 4, 0) ||
        copy_in(e, (void *)x.down_s, down_s, ds * 4, 0)) return -1;
    w.have[(size_t)(expert - e->n_local0) * 3 + 0] = w.have[(size_t)(expert - e->n_local0) * 3 + 1] =
        w.have[(size_t)(expert - e->n_local0) * 3 + 2] = 1;
    return 0;
}

// A whole named matrix filled with synthetic values on the GPU (no host copy of the weights ever
// exists): FP8 = uniform finite codes with the given scale grid, BF16 = bell-shaped values of
// standard deviation ~ 37837 * mul. The full-size model's 12.6 GB trunk is built this way.
extern "C" int g5b_engine_fill_matrix(g5b_engine *e, const char *name, int dtype, uint64_t seed, float mul,
                                      const float *scale_inv)
{
    if (e->finalized) return fail("fill after finalize");
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    DMat *m = nullptr;
    int rows = 0, cols = 0;
    if (!strcmp(name, "embed_tokens.weight")) { m = &e->embed; rows = c.vocab; cols = c.hidden; }
    else if (!strcmp(name, "lm_head.weight")) { m = &e->lm_head; rows = c.vocab; cols = c.hidden; }
    else {
        int l = -1, used = 0;
        if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= (int)e->L.size()) return fail("unknown tensor %s", name);
        auto it = e->names[l].find(name + used);
        if (it == e->names[l].end() || it->second.kind != 0) return fail("%s is not a matrix of layer %d", name, l);
        m = it->second.mat; rows = it->second.rows; cols = it->second.cols;
    }
    if (m->loaded()) return fail("%s is already loaded", name);
    const size_t n = (size_t)rows * cols;
    if (dtype == G5B_DT_BF16) {
        m->dt = dtype; m->rows = rows; m->cols = cols;
        if (e->dalloc(&m->w, n * 2)) return -1;
        fill_bf16_key(e->st, static_cast<uint16_t *>(m->w), synth_key(seed, name), mul, n);
    } else if (dtype == G5B_DT_FP8) {
        if (!scale_inv || c.fp8_block_r < 1 || c.fp8_block_c < 1) return fail("%s: FP8 needs a scale grid and the config's block size", name);
        if (n % 4) return fail("%s: synthetic FP8 matrices need a multiple of 4 elements", name);
        m->dt = dtype; m->rows = rows; m->cols = cols;
        m->br = c.fp8_block_r; m->bc = c.fp8_block_c; m->scols = (cols + m->bc - 1) / m->bc;
        const size_t ns = (size_t)((rows + m->br - 1) / m->br) * m->scols;
        if (e->dalloc(&m->w, n) || e->dalloc((void **)&m->s, ns * 4)) return -1;
        fill_codes_key(e->st, static_cast<uint8_t *>(m->w), synth_key(seed, name), n);
        if (copy_in(e, m->s, scale_inv, ns * 4, 0)) return -1;
    } else return fail("%s: synthetic matrices are BF16 or FP8", name);
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    return 0;
}

template <typename T>
static int walloc(g5b_engine *e, T **p, size_t count) { return e->dalloc((void **)p, count * sizeof(T)); }

extern "C" int g5b_engine_finalize(g5b_engine *e)
{
    if (e->finalized) return 0;
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    // A missing tensor must fail here: running with a NULL or zero weight gives plausible, wrong
    // tokens (the reference's bind refuses for the same reason, src/model/glm53f_bind.h:3-6).
    // Single-layer harnesses may leave embeddings and the head out; forward then refuses.
    for (int l = 0; l < (int)e->L.size(); l++) {
        Layer &w = e->L[l];
        for (auto &kv : e->names[l]) {
            const Target &t = kv.second;
            const bool ok = t.kind == 0 ? t.mat->loaded() : (*t.vec != nullptr);
            if (!ok && !e->partial) return fail("layer %d: tensor %s was never loaded", l, kv.first.c_str());
        }
        if (!w.is_dense && (w.expert_slab || !e->partial)) {
            if (!w.expert_slab) return fail("layer %d: no routed expert was loaded", l);
            if (w.router.dt == G5B_DT_FP8) return fail("layer %d: the router must be BF16 or FP32", l);
            for (int i = 0; i < e->n_local; i++)
                for (int k = 0; k < 3; k++)
                    if (!w.have[(size_t)i * 3 + k])
                        return fail("layer %d: routed expert %d is incomplete", l, e->n_local0 + i);
            if (c.n_shared == 1 && w.sh_gate.dt == w.expert_dt) {
                ExpertW &s = w.table[e->n_local];
                s.gate = (const uint8_t *)w.sh_gate.w; s.up = (const uint8_t *)w.sh_up.w; s.down = (const uint8_t *)w.sh_down.w;
                s.gate_s = w.sh_gate.s; s.up_s = w.sh_up.s; s.down_s = w.sh_down.s;
            }
            if (walloc(e, &w.table_dev, w.table.size())) return -1;
            CU(cudaMemcpyAsync(w.table_dev, w.table.data(), w.table.size() * sizeof(ExpertW), cudaMemcpyHostToDevice, e->st));
            CU(cudaStreamSynchronize(e->st));
        }
        // session state (reference: src/model/glm53f_model.c:194-228, always the latent form here)
        if (w.is_mla) {
            e->lat_seq = (size_t)e->cap * c.kv_lora;
            e->idx_seq = (size_t)2 * e->cap * c.index_dim +
                         (size_t)((e->cap + c.index_kpool - 1) / c.index_kpool) * c.index_dim;
            if (e->dalloc(&w.latent, e->n_seq * e->lat_seq * (e->latent_bf16 ? 2 : 4))) return -1;
            if (walloc(e, &w.idx_state, e->n_seq * e->idx_seq)) return -1;
        } else {
            const size_t P = (size_t)c.kda_heads * c.kda_head_dim;
            e->kda_seq = P * c.kda_head_dim + 3 * P * (size_t)(c.conv_k - 1);
            if (walloc(e, &w.kda_state, e->n_seq * e->kda_seq)) return -1;
        }
    }
    const size_t N = CHUNK, E = c.hidden, M = c.hc_mult, MIX = (2 + M) * M;
    const size_t P = (size_t)c.kda_heads * c.kda_head_dim, D = c.kda_head_dim;
    const size_t H = c.mla_heads, KL = c.kv_lora, stride = (size_t)c.index_topk + c.index_kpool;
    const size_t K = c.topk, I = c.moe_inter, SI = (size_t)c.moe_inter * c.n_shared;
    const size_t DI = c.dense_inter > (int)SI ? c.dense_inter : SI;
    if (walloc(e, &e->inv0, N) || walloc(e, &e->inv1, N) || walloc(e, &e->mix, N * MIX) ||
        walloc(e, &e->xc, N * E) || walloc(e, &e->xn, N * E) || walloc(e, &e->y, N * E) ||
        walloc(e, &e->post, N * M) || walloc(e, &e->comb, N * M * M)) return -1;
    if (walloc(e, &e->kq, N * P) || walloc(e, &e->kk, N * P) || walloc(e, &e->kv, N * P) ||
        walloc(e, &e->kz, N * P) || walloc(e, &e->kgb, N * P) || walloc(e, &e->ko, N * P) ||
        walloc(e, &e->kbraw, N * c.kda_heads) || walloc(e, &e->klr, N * 2 * D) ||
        walloc(e, &e->kscr.qn, N * P) || walloc(e, &e->kscr.kn, N * P) || walloc(e, &e->kscr.vn, N * P) ||
        walloc(e, &e->kscr.al, N * P) || walloc(e, &e->kscr.beta, N * c.kda_heads)) return -1;
    if (walloc(e, &e->mq_raw, N * c.q_lora) || walloc(e, &e->mct, N * KL) || walloc(e, &e->mwk, N * c.index_dim) ||
        walloc(e, &e->mgate, N * c.index_dim) || walloc(e, &e->mwp, N * c.index_heads) ||
        walloc(e, &e->mq, N * H * c.qk_nope) || walloc(e, &e->mqidx, N * (size_t)c.index_heads * c.index_dim) ||
        walloc(e, &e->mcb, N * H * KL) || walloc(e, &e->macc, N * H * c.v_head) ||
        walloc(e, &e->mscore, N * ((size_t)e->cap / c.index_kpool + 1)) || walloc(e, &e->minvq, N) ||
        walloc(e, &e->mqa, N * H * KL) || walloc(e, &e->mdsc, N * H * stride) ||
        walloc(e, &e->msel, N * stride) || walloc(e, &e->mnsel, N) ||
        walloc(e, &e->mstats, N * H * 2) || walloc(e, &e->mcount, N * H) ||
        walloc(e, &e->mpart, (size_t)MLA_PART_TOKENS * H * ((stride + 31) / 32) * KL)) return -1;
    e->mpart_bytes = (size_t)MLA_PART_TOKENS * H * ((stride + 31) / 32) * KL * sizeof(double);
    const size_t pairs = N * K + N;
    if (walloc(e, &e->rscore, N * c.n_experts) || walloc(e, &e->rw, N * K) || walloc(e, &e->ridx, N * K) ||
        walloc(e, &e->act, pairs * (I > SI ? I : SI)) || walloc(e, &e->contrib, pairs * E) ||
        walloc(e, &e->gu, N * 2 * DI) || walloc(e, &e->dact, N * DI) || walloc(e, &e->xinv, N) ||
        walloc(e, &e->hc_part, N * 32 * (MIX + 1)) || walloc(e, &e->hc_count, N) ||
        e->dalloc(&e->xterms, N * 2 * E * 2)) return -1;
    e->plan.max_slots = (int)((N * K < (size_t)e->n_local ? N * K : (size_t)e->n_local) + 1);
    e->plan.max_pairs = (int)pairs;
    if (walloc(e, &e->plan.n_slots, 1) || walloc(e, &e->plan.slot_expert, e->plan.max_slots) ||
        walloc(e, &e->plan.slot_off, e->plan.max_slots) || walloc(e, &e->plan.slot_cnt, e->plan.max_slots) ||
        walloc(e, &e->plan.pair_tok, pairs) || walloc(e, &e->plan.pair_dst, pairs)) return -1;
    if (walloc(e, &e->counter, CHUNK + 4) || walloc(e, &e->tile_done, E / 32 + 1) || walloc(e, &e->grid_sync, 2)) return -1;
    {
        int *hp = nullptr;
        CU(cudaHostAlloc((void **)&hp, 64, cudaHostAllocMapped));
        *hp = 0;
        e->err_host = hp;
        CU(cudaHostGetDevicePointer((void **)&e->err_dev, hp, 0));
    }
    if (walloc(e, &e->xm, N * E) || walloc(e, &e->inv_head, N) || walloc(e, &e->logits, N * (size_t)c.vocab) ||
        walloc(e, &e->am_v, N * 64) || walloc(e, &e->am_i, N * 64) || walloc(e, &e->am_out, (size_t)e->cap + N)) return -1;
    if (e->mtp && (walloc(e, &e->mtp_h, ((size_t)e->cap + N) * E) || walloc(e, &e->mtp_cat, N * 2 * E) ||
                   walloc(e, &e->mtp_x, N * E))) return -1;
    CU(cudaStreamSynchronize(e->st));
    {
        const int P = c.kda_heads * c.kda_head_dim;
        int max_c = e->mtp ? 2 * c.hidden : c.hidden;
        for (int v : {P, c.q_lora, c.kv_lora, c.kda_head_dim, c.mla_heads * c.v_head}) max_c = v > max_c ? v : max_c;
        for (int v : {c.dense_inter, c.moe_inter * c.n_shared}) max_c = v > max_c ? v : max_c;
        e->tc = tc_gemm_create(max_c, e->err_dev);
        if (!e->tc) return fail("the tensor-core projection path could not be set up (tensor-map encoder or scratch)");
    }
    e->cached_seq.assign((size_t)e->n_seq, 0);
    e->finalized = true;
    return 0;
}

// ------------------------------------------------------------------ sub-blocks ----
static MoeShape moe_shape(const g5b_engine *e, const Layer &w)
{
    const g5b_config &c = e->c;
    MoeShape s;
    s.E = c.hidden; s.I = c.moe_inter; s.NE = c.n_experts; s.K = c.topk;
    s.br = c.fp8_block_r; s.bc = c.fp8_block_c; s.dt = w.expert_dt < 0 ? G5B_DT_FP8 : w.expert_dt;
    s.n_local0 = e->n_local0; s.n_local = e->n_local;
    s.limit = c.swiglu_limit; s.routed_scale = c.routed_scale; s.norm_topk = c.norm_topk;
    return s;
}

static void prof_mark(g5b_engine *e, int slot)
{
    if (e->profile) cudaEventRecord(e->prof_ev[slot], e->st);
}
static void prof_collect(g5b_engine *e, int nslots)
{
    if (!e->profile) return;
    cudaEventSynchronize(e->prof_ev[nslots]);
    for (int i = 0; i < nslots; i++) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e->prof_ev[i], e->prof_ev[i + 1]);
        e->prof_ms[i] += ms;
    }
    e->prof_n++;
}

// x [n][E] (already normalised) -> out [n][E]. Router, plan, experts, combine.
// A MoE layer with the sequences split over the ranks (option "sequence_split"): x holds this
// rank's own n tokens, and every rank calls with the same n. The ranks' tokens are gathered
// everywhere (peer stores, arrival counters: the dispatch), every rank routes the gathered tokens
// in groups of at most CHUNK and multiplies them by the experts it owns, the contribution rows go
// to the exchange buffer of the rank a token lives on (the combine's transfer), and that rank
// sums its own tokens in top-k order with the shared expert, which it computed for its own tokens
// only. The groups are taken in rotated order so that the one holding the own tokens comes last:
// its router weights and shared rows are then still in place for the combine.
static int run_moe_seq_split(g5b_engine *e, Layer &w, const float *x, int n, float *out, int with_shared, const MoeShape &s)
{
    const g5b_config &c = e->c;
    const bool shared_in_plan = with_shared && c.n_shared == 1 && w.sh_gate.dt == s.dt;
    if (with_shared && !shared_in_plan) return fail("sequence_split needs the shared expert in the routed experts' format");
    const int N = e->ep_size, me = e->ep_rank;
    prof_mark(e, 0);
    ++e->ts_launches;
    const size_t area_off = EP_FLAG_BYTES + 2 * e->ep_rows_bytes + (size_t)(e->ts_launches & 1) * e->ts_area_bytes;
    TsReduce g{x, nullptr, 0, e->ep_peers_dev, me, N, n, c.hidden, n, area_off, 2 * N, e->ts_launches,
               (unsigned long long)e->ep_wait_ms * 1000000ull, e->err_dev, 1};
    ts_allreduce(e->st, g);
    prof_mark(e, 1);
    const float *all = reinterpret_cast<const float *>(e->ep_region + area_off);     // [N * n][hidden], rank order
    const int per = CHUNK / n > 0 ? CHUNK / n : 1;                                   // ranks per group
    const int groups = (N + per - 1) / per, mine = me / per;
    ++e->ep_step;
    for (int k = 1; k <= groups; k++) {
        const int gi = (mine + k) % groups, r0 = gi * per, r1 = r0 + per < N ? r0 + per : N;
        const int m = (r1 - r0) * n, g0 = r0 * n;
        const bool last = gi == mine;
        const float *xg = all + (size_t)g0 * c.hidden;
        router_plan(e->st, e->ridx, e->rw, e->rscore, xg, c.hidden, w.router.w, w.router.dt, w.bias, m, s, e->plan,
                    with_shared ? 1 : 0, e->counter, last ? me * n - g0 : 0, last ? n : 0);
        if (e->expert_path >= 1 && moe_mma_batch_supported(s, m)) {
            moe_mma_batch_gateup(e->st, e->act, e->xterms, e->xinv, xg, c.hidden, w.table_dev, e->plan, m, s, e->err_dev);
            moe_mma_batch_down(e->st, e->contrib, e->act, w.table_dev, e->plan, m, s, e->err_dev);
        } else {
            moe_gateup(e->st, e->act, xg, c.hidden, w.table_dev, e->plan, m, s);
            moe_down(e->st, e->contrib, e->act, w.table_dev, e->plan, m, s);
        }
        SeqExchange q{e->contrib, e->plan, e->ep_peers_dev, me, N, n, m, g0, c.topk, c.hidden, with_shared, last ? 1 : 0,
                      EP_FLAG_BYTES + (size_t)(e->ep_step & 1) * e->ep_rows_bytes, e->ep_step, e->ep_arrive, e->rw,
                      out, c.hidden, e->err_dev, (unsigned long long)e->ep_wait_ms * 1000000ull};
        const int want = (int)(((size_t)m * c.hidden + 255) / 256);
        seq_exchange(e->st, q, want < 8 ? 8 : want > 148 ? 148 : want);
    }
    prof_mark(e, 2); prof_mark(e, 3); prof_mark(e, 4);
    prof_collect(e, 4);
    return 0;
}

static int run_moe(g5b_engine *e, Layer &w, const float *x, int n, float *out, int with_shared)
{
    const g5b_config &c = e->c;
    if (!w.table_dev || !w.router.loaded() || !w.bias || (with_shared && !w.sh_down.loaded()))
        return fail("this layer's MoE weights were not loaded");
    if (e->ep_size > 1 && !e->ep_connected)
        return fail("expert-parallel engine: connect the ranks (g5b_engine_ep_connect) before running a MoE layer");
    const MoeShape s = moe_shape(e, w);
    if (e->seq_split && e->ep_size > 1) return run_moe_seq_split(e, w, x, n, out, with_shared, s);
    const bool shared_in_plan = with_shared && c.n_shared == 1 && w.sh_gate.dt == s.dt;
    const bool one_gpu_decode = e->ep_size == 1 && (shared_in_plan || !with_shared);
    prof_mark(e, 0);
    const bool ep_decode = e->ep_size > 1 && (shared_in_plan || !with_shared);
    if (e->expert_path == 2 && (one_gpu_decode || ep_decode) && moe_decode_supported(s, n)) {
        DecodeEp ep{e->ep_rank, e->ep_size, e->ep_peers_dev, EP_FLAG_BYTES + (size_t)((e->ep_step + 1) & 1) * e->ep_rows_bytes,
                    e->ep_decode_launches + 1, (unsigned long long)e->ep_wait_ms * 1000000ull};
        if (moe_decode(e->st, out, x, w.router.w, w.router.dt, w.bias, w.table_dev, e->rscore, e->ridx, e->rw, e->act,
                       e->contrib, s, with_shared, e->grid_sync, &e->grid_launches, e->tile_done, e->err_dev,
                       ep_decode ? &ep : nullptr) == 0) {
            if (ep_decode) { ++e->ep_step; ++e->ep_decode_launches; }
            prof_mark(e, 1); prof_mark(e, 2); prof_mark(e, 3); prof_mark(e, 4);
            prof_collect(e, 4);
            return 0;
        }
    }
    router_plan(e->st, e->ridx, e->rw, e->rscore, x, c.hidden, w.router.w, w.router.dt, w.bias, n, s, e->plan,
                shared_in_plan ? 1 : 0, e->counter);
    prof_mark(e, 1);
    auto exchange_and_combine = [&]() {
        // every rank computed the rows of the picks it owns: gather all rows everywhere and combine
        ++e->ep_step;
        EpExchange x{e->contrib, e->plan, e->ep_peers_dev, e->ep_rank, e->ep_size, n, c.topk, c.hidden, with_shared,
                     EP_FLAG_BYTES + (size_t)(e->ep_step & 1) * e->ep_rows_bytes, e->ep_step, e->ep_arrive, e->rw,
                     out, c.hidden, e->err_dev, (unsigned long long)e->ep_wait_ms * 1000000ull};
        const int want = (int)(((size_t)n * c.hidden + 255) / 256);
        ep_exchange_combine(e->st, x, want < 8 ? 8 : want > 148 ? 148 : want);
    };
    if (e->ep_size > 1 && e->expert_path >= 1 && (shared_in_plan || !with_shared) && moe_mma_supported(s, n)) {
        // batch 1 across ranks: the tensor-core kernels on this rank's picks, contributions only
        moe_mma_gateup(e->st, e->act, x, w.table_dev, e->plan, s, e->err_dev);
        prof_mark(e, 2);
        moe_mma_down(e->st, nullptr, e->contrib, e->act, e->rw, w.table_dev, e->plan, s, with_shared, e->tile_done, e->err_dev);
        prof_mark(e, 3);
        exchange_and_combine();
        prof_mark(e, 4);
        prof_collect(e, 4);
        return 0;
    }
    if (e->expert_path == 1 && one_gpu_decode && moe_mma_supported(s, n)) {
        moe_mma_gateup(e->st, e->act, x, w.table_dev, e->plan, s, e->err_dev);
        prof_mark(e, 2);
        moe_mma_down(e->st, out, e->contrib, e->act, e->rw, w.table_dev, e->plan, s, with_shared, e->tile_done, e->err_dev);
        prof_mark(e, 3);
        prof_mark(e, 4);
        prof_collect(e, 4);
        return 0;
    }
    if (e->expert_path >= 1 && (shared_in_plan || !with_shared) && moe_mma_batch_supported(s, n)) {
        // batches: the tensor-core pipeline with four tokens per weight stage
        moe_mma_batch_gateup(e->st, e->act, e->xterms, e->xinv, x, c.hidden, w.table_dev, e->plan, n, s, e->err_dev);
        prof_mark(e, 2);
        moe_mma_batch_down(e->st, e->contrib, e->act, w.table_dev, e->plan, n, s, e->err_dev);
        prof_mark(e, 3);
    } else {
        moe_gateup(e->st, e->act, x, c.hidden, w.table_dev, e->plan, n, s);
        prof_mark(e, 2);
        moe_down(e->st, e->contrib, e->act, w.table_dev, e->plan, n, s);
        prof_mark(e, 3);
    }
    if (with_shared && !shared_in_plan) {
        // a shared expert of another width or format goes through the plain MLP path
        const int SI = c.moe_inter * c.n_shared;
        GemvSeg g[2] = {make_seg(w.sh_gate, x, c.hidden, e->gu, 2 * SI), make_seg(w.sh_up, x, c.hidden, e->gu + SI, 2 * SI)};
        gemv_batch(e->st, g, 2, n);
        swiglu(e->st, e->dact, e->gu, SI, n, c.swiglu_limit);
        gemv(e->st, w.sh_down, e->dact, SI, e->contrib + (size_t)n * c.topk * c.hidden, c.hidden, n);
    }
    if (e->ep_size > 1) {
        exchange_and_combine();
    } else {
        moe_combine(e->st, out, c.hidden, e->contrib, e->rw, n, s, with_shared);
    }
    prof_mark(e, 4);
    prof_collect(e, 4);
    return 0;
}

static int proj_batch(g5b_engine *e, const GemvSeg *segs, int n, int T, bool early = false);
static int proj(g5b_engine *e, const DMat &m, const float *x, int ldx, float *y, int ldy, int T,
                const float *xinv = nullptr, const float *xw = nullptr);

static int run_mlp(g5b_engine *e, Layer &w, const float *x, int n, float *out)
{
    const g5b_config &c = e->c;
    const int DI = c.dense_inter;
    if (!w.d_gate.loaded() || !w.d_up.loaded() || !w.d_down.loaded()) return fail("this layer's dense MLP was not loaded");
    GemvSeg g[2] = {make_seg(w.d_gate, x, c.hidden, e->gu, 2 * DI), make_seg(w.d_up, x, c.hidden, e->gu + DI, 2 * DI)};
    if (proj_batch(e, g, 2, n)) return -1;
    swiglu(e->st, e->dact, e->gu, DI, n, c.swiglu_limit);
    return proj(e, w.d_down, e->dact, DI, out, c.hidden, n);
}

// From this point of the main stream on, fetch a matrix into L2 on the side stream: the kernels
// launched next on the main stream (latency-bound, few CTAs) run while the weights of the product
// after them arrive. Only worth it when the matrix fits L2 and is read once (one token).
static void prefetch_beside(g5b_engine *e, const DMat &m)
{
    if (!e->side || !e->side_ev || !m.loaded() || m.bytes() > ((size_t)96 << 20)) return;
    if (cudaEventRecord(e->side_ev, e->st) != cudaSuccess) return;
    if (cudaStreamWaitEvent(e->side, e->side_ev, 0) != cudaSuccess) return;
    l2_prefetch(e->side, m.w, m.bytes());
}

// Several products sharing (some of) their inputs: with 8 or more positions, FP8 (128 x 128 blocks)
// and BF16 matrices whose rows fill 128-row tiles go to the tcgen05 kernel, which reads the weights
// once; the rest (few rows, odd shapes) to the one-token kernel in one launch.
static int proj_batch(g5b_engine *e, const GemvSeg *segs, int n, int T, bool early)
{
    if (T < 8 || !e->tc || e->tensor_gemm == 0) { gemv_batch(e->st, segs, n, T, early); return 0; }
    tc_gemm_new_input(e->tc);
    GemvSeg rest[GEMV_MAX_SEG];
    int nr = 0;
    for (int i = 0; i < n; i++) {
        if (tc_gemm_takes(e->tc, segs[i], T)) {
            if (tc_gemm_run(e->tc, e->st, segs[i], T)) return fail("the tensor-core projection could not be launched");
        } else rest[nr++] = segs[i];
    }
    if (nr) gemv_batch(e->st, rest, nr, T);
    return 0;
}
static int proj(g5b_engine *e, const DMat &m, const float *x, int ldx, float *y, int ldy, int T,
                const float *xinv, const float *xw)
{
    GemvSeg s = make_seg(m, x, ldx, y, ldy, xinv, xw);
    return proj_batch(e, &s, 1, T);
}

// batch: the n rows are one new position of n different sequences (sequences 0..n-1), otherwise n
// consecutive positions of the current sequence.
// The sum over ranks of a column-split product's partial rows (e->ts_part -> out), in rank order.
static void trunk_allreduce(g5b_engine *e, float *out, int ldo, int n)
{
    ++e->ts_launches;
    TsReduce r{e->ts_part, out, ldo, e->ep_peers_dev, e->ep_rank, e->ep_size, n, e->c.hidden, CHUNK,
               EP_FLAG_BYTES + 2 * e->ep_rows_bytes + (size_t)(e->ts_launches & 1) * e->ts_area_bytes, 2 * e->ep_size,
               e->ts_launches, (unsigned long long)e->ep_wait_ms * 1000000ull, e->err_dev, 0};
    ts_allreduce(e->st, r);
}

static bool kda_heads_split(const g5b_engine *e, const Layer &w)
{
    const g5b_config &c = e->c;
    return e->tensor_split && !e->seq_split && e->ep_size > 1 && e->ep_connected && c.kda_heads % e->ep_size == 0 && (c.hidden % 4) == 0 &&
           w.kq.dt != G5B_DT_FP8 && w.kk.dt != G5B_DT_FP8 && w.kv.dt != G5B_DT_FP8 && w.ko.dt != G5B_DT_FP8 &&
           w.f_b.dt != G5B_DT_FP8 && w.g_b.dt != G5B_DT_FP8 && w.kb.dt != G5B_DT_FP8;
}

// batch: the n rows are one new position of n different sequences (sequences 0..n-1), otherwise n
// consecutive positions of the current sequence.
// Expert-parallel engines split the layer by heads as well (option "tensor_split", on by default):
// rank r multiplies the q / k / v / beta / low-rank rows of heads [r H / N, (r + 1) H / N), advances
// those heads' state only, and multiplies its heads' columns of the output projection; the partial
// output rows are summed over the ranks in rank order (ts_allreduce), so every rank continues with
// the same bits. A rank then holds a current state for its own heads only.
static int run_kda(g5b_engine *e, Layer &w, const float *x, int n, float *out, bool batch = false)
{
    const g5b_config &c = e->c;
    const int E = c.hidden, H = c.kda_heads, D = c.kda_head_dim, P = H * D;
    if (!w.kq.loaded() || !w.ko.loaded() || !w.g_b.loaded() || !w.f_b.loaded() || !w.kda_state || !w.dt_bias)
        return fail("this layer's KDA weights were not loaded");
    const bool ts = kda_heads_split(e, w);
    const int Hl = ts ? H / e->ep_size : H, h0 = ts ? e->ep_rank * Hl : 0, Pl = Hl * D, p0 = h0 * D;
    float *lrf = e->klr, *lrg = e->klr + (size_t)CHUNK * D;
    GemvSeg a[6] = {make_seg(row_slice(w.kq, p0, Pl), x, E, e->kq + p0, P), make_seg(row_slice(w.kk, p0, Pl), x, E, e->kk + p0, P),
                    make_seg(row_slice(w.kv, p0, Pl), x, E, e->kv + p0, P), make_seg(row_slice(w.kb, h0, Hl), x, E, e->kbraw + h0, H),
                    make_seg(w.f_a, x, E, lrf, D), make_seg(w.g_a, x, E, lrg, D)};
    if (proj_batch(e, a, 6, n, true)) return -1;
    // one new token: the recurrence kernel takes the two low-rank up-projections itself
    const bool lr_inside = n == 1 && !batch && w.f_b.dt == G5B_DT_BF16 && w.g_b.dt == G5B_DT_BF16 && (D == 64 || D == 128);
    const KdaLowRank lr{w.f_b.w, w.g_b.w, lrf, lrg};
    if (!lr_inside) {
        GemvSeg b[2] = {make_seg(row_slice(w.f_b, p0, Pl), lrf, D, e->kz + p0, P), make_seg(row_slice(w.g_b, p0, Pl), lrg, D, e->kgb + p0, P)};
        if (proj_batch(e, b, 2, n)) return -1;
    }
    KdaShape ks{H, D, c.conv_k, c.gate_lb, c.rms_eps};
    if (n == 1 && !ts) prefetch_beside(e, w.ko);        // the recurrence below leaves half the SMs and all of HBM idle
    if (batch)
        kda_core(e->st, e->ko, e->kq, e->kk, e->kv, e->kz, e->kbraw, e->kgb, w.q_conv, w.k_conv, w.v_conv,
                 w.A_log, w.dt_bias, w.o_norm, w.kda_state, 1, ks, n, e->kda_seq, nullptr, h0, Hl);
    else
        kda_core(e->st, e->ko, e->kq, e->kk, e->kv, e->kz, e->kbraw, e->kgb, w.q_conv, w.k_conv, w.v_conv,
                 w.A_log, w.dt_bias, w.o_norm, w.kda_state + (size_t)e->cur_seq * e->kda_seq, n, ks, 1, 0,
                 lr_inside ? &lr : nullptr, h0, Hl,
                 e->snap_first && n > 1 ? e->kda_snap[(size_t)(&w - e->L.data())] : nullptr, 0, &e->kscr);
    if (!ts) return proj(e, w.ko, e->ko, P, out, E, n);
    {
        GemvSeg o = make_seg(col_slice(w.ko, p0, Pl), e->ko + p0, P, e->ts_part, E);
        if (proj_batch(e, &o, 1, n)) return -1;
    }
    trunk_allreduce(e, out, E, n);
    return 0;
}

static MlaShape mla_shape(const g5b_engine *e)
{
    const g5b_config &c = e->c;
    MlaShape s;
    s.H = c.mla_heads; s.qn = c.qk_nope; s.vh = c.v_head; s.KL = c.kv_lora; s.q_lora = c.q_lora;
    s.E = c.hidden; s.cap = e->cap; s.ID = c.index_dim; s.IH = c.index_heads; s.KP = c.index_kpool;
    s.topk = c.index_topk; s.rms_eps = c.rms_eps; s.latent_bf16 = e->latent_bf16;
    return s;
}

// In a connected expert-parallel group (option "tensor_split") the MLA layer is split by heads too:
// every rank appends the same latent and indexer rows (those caches stay replicated, the selection
// is identical everywhere), but multiplies only its own heads' rows of q_b, absorbs, attends and
// projects values for those heads (the kernels see a layer of H / N heads: compact buffers, kv_b
// row-sliced to the heads' W_k | W_v rows), and multiplies its heads' columns of o_proj; the partial
// output rows are summed in rank order like the KDA layer's. FP8 slices must start on scale-block
// boundaries. The tensor-core attention core takes heads in groups of 16: a rank with fewer heads
// (8 at N = 8) pads the group with zero queries when the call is one new token (the padding
// relies on the single token's [heads][latent] rows being a prefix of the padded block), and keeps
// the layer whole otherwise.
static bool mla_heads_split(const g5b_engine *e, const Layer &w, const MlaShape &s, int n, bool batch)
{
    if (!e->tensor_split || e->seq_split || e->ep_size < 2 || !e->ep_connected) return false;
    const int N = e->ep_size;
    if (s.H % N || (s.E % 4)) return false;
    const int Hl = s.H / N;
    if (w.kv_b.dt == G5B_DT_FP8) return false;
    if (w.q_b.dt == G5B_DT_FP8 && (Hl * s.qn) % w.q_b.br) return false;
    if (w.mo.dt == G5B_DT_FP8 && (Hl * s.vh) % w.mo.bc) return false;
    if (w.mo.dt != G5B_DT_FP8 && (Hl * s.vh) % 8) return false;
    MlaShape sl = s; sl.H = Hl;
    if (e->mla_tensor && mla_flash_takes(s) && !mla_flash_takes(sl)) {                // keep the tensor-core core
        MlaShape sp = sl; sp.H = (Hl + 15) / 16 * 16;
        if (!(n == 1 && !batch && sp.H <= s.H && mla_flash_takes(sp))) return false;
    }
    return true;
}

static int run_mla(g5b_engine *e, Layer &w, const float *x, int n, int cached, float *out, bool batch = false)
{
    const g5b_config &c = e->c;
    const int E = c.hidden;
    MlaShape s = mla_shape(e);
    // the caches of the sequence(s) this call works on
    void *lat = static_cast<uint8_t *>(w.latent) + (batch ? 0 : (size_t)e->cur_seq * e->lat_seq * (e->latent_bf16 ? 2 : 4));
    float *ist = w.idx_state + (batch ? 0 : (size_t)e->cur_seq * e->idx_seq);
    if (batch) { s.batch = 1; s.lat_seq = e->lat_seq; s.idx_seq = e->idx_seq; }
    if (!w.q_a.loaded() || !w.kv_b.loaded() || !w.mo.loaded() || !w.wq_b.loaded() || !w.ape || !w.latent)
        return fail("this layer's MLA weights were not loaded");
    if (cached + (batch ? 1 : n) > e->cap) return fail("MLA cache position %d beyond capacity %d", cached + (batch ? 1 : n) - 1, e->cap);
    const bool ms = mla_heads_split(e, w, s, n, batch);
    const int Hl = ms ? s.H / e->ep_size : s.H, h0 = ms ? e->ep_rank * Hl : 0;
    MlaShape sl = s;                               // what the per-head kernels see
    sl.H = Hl;
    MlaShape sf = sl;                              // what the tensor-core attention core sees: heads padded to its group of 16
    bool flash = e->mla_tensor && mla_flash_takes(sl);
    if (!flash && ms && e->mla_tensor && n == 1 && !batch) {
        sf.H = (Hl + 15) / 16 * 16;
        flash = sf.H <= s.H && mla_flash_takes(sf);
        if (flash) CU(cudaMemsetAsync(e->mqa + (size_t)Hl * s.KL, 0, (size_t)(sf.H - Hl) * s.KL * sizeof(double), e->st));
    }
    const DMat qb = ms ? row_slice(w.q_b, h0 * s.qn, Hl * s.qn) : w.q_b;
    const DMat kvb = ms ? row_slice(w.kv_b, h0 * (s.qn + s.vh), Hl * (s.qn + s.vh)) : w.kv_b;
    GemvSeg a[5] = {make_seg(w.q_a, x, E, e->mq_raw, c.q_lora), make_seg(w.kv_a, x, E, e->mct, c.kv_lora),
                    make_seg(w.wk, x, E, e->mwk, c.index_dim), make_seg(w.igate, x, E, e->mgate, c.index_dim),
                    make_seg(w.wproj, x, E, e->mwp, c.index_heads)};
    if (proj_batch(e, a, 5, n, true)) return -1;
    mla_store(e->st, lat, ist, e->mct, w.kv_a_norm, e->mwk, e->mgate, w.k_norm_w, w.k_norm_b,
              w.ape, e->mq_raw, e->minvq, n, cached, s);
    // q = q_b(RMSNorm(q_a x)) and the indexer query, the norm applied on the way into the product
    GemvSeg b[2] = {make_seg(qb, e->mq_raw, c.q_lora, e->mq, Hl * c.qk_nope, e->minvq, w.q_a_norm),
                    make_seg(w.wq_b, e->mq_raw, c.q_lora, e->mqidx, c.index_heads * c.index_dim, e->minvq, w.q_a_norm)};
    if (proj_batch(e, b, 2, n, true)) return -1;
    // The indexer (pool scores, top-k, expansion: two latency-bound kernels) and the absorption of
    // W_k into the query need nothing from each other: the absorption runs on the side stream
    // meanwhile and the main stream takes it back before the scores.
    bool forked = false, join = false;
    if (e->side && e->side_ev && e->side_done && cudaEventRecord(e->side_ev, e->st) == cudaSuccess &&
        cudaStreamWaitEvent(e->side, e->side_ev, 0) == cudaSuccess) {
        mla_absorb(e->side, e->mqa, e->mq, kvb, n, sl);
        forked = true;
        join = cudaEventRecord(e->side_done, e->side) == cudaSuccess;
        if (!join) cudaStreamSynchronize(e->side);
    }
    dsa_select(e->st, e->msel, e->mnsel, ist, e->mqidx, e->mwp, e->mscore, n, cached, s);
    if (!forked) mla_absorb(e->st, e->mqa, e->mq, kvb, n, sl);
    else if (join && cudaStreamWaitEvent(e->st, e->side_done, 0) != cudaSuccess) cudaStreamSynchronize(e->side);
    if (flash)
        mla_attend_flash(e->st, e->mcb, e->mqa, lat, e->msel, e->mnsel, e->mpart, e->mpart_bytes, e->mdsc, n, cached, sf);
    else
        mla_attend(e->st, e->mcb, e->mqa, lat, e->msel, e->mnsel, e->mdsc, e->mpart, e->mstats, e->mcount, MLA_PART_TOKENS, n, cached, sl);
    mla_vout(e->st, e->macc, e->mcb, kvb, n, sl);
    if (ms) {
        GemvSeg o = make_seg(col_slice(w.mo, h0 * s.vh, Hl * s.vh), e->macc, Hl * c.v_head, e->ts_part, E);
        if (proj_batch(e, &o, 1, n, true)) return -1;
        trunk_allreduce(e, out, E, n);
    } else {
        GemvSeg o = make_seg(w.mo, e->macc, c.mla_heads * c.v_head, out, E);
        if (proj_batch(e, &o, 1, n, true)) return -1;
    }
    return 0;
}

static int run_hc_pre(g5b_engine *e, const HcW &hw, const float *h, int n)
{
    if (!hw.fn.loaded() || !hw.base || !hw.scale) return fail("this layer's mHC weights were not loaded");
    const g5b_config &c = e->c;
    const int M = c.hc_mult, E = c.hidden, MIX = (2 + M) * M;
    rms_factor(e->st, h, M * E, M * E, n, c.rms_eps, e->inv0);
    gemv(e->st, hw.fn, h, M * E, e->mix, MIX, n, e->inv0, nullptr);
    hc_finish(e->st, e->xc, e->post, e->comb, h, e->mix, hw, n, M, E, c.hc_iters, c.hc_eps);
    return 0;
}

// The stream expansion a decoder-layer site still owes (see run_layer).
static void flush_hc_post(g5b_engine *e)
{
    if (!e->post_h) return;
    hc_post(e->st, e->post_h, e->y, e->post, e->comb, e->post_n, e->c.hc_mult, e->c.hidden);
    e->post_h = nullptr;
}

// One decoder layer over n <= CHUNK positions (reference: glm53f_decoder_layer,
// src/core/glm53f_ops.c:1400-1433).
static int run_layer(g5b_engine *e, int l, float *h, int n, int cached, bool batch = false)
{
    const g5b_config &c = e->c;
    Layer &w = e->L[l];
    const int M = c.hc_mult, E = c.hidden;
    for (int site = 0; site < 2; site++) {
        if (!w.in_norm || !w.post_norm) return fail("this layer's norms were not loaded");
        const HcW &hw = w.hc[site];
        if (hw.fn.loaded() && hw.base && hw.scale && hc_pre_fused_supported(hw, M, E)) {
            // the previous site's stream expansion, if still owed to these positions, rides along
            const bool ride = e->post_h == h && e->post_n == n;
            if (!ride) flush_hc_post(e);
            hc_pre_fused(e->st, e->xn, e->post, e->comb, h, ride ? e->y : nullptr, hw, site ? w.post_norm : w.in_norm,
                         e->hc_part, e->hc_count, n, M, E, c.hc_iters, c.hc_eps, c.rms_eps);
            e->post_h = nullptr;
        } else {
            flush_hc_post(e);
            if (run_hc_pre(e, hw, h, n)) return -1;
            rms_factor(e->st, e->xc, E, E, n, c.rms_eps, e->inv1);
            rms_apply(e->st, e->xn, e->xc, site ? w.post_norm : w.in_norm, e->inv1, E, E, n);
        }
        int rc;
        if (site == 0) rc = w.is_mla ? run_mla(e, w, e->xn, n, cached, e->y, batch) : run_kda(e, w, e->xn, n, e->y, batch);
        else           rc = w.is_dense ? run_mlp(e, w, e->xn, n, e->y) : run_moe(e, w, e->xn, n, e->y, 1);
        if (rc) return rc;
        // owed: h' = hc_post(h, y). The next site on these positions applies it inside its own launch;
        // anything else that touches h calls flush_hc_post first.
        e->post_h = h; e->post_n = n;
    }
    return 0;
}

// A kernel whose bounded wait ran out wrote its code here; the step's result is then invalid.
static int check_device_error(g5b_engine *e)
{
    if (e->err_host && *e->err_host) {
        const int code = *e->err_host;
        *e->err_host = 0;
        // the grid-wide counters and tile counters of the interrupted launch are unusable: start over
        cudaMemsetAsync(e->grid_sync, 0, 2 * sizeof(unsigned long long), e->st);
        cudaMemsetAsync(e->tile_done, 0, ((size_t)e->c.hidden / 32 + 1) * sizeof(int), e->st);
        if (e->ep_arrive) cudaMemsetAsync(e->ep_arrive, 0, sizeof(int), e->st);
        cudaStreamSynchronize(e->st);
        e->grid_launches = 0;
        return fail("a device-side wait timed out (code %d); the result of this call is invalid", code);
    }
    return 0;
}

static int ensure_h(g5b_engine *e, size_t tokens)
{
    if (tokens <= e->h_tokens) return 0;
    const size_t per = (size_t)e->c.hc_mult * e->c.hidden;
    if (e->h) cudaFree(e->h);
    e->h = nullptr; e->h_tokens = 0;
    CU(cudaMalloc((void **)&e->h, tokens * per * 4));
    e->h_tokens = tokens;
    return 0;
}

static int ensure_ids(g5b_engine *e, size_t n)
{
    if (n <= e->ids_cap) return 0;
    if (e->ids_dev) cudaFree(e->ids_dev);
    e->ids_dev = nullptr; e->ids_cap = 0;
    CU(cudaMalloc((void **)&e->ids_dev, n * 4));
    e->ids_cap = n;
    return 0;
}

// Layers over T positions whose ids are already on the device, then the head for positions
// [first, T): logits of position t land in e->logits row (t - first) % CHUNK, arg-max in
// e->am_out[t].
// batch: the T ids are one new token for each of sequences 0..T-1 (T <= CHUNK), all at position
// e->cached; logits_host then receives all T rows.
// need_logits = false (greedy decode of one token): only the arg-max is wanted, so a connected
// expert-parallel group splits the head by vocabulary rows - rank r multiplies rows [r V / N,
// (r + 1) V / N), takes its own arg-max, and the ranks exchange (value, index) pairs and pick the
// first maximum in index order, which is the arg-max of the whole row.
static int forward_device(g5b_engine *e, const int *ids_dev, int T, bool all_positions, float *logits_host,
                          int *argmax_host, bool batch = false, bool need_logits = true)
{
    const g5b_config &c = e->c;
    const int M = c.hc_mult, E = c.hidden;
    if (!e->embed.loaded() || !e->lm_head.loaded() || !e->norm)
        return fail("forward needs embed_tokens, norm and lm_head");
    if (ensure_h(e, (size_t)T)) return -1;
    e->post_h = nullptr;                              // nothing is owed from a call that failed half-way
    embed_rows(e->st, e->h, e->embed, ids_dev, T, M);
    for (int l = 0; l < c.n_layers; l++)
        for (int t0 = 0; t0 < T; t0 += CHUNK) {
            const int n = T - t0 < CHUNK ? T - t0 : CHUNK;
            if (run_layer(e, l, e->h + (size_t)t0 * M * E, n, batch ? e->cached : e->cached + t0, batch)) return -1;
        }
    flush_hc_post(e);
    // with the MTP layer open every position's stream mean is kept, row t of this call
    // (src/model/glm53f_model.c:460-468)
    if (e->mtp && (size_t)T <= (size_t)e->cap + CHUNK) { head_mean(e->st, e->mtp_h, e->h, T, M, E); e->last_T = T; }
    const int first = all_positions ? 0 : T - 1;
    for (int t0 = first; t0 < T; t0 += CHUNK) {
        const int n = T - t0 < CHUNK ? T - t0 : CHUNK;
        head_mean(e->st, e->xm, e->h + (size_t)t0 * M * E, n, M, E);
        rms_factor(e->st, e->xm, E, E, n, c.rms_eps, e->inv_head);
        if (!need_logits && !logits_host && n == 1 && T == 1 && !batch && e->tensor_split && !e->seq_split && e->ep_size > 1 &&
            e->ep_connected && e->ep_size <= 8 && c.vocab >= 8 * e->ep_size) {
            const int per = (c.vocab + e->ep_size - 1) / e->ep_size, r0 = e->ep_rank * per;
            const int rows = c.vocab - r0 < per ? c.vocab - r0 : per;
            if (proj(e, row_slice(e->lm_head, r0, rows), e->xm, E, e->logits + r0, c.vocab, 1, e->inv_head, e->norm)) return -1;
            argmax_rows(e->st, e->am_out + t0, e->logits + r0, rows, 1, e->am_v, e->am_i);
            ++e->head_launches;
            HeadPick hp{e->logits + r0, e->am_out + t0, r0, e->ep_peers_dev, e->ep_rank, e->ep_size, EP_HEAD_WORD0,
                        e->head_launches, (unsigned long long)e->ep_wait_ms * 1000000ull, e->err_dev};
            head_pick_exchange(e->st, hp);
            continue;
        }
        if (proj(e, e->lm_head, e->xm, E, e->logits, c.vocab, n, e->inv_head, e->norm)) return -1;
        argmax_rows(e->st, e->am_out + t0, e->logits, c.vocab, n, e->am_v, e->am_i);
        if (logits_host && batch)
            CU(cudaMemcpyAsync(logits_host, e->logits, (size_t)n * c.vocab * 4, cudaMemcpyDeviceToHost, e->st));
        else if (logits_host && t0 + n == T)
            CU(cudaMemcpyAsync(logits_host, e->logits + (size_t)(n - 1) * c.vocab, (size_t)c.vocab * 4,
                               cudaMemcpyDeviceToHost, e->st));
    }
    if (argmax_host)
        CU(cudaMemcpyAsync(argmax_host, e->am_out + first, (size_t)(T - first) * 4, cudaMemcpyDeviceToHost, e->st));
    return 0;
}

extern "C" int g5b_engine_forward(g5b_engine *e, const int *ids, int T, float *logits, int *argmax_all)
{
    if (!e->finalized) return fail("forward before finalize");
    CU(cudaSetDevice(e->device));
    if (e->dirty) return fail("an earlier call failed half-way: reset the engine (g5b_engine_reset) first");
    if (T < 1) return fail("forward needs at least one token");
    if (e->cached + T > e->cap)
        return fail("%d cached + %d new positions exceed the session capacity %d", e->cached, T, e->cap);
    for (int t = 0; t < T; t++)
        if (ids[t] < 0 || ids[t] >= e->c.vocab) return fail("token id %d outside the vocabulary", ids[t]);
    if (ensure_ids(e, (size_t)T)) return -1;
    CU(cudaMemcpyAsync(e->ids_dev, ids, (size_t)T * 4, cudaMemcpyHostToDevice, e->st));
    // from here on the session state is being advanced: any failure leaves it undefined
    e->dirty = true;
    if (forward_device(e, e->ids_dev, T, argmax_all != nullptr, logits, argmax_all)) return -1;
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    if (check_device_error(e)) return -1;
    e->dirty = false;
    e->cached += T;
    return 0;
}

// Greedy decode without host round trips: each step's arg-max (already in device memory) is the
// next step's token id.
extern "C" int g5b_engine_decode_greedy(g5b_engine *e, int first, int n, int *out)
{
    if (!e->finalized) return fail("decode before finalize");
    CU(cudaSetDevice(e->device));
    if (e->dirty) return fail("an earlier call failed half-way: reset the engine (g5b_engine_reset) first");
    if (n < 1 || e->cached + n > e->cap) return fail("decode of %d tokens exceeds the session capacity", n);
    if (first < 0 || first >= e->c.vocab) return fail("token id %d outside the vocabulary", first);
    if (ensure_ids(e, (size_t)n + 1)) return -1;
    CU(cudaMemcpyAsync(e->ids_dev, &first, 4, cudaMemcpyHostToDevice, e->st));
    // The position count is committed only once every step is known to have succeeded; until then
    // the session is marked undefined, so that a failed call cannot be continued by accident.
    const int start = e->cached;
    e->dirty = true;
    for (int i = 0; i < n; i++) {
        e->cached = start + i;
        const int rc = forward_device(e, e->ids_dev + i, 1, false, nullptr, nullptr, false, false);
        if (rc) { e->cached = start; return -1; }
        CU(cudaMemcpyAsync(e->ids_dev + i + 1, e->am_out, 4, cudaMemcpyDeviceToDevice, e->st));
    }
    e->cached = start;
    CU(cudaMemcpyAsync(out, e->ids_dev + 1, (size_t)n * 4, cudaMemcpyDeviceToHost, e->st));
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    if (check_device_error(e)) return -1;
    e->dirty = false;
    e->cached = start + n;
    return 0;
}

// Sampled decode without host round trips: each step's token is drawn on the device from that
// step's logits (sample.cu) and is the next step's input. temperature <= 0 decodes greedily.
extern "C" int g5b_engine_decode_sampled(g5b_engine *e, int first, int n, float temperature, float top_p,
                                         uint64_t seed, int *out)
{
    if (!e->finalized) return fail("decode before finalize");
    if (!(temperature > 0.f)) return g5b_engine_decode_greedy(e, first, n, out);
    if (!(top_p > 0.f)) return fail("top_p must be positive (1 keeps every token)");
    CU(cudaSetDevice(e->device));
    if (e->dirty) return fail("an earlier call failed half-way: reset the engine (g5b_engine_reset) first");
    if (n < 1 || e->cached + n > e->cap) return fail("decode of %d tokens exceeds the session capacity", n);
    if (first < 0 || first >= e->c.vocab) return fail("token id %d outside the vocabulary", first);
    if (ensure_ids(e, (size_t)n + 1)) return -1;
    CU(cudaMemcpyAsync(e->ids_dev, &first, 4, cudaMemcpyHostToDevice, e->st));
    const int start = e->cached;
    e->dirty = true;
    for (int i = 0; i < n; i++) {
        e->cached = start + i;
        const int rc = forward_device(e, e->ids_dev + i, 1, false, nullptr, nullptr);
        if (rc) { e->cached = start; return -1; }
        // the step counter of the draw is the position the token will occupy
        sample_token(e->st, e->ids_dev + i + 1, e->logits, e->logits + e->c.vocab, e->c.vocab, temperature, top_p, seed,
                     (uint64_t)(start + i + 1));
    }
    e->cached = start;
    CU(cudaMemcpyAsync(out, e->ids_dev + 1, (size_t)n * 4, cudaMemcpyDeviceToHost, e->st));
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    if (check_device_error(e)) return -1;
    e->dirty = false;
    e->cached = start + n;
    return 0;
}

extern "C" void g5b_engine_reset(g5b_engine *e)
{
    cudaSetDevice(e->device);
    const g5b_config &c = e->c;
    const size_t P = (size_t)c.kda_heads * c.kda_head_dim;
    (void)P;
    for (auto &w : e->L)
        if (w.kda_state) cudaMemsetAsync(w.kda_state, 0, (size_t)e->n_seq * e->kda_seq * 4, e->st);
    cudaStreamSynchronize(e->st);
    e->cached = 0;
    e->mtp_cached = 0;
    e->dirty = false;
    e->post_h = nullptr;
    for (auto &v : e->cached_seq) v = 0;
}

// Stand-in for a long prefill: every sequence's session state (KDA state ~ 0.1 N(0,1), latent cache
// and indexer state ~ N(0,1), BF16-representable, from the hash generators) filled on the device
// and every sequence's position set to `positions`, so that a batch decode can be measured at a
// deep context without first running the prompts through the model.
extern "C" int g5b_engine_synth_session(g5b_engine *e, uint64_t seed, int positions)
{
    if (!e || !e->finalized) return fail("synth_session before finalize");
    if (positions < 0 || positions >= e->cap) return fail("%d positions do not leave room in a capacity of %d", positions, e->cap);
    CU(cudaSetDevice(e->device));
    const float unit = 1.0f / 37837.2f;
    // with the sequences split over the ranks, local sequence q is sequence rank * n_seq + q of the
    // whole batch and gets that sequence's values (an element's value is a hash of key + its index)
    const size_t first = e->seq_split ? (size_t)e->ep_rank * e->n_seq : 0;
    for (size_t l = 0; l < e->L.size(); l++) {
        Layer &w = e->L[l];
        char name[64];
        if (w.kda_state) {
            snprintf(name, sizeof name, "state.%zu.kda", l);
            fill_f32_key(e->st, w.kda_state, synth_key(seed, name) + first * e->kda_seq, 0.1f * unit, (size_t)e->n_seq * e->kda_seq);
        }
        if (w.latent) {
            snprintf(name, sizeof name, "state.%zu.latent", l);
            const uint64_t key = synth_key(seed, name) + first * e->lat_seq;
            if (e->latent_bf16) fill_bf16_key(e->st, static_cast<uint16_t *>(w.latent), key, unit, (size_t)e->n_seq * e->lat_seq);
            else                fill_f32_key(e->st, static_cast<float *>(w.latent), key, unit, (size_t)e->n_seq * e->lat_seq);
            snprintf(name, sizeof name, "state.%zu.indexer", l);
            fill_f32_key(e->st, w.idx_state, synth_key(seed, name) + first * e->idx_seq, unit, (size_t)e->n_seq * e->idx_seq);
        }
    }
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    e->cached = positions;
    for (auto &v : e->cached_seq) v = positions;
    e->dirty = false;
    return 0;
}

// Which sequence the single-sequence calls (forward, decode_greedy, layer ops, state access) address.
extern "C" int g5b_engine_use_sequence(g5b_engine *e, int seq)
{
    if (!e || !e->finalized) return fail("use_sequence before finalize");
    if (seq < 0 || seq >= e->n_seq) return fail("sequence %d of %d", seq, e->n_seq);
    e->cached_seq[(size_t)e->cur_seq] = e->cached;
    e->cur_seq = seq;
    e->cached = e->cached_seq[(size_t)seq];
    return 0;
}

// One new token for every sequence at once (lockstep decode): ids[s] continues sequence s; all
// sequences must hold the same number of positions. logits: [n_seq][vocab] or NULL; argmax:
// [n_seq] or NULL. Attention state and caches are per sequence, every weight is read once for
// the whole batch.
extern "C" int g5b_engine_decode_batch(g5b_engine *e, const int *ids, float *logits, int *argmax)
{
    if (!e || !e->finalized) return fail("decode_batch before finalize");
    CU(cudaSetDevice(e->device));
    if (e->dirty) return fail("an earlier call failed half-way: reset the engine (g5b_engine_reset) first");
    const int S = e->n_seq;
    e->cached_seq[(size_t)e->cur_seq] = e->cached;
    for (int q = 1; q < S; q++)
        if (e->cached_seq[(size_t)q] != e->cached_seq[0])
            return fail("decode_batch needs sequences of equal length (sequence %d holds %d positions, sequence 0 %d)", q,
                        e->cached_seq[(size_t)q], e->cached_seq[0]);
    const int pos = e->cached_seq[0];
    if (pos + 1 > e->cap) return fail("%d cached + 1 new position exceed the session capacity %d", pos, e->cap);
    for (int q = 0; q < S; q++)
        if (ids[q] < 0 || ids[q] >= e->c.vocab) return fail("token id %d outside the vocabulary", ids[q]);
    if (ensure_ids(e, (size_t)S)) return -1;
    CU(cudaMemcpyAsync(e->ids_dev, ids, (size_t)S * 4, cudaMemcpyHostToDevice, e->st));
    const int keep = e->cached;
    e->cached = pos;
    e->dirty = true;
    const int rc = forward_device(e, e->ids_dev, S, true, logits, argmax, true);
    e->cached = keep;
    if (rc) return -1;
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    if (check_device_error(e)) return -1;
    e->dirty = false;
    for (auto &v : e->cached_seq) v = pos + 1;
    e->cached = pos + 1;
    return 0;
}

extern "C" int g5b_engine_cached(const g5b_engine *e) { return e->cached; }

extern "C" void g5b_engine_free(g5b_engine *e)
{
    if (!e) return;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->st);
    tc_gemm_free(e->tc);
    for (void *p : e->owned) cudaFree(p);
    for (void *p : e->ep_opened) cudaIpcCloseMemHandle(p);
    for (void *p : e->ep_standins) cudaFree(p);
    if (e->ep_region) cudaFree(e->ep_region);
    if (e->h) cudaFree(e->h);
    if (e->ids_dev) cudaFree(e->ids_dev);
    if (e->flush_buf) cudaFree(e->flush_buf);
    if (e->err_host) cudaFreeHost((void *)e->err_host);
    for (int i = 0; i <= PROF_SLOTS; i++) cudaEventDestroy(e->prof_ev[i]);
    if (e->side) { cudaStreamSynchronize(e->side); cudaStreamDestroy(e->side); }
    if (e->side_ev) cudaEventDestroy(e->side_ev);
    if (e->side_done) cudaEventDestroy(e->side_done);
    cudaStreamDestroy(e->st);
    delete e;
}

extern "C" int g5b_engine_sync(g5b_engine *e)
{
    CU(cudaSetDevice(e->device));
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    return check_device_error(e);
}

extern "C" void *g5b_engine_stream(g5b_engine *e) { return (void *)e->st; }

// -------------------------------------------------------------- device-pointer ops ----
static int check_layer(g5b_engine *e, int layer, int n)
{
    if (!e->finalized) return fail("op before finalize");
    if (layer < 0 || layer >= (int)e->L.size()) return fail("layer %d out of range", layer);
    if (n < 1 || n > CHUNK) return fail("ops take 1..%d positions per call, got %d", CHUNK, n);
    if (cudaSetDevice(e->device) != cudaSuccess) return fail("cudaSetDevice failed");
    return 0;
}

extern "C" int g5b_dev_moe(g5b_engine *e, int layer, const float *x_dev, int T, float *out_dev)
{
    if (check_layer(e, layer, T)) return -1;
    if (e->L[layer].is_dense) return fail("layer %d has a dense MLP", layer);
    return run_moe(e, e->L[layer], x_dev, T, out_dev, 1);
}

extern "C" int g5b_dev_kda(g5b_engine *e, int layer, const float *x_dev, int T, float *out_dev)
{
    if (check_layer(e, layer, T)) return -1;
    if (e->L[layer].is_mla) return fail("layer %d is an MLA layer", layer);
    return run_kda(e, e->L[layer], x_dev, T, out_dev);
}

extern "C" int g5b_dev_mla(g5b_engine *e, int layer, const float *x_dev, int T, int cached, float *out_dev)
{
    if (check_layer(e, layer, T)) return -1;
    if (!e->L[layer].is_mla) return fail("layer %d is a KDA layer", layer);
    return run_mla(e, e->L[layer], x_dev, T, cached, out_dev);
}

extern "C" int g5b_dev_decoder_layer(g5b_engine *e, int layer, float *h_dev, int T, int cached)
{
    if (check_layer(e, layer, T)) return -1;
    e->post_h = nullptr;
    const int rc = run_layer(e, layer, h_dev, T, cached);
    if (rc) e->post_h = nullptr;
    flush_hc_post(e);
    return rc;
}

// ------------------------------------------------------------------ host-buffer ops ----
struct Staged {
    g5b_engine *e;
    std::vector<void *> bufs;
    ~Staged() { for (void *p : bufs) cudaFree(p); }
    float *in(const float *src, size_t n)
    {
        void *p = nullptr;
        if (cudaMalloc(&p, n * 4 + 16) != cudaSuccess) return nullptr;
        bufs.push_back(p);
        if (src) cudaMemcpyAsync(p, src, n * 4, cudaMemcpyHostToDevice, e->st);
        else     cudaMemsetAsync(p, 0, n * 4, e->st);
        return (float *)p;
    }
    int out(float *dst, const float *src, size_t n)
    {
        CU(cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaStreamSynchronize(e->st));
        CU(cudaGetLastError());
        return check_device_error(e);
    }
};

// Ops accept any T >= 1: the host entry points walk it in CHUNK-sized pieces.
static int check_op(g5b_engine *e, int layer, int T)
{
    if (T < 1) return fail("ops take at least one position, got %d", T);
    return check_layer(e, layer, 1);
}

#define FOR_CHUNKS(T) for (int t0 = 0, n_ = 0; (n_ = (T) - t0 < CHUNK ? (T) - t0 : CHUNK), t0 < (T); t0 += CHUNK)

// glm53f_mtp_feed (src/model/glm53f_mtp.c:100-144) on the MTP layer's own caches and position
// count: x = eh_proj([RMSNorm(embed(next), enorm), RMSNorm(h, hnorm)]); x += MLA(RMSNorm(x,
// input_layernorm)); x += MoE(RMSNorm(x, post_attention_layernorm)); for the last position the
// draft is the first-max arg-max of lm_head(RMSNorm(x, shared_head.norm)). The hidden states: T host
// rows `h`, else T device rows `h_dev`, else the rows the last forward call kept (from row 0).
// x_out: host [T][hidden] or NULL.
static int mtp_feed_rows(g5b_engine *e, const float *h, const float *h_dev, const int *next_ids, int T, int *draft, float *x_out)
{
    if (!e || !e->finalized || !e->mtp) return fail("the MTP layer is not enabled (g5b_engine_enable_mtp before loading)");
    CU(cudaSetDevice(e->device));
    const g5b_config &c = e->c;
    const int E = c.hidden;
    if (T < 1) return fail("mtp_feed needs at least one position");
    if (e->mtp_cached + T > e->cap) return fail("%d + %d MTP positions exceed the capacity %d", e->mtp_cached, T, e->cap);
    if (!h && T > e->cap + CHUNK) return fail("no kept hidden states for %d positions", T);
    for (int t = 0; t < T; t++)
        if (next_ids[t] < 0 || next_ids[t] >= c.vocab) return fail("token id %d outside the vocabulary", next_ids[t]);
    if (!e->embed.loaded() || !e->lm_head.loaded() || !e->eh.loaded() || !e->enorm || !e->hnorm || !e->head_norm)
        return fail("mtp_feed needs embed_tokens, lm_head and the MTP layer's tensors");
    Layer &w = e->L[(size_t)c.n_layers];
    if (ensure_ids(e, (size_t)T)) return -1;
    CU(cudaMemcpyAsync(e->ids_dev, next_ids, (size_t)T * 4, cudaMemcpyHostToDevice, e->st));
    Staged s{e};
    const float *hd = h_dev ? h_dev : e->mtp_h;          // device rows: the caller's, or the kept ones from row 0
    if (h) {
        hd = s.in(h, (size_t)T * E);
        if (!hd) return fail("out of device memory");
    }
    float *xo = nullptr;
    if (x_out) {
        xo = s.in(nullptr, (size_t)T * E);
        if (!xo) return fail("out of device memory");
    }
    e->post_h = nullptr;
    for (int t0 = 0; t0 < T; t0 += CHUNK) {
        const int n = T - t0 < CHUNK ? T - t0 : CHUNK;
        float *cat = e->mtp_cat, *x = e->mtp_x;
        embed_rows(e->st, cat, e->embed, e->ids_dev + t0, n, 2);                 // both halves; the second is replaced
        CU(cudaMemcpy2DAsync(cat + E, (size_t)2 * E * 4, hd + (size_t)t0 * E, (size_t)E * 4, (size_t)E * 4, (size_t)n,
                             cudaMemcpyDeviceToDevice, e->st));
        rms_factor(e->st, cat, E, 2 * E, n, c.rms_eps, e->inv0);
        rms_apply(e->st, cat, cat, e->enorm, e->inv0, E, 2 * E, n);
        rms_factor(e->st, cat + E, E, 2 * E, n, c.rms_eps, e->inv1);
        rms_apply(e->st, cat + E, cat + E, e->hnorm, e->inv1, E, 2 * E, n);
        if (proj(e, e->eh, cat, 2 * E, x, E, n)) return -1;
        rms_factor(e->st, x, E, E, n, c.rms_eps, e->inv1);
        rms_apply(e->st, e->xn, x, w.in_norm, e->inv1, E, E, n);
        if (run_mla(e, w, e->xn, n, e->mtp_cached + t0, e->y)) return -1;
        add_rows(e->st, x, e->y, (size_t)n * E);
        rms_factor(e->st, x, E, E, n, c.rms_eps, e->inv1);
        rms_apply(e->st, e->xn, x, w.post_norm, e->inv1, E, E, n);
        if (run_moe(e, w, e->xn, n, e->y, 1)) return -1;
        add_rows(e->st, x, e->y, (size_t)n * E);
        if (xo) CU(cudaMemcpyAsync(xo + (size_t)t0 * E, x, (size_t)n * E * 4, cudaMemcpyDeviceToDevice, e->st));
        if (draft && t0 + n == T) {
            const float *last = x + (size_t)(n - 1) * E;
            rms_factor(e->st, last, E, E, 1, c.rms_eps, e->inv_head);
            if (proj(e, e->lm_head, last, E, e->logits, c.vocab, 1, e->inv_head, e->head_norm)) return -1;
            argmax_rows(e->st, e->am_out, e->logits, c.vocab, 1, e->am_v, e->am_i);
            CU(cudaMemcpyAsync(draft, e->am_out, 4, cudaMemcpyDeviceToHost, e->st));
        }
    }
    if (x_out && s.out(x_out, xo, (size_t)T * E)) return -1;
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    if (check_device_error(e)) return -1;
    e->mtp_cached += T;
    return 0;
}

// Speculative greedy decode with the MTP layer as the drafter (the use glm53f_mtp.h:11-14 describes;
// the reference itself only counts how often a draft is right). Every pass feeds the model two
// positions, the current token and the draft of the one after it; the draft is kept only when
// the model's own arg-max for that position is the same token, so the tokens are those of greedy
// decode (a position verified in a two-position pass goes through the kernels for several
// positions, whose sums can differ from the one-position kernels' in the last bits). A rejected
// draft has already advanced the KDA states: during such a pass every KDA layer also writes its
// state as it is after the first position to a second buffer, and a rejection copies that back;
// latent and indexer rows of the rejected position are simply written again by the next pass. Needs the MTP layer fed up to, not including, the last cached position
// (after a prompt: its hidden states but the last with its tokens but the first), and the hidden
// state of the last position still kept (no other forward call in between).
// stats: [0] drafts made, [1] drafts accepted, [2] model passes.
extern "C" int g5b_engine_decode_speculative(g5b_engine *e, int first, int n, int *out, long *stats)
{
    if (!e || !e->finalized || !e->mtp) return fail("the MTP layer is not enabled (g5b_engine_enable_mtp before loading)");
    CU(cudaSetDevice(e->device));
    if (e->dirty) return fail("an earlier call failed half-way: reset the engine (g5b_engine_reset) first");
    if (n < 1 || e->cached + n + 1 > e->cap) return fail("speculative decode of %d tokens exceeds the session capacity", n);
    if (first < 0 || first >= e->c.vocab) return fail("token id %d outside the vocabulary", first);
    if (e->cached < 1 || e->mtp_cached != e->cached - 1)
        return fail("the MTP layer holds %d positions, the model %d: feed it the hidden states up to the last position but one first",
                    e->mtp_cached, e->cached);
    const g5b_config &c = e->c;
    const size_t E = (size_t)c.hidden;
    if (e->kda_snap.empty()) {
        e->kda_snap.assign((size_t)c.n_layers, nullptr);
        for (int l = 0; l < c.n_layers; l++)
            if (e->L[l].kda_state && walloc(e, &e->kda_snap[l], e->kda_seq)) return -1;
    }
    long drafts = 0, right = 0, passes = 0;
    int tok = first, got = 0;
    int h_row = e->last_T - 1;                    // row of the kept hidden states that belongs to the last cached position
    if (h_row < 0) return fail("no hidden state is kept: run the prompt first");
    while (got < n) {
        // the draft of the token after `tok`
        int draft = -1;
        if (mtp_feed_rows(e, nullptr, e->mtp_h + (size_t)h_row * E, &tok, 1, &draft, nullptr)) return -1;
        drafts++;
        if (got + 1 >= n) {
            // one token left to produce: no use for a second position
            int a = -1;
            if (g5b_engine_forward(e, &tok, 1, nullptr, &a)) return -1;
            passes++;
            out[got++] = a;
            right += a == draft;
            break;
        }
        const int pair[2] = {tok, draft};
        int am[2] = {-1, -1};
        e->snap_first = true;                     // every KDA layer also leaves its state after the first position
        const int frc = g5b_engine_forward(e, pair, 2, nullptr, am);
        e->snap_first = false;
        if (frc) return -1;
        passes++;
        if (am[0] == draft) {
            right++;
            out[got++] = am[0];
            out[got++] = am[1];
            // the MTP layer catches up with the accepted position: (its hidden state, the token after it)
            if (mtp_feed_rows(e, nullptr, e->mtp_h, &am[0], 1, nullptr, nullptr)) return -1;
            tok = am[1];
            h_row = 1;
        } else {
            // the second position was built on a wrong token: fall back to the state after the first
            for (int l = 0; l < c.n_layers; l++)
                if (e->kda_snap[l])
                    CU(cudaMemcpyAsync(e->L[l].kda_state + (size_t)e->cur_seq * e->kda_seq, e->kda_snap[l], e->kda_seq * 4,
                                       cudaMemcpyDeviceToDevice, e->st));
            CU(cudaStreamSynchronize(e->st));
            e->cached -= 1;
            out[got++] = am[0];
            tok = am[0];
            h_row = 0;
        }
    }
    if (stats) { stats[0] = drafts; stats[1] = right; stats[2] = passes; }
    return 0;
}

extern "C" int g5b_mtp_feed(g5b_engine *e, const float *h, const int *next_ids, int T, int *draft, float *x_out)
{
    return mtp_feed_rows(e, h, nullptr, next_ids, T, draft, x_out);
}

// The stream means the last forward call kept: T rows from row `first`, to the host.
extern "C" int g5b_mtp_hidden(g5b_engine *e, int first, int T, float *dst)
{
    if (!e || !e->finalized || !e->mtp) return fail("the MTP layer is not enabled");
    if (first < 0 || T < 1 || first + T > e->cap + CHUNK) return fail("rows outside the kept hidden states");
    CU(cudaSetDevice(e->device));
    CU(cudaMemcpyAsync(dst, e->mtp_h + (size_t)first * e->c.hidden, (size_t)T * e->c.hidden * 4, cudaMemcpyDeviceToHost, e->st));
    CU(cudaStreamSynchronize(e->st));
    return 0;
}


// Host buffers through the engine's own staging rows (no allocation per call): copy a piece in,
// run, copy the result out; one wait at the end. With pinned host memory the copies overlap the
// kernels of the neighbouring pieces.
// `direct_out`: the op's last kernel writes every output element exactly once with plain stores.
// If the caller's buffer is pinned and mapped, that kernel then writes straight into it (16 KB per
// token over PCIe as posted writes, visible once the stream has drained) and the copy engine's
// turn after the kernel - about 6 us of a 90 us call at batch 1 - is saved.
template <typename F>
static int host_op(g5b_engine *e, const float *x, int T, float *out, F &&run, bool direct_out = false)
{
    const size_t E = e->c.hidden;
    float *out_dev = nullptr;
    if (direct_out) {
        cudaPointerAttributes at{};
        if (cudaPointerGetAttributes(&at, out) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer)
            out_dev = static_cast<float *>(at.devicePointer);
        else
            cudaGetLastError();
    }
    FOR_CHUNKS(T) {
        CU(cudaMemcpyAsync(e->xn, x + t0 * E, n_ * E * 4, cudaMemcpyHostToDevice, e->st));
        if (run(e->xn, n_, out_dev ? out_dev + t0 * E : e->y, t0)) {
            cudaStreamSynchronize(e->st);            // copies on the caller's buffers must not outlive the call
            return -1;
        }
        if (!out_dev) CU(cudaMemcpyAsync(out + t0 * E, e->y, n_ * E * 4, cudaMemcpyDeviceToHost, e->st));
    }
    CU(cudaStreamSynchronize(e->st));
    CU(cudaGetLastError());
    return check_device_error(e);
}

extern "C" int g5b_op_moe(g5b_engine *e, int layer, const float *x, int T, float *out, int with_shared)
{
    if (check_op(e, layer, T)) return -1;
    if (e->L[layer].is_dense) return fail("layer %d has a dense MLP", layer);
    return host_op(e, x, T, out, [&](const float *xd, int n, float *od, int) {
        return run_moe(e, e->L[layer], xd, n, od, with_shared);
    }, e->ep_size <= 1);
}

extern "C" int g5b_op_router(g5b_engine *e, int layer, const float *x, int T, int *idx, float *w)
{
    if (check_op(e, layer, T)) return -1;
    if (e->L[layer].is_dense) return fail("layer %d has a dense MLP", layer);
    const size_t E = e->c.hidden, K = e->c.topk;
    Layer &lw = e->L[layer];
    Staged s{e};
    float *xd = s.in(x, (size_t)T * E);
    if (!xd) return fail("out of device memory");
    const MoeShape ms = moe_shape(e, lw);
    FOR_CHUNKS(T) {
        MoePlan none{};
        router_plan(e->st, e->ridx, e->rw, e->rscore, xd + t0 * E, (int)E, lw.router.w, lw.router.dt, lw.bias, n_, ms,
                    none, 0, e->counter);
        CU(cudaMemcpyAsync(idx + t0 * K, e->ridx, n_ * K * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaMemcpyAsync(w + t0 * K, e->rw, n_ * K * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaStreamSynchronize(e->st));
    }
    CU(cudaGetLastError());
    return 0;
}

// The expert picks and weights of the most recent MoE pass (its last chunk of T <= 64 positions),
// whatever entry point ran it - how a caller learns which experts a whole-layer op routed to.
extern "C" int g5b_engine_last_picks(g5b_engine *e, int T, int *idx, float *w)
{
    if (!e || !e->finalized) return fail("last_picks before finalize");
    if (T < 1 || T > CHUNK) return fail("last_picks covers 1..%d positions", CHUNK);
    CU(cudaSetDevice(e->device));
    const size_t n = (size_t)T * e->c.topk;
    if (idx) CU(cudaMemcpyAsync(idx, e->ridx, n * 4, cudaMemcpyDeviceToHost, e->st));
    if (w)   CU(cudaMemcpyAsync(w, e->rw, n * 4, cudaMemcpyDeviceToHost, e->st));
    CU(cudaStreamSynchronize(e->st));
    return 0;
}

extern "C" int g5b_op_mlp(g5b_engine *e, int layer, const float *x, int T, float *out)
{
    if (check_op(e, layer, T)) return -1;
    if (!e->L[layer].is_dense) return fail("layer %d is a MoE layer", layer);
    return host_op(e, x, T, out, [&](const float *xd, int n, float *od, int) {
        return run_mlp(e, e->L[layer], xd, n, od);
    });
}

extern "C" int g5b_op_kda(g5b_engine *e, int layer, const float *x, int T, float *out)
{
    if (check_op(e, layer, T)) return -1;
    if (e->L[layer].is_mla) return fail("layer %d is an MLA layer", layer);
    return host_op(e, x, T, out, [&](const float *xd, int n, float *od, int) {
        return run_kda(e, e->L[layer], xd, n, od);
    });
}

extern "C" int g5b_op_mla(g5b_engine *e, int layer, const float *x, int T, int cached, float *out,
                          int *sel_out, int *n_sel_out)
{
    if (check_op(e, layer, T)) return -1;
    if (!e->L[layer].is_mla) return fail("layer %d is a KDA layer", layer);
    int last_n = 0;
    if (host_op(e, x, T, out, [&](const float *xd, int n, float *od, int t0) {
            last_n = n;
            return run_mla(e, e->L[layer], xd, n, cached + t0, od);
        })) return -1;
    if (n_sel_out) {
        int ns = 0;
        CU(cudaMemcpyAsync(&ns, e->mnsel + last_n - 1, 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaStreamSynchronize(e->st));
        *n_sel_out = ns;
        if (sel_out && ns > 0) {
            CU(cudaMemcpyAsync(sel_out, e->msel + (size_t)(last_n - 1) * (e->c.index_topk + e->c.index_kpool),
                               (size_t)ns * 4, cudaMemcpyDeviceToHost, e->st));
            CU(cudaStreamSynchronize(e->st));
        }
    }
    return 0;
}

extern "C" int g5b_op_hc_pre(g5b_engine *e, int layer, int site, const float *h, int T, float *x,
                             float *post, float *comb)
{
    if (check_op(e, layer, T)) return -1;
    const size_t E = e->c.hidden, M = e->c.hc_mult;
    Staged s{e};
    float *hd = s.in(h, (size_t)T * M * E);
    if (!hd) return fail("out of device memory");
    FOR_CHUNKS(T) {
        if (run_hc_pre(e, e->L[layer].hc[site ? 1 : 0], hd + t0 * M * E, n_)) return -1;
        CU(cudaMemcpyAsync(x + t0 * E, e->xc, n_ * E * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaMemcpyAsync(post + t0 * M, e->post, n_ * M * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaMemcpyAsync(comb + t0 * M * M, e->comb, n_ * M * M * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaStreamSynchronize(e->st));
    }
    CU(cudaGetLastError());
    return 0;
}

extern "C" int g5b_op_hc_post(g5b_engine *e, float *h, const float *y, const float *post,
                              const float *comb, int T)
{
    if (check_op(e, 0, T)) return -1;
    const size_t E = e->c.hidden, M = e->c.hc_mult;
    Staged s{e};
    float *hd = s.in(h, (size_t)T * M * E), *yd = s.in(y, (size_t)T * E), *pd = s.in(post, (size_t)T * M),
          *cd = s.in(comb, (size_t)T * M * M);
    if (!hd || !yd || !pd || !cd) return fail("out of device memory");
    hc_post(e->st, hd, yd, pd, cd, T, (int)M, (int)E);
    return s.out(h, hd, (size_t)T * M * E);
}

extern "C" int g5b_op_decoder_layer(g5b_engine *e, int layer, float *h, int T, int cached)
{
    if (check_op(e, layer, T)) return -1;
    const size_t E = e->c.hidden, M = e->c.hc_mult;
    Staged s{e};
    float *hd = s.in(h, (size_t)T * M * E);
    if (!hd) return fail("out of device memory");
    FOR_CHUNKS(T) {
        e->post_h = nullptr;
        const int rc = run_layer(e, layer, hd + t0 * M * E, n_, cached + t0);
        if (rc) { e->post_h = nullptr; return -1; }
        flush_hc_post(e);
    }
    return s.out(h, hd, (size_t)T * M * E);
}

static DMat *find_mat(g5b_engine *e, const char *name)
{
    if (!strcmp(name, "embed_tokens.weight")) return &e->embed;
    if (!strcmp(name, "lm_head.weight")) return &e->lm_head;
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= (int)e->L.size()) return nullptr;
    auto it = e->names[l].find(name + used);
    if (it == e->names[l].end() || it->second.kind != 0 || !it->second.mat->loaded()) return nullptr;
    return it->second.mat;
}

extern "C" int g5b_op_matvec(g5b_engine *e, const char *name, const float *x, int T, float *y)
{
    CU(cudaSetDevice(e->device));
    if (T < 1) return fail("ops take at least one position, got %d", T);
    DMat *m = find_mat(e, name);
    if (!m) return fail("no loaded matrix named %s", name);
    Staged s{e};
    float *xd = s.in(x, (size_t)T * m->cols), *yd = s.in(nullptr, (size_t)T * m->rows);
    if (!xd || !yd) return fail("out of device memory");
    // the path the forward pass takes for this many positions (one-token kernels below 8, the
    // multi-token projection path from 8 on), a chunk at a time
    FOR_CHUNKS(T)
        if (proj(e, *m, xd + (size_t)t0 * m->cols, m->cols, yd + (size_t)t0 * m->rows, m->rows, n_)) return -1;
    return s.out(y, yd, (size_t)T * m->rows);
}

static float *state_ptr(g5b_engine *e, int layer, int kind, size_t *n, int *bf16)
{
    const g5b_config &c = e->c;
    Layer &w = e->L[layer];
    *bf16 = 0;
    if (kind == 0) {
        const size_t P = (size_t)c.kda_heads * c.kda_head_dim;
        *n = P * c.kda_head_dim + 3 * P * (size_t)(c.conv_k - 1);
        return w.kda_state ? w.kda_state + (size_t)e->cur_seq * e->kda_seq : nullptr;
    }
    if (kind == 1) {
        *n = (size_t)e->cap * c.kv_lora; *bf16 = e->latent_bf16;
        if (!w.latent) return nullptr;
        return (float *)(static_cast<uint8_t *>(w.latent) + (size_t)e->cur_seq * e->lat_seq * (e->latent_bf16 ? 2 : 4));
    }
    if (kind == 2) {
        *n = (size_t)2 * e->cap * c.index_dim + (size_t)((e->cap + c.index_kpool - 1) / c.index_kpool) * c.index_dim;
        return w.idx_state ? w.idx_state + (size_t)e->cur_seq * e->idx_seq : nullptr;
    }
    return nullptr;
}

extern "C" int g5b_state_write(g5b_engine *e, int layer, int kind, size_t offset, const float *src, size_t count)
{
    if (!e->finalized || layer < 0 || layer >= (int)e->L.size()) return fail("state access on a bad layer");
    CU(cudaSetDevice(e->device));
    size_t n = 0; int bf = 0;
    float *p = state_ptr(e, layer, kind, &n, &bf);
    if (!p || offset + count > n) return fail("state range outside the layer's state");
    if (!bf) {
        CU(cudaMemcpyAsync(p + offset, src, count * 4, cudaMemcpyHostToDevice, e->st));
    } else {
        Staged s{e};
        float *tmp = s.in(src, count);
        if (!tmp) return fail("out of device memory");
        f32_to_bf16(e->st, (uint16_t *)p + offset, tmp, count);
        CU(cudaStreamSynchronize(e->st));
    }
    CU(cudaStreamSynchronize(e->st));
    return 0;
}

extern "C" int g5b_state_read(g5b_engine *e, int layer, int kind, size_t offset, float *dst, size_t count)
{
    if (!e->finalized || layer < 0 || layer >= (int)e->L.size()) return fail("state access on a bad layer");
    CU(cudaSetDevice(e->device));
    size_t n = 0; int bf = 0;
    float *p = state_ptr(e, layer, kind, &n, &bf);
    if (!p || offset + count > n) return fail("state range outside the layer's state");
    if (!bf) {
        CU(cudaMemcpyAsync(dst, p + offset, count * 4, cudaMemcpyDeviceToHost, e->st));
        CU(cudaStreamSynchronize(e->st));
        return 0;
    }
    Staged s{e};
    float *tmp = s.in(nullptr, count);
    if (!tmp) return fail("out of device memory");
    bf16_to_f32(e->st, tmp, (const uint16_t *)p + offset, count);
    return s.out(dst, tmp, count);
}

// ------------------------------------------------------------ free-standing ops ----
static int with_device(int device, cudaStream_t *st)
{
    if (device < 0 || device >= g5b_device_count()) return fail("CUDA device %d is not available (no CPU path)", device);
    CU(cudaSetDevice(device));
    *st = nullptr;     // legacy default stream: these entry points are synchronous
    return 0;
}

struct Tmp {
    std::vector<void *> bufs;
    ~Tmp() { for (void *p : bufs) cudaFree(p); }
    void *up(const void *src, size_t bytes)
    {
        void *p = nullptr;
        if (cudaMalloc(&p, bytes + 16) != cudaSuccess) return nullptr;
        bufs.push_back(p);
        if (src) cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice);
        else     cudaMemset(p, 0, bytes);
        return p;
    }
};

extern "C" int g5b_matvec_host(const g5b_tensor *w, int br, int bc, const float *x, int T, float *y, int device)
{
    cudaStream_t st;
    if (with_device(device, &st)) return -1;
    Tmp t;
    DMat m;
    m.dt = w->dtype; m.rows = w->rows; m.cols = w->cols;
    const size_t n = (size_t)w->rows * w->cols;
    m.w = t.up(w->data, n * elt(w->dtype));
    if (w->dtype == G5B_DT_FP8) {
        if (br < 1 || bc < 1 || !w->scale_inv) return fail("FP8 matrix without block size or scales");
        m.br = br; m.bc = bc; m.scols = (w->cols + bc - 1) / bc;
        m.s = (float *)t.up(w->scale_inv, (size_t)((w->rows + br - 1) / br) * m.scols * 4);
    }
    float *xd = (float *)t.up(x, (size_t)T * w->cols * 4), *yd = (float *)t.up(nullptr, (size_t)T * w->rows * 4);
    if (!m.w || !xd || !yd) return fail("out of device memory");
    gemv(st, m, xd, w->cols, yd, w->rows, T);
    CU(cudaMemcpy(y, yd, (size_t)T * w->rows * 4, cudaMemcpyDeviceToHost));
    CU(cudaGetLastError());
    return 0;
}

extern "C" int g5b_rmsnorm_host(float *y, const float *x, const float *w, int n, int rows, float eps, int device)
{
    cudaStream_t st;
    if (with_device(device, &st)) return -1;
    Tmp t;
    float *xd = (float *)t.up(x, (size_t)rows * n * 4), *yd = (float *)t.up(nullptr, (size_t)rows * n * 4);
    float *wd = w ? (float *)t.up(w, (size_t)n * 4) : nullptr, *inv = (float *)t.up(nullptr, (size_t)rows * 4);
    if (!xd || !yd || !inv) return fail("out of device memory");
    rms_factor(st, xd, n, n, rows, eps, inv);
    rms_apply(st, yd, xd, wd, inv, n, n, rows);
    CU(cudaMemcpy(y, yd, (size_t)rows * n * 4, cudaMemcpyDeviceToHost));
    CU(cudaGetLastError());
    return 0;
}

// One draw from host logits: the sampler of g5b_engine_decode_sampled on its own.
extern "C" int g5b_sample_host(const float *logits, int V, float temperature, float top_p, uint64_t seed, uint64_t step,
                               int *token, int device)
{
    cudaStream_t st;
    if (with_device(device, &st)) return -1;
    if (V < 1 || !(temperature > 0.f) || !(top_p > 0.f)) return fail("sampling needs a vocabulary, temperature > 0 and top_p > 0");
    Tmp t;
    float *ld = (float *)t.up(logits, (size_t)V * 4), *pd = (float *)t.up(nullptr, (size_t)V * 4);
    int *od = (int *)t.up(nullptr, 4);
    if (!ld || !pd || !od) return fail("out of device memory");
    sample_token(st, od, ld, pd, V, temperature, top_p, seed, step);
    CU(cudaMemcpy(token, od, 4, cudaMemcpyDeviceToHost));
    CU(cudaGetLastError());
    return 0;
}

extern "C" int g5b_swiglu_host(float *y, const float *gu, int n, int rows, float limit, int device)
{
    cudaStream_t st;
    if (with_device(device, &st)) return -1;
    Tmp t;
    float *gd = (float *)t.up(gu, (size_t)rows * 2 * n * 4), *yd = (float *)t.up(nullptr, (size_t)rows * n * 4);
    if (!gd || !yd) return fail("out of device memory");
    swiglu(st, yd, gd, n, rows, limit);
    CU(cudaMemcpy(y, yd, (size_t)rows * n * 4, cudaMemcpyDeviceToHost));
    CU(cudaGetLastError());
    return 0;
}

extern "C" int g5b_shortconv_host(float *y, const float *x, const float *w, float *state, int channels, int k,
                                  int T, int device)
{
    cudaStream_t st;
    if (with_device(device, &st)) return -1;
    if (k - 1 > 16 || k < 1) return fail("conv kernel history %d above the limit of 16", k - 1);
    Tmp t;
    float *xd = (float *)t.up(x, (size_t)T * channels * 4), *yd = (float *)t.up(nullptr, (size_t)T * channels * 4);
    float *wd = (float *)t.up(w, (size_t)channels * k * 4);
    float *sd = state ? (float *)t.up(state, (size_t)channels * (k - 1) * 4) : nullptr;
    if (!xd || !yd || !wd) return fail("out of device memory");
    shortconv(st, yd, xd, wd, sd, channels, k, T);
    CU(cudaMemcpy(y, yd, (size_t)T * channels * 4, cudaMemcpyDeviceToHost));
    if (state) CU(cudaMemcpy(state, sd, (size_t)channels * (k - 1) * 4, cudaMemcpyDeviceToHost));
    CU(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------------ timing ----
// Time `iters` launches of one op ("moe", "kda", "mla", "mlp", "head", "layer", "layers", "layer_batch", "hc_site", "hc_site_post") between CUDA events on the
// engine's stream; before each launch `flush_bytes` of scratch are overwritten (0 = no flush) so
// that weights come from HBM, not from L2. ms_each receives the per-launch times. When the
// engine's "profile" option is on, the per-phase times of the MoE op accumulate in the profile.
extern "C" int g5b_time_op(g5b_engine *e, const char *op, int layer, const float *x_dev, int T, int cached,
                           float *out_dev, int iters, size_t flush_bytes, float *ms_total, float *ms_each)
{
    if (check_layer(e, layer, T)) return -1;
    if (flush_bytes > e->flush_bytes) {
        if (e->flush_buf) cudaFree(e->flush_buf);
        e->flush_buf = nullptr; e->flush_bytes = 0;
        CU(cudaMalloc(&e->flush_buf, flush_bytes));
        e->flush_bytes = flush_bytes;
    }
    // Every iteration is enqueued before the host waits for any of them: [flush, event, op, event]
    // repeated, then one wait. The events bracket the op alone, the flush runs between the timed
    // regions, and no host round trip sits between a step's end and the next step's launch - which
    // is how a decode loop runs, and what keeps expert-parallel ranks (separate host processes) from
    // timing each other's host wake-up jitter inside the op's wait for its peers.
    std::vector<cudaEvent_t> ev((size_t)2 * iters, nullptr);
    struct EvGuard { std::vector<cudaEvent_t> &v; ~EvGuard() { for (cudaEvent_t x : v) if (x) cudaEventDestroy(x); } } guard{ev};
    for (auto &x : ev) CU(cudaEventCreate(&x));
    double total = 0.0;
    for (int i = 0; i < iters; i++) {
        if (flush_bytes) flush_l2(e->st, e->flush_buf, flush_bytes);
        CU(cudaEventRecord(ev[2 * i], e->st));
        int rc;
        if (!strcmp(op, "moe"))        rc = g5b_dev_moe(e, layer, x_dev, T, out_dev);
        else if (!strcmp(op, "kda"))   rc = g5b_dev_kda(e, layer, x_dev, T, out_dev);
        else if (!strcmp(op, "mla"))   rc = g5b_dev_mla(e, layer, x_dev, T, cached, out_dev);
        else if (!strcmp(op, "layer")) rc = g5b_dev_decoder_layer(e, layer, out_dev, T, cached);
        else if (!strcmp(op, "layers")) {                  // every layer of the engine in order, one pass
            rc = 0;
            for (int l = 0; l < e->c.n_layers && !rc; l++) rc = run_layer(e, l, out_dev, T, cached);
            if (rc) e->post_h = nullptr;
            flush_hc_post(e);
        }
        else if (!strcmp(op, "layer_batch")) {             // T sequences, one new position each
            if (T > e->n_seq || T > CHUNK) rc = fail("layer_batch takes at most %d sequences", e->n_seq < CHUNK ? e->n_seq : CHUNK);
            else {
                e->post_h = nullptr;
                rc = run_layer(e, layer, out_dev, T, cached, true);
                if (rc) e->post_h = nullptr;
                flush_hc_post(e);
            }
        }
        else if (!strcmp(op, "hc_site") || !strcmp(op, "hc_site_post")) {
            // one mHC site of the layer on its own: gates, Sinkhorn, collapse and the sub-block's
            // RMSNorm, without / with the previous sub-block's stream expansion riding along
            const HcW &hw = e->L[layer].hc[0];
            if (!hw.fn.loaded() || !hc_pre_fused_supported(hw, e->c.hc_mult, e->c.hidden)) rc = fail("no fused mHC site for this layer");
            else {
                hc_pre_fused(e->st, e->xn, e->post, e->comb, out_dev, op[7] ? e->y : nullptr, hw, e->L[layer].in_norm,
                             e->hc_part, e->hc_count, T, e->c.hc_mult, e->c.hidden, e->c.hc_iters, e->c.hc_eps, e->c.rms_eps);
                rc = 0;
            }
        }
        else if (!strcmp(op, "head")) {                    // mean of the streams, final norm, lm_head, arg-max
            if (!e->lm_head.loaded() || !e->norm) rc = fail("the head was not loaded");
            else {
                head_mean(e->st, e->xm, out_dev, T, e->c.hc_mult, e->c.hidden);
                rms_factor(e->st, e->xm, e->c.hidden, e->c.hidden, T, e->c.rms_eps, e->inv_head);
                rc = proj(e, e->lm_head, e->xm, e->c.hidden, e->logits, e->c.vocab, T, e->inv_head, e->norm);
                if (!rc) argmax_rows(e->st, e->am_out, e->logits, e->c.vocab, T, e->am_v, e->am_i);
            }
        }
        else if (!strcmp(op, "mlp")) {
            rc = e->L[layer].is_dense ? run_mlp(e, e->L[layer], x_dev, T, out_dev) : fail("layer %d is a MoE layer", layer);
        }
        else rc = fail("unknown op %s", op);
        if (rc) { cudaStreamSynchronize(e->st); return -1; }
        CU(cudaEventRecord(ev[2 * i + 1], e->st));
    }
    CU(cudaStreamSynchronize(e->st));
    for (int i = 0; i < iters; i++) {
        float ms = 0.f;
        CU(cudaEventElapsedTime(&ms, ev[2 * i], ev[2 * i + 1]));
        if (ms_each) ms_each[i] = ms;
        total += ms;
    }
    CU(cudaGetLastError());
    if (ms_total) *ms_total = (float)total;
    return check_device_error(e);
}

// Time `iters` products of one loaded matrix with T positions (the path the forward pass takes for
// that many positions), events around each product, L2 flushed before each.
extern "C" int g5b_time_matvec(g5b_engine *e, const char *name, const float *x_dev, int T, float *y_dev, int iters,
                               size_t flush_bytes, float *ms_each)
{
    if (!e || !e->finalized) return fail("time_matvec before finalize");
    CU(cudaSetDevice(e->device));
    if (T < 1 || T > CHUNK) return fail("time_matvec takes 1..%d positions", CHUNK);
    DMat *m = find_mat(e, name);
    if (!m) return fail("no loaded matrix named %s", name);
    if (flush_bytes > e->flush_bytes) {
        if (e->flush_buf) cudaFree(e->flush_buf);
        e->flush_buf = nullptr; e->flush_bytes = 0;
        CU(cudaMalloc(&e->flush_buf, flush_bytes));
        e->flush_bytes = flush_bytes;
    }
    std::vector<cudaEvent_t> ev((size_t)2 * iters, nullptr);
    struct EvGuard { std::vector<cudaEvent_t> &v; ~EvGuard() { for (cudaEvent_t x : v) if (x) cudaEventDestroy(x); } } guard{ev};
    for (auto &x : ev) CU(cudaEventCreate(&x));
    for (int i = 0; i < iters; i++) {
        if (flush_bytes) flush_l2(e->st, e->flush_buf, flush_bytes);
        CU(cudaEventRecord(ev[2 * i], e->st));
        if (proj(e, *m, x_dev, m->cols, y_dev, m->rows, T)) { cudaStreamSynchronize(e->st); return -1; }
        CU(cudaEventRecord(ev[2 * i + 1], e->st));
    }
    CU(cudaStreamSynchronize(e->st));
    for (int i = 0; i < iters; i++) CU(cudaEventElapsedTime(&ms_each[i], ev[2 * i], ev[2 * i + 1]));
    CU(cudaGetLastError());
    return check_device_error(e);
}

extern "C" int g5b_engine_profile_read(g5b_engine *e, float *ms, int n, long *count, int reset)
{
    for (int i = 0; i < n && i < PROF_SLOTS; i++) ms[i] = e->prof_ms[i];
    if (count) *count = e->prof_n;
    if (reset) { memset(e->prof_ms, 0, sizeof e->prof_ms); e->prof_n = 0; }
    return 0;
}

// ------------------------------------------------------------- expert parallel ----

static int ep_alloc(g5b_engine *e)
{
    if (e->ep_region) return 0;
    e->ep_rows_bytes = (size_t)CHUNK * e->c.topk * e->c.hidden * 4;
    e->ts_area_bytes = (size_t)e->ep_size * CHUNK * e->c.hidden * 4;
    const size_t bytes = EP_FLAG_BYTES + 2 * e->ep_rows_bytes + 2 * e->ts_area_bytes;
    CU(cudaMalloc((void **)&e->ep_region, bytes));       // an allocation of its own: it is what peers map
    CU(cudaMemset(e->ep_region, 0, bytes));
    if (e->dalloc((void **)&e->ep_peers_dev, sizeof(void *) * (size_t)e->ep_size)) return -1;
    if (e->dalloc((void **)&e->ep_arrive, sizeof(int))) return -1;
    if (e->dalloc((void **)&e->ts_part, (size_t)CHUNK * e->c.hidden * 4)) return -1;
    CU(cudaStreamSynchronize(e->st));
    return 0;
}

static int ep_publish_peers(g5b_engine *e, const std::vector<void *> &peers)
{
    CU(cudaMemcpy(e->ep_peers_dev, peers.data(), sizeof(void *) * peers.size(), cudaMemcpyHostToDevice));
    e->ep_connected = true;
    e->ep_step = 0;
    e->ep_decode_launches = 0;
    e->ts_launches = 0;
    e->head_launches = 0;
    return 0;
}

extern "C" size_t g5b_engine_ep_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int g5b_engine_ep_export(g5b_engine *e, void *handle_out)
{
    if (!e || !handle_out) return fail("null argument");
    if (e->ep_size == 1) { memset(handle_out, 0, sizeof(cudaIpcMemHandle_t)); return 0; }
    if (!e->finalized) return fail("export the exchange handle after finalize");
    CU(cudaSetDevice(e->device));
    if (ep_alloc(e)) return -1;
    CU(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle_out), e->ep_region));
    return 0;
}

extern "C" int g5b_engine_ep_connect(g5b_engine *e, const void *all_handles)
{
    if (!e) return fail("null engine");
    if (e->ep_size == 1) return 0;
    if (!all_handles) return fail("null handle array");
    if (!e->finalized) return fail("connect after finalize");
    if (e->ep_connected) return fail("the ranks are already connected");
    CU(cudaSetDevice(e->device));
    if (ep_alloc(e)) return -1;
    const cudaIpcMemHandle_t *h = static_cast<const cudaIpcMemHandle_t *>(all_handles);
    std::vector<void *> peers((size_t)e->ep_size, nullptr);
    for (int r = 0; r < e->ep_size; r++) {
        if (r == e->ep_rank) { peers[r] = e->ep_region; continue; }
        void *p = nullptr;
        const cudaError_t rc = cudaIpcOpenMemHandle(&p, h[r], cudaIpcMemLazyEnablePeerAccess);
        if (rc != cudaSuccess) {
            cudaGetLastError();
            return fail("rank %d cannot map rank %d's exchange region: %s", e->ep_rank, r, cudaGetErrorString(rc));
        }
        e->ep_opened.push_back(p);
        peers[r] = p;
    }
    return ep_publish_peers(e, peers);
}

// The same wiring for ranks that live in ONE process, one engine per device (a host that drives
// several GPUs from threads of one process, like the reference's own multi-device backend): no
// handles, the devices are given access to each other's memory and every engine gets the others'
// exchange regions directly. engines[r] must be rank r of n, each on a device of its own. The
// caller then runs every step on all engines at the same time, one host thread per engine.
extern "C" int g5b_engine_ep_connect_local(g5b_engine *const *engines, int n)
{
    if (!engines || n < 2) return fail("connect_local needs at least two engines");
    for (int r = 0; r < n; r++) {
        g5b_engine *e = engines[r];
        if (!e || !e->finalized) return fail("connect_local: engine %d is not finalized", r);
        if (e->ep_size != n || e->ep_rank != r) return fail("connect_local: engine %d is rank %d of %d", r, e ? e->ep_rank : -1, e ? e->ep_size : -1);
        if (e->ep_connected) return fail("the ranks are already connected");
        for (int q = 0; q < r; q++)
            if (engines[q]->device == e->device)
                return fail("connect_local: ranks %d and %d share device %d (kernels that wait for each other need a GPU each)", q, r, e->device);
    }
    for (int r = 0; r < n; r++) {
        CU(cudaSetDevice(engines[r]->device));
        if (ep_alloc(engines[r])) return -1;
    }
    for (int r = 0; r < n; r++) {
        g5b_engine *e = engines[r];
        CU(cudaSetDevice(e->device));
        std::vector<void *> peers((size_t)n, nullptr);
        for (int q = 0; q < n; q++) {
            peers[q] = engines[q]->ep_region;
            if (q == r) continue;
            int can = 0;
            CU(cudaDeviceCanAccessPeer(&can, e->device, engines[q]->device));
            if (!can) return fail("device %d cannot access device %d's memory", e->device, engines[q]->device);
            const cudaError_t rc = cudaDeviceEnablePeerAccess(engines[q]->device, 0);
            if (rc != cudaSuccess && rc != cudaErrorPeerAccessAlreadyEnabled)
                return fail("peer access from device %d to %d: %s", e->device, engines[q]->device, cudaGetErrorString(rc));
            cudaGetLastError();
        }
        if (ep_publish_peers(e, peers)) return -1;
    }
    return 0;
}

// Re-align the ranks after a step that failed on some of them. Host-side and collective: every rank
// calls it, and the caller's own transport must order the calls so that no rank has a MoE kernel in
// flight and none starts one before all have returned (a barrier before and one after). It forgets
// every published step word of this rank's region and restarts the step count at zero.
extern "C" int g5b_engine_ep_resync(g5b_engine *e)
{
    if (!e) return fail("null engine");
    if (e->ep_size == 1) return 0;
    if (!e->ep_connected) return fail("resync before the ranks are connected");
    CU(cudaSetDevice(e->device));
    CU(cudaStreamSynchronize(e->st));
    CU(cudaMemsetAsync(e->ep_region, 0, EP_FLAG_BYTES, e->st));
    CU(cudaMemsetAsync(e->ep_arrive, 0, sizeof(int), e->st));
    CU(cudaStreamSynchronize(e->st));
    if (e->err_host) *e->err_host = 0;
    e->ep_step = 0;
    e->ep_decode_launches = 0;
    e->ts_launches = 0;
    e->head_launches = 0;
    return 0;
}

// Stand-in peers in this GPU's own memory that nobody ever writes: lets one GPU exercise the
// delivery code and the bounded wait (which then runs out and is reported), nothing else.
static int ep_loopback(g5b_engine *e)
{
    if (e->ep_size == 1) return 0;
    if (!e->finalized) return fail("ep_loopback after finalize");
    if (e->ep_connected) return fail("the ranks are already connected");
    if (ep_alloc(e)) return -1;
    std::vector<void *> peers((size_t)e->ep_size, nullptr);
    for (int r = 0; r < e->ep_size; r++) {
        if (r == e->ep_rank) { peers[r] = e->ep_region; continue; }
        void *p = nullptr;
        CU(cudaMalloc(&p, EP_FLAG_BYTES + 2 * e->ep_rows_bytes + 2 * e->ts_area_bytes));
        CU(cudaMemset(p, 0, EP_FLAG_BYTES + 2 * e->ep_rows_bytes + 2 * e->ts_area_bytes));
        e->ep_standins.push_back(p);
        peers[r] = p;
    }
    return ep_publish_peers(e, peers);
}

