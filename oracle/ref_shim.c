/*
 * ref_shim.c - the UNMODIFIED reference engine behind the same flat entry points as the
 * oracle (glm53f_oracle.h), with the prefix ref_ instead of orc_.
 *
 * TEST INFRASTRUCTURE ONLY. This file contains no arithmetic of its own: every result comes
 * from the reference's functions (glm53f_mm, glm53f_moe, glm53f_kda_layer, glm53f_mla,
 * glm53f_dsa_*, glm53f_decoder_layer, glm53f_model_forward, ...). It is compiled against the
 * reference's headers where they lie and linked with the reference's objects by the Makefile
 * beside it, into oracle/_ref/, only when the reference tree is present. It serves two
 * purposes: proving that the oracle restatement is bit-identical to the reference, and being
 * the timed CPU baseline ("kind": "reference") of the benchmark.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "glm53f_b200.h"
#include "glm53f_model.h"      /* reference: src/model/glm53f_model.h */
/* The reference's MTP layer keeps its struct private to its .c file and can only be opened from a
 * checkpoint on disk. To drive glm53f_mtp_feed from tensors in memory, the reference's source file
 * is compiled as part of this translation unit, where it lies (the Makefile leaves it out of the
 * list of separately compiled files), and the struct is filled below by ref_model_enable_mtp. */
#include "glm53f_mtp.c"

typedef struct {
    Glm53fExpertSrc src;       /* first member: &src is what Glm53fMoeW.src points at */
    Glm53fExpertQ  *q;         /* [n_layers][n_experts] */
    int             n_experts;
} RamExperts;

typedef struct {
    Glm53fModel m;
    RamExperts  ram;
    int         from_dir, latent, finalized, mtp;
    void      **owned;
    size_t      n_owned, cap_owned;
} RefModel;

static void *own(RefModel *r, void *p)
{
    if (r->n_owned == r->cap_owned) {
        r->cap_owned = r->cap_owned ? 2 * r->cap_owned : 256;
        r->owned = (void **)realloc(r->owned, r->cap_owned * sizeof(void *));
    }
    r->owned[r->n_owned++] = p;
    return p;
}

/* Glm53fExpertSrc.get over experts held in RAM (contract: include/glm53f/glm53f.h:216-228). */
static int ram_get(Glm53fExpertSrc *self, int layer, int expert, Glm53fExpertQ *out)
{
    RamExperts *r = (RamExperts *)self;
    const Glm53fExpertQ *q = &r->q[(size_t)layer * r->n_experts + expert];
    if (!q->gate.w || !q->up.w || !q->down.w) return -1;
    *out = *q;
    return 0;
}

static void to_cfg(Glm53fCfg *c, const g5b_config *g, const uint8_t *is_mla, const uint8_t *is_dense)
{
    memset(c, 0, sizeof *c);
    c->hidden = g->hidden; c->n_layers = g->n_layers; c->vocab = g->vocab; c->rms_eps = g->rms_eps;
    c->hc_mult = g->hc_mult; c->hc_iters = g->hc_iters; c->hc_eps = g->hc_eps;
    c->kda_heads = g->kda_heads; c->kda_head_dim = g->kda_head_dim; c->conv_k = g->conv_k;
    c->gate_lb = g->gate_lb;
    c->n_heads = g->mla_heads; c->q_lora = g->q_lora; c->kv_lora = g->kv_lora;
    c->qk_nope = g->qk_nope; c->v_head = g->v_head;
    c->index_topk = g->index_topk; c->index_kpool = g->index_kpool;
    c->index_heads = g->index_heads; c->index_dim = g->index_dim; c->index_tail = 1;
    c->n_experts = g->n_experts; c->topk = g->topk; c->n_shared = g->n_shared;
    c->moe_inter = g->moe_inter; c->dense_inter = g->dense_inter;
    c->routed_scale = g->routed_scale; c->norm_topk = g->norm_topk; c->swiglu_limit = g->swiglu_limit;
    c->fp8_block_r = g->fp8_block_r; c->fp8_block_c = g->fp8_block_c;
    for (int l = 0; l < g->n_layers; l++) { c->is_mla[l] = is_mla[l]; c->is_dense[l] = is_dense[l]; }
}

void *ref_model_create(const g5b_config *cfg, const uint8_t *is_mla, const uint8_t *is_dense,
                       int cap, int kv_mode)
{
    RefModel *r = (RefModel *)calloc(1, sizeof *r);
    Glm53fModel *m = &r->m;
    to_cfg(&m->cfg, cfg, is_mla, is_dense);
    m->cap = cap < 1 ? 1 : cap;
    m->n_bound = cfg->n_layers;
    m->lay = (Glm53fLayerBind *)calloc((size_t)cfg->n_layers, sizeof *m->lay);
    r->latent = kv_mode == 2 || (kv_mode == 0 && m->cap > glm53f_dense_attn_limit(&m->cfg));
    r->ram.src.get = ram_get;
    r->ram.n_experts = cfg->n_experts;
    r->ram.q = (Glm53fExpertQ *)calloc((size_t)(cfg->n_layers + 1) * cfg->n_experts, sizeof(Glm53fExpertQ));  /* + the MTP layer */
    for (int l = 0; l < cfg->n_layers; l++) {
        Glm53fLayerW *w = &m->lay[l].w;
        w->is_mla = is_mla[l]; w->is_dense = is_dense[l];
        w->moe.src = &r->ram.src;
        w->moe.layer = l;
    }
    glm53f_quiet = 1;
    return r;
}

/* Checkpoint layer n_layers as the reference's MTP layer: the struct glm53f_mtp_open would build
 * (src/model/glm53f_mtp.c:29-84), with weights arriving through ref_model_load and the experts in
 * RAM like the trunk's. Call before loading. */
int ref_model_enable_mtp(void *h)
{
    RefModel *r = (RefModel *)h;
    if (r->mtp || r->finalized) return -1;
    Glm53fMtp *t = (Glm53fMtp *)calloc(1, sizeof *t);
    t->b.w.w.is_mla = 1;
    t->b.w.w.is_dense = 0;
    t->b.w.w.moe.src = &r->ram.src;
    t->b.w.w.moe.layer = r->m.cfg.n_layers;
    t->b.w.w.moe.prefetch_n = 0;
    r->m.mtp = t;
    r->mtp = 1;
    return 0;
}

static int put_mat(RefModel *r, Glm53fMat *dst, const g5b_tensor *t, int rows, int cols)
{
    const Glm53fCfg *c = &r->m.cfg;
    if (t->rows != rows || t->cols != cols) return -1;
    const size_t n = (size_t)rows * cols;
    const size_t eb = t->dtype == G5B_DT_F32 ? 4 : t->dtype == G5B_DT_BF16 ? 2 : 1;
    memset(dst, 0, sizeof *dst);
    void *w = own(r, malloc(n * eb));
    memcpy(w, t->data, n * eb);
    dst->w = w; dst->rows = rows; dst->cols = cols;
    dst->dt = t->dtype == G5B_DT_F32 ? GLM53F_WF32 : t->dtype == G5B_DT_BF16 ? GLM53F_WBF16 : GLM53F_WF8;
    if (t->dtype == G5B_DT_FP8) {
        if (!t->scale_inv) return -1;
        dst->br = c->fp8_block_r; dst->bc = c->fp8_block_c;
        dst->scols = (cols + dst->bc - 1) / dst->bc;
        const size_t ns = (size_t)((rows + dst->br - 1) / dst->br) * dst->scols;
        float *s = (float *)own(r, malloc(ns * sizeof(float)));
        memcpy(s, t->scale_inv, ns * sizeof(float));
        dst->s = s;
    }
    return 0;
}

static int put_vec(RefModel *r, const float **dst, const g5b_tensor *t, size_t n)
{
    if ((size_t)t->rows * (size_t)t->cols != n) return -1;
    float *v = (float *)own(r, malloc(n * sizeof(float)));
    if (t->dtype == G5B_DT_F32) memcpy(v, t->data, n * sizeof(float));
    else if (t->dtype == G5B_DT_BF16)
        for (size_t i = 0; i < n; i++) v[i] = glm53f_bf16f(((const uint16_t *)t->data)[i]);
    else return -1;
    *dst = v;
    return 0;
}

int ref_model_load(void *h, const char *name, const g5b_tensor *t)
{
    RefModel *r = (RefModel *)h;
    Glm53fModel *m = &r->m;
    const Glm53fCfg *c = &m->cfg;
    const int E = c->hidden, M = c->hc_mult, MIX = (2 + M) * M;
    if (!strcmp(name, "embed_tokens.weight")) return put_mat(r, &m->mb.embed, t, c->vocab, E);
    if (!strcmp(name, "lm_head.weight"))      return put_mat(r, &m->mb.lm_head, t, c->vocab, E);
    if (!strcmp(name, "norm.weight"))         return put_vec(r, &m->mb.norm, t, (size_t)E);
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= c->n_layers + (r->mtp ? 1 : 0)) return -1;
    const char *p = name + used;
    Glm53fLayerW *w = l < c->n_layers ? &m->lay[l].w : &m->mtp->b.w.w;
    if (l == c->n_layers) {
        Glm53fMtpW *mw = &m->mtp->b.w;
        if (!strcmp(p, "enorm.weight")) return put_vec(r, &mw->enorm, t, (size_t)E);
        if (!strcmp(p, "hnorm.weight")) return put_vec(r, &mw->hnorm, t, (size_t)E);
        if (!strcmp(p, "shared_head.norm.weight")) return put_vec(r, &mw->head_norm, t, (size_t)E);
        if (!strcmp(p, "eh_proj.weight")) return put_mat(r, &mw->eh, t, E, 2 * E);
    }
    const int H = c->kda_heads, D = c->kda_head_dim, P = H * D, MH = c->n_heads;
    const int IH = c->index_heads, ID = c->index_dim, SI = c->moe_inter * c->n_shared;
#define MAT(nm, field, R, C) if (!strcmp(p, nm)) return put_mat(r, &w->field, t, R, C)
#define VEC(nm, field, N)    if (!strcmp(p, nm)) return put_vec(r, &w->field, t, (size_t)(N))
    VEC("input_layernorm.weight", in_norm, E);
    VEC("post_attention_layernorm.weight", post_norm, E);
    MAT("hc_attn_fn", attn_hc.fn, MIX, M * E); VEC("hc_attn_base", attn_hc.base, MIX); VEC("hc_attn_scale", attn_hc.scale, 3);
    MAT("hc_ffn_fn", ffn_hc.fn, MIX, M * E);   VEC("hc_ffn_base", ffn_hc.base, MIX);   VEC("hc_ffn_scale", ffn_hc.scale, 3);
    if (w->is_mla) {
        MAT("self_attn.q_a_proj.weight", mla.q_a, c->q_lora, E);
        VEC("self_attn.q_a_layernorm.weight", mla.q_a_norm, c->q_lora);
        MAT("self_attn.q_b_proj.weight", mla.q_b, MH * c->qk_nope, c->q_lora);
        MAT("self_attn.kv_a_proj_with_mqa.weight", mla.kv_a, c->kv_lora, E);
        VEC("self_attn.kv_a_layernorm.weight", mla.kv_a_norm, c->kv_lora);
        MAT("self_attn.kv_b_proj.weight", mla.kv_b, MH * (c->qk_nope + c->v_head), c->kv_lora);
        MAT("self_attn.o_proj.weight", mla.o, E, MH * c->v_head);
        MAT("self_attn.indexer.wq_b.weight", mla.idx.wq_b, IH * ID, c->q_lora);
        MAT("self_attn.indexer.wk.weight", mla.idx.wk, ID, E);
        VEC("self_attn.indexer.k_norm.weight", mla.idx.k_norm_w, ID);
        VEC("self_attn.indexer.k_norm.bias", mla.idx.k_norm_b, ID);
        MAT("self_attn.indexer.weights_proj.weight", mla.idx.wproj, IH, E);
        MAT("self_attn.indexer.index_kpool_compress_gate", mla.idx.gate, ID, E);
        VEC("self_attn.indexer.index_kpool_compress_ape", mla.idx.ape, c->index_kpool * ID);
    } else {
        MAT("self_attn.q_proj.weight", kda.q, P, E);
        MAT("self_attn.k_proj.weight", kda.k, P, E);
        MAT("self_attn.v_proj.weight", kda.v, P, E);
        VEC("self_attn.q_conv1d.weight", kda.q_conv, P * c->conv_k);
        VEC("self_attn.k_conv1d.weight", kda.k_conv, P * c->conv_k);
        VEC("self_attn.v_conv1d.weight", kda.v_conv, P * c->conv_k);
        MAT("self_attn.f_a_proj.weight", kda.f_a, D, E);
        MAT("self_attn.f_b_proj.weight", kda.f_b, P, D);
        VEC("self_attn.A_log", kda.A_log, H);
        VEC("self_attn.dt_bias", kda.dt_bias, P);
        MAT("self_attn.b_proj.weight", kda.b, H, E);
        MAT("self_attn.g_a_proj.weight", kda.g_a, D, E);
        MAT("self_attn.g_b_proj.weight", kda.g_b, P, D);
        VEC("self_attn.o_norm.weight", kda.o_norm, D);
        MAT("self_attn.o_proj.weight", kda.o, E, P);
    }
    if (w->is_dense) {
        MAT("mlp.gate_proj.weight", d_gate, c->dense_inter, E);
        MAT("mlp.up_proj.weight", d_up, c->dense_inter, E);
        MAT("mlp.down_proj.weight", d_down, E, c->dense_inter);
    } else {
        VEC("mlp.gate.weight", moe.gate, (size_t)c->n_experts * E);
        VEC("mlp.gate.e_score_correction_bias", moe.bias, c->n_experts);
        MAT("mlp.shared_experts.gate_proj.weight", moe.sh_gate, SI, E);
        MAT("mlp.shared_experts.up_proj.weight", moe.sh_up, SI, E);
        MAT("mlp.shared_experts.down_proj.weight", moe.sh_down, E, SI);
        int ex = -1, n2 = 0;
        if (sscanf(p, "mlp.experts.%d.%n", &ex, &n2) == 1 && ex >= 0 && ex < c->n_experts) {
            Glm53fExpertQ *q = &r->ram.q[(size_t)l * c->n_experts + ex];
            const char *s = p + n2;
            if (!strcmp(s, "gate_proj.weight")) return put_mat(r, &q->gate, t, c->moe_inter, E);
            if (!strcmp(s, "up_proj.weight"))   return put_mat(r, &q->up, t, c->moe_inter, E);
            if (!strcmp(s, "down_proj.weight")) return put_mat(r, &q->down, t, E, c->moe_inter);
        }
    }
#undef MAT
#undef VEC
    return -1;
}

/* Session state exactly as glm53f_model_open allocates it (glm53f_model.c:194-228). */
int ref_model_finalize(void *h)
{
    RefModel *r = (RefModel *)h;
    Glm53fModel *m = &r->m;
    const Glm53fCfg *c = &m->cfg;
    m->state = (float *)calloc(glm53f_kda_state_floats(c) * (size_t)m->n_bound, sizeof(float));
    m->kv  = (float **)calloc((size_t)m->n_bound, sizeof(float *));
    m->idx = (float **)calloc((size_t)m->n_bound, sizeof(float *));
    if (r->latent) m->ckv = (float **)calloc((size_t)m->n_bound, sizeof(float *));
    for (int l = 0; l < m->n_bound; l++) {
        if (!glm53f_is_mla(c, l)) continue;
        const size_t n = r->latent ? (size_t)m->cap * c->kv_lora
                                   : (size_t)m->cap * glm53f_kv_floats_per_pos(c);
        if (r->latent) m->ckv[l] = (float *)calloc(n, sizeof(float));
        else           m->kv[l]  = (float *)calloc(n, sizeof(float));
        m->idx[l] = (float *)calloc(glm53f_dsa_state_floats(c, m->cap), sizeof(float));
    }
    if (r->mtp) {                       /* the buffers of glm53f_mtp_open (glm53f_mtp.c:55-73) */
        Glm53fMtp *t = m->mtp;
        const size_t E = (size_t)c->hidden;
        t->cap = m->cap; t->maxT = m->cap;
        if (r->latent) t->ckv = (float *)calloc((size_t)m->cap * c->kv_lora, sizeof(float));
        else           t->kv  = (float *)malloc((size_t)m->cap * glm53f_kv_floats_per_pos(c) * sizeof(float));
        t->istate = (float *)calloc(glm53f_dsa_state_floats(c, m->cap), sizeof(float));
        t->x = (float *)malloc((size_t)t->maxT * E * sizeof(float));
        t->y = (float *)malloc((size_t)t->maxT * E * sizeof(float));
        t->cat = (float *)malloc((size_t)t->maxT * 2 * E * sizeof(float));
        t->lg = (float *)malloc((size_t)c->vocab * sizeof(float));
        t->scratch = (float *)malloc(work_floats(c, t->maxT, m->cap) * sizeof(float));
        m->mtp_h = (float *)calloc((size_t)m->cap * E, sizeof(float));
    }
    r->finalized = 1;
    return 0;
}

/* glm53f_mtp_feed; h == NULL feeds the hidden states the last forward call kept. x_out: the
 * layer's output rows (the reference's own buffer). */
int ref_mtp_feed(void *h, const float *hid, const int *next_ids, int T, int *draft, float *x_out)
{
    RefModel *r = (RefModel *)h;
    if (!r->mtp || !r->finalized) return -1;
    const int rc = glm53f_mtp_feed(&r->m, hid ? hid : r->m.mtp_h, next_ids, T, draft);
    if (rc == 0 && x_out) memcpy(x_out, r->m.mtp->x, (size_t)T * r->m.cfg.hidden * sizeof(float));
    return rc;
}

int ref_mtp_hidden(void *h, int first, int T, float *dst)
{
    RefModel *r = (RefModel *)h;
    if (!r->m.mtp_h || first < 0 || first + T > r->m.cap) return -1;
    memcpy(dst, r->m.mtp_h + (size_t)first * r->m.cfg.hidden, (size_t)T * r->m.cfg.hidden * sizeof(float));
    return 0;
}

/* The reference's own loader end to end: a checkpoint directory (config.json + safetensors). */
void *ref_open_dir(const char *dir, int cap, int kv_mode)
{
    RefModel *r = (RefModel *)calloc(1, sizeof *r);
    glm53f_quiet = 1;
    if (glm53f_model_open(&r->m, dir, NULL, 0.05, -1, cap, 0, 0, 0, kv_mode) != 0) { free(r); return NULL; }
    r->from_dir = 1;
    r->finalized = 1;
    r->latent = r->m.ckv != NULL;
    return r;
}

int ref_model_forward(void *h, const int *ids, int T, float *logits, int *argmax_all)
{
    RefModel *r = (RefModel *)h;
    if (!r->finalized) return -1;
    return glm53f_model_forward(&r->m, ids, T, logits, argmax_all);
}

void ref_model_reset(void *h)
{
    glm53f_model_reset(&((RefModel *)h)->m);
    glm53f_mtp_reset(&((RefModel *)h)->m);
}
int  ref_model_cached(void *h) { return ((RefModel *)h)->m.cached; }
int  ref_model_vocab(void *h) { return ((RefModel *)h)->m.cfg.vocab; }

void ref_model_free(void *h)
{
    RefModel *r = (RefModel *)h;
    if (!r) return;
    if (r->from_dir) { glm53f_model_close(&r->m); free(r); return; }
    Glm53fModel *m = &r->m;
    for (int l = 0; l < m->n_bound; l++) {
        if (m->kv) free(m->kv[l]);
        if (m->idx) free(m->idx[l]);
        if (m->ckv) free(m->ckv[l]);
    }
    free(m->kv); free(m->idx); free(m->ckv); free(m->state); free(m->lay);
    if (m->mtp) {
        Glm53fMtp *t = m->mtp;
        free(t->kv); free(t->ckv); free(t->istate); free(t->x); free(t->y); free(t->cat); free(t->lg);
        free(t->scratch); free(t); free(m->mtp_h);
    }
    for (size_t i = 0; i < r->n_owned; i++) free(r->owned[i]);
    free(r->owned); free(r->ram.q); free(r);
}

/* ----------------------------------------------------------------- op entries ---- */
int ref_matvec_host(const g5b_tensor *w, int br, int bc, const float *x, int T, float *y)
{
    Glm53fMat m;
    memset(&m, 0, sizeof m);
    m.w = w->data; m.s = w->scale_inv; m.rows = w->rows; m.cols = w->cols;
    m.dt = w->dtype == G5B_DT_F32 ? GLM53F_WF32 : w->dtype == G5B_DT_BF16 ? GLM53F_WBF16 : GLM53F_WF8;
    m.br = br; m.bc = bc; m.scols = bc > 0 ? (w->cols + bc - 1) / bc : 0;
    if (T == 1) glm53f_mm(y, x, &m); else glm53f_mm_batch(y, x, T, &m);
    return 0;
}

int ref_rmsnorm_host(float *y, const float *x, const float *w, int n, int rows, float eps)
{
    for (int r = 0; r < rows; r++) glm53f_rmsnorm(y + (size_t)r * n, x + (size_t)r * n, w, n, eps);
    return 0;
}

int ref_swiglu_host(float *y, const float *gu, int n, int rows, float limit)
{
    for (int r = 0; r < rows; r++) glm53f_swiglu_clamp(y + (size_t)r * n, gu + (size_t)r * 2 * n, n, limit);
    return 0;
}

int ref_shortconv_host(float *y, const float *x, const float *w, float *state, int channels, int k, int T)
{
    glm53f_shortconv(y, x, w, state, channels, k, T);
    return 0;
}

int ref_op_hc_pre(void *h, int layer, int site, const float *hs, int T, float *x, float *post, float *comb)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    const size_t E = (size_t)c->hidden, M = (size_t)c->hc_mult;
    float *scratch = (float *)malloc(glm53f_hc_scratch(c) * sizeof(float));
    const Glm53fLayerW *w = &r->m.lay[layer].w;
    for (int t = 0; t < T; t++)
        glm53f_hc_pre(x + t * E, post + t * M, comb + t * M * M, hs + t * M * E,
                      site ? &w->ffn_hc : &w->attn_hc, c, scratch);
    free(scratch);
    return 0;
}

int ref_op_hc_post(void *h, float *hs, const float *y, const float *post, const float *comb, int T)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    const size_t E = (size_t)c->hidden, M = (size_t)c->hc_mult;
    float *scratch = (float *)malloc(M * E * sizeof(float));
    for (int t = 0; t < T; t++)
        glm53f_hc_post(hs + t * M * E, y + t * E, post + t * M, comb + t * M * M, c, scratch);
    free(scratch);
    return 0;
}

int ref_op_kda(void *h, int layer, const float *x, int T, float *out)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    float *scratch = (float *)malloc(glm53f_kda_scratch(c, T) * sizeof(float));
    glm53f_kda_layer(out, x, &r->m.lay[layer].w.kda, c, T,
                     r->m.state + glm53f_kda_state_floats(c) * (size_t)layer, scratch);
    free(scratch);
    return 0;
}

int ref_op_mla(void *h, int layer, const float *x, int T, int cached, float *out,
               int *sel_out, int *n_sel_out)
{
    RefModel *r = (RefModel *)h;
    Glm53fModel *m = &r->m;
    const Glm53fCfg *c = &m->cfg;
    const Glm53fMlaW *w = &m->lay[layer].w.mla;
    float *scratch = (float *)malloc(glm53f_mla_scratch(c, T, m->cap) * sizeof(float));
    glm53f_mla(out, x, w, c, T, scratch, m->kv[layer], cached, m->cap, m->idx[layer],
               m->ckv ? m->ckv[layer] : NULL);
    if (n_sel_out) {
        /* the selection is a pure function of the indexer state: ask again for the last query */
        const float *xt = x + (size_t)(T - 1) * c->hidden;
        float *ql = (float *)malloc((size_t)c->q_lora * sizeof(float));
        float *ds = (float *)malloc(glm53f_dsa_scratch(c, m->cap) * sizeof(float));
        int *sel = (int *)malloc((size_t)(c->index_topk + c->index_kpool) * sizeof(int));
        glm53f_mm(ql, xt, &w->q_a);
        glm53f_rmsnorm(ql, ql, w->q_a_norm, c->q_lora, c->rms_eps);
        const int n = glm53f_dsa_select(sel, m->idx[layer], xt, ql, &w->idx, c, cached + T - 1, m->cap, ds);
        *n_sel_out = n;
        if (sel_out && n > 0) memcpy(sel_out, sel, (size_t)n * sizeof(int));
        free(ql); free(ds); free(sel);
    }
    free(scratch);
    return 0;
}

int ref_op_router(void *h, int layer, const float *x, int T, int *idx, float *wt)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    for (int t = 0; t < T; t++)
        glm53f_router(idx + (size_t)t * c->topk, wt + (size_t)t * c->topk, x + (size_t)t * c->hidden,
                      &r->m.lay[layer].w.moe, c);
    return 0;
}

int ref_op_moe(void *h, int layer, const float *x, int T, float *out, int with_shared)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    float *scratch = (float *)malloc(glm53f_moe_scratch(c, T) * sizeof(float));
    const long drops = glm53f_expert_drops;
    if (with_shared) glm53f_moe(out, x, &r->m.lay[layer].w.moe, c, T, scratch);
    else             glm53f_moe_routed(out, x, &r->m.lay[layer].w.moe, c, T, scratch);
    free(scratch);
    return glm53f_expert_drops == drops ? 0 : -1;
}

int ref_op_mlp(void *h, int layer, const float *x, int T, float *out)
{
    RefModel *r = (RefModel *)h;
    const Glm53fCfg *c = &r->m.cfg;
    const Glm53fLayerW *w = &r->m.lay[layer].w;
    float *scratch = (float *)malloc(glm53f_mlp_scratch(c) * sizeof(float));
    for (int t = 0; t < T; t++)
        glm53f_mlp(out + (size_t)t * c->hidden, x + (size_t)t * c->hidden, &w->d_gate, &w->d_up,
                   &w->d_down, c->swiglu_limit, scratch);
    free(scratch);
    return 0;
}

int ref_op_decoder_layer(void *h, int layer, float *hs, int T, int cached)
{
    RefModel *r = (RefModel *)h;
    Glm53fModel *m = &r->m;
    const Glm53fCfg *c = &m->cfg;
    float *scratch = (float *)malloc(glm53f_layer_scratch(c, T, m->cap) * sizeof(float));
    const long drops = glm53f_expert_drops;
    glm53f_decoder_layer(hs, &m->lay[layer].w, c, T,
                         m->state + glm53f_kda_state_floats(c) * (size_t)layer, scratch,
                         m->kv[layer], cached, m->cap, m->idx[layer], m->ckv ? m->ckv[layer] : NULL);
    free(scratch);
    return glm53f_expert_drops == drops ? 0 : -1;
}

static float *ref_state_ptr(RefModel *r, int layer, int kind, size_t *n)
{
    Glm53fModel *m = &r->m;
    const Glm53fCfg *c = &m->cfg;
    if (kind == 0) { *n = glm53f_kda_state_floats(c); return m->state + *n * (size_t)layer; }
    if (kind == 1) { *n = (size_t)m->cap * c->kv_lora; return m->ckv ? m->ckv[layer] : NULL; }
    if (kind == 2) { *n = glm53f_dsa_state_floats(c, m->cap); return m->idx[layer]; }
    return NULL;
}

int ref_state_write(void *h, int layer, int kind, size_t offset, const float *src, size_t count)
{
    size_t n = 0;
    float *p = ref_state_ptr((RefModel *)h, layer, kind, &n);
    if (!p || offset + count > n) return -1;
    memcpy(p + offset, src, count * sizeof(float));
    return 0;
}

int ref_state_read(void *h, int layer, int kind, size_t offset, float *dst, size_t count)
{
    size_t n = 0;
    float *p = ref_state_ptr((RefModel *)h, layer, kind, &n);
    if (!p || offset + count > n) return -1;
    memcpy(dst, p + offset, count * sizeof(float));
    return 0;
}
