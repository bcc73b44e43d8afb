/*
 * glm53f_gpu_b200.c - the reference project's backend ABI on top of libglm53f_b200.
 *
 * This is the file a maintainer of josesilva05/glm-5.3-flash-in-c adds to build its model driver
 * (src/model/glm53f_model.c, compiled with -DGLM53F_CUDA) against this engine instead of its
 * own src/gpu/: it exports the five symbols of src/gpu/glm53f_gpu.h:38-53 and nothing else. It is
 * compiled against the reference's headers where they lie (never copied here) and contains no
 * arithmetic: it reads the weights the reference has already bound (Glm53fLayerW,
 * include/glm53f/glm53f.h:249-257), hands them to g5b_engine_load under their checkpoint names,
 * pulls every routed expert once through the reference's own expert source
 * (Glm53fExpertSrc.get, glm53f.h:216-228) so that they become HBM resident, and forwards calls.
 *
 * Differences from the backend it replaces, visible to the driver: routed experts, router,
 * embedding gather and arg-max run on the GPU (the reference kept them on the CPU,
 * src/gpu/glm53f_gpu.c:1024-1040,1062-1066). With several devices (ndev > 1) the reference places
 * consecutive layers on consecutive devices (src/gpu/glm53f_gpu.c:758-790); here the devices form an
 * expert-parallel group instead - one engine per device, 1 / ndev of the routed experts each, the
 * trunk split by heads - and every call runs on all of them at once, one host thread per device.
 * ndev <= 0 ("all" in the reference) takes device 0 only: a group is formed only when asked for.
 */
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "glm53f_b200.h"
#include "glm53f_gpu.h"        /* reference: src/gpu/glm53f_gpu.h   */
#include "glm53f_model.h"      /* reference: src/model/glm53f_model.h */

#define B200_MAX_DEV 8
struct Glm53fGpu {
    g5b_engine *e;                      /* rank 0: its logits are the call's result */
    g5b_engine *all[B200_MAX_DEV];
    int n;
};

int glm53f_gpu_device_count(void) { return g5b_device_count(); }

static int put_mat(g5b_engine *e, const char *name, const Glm53fMat *m)
{
    g5b_tensor t;
    memset(&t, 0, sizeof t);
    t.data = m->w;
    t.scale_inv = m->s;
    t.dtype = m->dt == GLM53F_WF32 ? G5B_DT_F32 : m->dt == GLM53F_WBF16 ? G5B_DT_BF16 : G5B_DT_FP8;
    t.rows = m->rows;
    t.cols = m->cols;
    if (m->dt == GLM53F_WI4) { fprintf(stderr, "glm53f_b200: %s is int4, an approximation this engine does not load\n", name); return -1; }
    return g5b_engine_load(e, name, &t);
}

static int put_vec(g5b_engine *e, const char *name, const float *v, int n)
{
    g5b_tensor t;
    memset(&t, 0, sizeof t);
    t.data = v;
    t.dtype = G5B_DT_F32;
    t.rows = n;
    t.cols = 1;
    return g5b_engine_load(e, name, &t);
}

#define MAT(suffix, field)                                                         \
    do { snprintf(nm, sizeof nm, "layers.%d." suffix, L); if (put_mat(e, nm, &(field))) return -1; } while (0)
#define VEC(suffix, field, n)                                                      \
    do { snprintf(nm, sizeof nm, "layers.%d." suffix, L); if (put_vec(e, nm, (field), (n))) return -1; } while (0)

static int upload_layer(g5b_engine *e, struct Glm53fModel *m, int L)
{
    const Glm53fCfg *c = &m->cfg;
    const Glm53fLayerW *w = &m->lay[L].w;
    const int E = c->hidden, M = c->hc_mult, MIX = (2 + M) * M;
    char nm[160];
    VEC("input_layernorm.weight", w->in_norm, E);
    VEC("post_attention_layernorm.weight", w->post_norm, E);
    MAT("hc_attn_fn", w->attn_hc.fn); VEC("hc_attn_base", w->attn_hc.base, MIX); VEC("hc_attn_scale", w->attn_hc.scale, 3);
    MAT("hc_ffn_fn", w->ffn_hc.fn);   VEC("hc_ffn_base", w->ffn_hc.base, MIX);   VEC("hc_ffn_scale", w->ffn_hc.scale, 3);
    if (w->is_mla) {
        const Glm53fMlaW *a = &w->mla;
        MAT("self_attn.q_a_proj.weight", a->q_a);
        VEC("self_attn.q_a_layernorm.weight", a->q_a_norm, c->q_lora);
        MAT("self_attn.q_b_proj.weight", a->q_b);
        MAT("self_attn.kv_a_proj_with_mqa.weight", a->kv_a);
        VEC("self_attn.kv_a_layernorm.weight", a->kv_a_norm, c->kv_lora);
        MAT("self_attn.kv_b_proj.weight", a->kv_b);
        MAT("self_attn.o_proj.weight", a->o);
        MAT("self_attn.indexer.wq_b.weight", a->idx.wq_b);
        MAT("self_attn.indexer.wk.weight", a->idx.wk);
        VEC("self_attn.indexer.k_norm.weight", a->idx.k_norm_w, c->index_dim);
        VEC("self_attn.indexer.k_norm.bias", a->idx.k_norm_b, c->index_dim);
        MAT("self_attn.indexer.weights_proj.weight", a->idx.wproj);
        MAT("self_attn.indexer.index_kpool_compress_gate", a->idx.gate);
        VEC("self_attn.indexer.index_kpool_compress_ape", a->idx.ape, c->index_kpool * c->index_dim);
    } else {
        const Glm53fKdaW *k = &w->kda;
        const int H = c->kda_heads, D = c->kda_head_dim, P = H * D;
        MAT("self_attn.q_proj.weight", k->q); MAT("self_attn.k_proj.weight", k->k); MAT("self_attn.v_proj.weight", k->v);
        VEC("self_attn.q_conv1d.weight", k->q_conv, P * c->conv_k);
        VEC("self_attn.k_conv1d.weight", k->k_conv, P * c->conv_k);
        VEC("self_attn.v_conv1d.weight", k->v_conv, P * c->conv_k);
        MAT("self_attn.f_a_proj.weight", k->f_a); MAT("self_attn.f_b_proj.weight", k->f_b);
        VEC("self_attn.A_log", k->A_log, H); VEC("self_attn.dt_bias", k->dt_bias, P);
        MAT("self_attn.b_proj.weight", k->b);
        MAT("self_attn.g_a_proj.weight", k->g_a); MAT("self_attn.g_b_proj.weight", k->g_b);
        VEC("self_attn.o_norm.weight", k->o_norm, D);
        MAT("self_attn.o_proj.weight", k->o);
    }
    if (w->is_dense) {
        MAT("mlp.gate_proj.weight", w->d_gate); MAT("mlp.up_proj.weight", w->d_up); MAT("mlp.down_proj.weight", w->d_down);
        return 0;
    }
    /* The router arrives widened to FP32 (src/model/glm53f_bind.c:199): a matrix to this engine. */
    {
        g5b_tensor t;
        memset(&t, 0, sizeof t);
        t.data = w->moe.gate; t.dtype = G5B_DT_F32; t.rows = c->n_experts; t.cols = E;
        snprintf(nm, sizeof nm, "layers.%d.mlp.gate.weight", L);
        if (g5b_engine_load(e, nm, &t)) return -1;
    }
    VEC("mlp.gate.e_score_correction_bias", w->moe.bias, c->n_experts);
    MAT("mlp.shared_experts.gate_proj.weight", w->moe.sh_gate);
    MAT("mlp.shared_experts.up_proj.weight", w->moe.sh_up);
    MAT("mlp.shared_experts.down_proj.weight", w->moe.sh_down);
    Glm53fExpertSrc *src = w->moe.src;
    for (int x = 0; x < c->n_experts; x++) {
        Glm53fExpertQ q;
        if (!src || src->get(src, L, x, &q) != 0) {
            fprintf(stderr, "glm53f_b200: layer %d expert %d could not be read\n", L, x);
            return -1;
        }
        int rc = 0;
        snprintf(nm, sizeof nm, "layers.%d.mlp.experts.%d.gate_proj.weight", L, x); rc |= put_mat(e, nm, &q.gate);
        snprintf(nm, sizeof nm, "layers.%d.mlp.experts.%d.up_proj.weight", L, x);   rc |= put_mat(e, nm, &q.up);
        snprintf(nm, sizeof nm, "layers.%d.mlp.experts.%d.down_proj.weight", L, x); rc |= put_mat(e, nm, &q.down);
        if (src->release) src->release(src, L, x);
        if (rc) return -1;
    }
    return 0;
}

Glm53fGpu *glm53f_gpu_create(struct Glm53fModel *m, const int *devices, int ndev)
{
    const Glm53fCfg *c = &m->cfg;
    g5b_config g;
    memset(&g, 0, sizeof g);
    g.hidden = c->hidden; g.n_layers = m->n_bound; g.vocab = c->vocab; g.rms_eps = c->rms_eps;
    g.hc_mult = c->hc_mult; g.hc_iters = c->hc_iters; g.hc_eps = c->hc_eps;
    g.kda_heads = c->kda_heads; g.kda_head_dim = c->kda_head_dim; g.conv_k = c->conv_k; g.gate_lb = c->gate_lb;
    g.mla_heads = c->n_heads; g.q_lora = c->q_lora; g.kv_lora = c->kv_lora; g.qk_nope = c->qk_nope; g.v_head = c->v_head;
    g.index_topk = c->index_topk; g.index_kpool = c->index_kpool; g.index_heads = c->index_heads; g.index_dim = c->index_dim;
    g.n_experts = c->n_experts; g.topk = c->topk; g.n_shared = c->n_shared; g.moe_inter = c->moe_inter;
    g.dense_inter = c->dense_inter; g.routed_scale = c->routed_scale; g.norm_topk = c->norm_topk;
    g.swiglu_limit = c->swiglu_limit; g.fp8_block_r = c->fp8_block_r; g.fp8_block_c = c->fp8_block_c;

    /* one engine per device; the devices become an expert-parallel group when the experts divide */
    int n = (devices && ndev > 1) ? ndev : 1;
    if (n > B200_MAX_DEV) n = B200_MAX_DEV;
    while (n > 1 && c->n_experts % n) n--;
    Glm53fGpu *gpu = (Glm53fGpu *)calloc(1, sizeof *gpu);
    gpu->n = n;
    int rc = 0;
    for (int r = 0; r < n && !rc; r++) {
        const int device = (devices && ndev > 0) ? devices[r] : 0;
        g5b_engine *e = g5b_engine_create(&g, c->is_mla, c->is_dense, m->cap, device, r, n);
        if (!e) { rc = -1; break; }
        gpu->all[r] = e;
        /* every engine is offered every tensor; routed experts of other ranks are skipped by the engine */
        rc = put_mat(e, "embed_tokens.weight", &m->mb.embed) | put_mat(e, "lm_head.weight", &m->mb.lm_head) |
             put_vec(e, "norm.weight", m->mb.norm, c->hidden);
        for (int L = 0; L < m->n_bound && !rc; L++) rc = upload_layer(e, m, L);
        if (!rc) rc = g5b_engine_finalize(e);
    }
    if (!rc && n > 1) rc = g5b_engine_ep_connect_local(gpu->all, n);
    if (rc) {
        fprintf(stderr, "glm53f_b200: %s\n", g5b_last_error());
        for (int r = 0; r < n; r++) if (gpu->all[r]) g5b_engine_free(gpu->all[r]);
        free(gpu);
        return NULL;
    }
    gpu->e = gpu->all[0];
    if (!glm53f_quiet)
        printf("B200 engine: %d layers resident on %d device(s), %d routed experts per layer and device\n",
               m->n_bound, n, c->n_experts / n);
    return gpu;
}

void glm53f_gpu_free(Glm53fGpu *g)
{
    if (!g) return;
    for (int r = 0; r < g->n; r++) g5b_engine_free(g->all[r]);
    free(g);
}

/* One rank's share of a forward call (ranks other than 0 need no logits). */
typedef struct { g5b_engine *e; const int *ids; int T; int rc; } RankCall;
static void *rank_forward(void *p)
{
    RankCall *c = (RankCall *)p;
    c->rc = g5b_engine_forward(c->e, c->ids, c->T, NULL, NULL);
    return NULL;
}

int glm53f_gpu_forward(Glm53fGpu *g, struct Glm53fModel *m, const int *ids, int T, float *logits, int *argmax_all)
{
    m->layers_completed = 0;
    pthread_t th[B200_MAX_DEV];
    RankCall call[B200_MAX_DEV];
    int started = 0, rc = 0;
    for (int r = 1; r < g->n; r++) {
        call[r].e = g->all[r]; call[r].ids = ids; call[r].T = T; call[r].rc = -1;
        if (pthread_create(&th[r], NULL, rank_forward, &call[r]) != 0) { rc = -1; break; }
        started = r;
    }
    /* rank 0 runs even if a thread could not be started: its exchange then times out and reports */
    if (g5b_engine_forward(g->e, ids, T, logits, argmax_all) != 0) rc = -1;
    for (int r = 1; r <= started; r++) {
        pthread_join(th[r], NULL);
        if (call[r].rc != 0) rc = -1;
    }
    if (rc) return -1;
    m->layers_completed = m->n_bound;
    m->cached += T;
    return 0;
}

void glm53f_gpu_reset(Glm53fGpu *g)
{
    for (int r = 0; r < g->n; r++) g5b_engine_reset(g->all[r]);
}
