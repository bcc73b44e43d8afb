/*
 * glm53f_oracle.c - see glm53f_oracle.h. TEST INFRASTRUCTURE: the CPU checker, never the
 * product. Scalar C, compiled with -ffp-contract=off so that no sum is fused differently
 * from the reference build (reference CMakeLists.txt:42). Citations are path:line into
 * josesilva05/glm-5.3-flash-in-c.
 */
#include "glm53f_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ storage ---- */
typedef struct {
    void  *w;
    float *s;
    int dt, rows, cols, br, bc, scols;
} OMat;

typedef struct {
    OMat   fn;
    float *base, *scale;
} OHc;

typedef struct {
    OHc    hc[2];                       /* 0 attention site, 1 feed-forward site */
    float *in_norm, *post_norm;
    int    is_mla, is_dense;
    /* KDA */
    OMat   kq, kk, kv, f_a, f_b, kb, g_a, g_b, ko;
    float *q_conv, *k_conv, *v_conv, *A_log, *dt_bias, *o_norm;
    /* MLA + indexer */
    OMat   q_a, q_b, kv_a, kv_b, mo, wq_b, wk, wproj, igate;
    float *q_a_norm, *kv_a_norm, *k_norm_w, *k_norm_b, *ape;
    /* feed-forward */
    OMat   d_gate, d_up, d_down, sh_gate, sh_up, sh_down;
    float *router, *bias;
    OMat  *experts;                     /* [n_experts][3] gate, up, down */
    /* session state */
    float *kda_state, *kvc, *ckv, *idx;
} OLayer;

struct orc_model {
    g5b_config c;
    int     cap, cached, latent, finalized;
    OLayer *L;                          /* n_layers entries, one more (the MTP layer) with `mtp` */
    OMat    embed, lm_head;
    float  *norm;
    /* the multi-token-prediction layer (checkpoint layer n_layers), orc_model_enable_mtp */
    int     mtp, mtp_cached;
    float  *enorm, *hnorm, *head_norm;
    OMat    eh;
    float  *mtp_h;                      /* [cap][hidden]: mean of the streams of every position fed */
};
static int n_slots(const orc_model *m) { return m->c.n_layers + (m->mtp ? 1 : 0); }

static float bf16f(uint16_t h)
{
    union { uint32_t u; float f; } v;
    v.u = (uint32_t)h << 16;
    return v.f;
}

/* E4M3FN code to float (reference: src/core/glm53f_ops.c:51-72): bias 7, exponent 0 is
 * subnormal m/8 * 2^-6, only s.1111.111 is NaN, there is no infinity. */
static float E4M3[256];
static int   e4m3_built = 0;
static void build_e4m3(void)
{
    if (e4m3_built) return;
    for (int code = 0; code < 256; code++) {
        const int neg = code >> 7, ex = (code >> 3) & 15, man = code & 7;
        double mag;
        if (ex == 15 && man == 7) mag = NAN;
        else if (ex == 0)         mag = ldexp((double)man / 8.0, -6);
        else                      mag = ldexp(1.0 + (double)man / 8.0, ex - 7);
        E4M3[code] = (float)(neg ? -mag : mag);
    }
    e4m3_built = 1;
}

static float sigm(float x) { return 1.0f / (1.0f + expf(-x)); }   /* glm53f_ops.c:46 */

/* ------------------------------------------------------------------- matvec ---- */
/* Sixteen interleaved double accumulators, element i+l into accumulator l, folded as
 * ((a0+a4)+(a8+a12)) + ... then the four folds pairwise; leftover elements are added to the
 * total one by one (glm53f_ops.c:77-98 for F32, :101-154 for BF16; the AVX2 and scalar forms
 * of the reference are the same sums). */
static float dot16(const void *row, int dt, const float *x, int n)
{
    double a[16];
    for (int l = 0; l < 16; l++) a[l] = 0.0;
    const float *rf = (const float *)row;
    const uint16_t *rh = (const uint16_t *)row;
    int i = 0;
    for (; i + 15 < n; i += 16)
        for (int l = 0; l < 16; l++) {
            const double wv = dt == G5B_DT_BF16 ? (double)bf16f(rh[i + l]) : (double)rf[i + l];
            a[l] = fma(wv, (double)x[i + l], a[l]);
        }
    const double f0 = (a[0] + a[4]) + (a[8] + a[12]);
    const double f1 = (a[1] + a[5]) + (a[9] + a[13]);
    const double f2 = (a[2] + a[6]) + (a[10] + a[14]);
    const double f3 = (a[3] + a[7]) + (a[11] + a[15]);
    double total = (f0 + f1) + (f2 + f3);
    for (; i < n; i++) {
        const double wv = dt == G5B_DT_BF16 ? (double)bf16f(rh[i]) : (double)rf[i];
        total = fma(wv, (double)x[i], total);
    }
    return (float)total;
}

/* FP8 row (glm53f_ops.c:185-228): per column block, eight float lanes of fmaf (lane l takes
 * columns congruent to l mod 8, whole groups of eight only), lanes folded in double as
 * ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)), leftover columns added as double products, the block
 * sum multiplied by the block scale in double, blocks added in order. */
static float dot_fp8(const uint8_t *row, const float *srow, const float *x, int n, int bc)
{
    double total = 0.0;
    int blk = 0;
    for (int c0 = 0; c0 < n; c0 += bc, blk++) {
        const int c1 = c0 + bc < n ? c0 + bc : n;
        float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int j = c0;
        for (; j + 8 <= c1; j += 8)
            for (int l = 0; l < 8; l++) lane[l] = fmaf(E4M3[row[j + l]], x[j + l], lane[l]);
        double bs = (((double)lane[0] + lane[4]) + ((double)lane[2] + lane[6]))
                  + (((double)lane[1] + lane[5]) + ((double)lane[3] + lane[7]));
        for (; j < c1; j++) bs += (double)E4M3[row[j]] * (double)x[j];
        total += bs * (double)srow[blk];
    }
    return (float)total;
}

/* y[rows] = M x (glm53f_mm, glm53f_ops.c:446-458). glm53f_mm_batch (:378-444) is the same sum
 * per input, so T inputs are T independent calls. */
static void mv(float *y, const float *x, const OMat *m)
{
    if (!m->w) { fprintf(stderr, "oracle: multiply through an unloaded matrix\n"); abort(); }
    int r;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) if (m->rows > 64)
#endif
    for (r = 0; r < m->rows; r++) {
        if (m->dt == G5B_DT_FP8)
            y[r] = dot_fp8((const uint8_t *)m->w + (size_t)r * m->cols,
                           m->s + (size_t)(r / m->br) * m->scols, x, m->cols, m->bc);
        else if (m->dt == G5B_DT_BF16)
            y[r] = dot16((const uint16_t *)m->w + (size_t)r * m->cols, G5B_DT_BF16, x, m->cols);
        else
            y[r] = dot16((const float *)m->w + (size_t)r * m->cols, G5B_DT_F32, x, m->cols);
    }
}

/* glm53f_rmsnorm, glm53f_ops.c:473-480. */
static void rmsnorm(float *y, const float *x, const float *w, int n, float eps)
{
    double ss = 0.0;
    for (int i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    const float inv = (float)(1.0 / sqrt(ss / (double)n + (double)eps));
    for (int i = 0; i < n; i++) y[i] = w ? w[i] * (x[i] * inv) : x[i] * inv;
}

/* glm53f_swiglu_clamp, glm53f_ops.c:486-494: the gate is clamped from above only. */
static void swiglu(float *y, const float *gu, int n, float lim)
{
    for (int i = 0; i < n; i++) {
        const float g = gu[i] > lim ? lim : gu[i];
        float u = gu[n + i];
        u = u > lim ? lim : (u < -lim ? -lim : u);
        y[i] = (g * sigm(g)) * u;
    }
}

/* glm53f_mlp, glm53f_ops.c:503-511. */
static void mlp(float *out, const float *x, const OMat *g, const OMat *u, const OMat *d, float lim)
{
    const int I = g->rows;
    float *gu = (float *)malloc((size_t)3 * I * sizeof(float));
    mv(gu, x, g);
    mv(gu + I, x, u);
    swiglu(gu + 2 * I, gu, I, lim);
    mv(out, gu + 2 * I, d);
    free(gu);
}

/* glm53f_shortconv, glm53f_ops.c:517-542: taps oldest to newest, w[k-1] on the current input,
 * the current term first, then history terms added in order; SiLU; history shifts. */
static void shortconv(float *y, const float *x, const float *w, float *state, int ch, int k, int T)
{
    const int hist = k - 1;
    for (int c = 0; c < ch; c++) {
        float past[16];
        for (int j = 0; j < hist; j++) past[j] = state ? state[(size_t)c * hist + j] : 0.0f;
        for (int t = 0; t < T; t++) {
            const float cur = x[(size_t)t * ch + c];
            float acc = w[(size_t)c * k + hist] * cur;
            for (int j = 0; j < hist; j++) acc += w[(size_t)c * k + j] * past[j];
            for (int j = 0; j + 1 < hist; j++) past[j] = past[j + 1];
            if (hist > 0) past[hist - 1] = cur;
            y[(size_t)t * ch + c] = acc * sigm(acc);
        }
        if (state) for (int j = 0; j < hist; j++) state[(size_t)c * hist + j] = past[j];
    }
}

/* ---------------------------------------------------------------------- mHC ---- */
/* glm53f_hc_pre, glm53f_ops.c:560-608. */
static void hc_pre(float *x, float *post, float *comb, const float *h, const OHc *w,
                   const g5b_config *c)
{
    const int M = c->hc_mult, E = c->hidden, ME = M * E, MIX = (2 + M) * M;
    float *flat = (float *)malloc(((size_t)ME + MIX) * sizeof(float));
    float *mix = flat + ME;
    rmsnorm(flat, h, NULL, ME, c->rms_eps);
    mv(mix, flat, &w->fn);

    double pre[G5B_MAX_HC], cm[G5B_MAX_HC * G5B_MAX_HC];
    const double eps = (double)c->hc_eps;
    for (int i = 0; i < M; i++) {
        pre[i]  = (double)sigm(mix[i] * w->scale[0] + w->base[i]) + eps;
        post[i] = 2.0f * sigm(mix[M + i] * w->scale[1] + w->base[M + i]);
    }
    for (int i = 0; i < M; i++) {
        double lg[G5B_MAX_HC], top = -INFINITY, z = 0.0;
        for (int j = 0; j < M; j++) {
            const int k = 2 * M + i * M + j;
            lg[j] = (double)(mix[k] * w->scale[2] + w->base[k]);
            if (lg[j] > top) top = lg[j];
        }
        for (int j = 0; j < M; j++) z += exp(lg[j] - top);
        for (int j = 0; j < M; j++) cm[i * M + j] = exp(lg[j] - top) / z + eps;
    }
    /* Sinkhorn: columns first, then (iters-1) x (rows, columns); every division is by
     * (sum + eps) (glm53f_ops.c:591-598). */
    for (int pass = 0; pass < 2 * c->hc_iters - 1; pass++) {
        const int by_col = (pass % 2) == 0;
        for (int a = 0; a < M; a++) {
            double s = 0.0;
            for (int b = 0; b < M; b++) s += by_col ? cm[b * M + a] : cm[a * M + b];
            for (int b = 0; b < M; b++) {
                if (by_col) cm[b * M + a] /= (s + eps);
                else        cm[a * M + b] /= (s + eps);
            }
        }
    }
    for (int k = 0; k < M * M; k++) comb[k] = (float)cm[k];
    for (int d = 0; d < E; d++) {
        double s = 0.0;
        for (int i = 0; i < M; i++) s += pre[i] * (double)h[(size_t)i * E + d];
        x[d] = (float)s;
    }
    free(flat);
}

/* glm53f_hc_post, glm53f_ops.c:612-625: h'[j] = post[j]*y + sum_i comb[i][j]*h[i]. */
static void hc_post(float *h, const float *y, const float *post, const float *comb,
                    const g5b_config *c)
{
    const int M = c->hc_mult, E = c->hidden;
    float *nh = (float *)malloc((size_t)M * E * sizeof(float));
    for (int j = 0; j < M; j++)
        for (int d = 0; d < E; d++) {
            double s = (double)post[j] * (double)y[d];
            for (int i = 0; i < M; i++) s += (double)comb[i * M + j] * (double)h[(size_t)i * E + d];
            nh[(size_t)j * E + d] = (float)s;
        }
    memcpy(h, nh, (size_t)M * E * sizeof(float));
    free(nh);
}

/* ---------------------------------------------------------------------- KDA ---- */
/* kda_step, glm53f_ops.c:630-658. S is [dk][dv]; four passes, each summing over the key index
 * in ascending order in FP32. */
static void delta_step(float *S, float *o, const float *q, const float *k, const float *v,
                       const float *alpha, float beta, int D)
{
    float *u = (float *)malloc((size_t)D * sizeof(float));
    for (int i = 0; i < D; i++)
        for (int j = 0; j < D; j++) S[(size_t)i * D + j] *= alpha[i];
    for (int j = 0; j < D; j++) u[j] = 0.0f;
    for (int i = 0; i < D; i++)
        for (int j = 0; j < D; j++) u[j] += S[(size_t)i * D + j] * k[i];
    for (int j = 0; j < D; j++) u[j] = (v[j] - u[j]) * beta;
    for (int i = 0; i < D; i++)
        for (int j = 0; j < D; j++) S[(size_t)i * D + j] += k[i] * u[j];
    for (int j = 0; j < D; j++) o[j] = 0.0f;
    for (int i = 0; i < D; i++)
        for (int j = 0; j < D; j++) o[j] += S[(size_t)i * D + j] * q[i];
    free(u);
}

/* l2norm_, glm53f_ops.c:661-667: divide by sqrt(SUM of squares + eps). */
static void l2norm(float *v, int n, float eps)
{
    double ss = 0.0;
    for (int i = 0; i < n; i++) ss += (double)v[i] * (double)v[i];
    const float inv = (float)(1.0 / sqrt(ss + (double)eps));
    for (int i = 0; i < n; i++) v[i] *= inv;
}

/* glm53f_kda_layer, glm53f_ops.c:687-755. */
static void kda_layer(float *out, const float *x, const OLayer *w, const g5b_config *c, int T,
                      float *state)
{
    const int E = c->hidden, H = c->kda_heads, D = c->kda_head_dim, P = H * D;
    const int K = c->conv_k, hist = K - 1;
    const size_t TP = (size_t)T * P;
    float *q = (float *)malloc((6 * TP + (size_t)T * H + 2 * (size_t)P + 2 * (size_t)D) * sizeof(float));
    float *k = q + TP, *v = k + TP, *z = v + TP, *al = z + TP, *o = al + TP;
    float *bt = o + TP, *gb = bt + (size_t)T * H, *qs = gb + P, *lr = qs + P;

    for (int t = 0; t < T; t++) {
        const float *xt = x + (size_t)t * E;
        mv(q + (size_t)t * P, xt, &w->kq);
        mv(k + (size_t)t * P, xt, &w->kk);
        mv(v + (size_t)t * P, xt, &w->kv);
        mv(bt + (size_t)t * H, xt, &w->kb);
        mv(lr, xt, &w->f_a);
        mv(z + (size_t)t * P, lr, &w->f_b);
    }
    float *cs = state + (size_t)H * D * D;
    shortconv(q, q, w->q_conv, cs, P, K, T);
    shortconv(k, k, w->k_conv, cs + (size_t)P * hist, P, K, T);
    shortconv(v, v, w->v_conv, cs + (size_t)2 * P * hist, P, K, T);

    for (int t = 0; t < T; t++)
        for (int h = 0; h < H; h++) {
            const size_t off = (size_t)t * P + (size_t)h * D;
            l2norm(q + off, D, 1e-6f);
            l2norm(k + off, D, 1e-6f);
            bt[(size_t)t * H + h] = sigm(bt[(size_t)t * H + h]);
            const float a = expf(w->A_log[h]);
            for (int d = 0; d < D; d++) {
                const float g = c->gate_lb * sigm(a * (z[off + d] + w->dt_bias[(size_t)h * D + d]));
                al[off + d] = expf(g);
            }
        }
    const float qscale = 1.0f / sqrtf((float)D);
    for (int h = 0; h < H; h++)
        for (int t = 0; t < T; t++) {
            const size_t off = (size_t)t * P + (size_t)h * D;
            for (int i = 0; i < D; i++) qs[i] = q[off + i] * qscale;
            delta_step(state + (size_t)h * D * D, o + off, qs, k + off, v + off, al + off,
                       bt[(size_t)t * H + h], D);
        }
    for (int t = 0; t < T; t++) {
        const float *xt = x + (size_t)t * E;
        float *ot = o + (size_t)t * P;
        mv(lr, xt, &w->g_a);
        mv(gb, lr, &w->g_b);
        for (int h = 0; h < H; h++) {
            float *oh = ot + (size_t)h * D;
            rmsnorm(oh, oh, w->o_norm, D, c->rms_eps);
            for (int d = 0; d < D; d++) oh[d] *= sigm(gb[(size_t)h * D + d]);
        }
        mv(out + (size_t)t * E, ot, &w->ko);
    }
    free(q);
}

/* ---------------------------------------------------------------------- DSA ---- */
/* State layout (glm53f_dsa.c:44-53): keys [cap][D], then gate values [cap][D], then pool keys
 * [ceil(cap/kpool)][D]. */
static size_t dsa_floats(const g5b_config *c, int cap)
{
    return (size_t)2 * cap * c->index_dim +
           (size_t)((cap + c->index_kpool - 1) / c->index_kpool) * c->index_dim;
}
static float *dsa_key(float *st, const g5b_config *c, int pos) { return st + (size_t)pos * c->index_dim; }
static float *dsa_gate(float *st, const g5b_config *c, int cap, int pos)
{
    return st + ((size_t)cap + pos) * c->index_dim;
}
static float *dsa_pool(float *st, const g5b_config *c, int cap, int pool)
{
    return st + ((size_t)2 * cap + pool) * c->index_dim;
}

/* glm53f_dsa_append, glm53f_dsa.c:62-106: key = LayerNorm(wk x) (biased variance, eps 1e-6,
 * FP64), gate = gate x; a pool is closed when its last position arrives: per channel a
 * softmax over the pool's (gate + ape) weights the keys. */
static void dsa_append(float *st, const float *x, const OLayer *w, const g5b_config *c, int T,
                       int cached, int cap)
{
    const int D = c->index_dim, K = c->index_kpool, E = c->hidden;
    float *raw = (float *)malloc((size_t)D * sizeof(float));
    for (int t = 0; t < T; t++) {
        const int pos = cached + t;
        const float *xt = x + (size_t)t * E;
        mv(raw, xt, &w->wk);
        double mean = 0.0, var = 0.0;
        for (int i = 0; i < D; i++) mean += (double)raw[i];
        mean /= (double)D;
        for (int i = 0; i < D; i++) { const double d = (double)raw[i] - mean; var += d * d; }
        var /= (double)D;
        const double inv = 1.0 / sqrt(var + 1e-6);
        float *kp = dsa_key(st, c, pos);
        for (int i = 0; i < D; i++)
            kp[i] = (float)(((double)raw[i] - mean) * inv) * w->k_norm_w[i] + w->k_norm_b[i];
        mv(dsa_gate(st, c, cap, pos), xt, &w->igate);
        if ((pos + 1) % K) continue;
        const int pool = (pos + 1) / K - 1;
        float *pk = dsa_pool(st, c, cap, pool);
        for (int i = 0; i < D; i++) {
            double top = -INFINITY, z = 0.0, acc = 0.0;
            for (int j = 0; j < K; j++) {
                const double l = (double)dsa_gate(st, c, cap, pool * K + j)[i] + (double)w->ape[j * D + i];
                if (l > top) top = l;
            }
            for (int j = 0; j < K; j++)
                z += exp((double)dsa_gate(st, c, cap, pool * K + j)[i] + (double)w->ape[j * D + i] - top);
            for (int j = 0; j < K; j++) {
                const double p = exp((double)dsa_gate(st, c, cap, pool * K + j)[i] +
                                     (double)w->ape[j * D + i] - top) / z;
                acc += p * (double)dsa_key(st, c, pool * K + j)[i];
            }
            pk[i] = (float)acc;
        }
    }
    free(raw);
}

typedef struct { float s; int i; } Ranked;
static int by_score_then_index(const void *a, const void *b)
{
    const Ranked *p = (const Ranked *)a, *q = (const Ranked *)b;
    if (p->s != q->s) return p->s > q->s ? -1 : 1;
    return (p->i > q->i) - (p->i < q->i);
}
static int by_int(const void *a, const void *b)
{
    const int p = *(const int *)a, q = *(const int *)b;
    return (p > q) - (p < q);
}

/* glm53f_dsa_select, glm53f_dsa.c:124-171. Returns -1 when every visible position is kept. */
static int dsa_select(int *sel, float *st, const float *x_t, const float *q_resid,
                      const OLayer *w, const g5b_config *c, int p, int cap)
{
    const int D = c->index_dim, HI = c->index_heads, K = c->index_kpool;
    const int np = (p + 1) / K;
    int keep = c->index_topk / K;
    if (np <= keep) return -1;
    float *q = (float *)malloc(((size_t)HI * D + HI + np) * sizeof(float));
    float *wt = q + (size_t)HI * D, *score = wt + HI;
    mv(q, q_resid, &w->wq_b);
    mv(wt, x_t, &w->wproj);
    const float hscale = 1.0f / sqrtf((float)HI), dscale = 1.0f / sqrtf((float)D);
    for (int pp = 0; pp < np; pp++) {
        const float *pk = dsa_pool(st, c, cap, pp);
        double acc = 0.0;
        for (int h = 0; h < HI; h++) {
            double d = 0.0;
            for (int i = 0; i < D; i++) d += (double)q[(size_t)h * D + i] * (double)pk[i];
            d *= (double)dscale;
            if (d > 0.0) acc += (double)wt[h] * (double)hscale * d;
        }
        score[pp] = (float)acc;
    }
    Ranked *rank = (Ranked *)malloc((size_t)np * sizeof *rank);
    int *pools = (int *)malloc((size_t)keep * sizeof *pools);
    for (int pp = 0; pp < np; pp++) { rank[pp].s = score[pp]; rank[pp].i = pp; }
    qsort(rank, (size_t)np, sizeof *rank, by_score_then_index);
    for (int i = 0; i < keep; i++) pools[i] = rank[i].i;
    qsort(pools, (size_t)keep, sizeof(int), by_int);
    int n = 0;
    for (int i = 0; i < keep; i++)
        for (int j = 0; j < K; j++) sel[n++] = pools[i] * K + j;
    for (int j = np * K; j <= p; j++) sel[n++] = j;
    free(rank); free(pools); free(q);
    return n;
}

/* ---------------------------------------------------------------------- MLA ---- */
/* glm53f_mla, glm53f_ops.c:828-937, both cache forms. sel_out/n_sel_out report the last
 * query's selection. */
static void mla(float *out, const float *x, const OLayer *w, const g5b_config *c, int T,
                float *kvc, int cached, int cap, float *istate, float *ckv,
                int *sel_out, int *n_sel_out)
{
    const int E = c->hidden, H = c->mla_heads, qn = c->qk_nope, vh = c->v_head, KL = c->kv_lora;
    const int kvd = qn + vh;
    const float scale = 1.0f / sqrtf((float)qn);
    float *q   = (float *)malloc(((size_t)T * H * qn + (size_t)T * c->q_lora + KL +
                                  (size_t)T * H * vh) * sizeof(float));
    float *ql  = q + (size_t)T * H * qn;
    float *ct  = ql + (size_t)T * c->q_lora;
    float *acc = ct + KL;
    int   *sel = (int *)malloc((size_t)(c->index_topk + c->index_kpool) * sizeof(int));

    for (int t = 0; t < T; t++) {
        const float *xt = x + (size_t)t * E;
        float *qlt = ql + (size_t)t * c->q_lora;
        mv(qlt, xt, &w->q_a);
        rmsnorm(qlt, qlt, w->q_a_norm, c->q_lora, c->rms_eps);
        mv(q + (size_t)t * H * qn, qlt, &w->q_b);
        mv(ct, xt, &w->kv_a);
        rmsnorm(ct, ct, w->kv_a_norm, KL, c->rms_eps);
        if (ckv) memcpy(ckv + (size_t)(cached + t) * KL, ct, (size_t)KL * sizeof(float));
        else     mv(kvc + (size_t)(cached + t) * H * kvd, ct, &w->kv_b);
    }
    if (istate) dsa_append(istate, x, w, c, T, cached, cap);

    for (int t = 0; t < T; t++) {
        const int p = cached + t;
        const int nsel = istate ? dsa_select(sel, istate, x + (size_t)t * E,
                                             ql + (size_t)t * c->q_lora, w, c, p, cap) : -1;
        const int nvis = nsel < 0 ? p + 1 : nsel;
        if (t == T - 1 && n_sel_out) {
            *n_sel_out = nsel;
            if (sel_out && nsel > 0) memcpy(sel_out, sel, (size_t)nsel * sizeof(int));
        }
        int h;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
        for (h = 0; h < H; h++) {
            const float *qt = q + ((size_t)t * H + h) * qn;
            float  *s  = (float *)malloc((size_t)nvis * sizeof(float));
            double top = -INFINITY, z = 0.0;
            float *o = acc + ((size_t)t * H + h) * vh;
            if (ckv) {
                /* absorbed form: qa = W_k^T q in double (matmul_transposed, :793-814) */
                double *qa = (double *)calloc((size_t)2 * KL, sizeof(double));
                double *cb = qa + KL;
                for (int i = 0; i < qn; i++) {
                    const double qi = (double)qt[i];
                    if (qi == 0.0) continue;
                    const int r = h * kvd + i;
                    for (int cc = 0; cc < KL; cc++) {
                        double wv;
                        if (w->kv_b.dt == G5B_DT_BF16)
                            wv = (double)bf16f(((const uint16_t *)w->kv_b.w)[(size_t)r * KL + cc]);
                        else if (w->kv_b.dt == G5B_DT_FP8)
                            wv = (double)E4M3[((const uint8_t *)w->kv_b.w)[(size_t)r * KL + cc]] *
                                 (double)w->kv_b.s[(size_t)(r / w->kv_b.br) * w->kv_b.scols + cc / w->kv_b.bc];
                        else
                            wv = (double)((const float *)w->kv_b.w)[(size_t)r * KL + cc];
                        qa[cc] += qi * wv;
                    }
                }
                for (int jj = 0; jj < nvis; jj++) {
                    const float *cj = ckv + (size_t)(nsel < 0 ? jj : sel[jj]) * KL;
                    double d = 0.0;
                    for (int i = 0; i < KL; i++) d += qa[i] * (double)cj[i];
                    d *= scale;
                    s[jj] = (float)d;
                    if (d > top) top = d;
                }
                for (int jj = 0; jj < nvis; jj++) z += exp((double)s[jj] - top);
                for (int jj = 0; jj < nvis; jj++) {
                    const float *cj = ckv + (size_t)(nsel < 0 ? jj : sel[jj]) * KL;
                    const double pr = exp((double)s[jj] - top) / z;
                    for (int i = 0; i < KL; i++) cb[i] += pr * (double)cj[i];
                }
                float *cbf = (float *)malloc((size_t)KL * sizeof(float));
                for (int i = 0; i < KL; i++) cbf[i] = (float)cb[i];
                OMat wv = w->kv_b;                       /* row_slice, :781-790 */
                const int r0 = h * kvd + qn;
                wv.rows = vh;
                if (wv.dt == G5B_DT_BF16)      wv.w = (uint16_t *)wv.w + (size_t)r0 * KL;
                else if (wv.dt == G5B_DT_FP8) { wv.w = (uint8_t *)wv.w + (size_t)r0 * KL;
                                                wv.s = wv.s + (size_t)(r0 / wv.br) * wv.scols; }
                else                           wv.w = (float *)wv.w + (size_t)r0 * KL;
                /* mv() would nest an OpenMP region; rows are few, run them here */
                for (int r = 0; r < vh; r++) {
                    if (wv.dt == G5B_DT_FP8)
                        o[r] = dot_fp8((const uint8_t *)wv.w + (size_t)r * KL,
                                       wv.s + (size_t)(r / wv.br) * wv.scols, cbf, KL, wv.bc);
                    else if (wv.dt == G5B_DT_BF16)
                        o[r] = dot16((const uint16_t *)wv.w + (size_t)r * KL, G5B_DT_BF16, cbf, KL);
                    else
                        o[r] = dot16((const float *)wv.w + (size_t)r * KL, G5B_DT_F32, cbf, KL);
                }
                free(cbf); free(qa); free(s);
                continue;
            }
            for (int jj = 0; jj < nvis; jj++) {
                const float *kj = kvc + ((size_t)(nsel < 0 ? jj : sel[jj]) * H + h) * kvd;
                double d = 0.0;
                for (int i = 0; i < qn; i++) d += (double)qt[i] * (double)kj[i];
                d *= scale;
                s[jj] = (float)d;
                if (d > top) top = d;
            }
            for (int jj = 0; jj < nvis; jj++) z += exp((double)s[jj] - top);
            double *tmp = (double *)calloc((size_t)vh, sizeof(double));
            for (int jj = 0; jj < nvis; jj++) {
                const float *vj = kvc + ((size_t)(nsel < 0 ? jj : sel[jj]) * H + h) * kvd + qn;
                const double pr = exp((double)s[jj] - top) / z;
                for (int i = 0; i < vh; i++) tmp[i] += pr * (double)vj[i];
            }
            for (int i = 0; i < vh; i++) o[i] = (float)tmp[i];
            free(tmp); free(s);
        }
        mv(out + (size_t)t * E, acc + (size_t)t * H * vh, &w->mo);
    }
    free(q); free(sel);
}

/* ---------------------------------------------------------------- router, MoE ---- */
/* glm53f_router, glm53f_ops.c:945-976. */
static int router(int *idx, float *wt, const float *x, const OLayer *w, const g5b_config *c)
{
    const int NE = c->n_experts, E = c->hidden, K = c->topk;
    float score[G5B_MAX_EXPERTS], choice[G5B_MAX_EXPERTS];
    for (int e = 0; e < NE; e++) {
        const float *row = w->router + (size_t)e * E;
        double acc = 0.0;
        for (int i = 0; i < E; i++) acc += (double)row[i] * (double)x[i];
        score[e]  = sigm((float)acc);
        choice[e] = score[e] + w->bias[e];
    }
    for (int j = 0; j < K; j++) {
        int best = -1;
        float bv = -INFINITY;
        for (int e = 0; e < NE; e++)
            if (choice[e] > bv) { bv = choice[e]; best = e; }
        if (best < 0) return -1;
        idx[j] = best;
        wt[j] = score[best];
        choice[best] = -INFINITY;
    }
    if (c->norm_topk) {
        double s = 0.0;
        for (int j = 0; j < K; j++) s += (double)wt[j];
        for (int j = 0; j < K; j++) wt[j] = (float)((double)wt[j] / (s + 1e-20));
    }
    for (int j = 0; j < K; j++) wt[j] *= c->routed_scale;
    return 0;
}

/* moe_chunk, glm53f_ops.c:1144-1342, without its streaming/prefetch machinery: per token, the
 * K expert outputs are kept as floats and summed in top-k order in double with the router
 * weights (:1329-1337); the shared expert is added afterwards in FP32 (:1339-1340). Batched
 * experts use glm53f_mm_batch, which is the same sum per token, so tokens are independent. */
static int moe(float *out, const float *x, const OLayer *w, const g5b_config *c, int T,
               int with_shared)
{
    const int E = c->hidden, K = c->topk, I = c->moe_inter;
    float *contrib = (float *)malloc(((size_t)K * E + 3 * (size_t)I + E) * sizeof(float));
    float *gu = contrib + (size_t)K * E, *sho = gu + 3 * (size_t)I;
    int rc = 0;
    for (int t = 0; t < T && rc == 0; t++) {
        const float *xt = x + (size_t)t * E;
        int idx[G5B_MAX_TOPK];
        float wt[G5B_MAX_TOPK];
        if (router(idx, wt, xt, w, c) != 0) { rc = -1; break; }
        for (int j = 0; j < K; j++) {
            const OMat *ex = w->experts ? w->experts + (size_t)idx[j] * 3 : NULL;
            if (!ex || !ex[0].w || !ex[1].w || !ex[2].w) {
                fprintf(stderr, "oracle: routed expert %d was not loaded\n", idx[j]);
                rc = -1; break;
            }
            mv(gu, xt, &ex[0]);
            mv(gu + I, xt, &ex[1]);
            swiglu(gu + 2 * I, gu, I, c->swiglu_limit);
            mv(contrib + (size_t)j * E, gu + 2 * I, &ex[2]);
        }
        if (rc) break;
        float *ot = out + (size_t)t * E;
        for (int d = 0; d < E; d++) {
            double s = 0.0;
            for (int j = 0; j < K; j++) s += (double)wt[j] * (double)contrib[(size_t)j * E + d];
            ot[d] = (float)s;
        }
        if (with_shared) {
            mlp(sho, xt, &w->sh_gate, &w->sh_up, &w->sh_down, c->swiglu_limit);
            for (int d = 0; d < E; d++) ot[d] += sho[d];
        }
    }
    free(contrib);
    return rc;
}

/* glm53f_decoder_layer, glm53f_ops.c:1400-1433. */
static int decoder_layer(orc_model *m, int L, float *h, int T, int cached)
{
    const g5b_config *c = &m->c;
    OLayer *w = &m->L[L];
    const size_t E = (size_t)c->hidden, M = (size_t)c->hc_mult;
    float *xc = (float *)malloc((3 * T * E + T * M * (1 + M)) * sizeof(float));
    float *xn = xc + T * E, *y = xn + T * E, *post = y + T * E, *comb = post + T * M;
    int rc = 0;
    for (int site = 0; site < 2 && rc == 0; site++) {
        for (int t = 0; t < T; t++)
            hc_pre(xc + t * E, post + t * M, comb + t * M * M, h + t * M * E, &w->hc[site], c);
        for (int t = 0; t < T; t++)
            rmsnorm(xn + t * E, xc + t * E, site ? w->post_norm : w->in_norm, c->hidden, c->rms_eps);
        if (site == 0) {
            if (w->is_mla) mla(y, xn, w, c, T, w->kvc, cached, m->cap, w->idx, w->ckv, NULL, NULL);
            else           kda_layer(y, xn, w, c, T, w->kda_state);
        } else if (w->is_dense) {
            for (int t = 0; t < T; t++)
                mlp(y + t * E, xn + t * E, &w->d_gate, &w->d_up, &w->d_down, c->swiglu_limit);
        } else {
            rc = moe(y, xn, w, c, T, 1);
        }
        for (int t = 0; t < T && rc == 0; t++)
            hc_post(h + t * M * E, y + t * E, post + t * M, comb + t * M * M, c);
    }
    free(xc);
    return rc;
}

/* ------------------------------------------------------------------- loading ---- */
static int keep_mat(OMat *dst, const g5b_tensor *t, const g5b_config *c, int rows, int cols,
                    const char *name)
{
    if (t->rows != rows || t->cols != cols) {
        fprintf(stderr, "oracle: %s is %d x %d, expected %d x %d\n", name, t->rows, t->cols, rows, cols);
        return -1;
    }
    const size_t n = (size_t)rows * cols;
    const size_t eb = t->dtype == G5B_DT_F32 ? 4 : t->dtype == G5B_DT_BF16 ? 2 : 1;
    free(dst->w); free(dst->s);
    memset(dst, 0, sizeof *dst);
    dst->w = malloc(n * eb);
    memcpy(dst->w, t->data, n * eb);
    dst->dt = t->dtype; dst->rows = rows; dst->cols = cols;
    if (t->dtype == G5B_DT_FP8) {
        if (!t->scale_inv || c->fp8_block_r < 1 || c->fp8_block_c < 1) {
            fprintf(stderr, "oracle: %s is FP8 without a scale grid\n", name);
            return -1;
        }
        dst->br = c->fp8_block_r; dst->bc = c->fp8_block_c;
        dst->scols = (cols + dst->bc - 1) / dst->bc;
        const size_t ns = (size_t)((rows + dst->br - 1) / dst->br) * dst->scols;
        dst->s = (float *)malloc(ns * sizeof(float));
        memcpy(dst->s, t->scale_inv, ns * sizeof(float));
    }
    return 0;
}

/* Vectors (and the router matrix) are widened to FP32 as the reference's bind does
 * (src/model/glm53f_bind.c:130-133,199). */
static int keep_vec(float **dst, const g5b_tensor *t, size_t n, const char *name)
{
    if ((size_t)t->rows * (size_t)t->cols != n) {
        fprintf(stderr, "oracle: %s has %zu values, expected %zu\n", name,
                (size_t)t->rows * (size_t)t->cols, n);
        return -1;
    }
    free(*dst);
    *dst = (float *)malloc(n * sizeof(float));
    if (t->dtype == G5B_DT_F32) memcpy(*dst, t->data, n * sizeof(float));
    else if (t->dtype == G5B_DT_BF16)
        for (size_t i = 0; i < n; i++) (*dst)[i] = bf16f(((const uint16_t *)t->data)[i]);
    else { fprintf(stderr, "oracle: %s must be a float vector\n", name); return -1; }
    return 0;
}

orc_model *orc_model_create(const g5b_config *cfg, const uint8_t *is_mla,
                            const uint8_t *is_dense, int cap, int kv_mode)
{
    build_e4m3();
    orc_model *m = (orc_model *)calloc(1, sizeof *m);
    m->c = *cfg;
    m->cap = cap < 1 ? 1 : cap;
    const int dense_limit = cfg->index_topk + cfg->index_kpool - 1;
    m->latent = kv_mode == 2 || (kv_mode == 0 && m->cap > dense_limit);
    m->L = (OLayer *)calloc((size_t)cfg->n_layers, sizeof *m->L);
    for (int l = 0; l < cfg->n_layers; l++) {
        m->L[l].is_mla = is_mla[l];
        m->L[l].is_dense = is_dense[l];
        if (!is_dense[l]) m->L[l].experts = (OMat *)calloc((size_t)cfg->n_experts * 3, sizeof(OMat));
    }
    return m;
}

/* Adds checkpoint layer n_layers, the multi-token-prediction layer: an MLA + MoE layer of the
 * model's shapes without mHC mixers, two input norms, the projection of [norm(embedding),
 * norm(hidden)] and the norm before the shared lm_head (plan_mtp, src/model/glm53f_bind.c:208-249).
 * Call before loading. */
int orc_model_enable_mtp(orc_model *m)
{
    if (m->finalized || m->mtp) return -1;
    const int n = m->c.n_layers;
    m->L = (OLayer *)realloc(m->L, (size_t)(n + 1) * sizeof *m->L);
    memset(&m->L[n], 0, sizeof m->L[n]);
    m->L[n].is_mla = 1;
    m->L[n].is_dense = 0;
    m->L[n].experts = (OMat *)calloc((size_t)m->c.n_experts * 3, sizeof(OMat));
    m->mtp = 1;
    return 0;
}

int orc_model_load(orc_model *m, const char *name, const g5b_tensor *t)
{
    const g5b_config *c = &m->c;
    const int E = c->hidden, M = c->hc_mult, MIX = (2 + M) * M;
    if (!strcmp(name, "embed_tokens.weight")) return keep_mat(&m->embed, t, c, c->vocab, E, name);
    if (!strcmp(name, "lm_head.weight"))      return keep_mat(&m->lm_head, t, c, c->vocab, E, name);
    if (!strcmp(name, "norm.weight"))         return keep_vec(&m->norm, t, (size_t)E, name);
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= n_slots(m)) {
        fprintf(stderr, "oracle: unknown tensor %s\n", name);
        return -1;
    }
    const char *r = name + used;
    OLayer *w = &m->L[l];
    if (l == c->n_layers) {
        if (!strcmp(r, "enorm.weight")) return keep_vec(&m->enorm, t, (size_t)E, name);
        if (!strcmp(r, "hnorm.weight")) return keep_vec(&m->hnorm, t, (size_t)E, name);
        if (!strcmp(r, "shared_head.norm.weight")) return keep_vec(&m->head_norm, t, (size_t)E, name);
        if (!strcmp(r, "eh_proj.weight")) return keep_mat(&m->eh, t, c, E, 2 * E, name);
    }
    const int H = c->kda_heads, D = c->kda_head_dim, P = H * D;
    const int MH = c->mla_heads, IH = c->index_heads, ID = c->index_dim;
    const int SI = c->moe_inter * c->n_shared;
#define MAT(nm, field, R, C) if (!strcmp(r, nm)) return keep_mat(&w->field, t, c, R, C, name)
#define VEC(nm, field, N)    if (!strcmp(r, nm)) return keep_vec(&w->field, t, (size_t)(N), name)
    VEC("input_layernorm.weight", in_norm, E);
    VEC("post_attention_layernorm.weight", post_norm, E);
    MAT("hc_attn_fn", hc[0].fn, MIX, M * E);  VEC("hc_attn_base", hc[0].base, MIX);  VEC("hc_attn_scale", hc[0].scale, 3);
    MAT("hc_ffn_fn", hc[1].fn, MIX, M * E);   VEC("hc_ffn_base", hc[1].base, MIX);   VEC("hc_ffn_scale", hc[1].scale, 3);
    if (w->is_mla) {
        MAT("self_attn.q_a_proj.weight", q_a, c->q_lora, E);
        VEC("self_attn.q_a_layernorm.weight", q_a_norm, c->q_lora);
        MAT("self_attn.q_b_proj.weight", q_b, MH * c->qk_nope, c->q_lora);
        MAT("self_attn.kv_a_proj_with_mqa.weight", kv_a, c->kv_lora, E);
        VEC("self_attn.kv_a_layernorm.weight", kv_a_norm, c->kv_lora);
        MAT("self_attn.kv_b_proj.weight", kv_b, MH * (c->qk_nope + c->v_head), c->kv_lora);
        MAT("self_attn.o_proj.weight", mo, E, MH * c->v_head);
        MAT("self_attn.indexer.wq_b.weight", wq_b, IH * ID, c->q_lora);
        MAT("self_attn.indexer.wk.weight", wk, ID, E);
        VEC("self_attn.indexer.k_norm.weight", k_norm_w, ID);
        VEC("self_attn.indexer.k_norm.bias", k_norm_b, ID);
        MAT("self_attn.indexer.weights_proj.weight", wproj, IH, E);
        MAT("self_attn.indexer.index_kpool_compress_gate", igate, ID, E);
        VEC("self_attn.indexer.index_kpool_compress_ape", ape, c->index_kpool * ID);
    } else {
        MAT("self_attn.q_proj.weight", kq, P, E);
        MAT("self_attn.k_proj.weight", kk, P, E);
        MAT("self_attn.v_proj.weight", kv, P, E);
        VEC("self_attn.q_conv1d.weight", q_conv, P * c->conv_k);
        VEC("self_attn.k_conv1d.weight", k_conv, P * c->conv_k);
        VEC("self_attn.v_conv1d.weight", v_conv, P * c->conv_k);
        MAT("self_attn.f_a_proj.weight", f_a, D, E);
        MAT("self_attn.f_b_proj.weight", f_b, P, D);
        VEC("self_attn.A_log", A_log, H);
        VEC("self_attn.dt_bias", dt_bias, P);
        MAT("self_attn.b_proj.weight", kb, H, E);
        MAT("self_attn.g_a_proj.weight", g_a, D, E);
        MAT("self_attn.g_b_proj.weight", g_b, P, D);
        VEC("self_attn.o_norm.weight", o_norm, D);
        MAT("self_attn.o_proj.weight", ko, E, P);
    }
    if (w->is_dense) {
        MAT("mlp.gate_proj.weight", d_gate, c->dense_inter, E);
        MAT("mlp.up_proj.weight", d_up, c->dense_inter, E);
        MAT("mlp.down_proj.weight", d_down, E, c->dense_inter);
    } else {
        VEC("mlp.gate.weight", router, (size_t)c->n_experts * E);
        VEC("mlp.gate.e_score_correction_bias", bias, c->n_experts);
        MAT("mlp.shared_experts.gate_proj.weight", sh_gate, SI, E);
        MAT("mlp.shared_experts.up_proj.weight", sh_up, SI, E);
        MAT("mlp.shared_experts.down_proj.weight", sh_down, E, SI);
        int ex = -1, n2 = 0;
        if (sscanf(r, "mlp.experts.%d.%n", &ex, &n2) == 1 && ex >= 0 && ex < c->n_experts) {
            const char *p = r + n2;
            OMat *q = w->experts + (size_t)ex * 3;
            if (!strcmp(p, "gate_proj.weight")) return keep_mat(&q[0], t, c, c->moe_inter, E, name);
            if (!strcmp(p, "up_proj.weight"))   return keep_mat(&q[1], t, c, c->moe_inter, E, name);
            if (!strcmp(p, "down_proj.weight")) return keep_mat(&q[2], t, c, E, c->moe_inter, name);
        }
    }
#undef MAT
#undef VEC
    fprintf(stderr, "oracle: tensor %s does not belong to layer %d of this config\n", name, l);
    return -1;
}

static size_t kda_floats(const g5b_config *c)
{
    const size_t P = (size_t)c->kda_heads * c->kda_head_dim;
    return P * c->kda_head_dim + 3 * P * (size_t)(c->conv_k - 1);
}

/* Session state as glm53f_model_open allocates it (glm53f_model.c:194-228). */
int orc_model_finalize(orc_model *m)
{
    const g5b_config *c = &m->c;
    if (m->mtp) m->mtp_h = (float *)calloc((size_t)m->cap * c->hidden, sizeof(float));
    for (int l = 0; l < n_slots(m); l++) {
        OLayer *w = &m->L[l];
        if (w->is_mla) {
            const size_t per = m->latent ? (size_t)c->kv_lora
                                         : (size_t)c->mla_heads * (c->qk_nope + c->v_head);
            float *kv = (float *)calloc((size_t)m->cap * per, sizeof(float));
            if (m->latent) w->ckv = kv; else w->kvc = kv;
            w->idx = (float *)calloc(dsa_floats(c, m->cap), sizeof(float));
        } else {
            w->kda_state = (float *)calloc(kda_floats(c), sizeof(float));
        }
    }
    m->finalized = 1;
    return 0;
}

void orc_model_reset(orc_model *m)
{
    for (int l = 0; l < m->c.n_layers; l++)
        if (m->L[l].kda_state) memset(m->L[l].kda_state, 0, kda_floats(&m->c) * sizeof(float));
    m->cached = 0;
    m->mtp_cached = 0;
}

int orc_model_cached(const orc_model *m) { return m->cached; }

/* forward_cpu, glm53f_model.c:410-479: embedding row copied into every stream, layers in
 * order, then per position the FP64 mean of the streams, final RMSNorm, lm_head, first-max
 * argmax (:361-366). Chunking in the reference does not change any sum. */
int orc_model_forward(orc_model *m, const int *ids, int T, float *logits, int *argmax_all)
{
    const g5b_config *c = &m->c;
    const int E = c->hidden, M = c->hc_mult;
    if (!m->finalized || T < 1 || m->cached + T > m->cap) return -1;
    for (int t = 0; t < T; t++) if (ids[t] < 0 || ids[t] >= c->vocab) return -1;
    float *h = (float *)malloc((size_t)T * M * E * sizeof(float));
    for (int t = 0; t < T; t++) {
        float *ht = h + (size_t)t * M * E;
        for (int i = 0; i < E; i++)
            ht[i] = m->embed.dt == G5B_DT_BF16
                  ? bf16f(((const uint16_t *)m->embed.w)[(size_t)ids[t] * E + i])
                  : ((const float *)m->embed.w)[(size_t)ids[t] * E + i];
        for (int s = 1; s < M; s++) memcpy(ht + (size_t)s * E, ht, (size_t)E * sizeof(float));
    }
    int rc = 0;
    for (int l = 0; l < c->n_layers && rc == 0; l++) rc = decoder_layer(m, l, h, T, m->cached);
    if (rc == 0) {
        float *xm = (float *)malloc(((size_t)2 * E + c->vocab) * sizeof(float));
        float *lg = xm + 2 * E;
        /* with the MTP layer open every position's mean is computed and kept (glm53f_model.c:460-468) */
        for (int t = (argmax_all || m->mtp_h) ? 0 : T - 1; t < T; t++) {
            const float *ht = h + (size_t)t * M * E;
            for (int d = 0; d < E; d++) {
                double s = 0.0;
                for (int i = 0; i < M; i++) s += (double)ht[(size_t)i * E + d];
                xm[d] = (float)(s / M);
            }
            if (m->mtp_h) memcpy(m->mtp_h + (size_t)t * E, xm, (size_t)E * sizeof(float));
            if (!argmax_all && t < T - 1) continue;
            rmsnorm(xm + E, xm, m->norm, E, c->rms_eps);
            mv(lg, xm + E, &m->lm_head);
            if (argmax_all) {
                int b = 0;
                for (int i = 1; i < c->vocab; i++) if (lg[i] > lg[b]) b = i;
                argmax_all[t] = b;
            }
        }
        if (logits) memcpy(logits, lg, (size_t)c->vocab * sizeof(float));
        free(xm);
        m->cached += T;
    }
    free(h);
    return rc;
}

/* glm53f_mtp_feed, src/model/glm53f_mtp.c:100-144. h: T hidden states (means of the streams,
 * before the final norm; NULL = the rows the last forward call kept), next_ids[t]: the token that
 * follows position t. x = eh_proj([RMSNorm(embed(next), enorm), RMSNorm(h, hnorm)]), then a plain
 * pre-norm residual MLA + MoE layer on the MTP layer's own caches at its own position count, and for
 * the last position the draft = first-max arg-max of lm_head(RMSNorm(x, shared_head.norm)).
 * x_out (may be NULL) receives the T rows of x after the layer. */
int orc_mtp_feed(orc_model *m, const float *h, const int *next_ids, int T, int *draft, float *x_out)
{
    const g5b_config *c = &m->c;
    const int E = c->hidden;
    if (!m->mtp || !m->finalized || T < 1 || m->mtp_cached + T > m->cap) return -1;
    if (!m->enorm || !m->hnorm || !m->head_norm || !m->eh.w) return -1;
    if (!h) h = m->mtp_h;
    OLayer *w = &m->L[c->n_layers];
    float *x = (float *)malloc((size_t)T * E * 4 * sizeof(float));
    float *y = x + (size_t)T * E, *cat = y + (size_t)T * E;        /* cat: [T][2E] */
    for (int i = 0; i < T; i++) {
        if (next_ids[i] < 0 || next_ids[i] >= c->vocab) { free(x); return -1; }
        float *ci = cat + (size_t)i * 2 * E;
        for (int d = 0; d < E; d++)
            ci[d] = m->embed.dt == G5B_DT_BF16
                  ? bf16f(((const uint16_t *)m->embed.w)[(size_t)next_ids[i] * E + d])
                  : ((const float *)m->embed.w)[(size_t)next_ids[i] * E + d];
        rmsnorm(ci, ci, m->enorm, E, c->rms_eps);
        rmsnorm(ci + E, h + (size_t)i * E, m->hnorm, E, c->rms_eps);
        mv(x + (size_t)i * E, ci, &m->eh);
    }
    for (int i = 0; i < T; i++) rmsnorm(y + (size_t)i * E, x + (size_t)i * E, w->in_norm, E, c->rms_eps);
    mla(cat, y, w, c, T, w->kvc, m->mtp_cached, m->cap, w->idx, w->ckv, NULL, NULL);
    for (size_t i = 0; i < (size_t)T * E; i++) x[i] += cat[i];
    for (int i = 0; i < T; i++) rmsnorm(y + (size_t)i * E, x + (size_t)i * E, w->post_norm, E, c->rms_eps);
    const int rc = moe(cat, y, w, c, T, 1);
    for (size_t i = 0; i < (size_t)T * E; i++) x[i] += cat[i];
    m->mtp_cached += T;
    if (rc == 0 && draft) {
        float *lg = (float *)malloc((size_t)c->vocab * sizeof(float));
        rmsnorm(y, x + (size_t)(T - 1) * E, m->head_norm, E, c->rms_eps);
        mv(lg, y, &m->lm_head);
        int b = 0;
        for (int i = 1; i < c->vocab; i++) if (lg[i] > lg[b]) b = i;
        *draft = b;
        free(lg);
    }
    if (x_out) memcpy(x_out, x, (size_t)T * E * sizeof(float));
    free(x);
    return rc;
}

/* The hidden states (means of the streams) the last forward call kept: T rows from row `first`. */
int orc_mtp_hidden(const orc_model *m, int first, int T, float *dst)
{
    if (!m->mtp_h || first < 0 || first + T > m->cap) return -1;
    memcpy(dst, m->mtp_h + (size_t)first * m->c.hidden, (size_t)T * m->c.hidden * sizeof(float));
    return 0;
}

static void drop_mat(OMat *m) { free(m->w); free(m->s); }

void orc_model_free(orc_model *m)
{
    if (!m) return;
    for (int l = 0; l < n_slots(m); l++) {
        OLayer *w = &m->L[l];
        OMat *mats[] = { &w->hc[0].fn, &w->hc[1].fn, &w->kq, &w->kk, &w->kv, &w->f_a, &w->f_b, &w->kb,
                         &w->g_a, &w->g_b, &w->ko, &w->q_a, &w->q_b, &w->kv_a, &w->kv_b, &w->mo,
                         &w->wq_b, &w->wk, &w->wproj, &w->igate, &w->d_gate, &w->d_up, &w->d_down,
                         &w->sh_gate, &w->sh_up, &w->sh_down };
        for (size_t i = 0; i < sizeof mats / sizeof *mats; i++) drop_mat(mats[i]);
        float *vecs[] = { w->hc[0].base, w->hc[0].scale, w->hc[1].base, w->hc[1].scale, w->in_norm,
                          w->post_norm, w->q_conv, w->k_conv, w->v_conv, w->A_log, w->dt_bias,
                          w->o_norm, w->q_a_norm, w->kv_a_norm, w->k_norm_w, w->k_norm_b, w->ape,
                          w->router, w->bias, w->kda_state, w->kvc, w->ckv, w->idx };
        for (size_t i = 0; i < sizeof vecs / sizeof *vecs; i++) free(vecs[i]);
        if (w->experts) {
            for (int e = 0; e < m->c.n_experts * 3; e++) drop_mat(&w->experts[e]);
            free(w->experts);
        }
    }
    drop_mat(&m->embed); drop_mat(&m->lm_head); drop_mat(&m->eh);
    free(m->enorm); free(m->hnorm); free(m->head_norm); free(m->mtp_h);
    free(m->norm); free(m->L); free(m);
}

/* ----------------------------------------------------------------- op entries ---- */
int orc_matvec_host(const g5b_tensor *w, int br, int bc, const float *x, int T, float *y)
{
    build_e4m3();
    OMat m;
    memset(&m, 0, sizeof m);
    m.w = (void *)w->data; m.s = (float *)w->scale_inv; m.dt = w->dtype;
    m.rows = w->rows; m.cols = w->cols; m.br = br; m.bc = bc;
    m.scols = bc > 0 ? (w->cols + bc - 1) / bc : 0;
    for (int t = 0; t < T; t++) mv(y + (size_t)t * m.rows, x + (size_t)t * m.cols, &m);
    return 0;
}

int orc_rmsnorm_host(float *y, const float *x, const float *w, int n, int rows, float eps)
{
    for (int r = 0; r < rows; r++) rmsnorm(y + (size_t)r * n, x + (size_t)r * n, w, n, eps);
    return 0;
}

int orc_swiglu_host(float *y, const float *gu, int n, int rows, float limit)
{
    for (int r = 0; r < rows; r++) swiglu(y + (size_t)r * n, gu + (size_t)r * 2 * n, n, limit);
    return 0;
}

int orc_shortconv_host(float *y, const float *x, const float *w, float *state, int channels,
                       int k, int T)
{
    if (k - 1 > 16) return -1;
    shortconv(y, x, w, state, channels, k, T);
    return 0;
}

static OMat *find_mat(orc_model *m, const char *name)
{
    if (!strcmp(name, "embed_tokens.weight")) return &m->embed;
    if (!strcmp(name, "lm_head.weight")) return &m->lm_head;
    int l = -1, used = 0;
    if (sscanf(name, "layers.%d.%n", &l, &used) != 1 || l < 0 || l >= m->c.n_layers) return NULL;
    const char *r = name + used;
    OLayer *w = &m->L[l];
    struct { const char *n; OMat *p; } tab[] = {
        { "hc_attn_fn", &w->hc[0].fn }, { "hc_ffn_fn", &w->hc[1].fn },
        { "self_attn.q_proj.weight", &w->kq }, { "self_attn.k_proj.weight", &w->kk },
        { "self_attn.v_proj.weight", &w->kv }, { "self_attn.f_a_proj.weight", &w->f_a },
        { "self_attn.f_b_proj.weight", &w->f_b }, { "self_attn.b_proj.weight", &w->kb },
        { "self_attn.g_a_proj.weight", &w->g_a }, { "self_attn.g_b_proj.weight", &w->g_b },
        { "self_attn.o_proj.weight", w->is_mla ? &w->mo : &w->ko },
        { "self_attn.q_a_proj.weight", &w->q_a }, { "self_attn.q_b_proj.weight", &w->q_b },
        { "self_attn.kv_a_proj_with_mqa.weight", &w->kv_a }, { "self_attn.kv_b_proj.weight", &w->kv_b },
        { "self_attn.indexer.wq_b.weight", &w->wq_b }, { "self_attn.indexer.wk.weight", &w->wk },
        { "self_attn.indexer.weights_proj.weight", &w->wproj },
        { "self_attn.indexer.index_kpool_compress_gate", &w->igate },
        { "mlp.gate_proj.weight", &w->d_gate }, { "mlp.up_proj.weight", &w->d_up },
        { "mlp.down_proj.weight", &w->d_down },
        { "mlp.shared_experts.gate_proj.weight", &w->sh_gate },
        { "mlp.shared_experts.up_proj.weight", &w->sh_up },
        { "mlp.shared_experts.down_proj.weight", &w->sh_down },
    };
    for (size_t i = 0; i < sizeof tab / sizeof *tab; i++)
        if (!strcmp(r, tab[i].n)) return tab[i].p->w ? tab[i].p : NULL;
    int ex = -1, n2 = 0;
    if (w->experts && sscanf(r, "mlp.experts.%d.%n", &ex, &n2) == 1 && ex >= 0 && ex < m->c.n_experts) {
        const char *p = r + n2;
        OMat *q = w->experts + (size_t)ex * 3;
        const int which = !strcmp(p, "gate_proj.weight") ? 0 : !strcmp(p, "up_proj.weight") ? 1
                        : !strcmp(p, "down_proj.weight") ? 2 : -1;
        if (which >= 0 && q[which].w) return &q[which];
    }
    return NULL;
}

int orc_op_matvec(orc_model *m, const char *name, const float *x, int T, float *y)
{
    OMat *mat = find_mat(m, name);
    if (!mat) return -1;
    for (int t = 0; t < T; t++) mv(y + (size_t)t * mat->rows, x + (size_t)t * mat->cols, mat);
    return 0;
}

int orc_op_hc_pre(orc_model *m, int layer, int site, const float *h, int T, float *x,
                  float *post, float *comb)
{
    const size_t E = (size_t)m->c.hidden, M = (size_t)m->c.hc_mult;
    for (int t = 0; t < T; t++)
        hc_pre(x + t * E, post + t * M, comb + t * M * M, h + t * M * E, &m->L[layer].hc[site], &m->c);
    return 0;
}

int orc_op_hc_post(orc_model *m, float *h, const float *y, const float *post,
                   const float *comb, int T)
{
    const size_t E = (size_t)m->c.hidden, M = (size_t)m->c.hc_mult;
    for (int t = 0; t < T; t++)
        hc_post(h + t * M * E, y + t * E, post + t * M, comb + t * M * M, &m->c);
    return 0;
}

int orc_op_kda(orc_model *m, int layer, const float *x, int T, float *out)
{
    if (m->L[layer].is_mla || !m->L[layer].kda_state) return -1;
    kda_layer(out, x, &m->L[layer], &m->c, T, m->L[layer].kda_state);
    return 0;
}

int orc_op_mla(orc_model *m, int layer, const float *x, int T, int cached, float *out,
               int *sel_out, int *n_sel_out)
{
    OLayer *w = &m->L[layer];
    if (!w->is_mla || !w->idx || cached + T > m->cap) return -1;
    mla(out, x, w, &m->c, T, w->kvc, cached, m->cap, w->idx, w->ckv, sel_out, n_sel_out);
    return 0;
}

int orc_op_router(orc_model *m, int layer, const float *x, int T, int *idx, float *w)
{
    for (int t = 0; t < T; t++)
        if (router(idx + (size_t)t * m->c.topk, w + (size_t)t * m->c.topk,
                   x + (size_t)t * m->c.hidden, &m->L[layer], &m->c) != 0) return -1;
    return 0;
}

int orc_op_moe(orc_model *m, int layer, const float *x, int T, float *out, int with_shared)
{
    if (m->L[layer].is_dense) return -1;
    return moe(out, x, &m->L[layer], &m->c, T, with_shared);
}

int orc_op_mlp(orc_model *m, int layer, const float *x, int T, float *out)
{
    OLayer *w = &m->L[layer];
    if (!w->is_dense) return -1;
    for (int t = 0; t < T; t++)
        mlp(out + (size_t)t * m->c.hidden, x + (size_t)t * m->c.hidden, &w->d_gate, &w->d_up,
            &w->d_down, m->c.swiglu_limit);
    return 0;
}

int orc_op_decoder_layer(orc_model *m, int layer, float *h, int T, int cached)
{
    return decoder_layer(m, layer, h, T, cached);
}

static float *state_ptr(orc_model *m, int layer, int kind, size_t *n)
{
    OLayer *w = &m->L[layer];
    if (kind == 0) { *n = kda_floats(&m->c); return w->kda_state; }
    if (kind == 1) { *n = (size_t)m->cap * m->c.kv_lora; return w->ckv; }
    if (kind == 2) { *n = dsa_floats(&m->c, m->cap); return w->idx; }
    return NULL;
}

int orc_state_write(orc_model *m, int layer, int kind, size_t offset, const float *src, size_t count)
{
    size_t n = 0;
    float *p = state_ptr(m, layer, kind, &n);
    if (!p || offset + count > n) return -1;
    memcpy(p + offset, src, count * sizeof(float));
    return 0;
}

int orc_state_read(orc_model *m, int layer, int kind, size_t offset, float *dst, size_t count)
{
    size_t n = 0;
    float *p = state_ptr(m, layer, kind, &n);
    if (!p || offset + count > n) return -1;
    memcpy(dst, p + offset, count * sizeof(float));
    return 0;
}

/* ------------------------------------------------------- synthetic experts ---- */
/* Counter-based generator shared with the engine's device fill: a 64-bit mix of the stream
 * key and the index of a group of four codes gives four 16-bit draws; each is scaled to
 * 0..253 and mapped past 0x7f, so the 254 finite E4M3 codes are (near) equally likely and
 * NaN codes never appear. */
static uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* The generators of g5b_engine_fill_matrix, restated: key = mix64(seed ^ mix64(FNV-1a(name))). */
static uint64_t synth_key(uint64_t seed, const char *name)
{
    uint64_t h = 0xcbf29ce484222325ull;
    for (const unsigned char *p = (const unsigned char *)name; *p; p++) { h ^= *p; h *= 0x100000001b3ull; }
    return mix64(seed ^ mix64(h));
}

void orc_synth_matrix_codes(uint8_t *dst, uint64_t seed, const char *name, size_t count)
{
    const uint64_t key = synth_key(seed, name);
    for (size_t g = 0; g * 4 < count; g++) {
        const uint64_t h = mix64(key + g);
        for (int j = 0; j < 4 && g * 4 + j < count; j++) {
            const uint32_t v = (uint32_t)(((h >> (16 * j)) & 0xffffu) * 254u) >> 16;
            dst[g * 4 + j] = (uint8_t)(v + (v >= 127u));
        }
    }
}

void orc_synth_matrix_bf16(uint16_t *dst, uint64_t seed, const char *name, float mul, size_t count)
{
    const uint64_t key = synth_key(seed, name);
    for (size_t i = 0; i < count; i++) {
        const uint64_t h = mix64(key + i);
        const int c = (int)((h & 0xffffu) + ((h >> 16) & 0xffffu) + ((h >> 32) & 0xffffu) + (h >> 48)) - 131070;
        const float v = (float)c * mul;
        uint32_t u;
        memcpy(&u, &v, 4);
        u += 0x7fffu + ((u >> 16) & 1u);               /* round to nearest even; values are finite */
        dst[i] = (uint16_t)(u >> 16);
    }
}

void orc_synth_codes(uint8_t *dst, uint64_t seed, int layer, int expert, int which, size_t count)
{
    const uint64_t key = mix64(seed ^ mix64(((uint64_t)layer << 40) ^ ((uint64_t)expert << 8) ^ (uint64_t)which));
    for (size_t g = 0; g * 4 < count; g++) {
        const uint64_t h = mix64(key + g);
        for (int j = 0; j < 4 && g * 4 + j < count; j++) {
            const uint32_t v = (uint32_t)(((h >> (16 * j)) & 0xffffu) * 254u) >> 16;
            dst[g * 4 + j] = (uint8_t)(v + (v >= 127u));
        }
    }
}
