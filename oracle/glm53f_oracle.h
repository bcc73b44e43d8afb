/*
 * glm53f_oracle.h - CPU restatement of the reference's per-token forward pass.
 *
 * TEST INFRASTRUCTURE ONLY. This is the checker the GPU engine is compared against; nothing
 * in the product library links, loads or calls it. It restates, in plain scalar C, the
 * arithmetic of josesilva05/glm-5.3-flash-in-c's numeric core (src/core/glm53f_ops.c,
 * src/core/glm53f_dsa.c) and of its model driver's forward loop (src/model/glm53f_model.c:
 * 410-479), keeping the order of every floating-point sum, so that on the same inputs it
 * reproduces the reference bit for bit. Each function names the reference lines it follows.
 *
 * Parity pins: (1) the reference's golden vectors produced by the transformers
 * implementation (tests/fixtures/glm_tiny/ref.json, gates of tests/unit/test_glm_tiny.c:
 * 77-136), (2) the known-answer shapes of tests/unit/test_fp8.c:153-157, (3) bit-equality
 * with the reference itself wherever the reference objects were built beside this file.
 *
 * The entry points have the same shape as the engine's layer ops (include/glm53f_b200.h)
 * so one test body can drive either.
 */
#ifndef GLM53F_ORACLE_H
#define GLM53F_ORACLE_H

#include "glm53f_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct orc_model orc_model;

/* kv_mode: 0 = the reference's choice (latent cache when cap exceeds the dense-attention
 * limit, expanded keys/values below it: glm53f_model.c:138,201), 1 = expanded, 2 = latent. */
orc_model *orc_model_create(const g5b_config *cfg, const uint8_t *is_mla,
                            const uint8_t *is_dense, int cap, int kv_mode);
int  orc_model_load(orc_model *m, const char *name, const g5b_tensor *t);  /* copies */
int  orc_model_finalize(orc_model *m);
int  orc_model_forward(orc_model *m, const int *ids, int T, float *logits, int *argmax_all);
void orc_model_reset(orc_model *m);
void orc_model_free(orc_model *m);
int  orc_model_cached(const orc_model *m);
/* The multi-token-prediction layer (src/model/glm53f_mtp.c): enable before loading "layers.<n_layers>.*". */
int  orc_model_enable_mtp(orc_model *m);
int  orc_mtp_feed(orc_model *m, const float *h, const int *next_ids, int T, int *draft, float *x_out);
int  orc_mtp_hidden(const orc_model *m, int first, int T, float *dst);

int orc_matvec_host(const g5b_tensor *w, int br, int bc, const float *x, int T, float *y);
int orc_rmsnorm_host(float *y, const float *x, const float *w, int n, int rows, float eps);
int orc_swiglu_host(float *y, const float *gu, int n, int rows, float limit);
int orc_shortconv_host(float *y, const float *x, const float *w, float *state, int channels,
                       int k, int T);

int orc_op_matvec(orc_model *m, const char *name, const float *x, int T, float *y);
int orc_op_hc_pre(orc_model *m, int layer, int site, const float *h, int T, float *x,
                  float *post, float *comb);
int orc_op_hc_post(orc_model *m, float *h, const float *y, const float *post,
                   const float *comb, int T);
int orc_op_kda(orc_model *m, int layer, const float *x, int T, float *out);
int orc_op_mla(orc_model *m, int layer, const float *x, int T, int cached, float *out,
               int *sel_out, int *n_sel_out);
int orc_op_router(orc_model *m, int layer, const float *x, int T, int *idx, float *w);
int orc_op_moe(orc_model *m, int layer, const float *x, int T, float *out, int with_shared);
int orc_op_mlp(orc_model *m, int layer, const float *x, int T, float *out);
int orc_op_decoder_layer(orc_model *m, int layer, float *h, int T, int cached);
int orc_state_write(orc_model *m, int layer, int kind, size_t offset, const float *src,
                    size_t count);
int orc_state_read(orc_model *m, int layer, int kind, size_t offset, float *dst,
                   size_t count);

/* The synthetic expert generator of g5b_engine_fill_expert, on the CPU: writes rows*cols
 * E4M3 codes of matrix `which` (0 gate, 1 up, 2 down) of (layer, expert). */
void orc_synth_codes(uint8_t *dst, uint64_t seed, int layer, int expert, int which,
                     size_t count);

/* The named-matrix generators of g5b_engine_fill_matrix, on the CPU. */
void orc_synth_matrix_codes(uint8_t *dst, uint64_t seed, const char *name, size_t count);
void orc_synth_matrix_bf16(uint16_t *dst, uint64_t seed, const char *name, float mul, size_t count);

#ifdef __cplusplus
}
#endif

#endif
