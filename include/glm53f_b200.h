/*
 * glm53f_b200.h - C ABI of the B200 decode engine for the GLM-5.3-Flash architecture.
 *
 * The library behind this header (libglm53f_b200.so) is hand-written CUDA for sm_100a. It
 * replaces one path of josesilva05/glm-5.3-flash-in-c: the per-token forward pass that its
 * model driver hands to a backend (src/model/glm53f_model.c:382-384) and the numeric ops
 * that pass is made of (include/glm53f/glm53f.h:136-360). Nothing here takes or returns a
 * torch type; every argument is a plain pointer, size or handle.
 *
 * Three groups of entry points:
 *
 *   1. ENGINE      create / load / finalize / forward / reset / free. This is the contract
 *                  of the reference backend ABI (src/gpu/glm53f_gpu.h:38-50) with the
 *                  reference's opaque `struct Glm53fModel *` argument replaced by a flat
 *                  config plus tensors loaded by checkpoint name (the name table of
 *                  src/model/glm53f_bind.c:139-206,311-317 and src/io/glm53f_load.c:11).
 *   2. LAYER OPS   one entry point per op function of the reference, host buffers in and
 *                  out, running on the loaded layer's weights and the engine's session
 *                  state. These are what the parity tests and the benchmark call.
 *   3. DEVICE OPS  the same hot ops with device pointers and no copies, for callers that
 *                  already hold activations in HBM (the reference's gk_* launcher layer,
 *                  src/gpu/glm53f_gpu_kernels.h:18-93).
 *
 * Error convention (reference: glm53f_model.h:61-64, glm53f_gpu_kernels.cu:668-686): every
 * int function returns 0 on success and -1 on failure; on failure outputs are untouched or
 * undefined, a message is kept for g5b_last_error(), and nothing falls back to a CPU
 * implementation. The library has no CPU compute path at all.
 *
 * Threading: one caller thread per engine, like the reference model (not re-entrant).
 */
#ifndef GLM53F_B200_H
#define GLM53F_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Storage formats of a weight matrix (reference: enum at glm53f.h:122; int4 is an
 * approximation format of the reference's SSD cache and is not part of this engine). */
#define G5B_DT_F32  0
#define G5B_DT_BF16 1
#define G5B_DT_FP8  2   /* E4M3FN codes + FP32 block scales ("weight_scale_inv") */

/* Engine limits (reference: glm53f.h:42-45,377; glm53f_cfg.h:259-283). */
#define G5B_MAX_LAYERS    256
#define G5B_MAX_TOPK      64
#define G5B_MAX_HC        8
#define G5B_MAX_EXPERTS   1024
#define G5B_MAX_POSITIONS 32768

/* Model shape. Field for field the information of the reference's Glm53fCfg
 * (glm53f.h:48-95) without its layer-type arrays, which are passed beside it. */
typedef struct g5b_config {
    int32_t hidden, n_layers, vocab;
    float   rms_eps;
    int32_t hc_mult, hc_iters;           /* mHC residual streams, Sinkhorn iterations */
    float   hc_eps;
    int32_t kda_heads, kda_head_dim, conv_k;
    float   gate_lb;                      /* KDA gate lower bound (-5) */
    int32_t mla_heads, q_lora, kv_lora, qk_nope, v_head;
    int32_t index_topk, index_kpool, index_heads, index_dim;
    int32_t n_experts, topk, n_shared, moe_inter, dense_inter;
    float   routed_scale;
    int32_t norm_topk;
    float   swiglu_limit;
    int32_t fp8_block_r, fp8_block_c;     /* 128 x 128 in the released checkpoint */
} g5b_config;

/* One tensor handed to a loader. FP8 tensors carry their scale grid
 * [ceil(rows/fp8_block_r)][ceil(cols/fp8_block_c)] in scale_inv. Vectors use rows = n,
 * cols = 1. `on_device` != 0 means data/scale_inv already live in the engine GPU's memory
 * (the engine copies them device to device into its own layout). */
typedef struct g5b_tensor {
    const void  *data;
    const float *scale_inv;
    int32_t      dtype, rows, cols, on_device;
} g5b_tensor;

typedef struct g5b_engine g5b_engine;

/* Message of the most recent failure on this thread ("" if none). */
const char *g5b_last_error(void);

/* ------------------------------------------------------------------- ENGINE ---- */

/* Number of CUDA devices; 0 if none. Replaces glm53f_gpu_device_count (glm53f_gpu.h:42). */
int g5b_device_count(void);

/* Create an engine on one GPU for `cap` positions per session. is_mla / is_dense hold
 * cfg->n_layers flags each (the reference's Glm53fCfg.is_mla / is_dense). Routed experts are
 * expert-parallel: this engine owns experts [ep_rank*n_experts/ep_size,
 * (ep_rank+1)*n_experts/ep_size) of every MoE layer and only those are accepted by
 * g5b_engine_load; the trunk is replicated. ep_size = 1 keeps everything on this GPU.
 * Replaces glm53f_gpu_create (glm53f_gpu.h:46), which placed whole layers on devices and left
 * routed experts on the CPU. Returns NULL on failure. */
g5b_engine *g5b_engine_create(const g5b_config *cfg, const uint8_t *is_mla,
                              const uint8_t *is_dense, int cap, int device,
                              int ep_rank, int ep_size);

/* Upload one checkpoint tensor by its name below "model.language_model." (for example
 * "layers.3.self_attn.q_a_proj.weight", "layers.3.mlp.experts.17.down_proj.weight",
 * "embed_tokens.weight", "norm.weight") or "lm_head.weight". Names, shapes and dtypes follow
 * glm53f_bind.c:139-206,311-317 and glm53f_load.c:11-63; a wrong shape or dtype is refused.
 * Replaces upload_layer (src/gpu/glm53f_gpu.c:662-708) and the SSD expert cache
 * (src/cache/glm53f_cache.c): every routed expert becomes HBM resident. An expert outside
 * this engine's expert-parallel range is ignored and reported as success. */
int g5b_engine_load(g5b_engine *e, const char *name, const g5b_tensor *t);

/* Stream a whole checkpoint directory (every *.safetensors file in it) into the engine: each tensor
 * of "model.language_model." (and "lm_head.weight") that this engine owns is read in pieces of at
 * most 32 MB by `threads` reader threads into pinned staging buffers and copied to its final place in
 * HBM; routed experts of other expert-parallel ranks and layers beyond the engine's are never read.
 * Names, shapes and dtypes are checked like g5b_engine_load's. Replaces the reference's load path
 * (src/io/glm53f_st.c, src/model/glm53f_bind.c:139-206,311-331, src/io/glm53f_load.c:15-99 and the
 * SSD expert cache they feed). Call g5b_engine_finalize afterwards. */
int g5b_engine_load_checkpoint(g5b_engine *e, const char *directory, int threads);
/* Lower level of the same: reserve a named matrix's place and get the device addresses to write
 * its bytes (and FP8 scale grid) to; NULL addresses with success for another rank's expert. */
int g5b_engine_reserve(g5b_engine *e, const char *name, int dtype, int rows, int cols, void **data_dev,
                       float **scale_dev);

/* Fill one routed expert of a MoE layer with synthetic weights generated on the GPU: E4M3
 * codes uniform over the 254 finite codes from a counter-based hash of (seed, layer, expert,
 * matrix, element index), so the CPU can regenerate any single expert bit for bit. Scale
 * grids (three, in gate/up/down order, host memory) are uploaded as given. */
int g5b_engine_fill_expert(g5b_engine *e, int layer, int expert, uint64_t seed,
                           const float *gate_s, const float *up_s, const float *down_s);

/* Fill one whole named matrix (any matrix g5b_engine_load accepts except a routed expert's) with
 * synthetic weights generated on the GPU from a hash of (seed, tensor name, element index), so that
 * no host copy of the weights ever exists and the CPU can still regenerate any single tensor bit
 * for bit: FP8 = E4M3 codes uniform over the 254 finite codes with the given scale grid (host
 * memory); BF16 = a bell-shaped distribution (sum of four uniform 16-bit fields, centred) times
 * `mul`, i.e. standard deviation 37837.2 * mul. This is how the full-size random-init model's
 * trunk is built without a checkpoint (no counterpart in the reference, which loads safetensors). */
int g5b_engine_fill_matrix(g5b_engine *e, const char *name, int dtype, uint64_t seed, float mul,
                           const float *scale_inv);

/* Benchmarks only: fill every sequence's session state with synthetic values on the GPU and set every
 * sequence's position to `positions`, standing in for prompts of that length (no counterpart in the
 * reference; the decode kernels do the work they would do after a real prefill of that depth). */
int g5b_engine_synth_session(g5b_engine *e, uint64_t seed, int positions);

/* Engine options, by name. "latent_bf16" (before finalize): keep the MLA latent cache in BF16
 * instead of FP32, half the bytes per position. "profile": record per-phase events in MoE ops.
 * "sequences" (before finalize), "ep_wait_ms", "ep_loopback": see below. "expert_path": which
 * batch-1 expert kernels run (0 register kernels, 1 tensor-core kernels as three launches, 2 the
 * whole layer as one kernel, the default); "allow_partial": finalize accepts missing tensors
 * (single-layer harnesses). "tensor_gemm" (default 1): matrices times 8..64 positions go through the
 * tcgen05 kernel instead of repeated one-token passes. "mla_tensor" (default 1): with the BF16
 * latent cache the attention core runs on the tensor cores. "tensor_split" (default 1; it cannot
 * change once a split layer has run): in a connected expert-parallel group every rank runs the KDA
 * layers for its own H / ep_size heads only and the ranks sum their partial output rows in rank
 * order; the kind-0 state keeps its full layout on every rank, but a rank advances only the
 * entries of its own heads [rank H / ep_size, (rank + 1) H / ep_size): g5b_state_read returns stale
 * values for the others, and a caller that wants the whole state takes each head from its rank. */
int g5b_engine_set_option(g5b_engine *e, const char *name, int value);

/* Check that every tensor the config implies has been loaded, then allocate the session
 * state (KDA recurrent + conv state, MLA latent cache, DSA indexer state) and work buffers. */
int g5b_engine_finalize(g5b_engine *e);

/* Feed T tokens after the positions already consumed. logits (vocab floats, may be NULL)
 * receives the last position's logits; argmax_all (T ints, may be NULL) the argmax at every
 * position. Same contract as glm53f_model_forward / glm53f_gpu_forward
 * (glm53f_model.h:59-64, glm53f_gpu.h:49-50). */
int g5b_engine_forward(g5b_engine *e, const int *ids, int T, float *logits, int *argmax_all);

/* A forward / decode call that fails after it began to advance the session (a launch error, a
 * device-side wait that ran out) leaves the KDA state, the caches and the position count out of
 * step with each other: the engine then refuses further forward / decode calls until
 * g5b_engine_reset (the reference: "session must be reset", glm53f_model.h:61-64).
 * Forget every carried position (glm53f_gpu_reset, glm53f_gpu.h:53). */
void g5b_engine_reset(g5b_engine *e);
void g5b_engine_free(g5b_engine *e);       /* glm53f_gpu_free, glm53f_gpu.h:47 */
int  g5b_engine_cached(const g5b_engine *e);  /* positions consumed so far */

/* Greedy decode on the device: feed `first` and generate n tokens without returning to the
 * host between steps (the reference's CLI loop, src/cli/glm53f_run.c:469-524, round-trips
 * logits to the host and takes the argmax there). out receives n token ids. */
int g5b_engine_decode_greedy(g5b_engine *e, int first, int n, int *out);

/* Sampled decode on the device (no counterpart in the reference, which is greedy only,
 * src/cli/glm53f_run.c:492-494): as g5b_engine_decode_greedy, but each token is drawn from the
 * step's logits: p = softmax(logits / temperature), truncated to the nucleus (every token at least
 * as probable as the least probable one needed to reach top_p of the mass; top_p >= 1 keeps all),
 * one draw per step from a counter-based generator of (seed, position), so a run is reproducible
 * and independent of how it is split into calls. temperature <= 0 decodes greedily. */
int g5b_engine_decode_sampled(g5b_engine *e, int first, int n, float temperature, float top_p,
                              uint64_t seed, int *out);
/* The sampler on its own: one draw from V host logits; `step` is the generator's counter. */
int g5b_sample_host(const float *logits, int V, float temperature, float top_p, uint64_t seed,
                    uint64_t step, int *token, int device);

/* Several independent sequences on one engine (no counterpart in the reference, which holds one
 * session per model, src/model/glm53f_model.h:53-75; the benchmark's batch-64 decode needs it).
 * Option "sequences" = S (g5b_engine_set_option before finalize, 1..64) gives every layer S copies
 * of its session state. g5b_engine_use_sequence picks the sequence that forward / decode_greedy /
 * the layer ops / g5b_state_* address (each sequence keeps its own position count), e.g. to
 * prefill S prompts one after the other. g5b_engine_decode_batch then advances all S sequences by
 * one token in a single pass: ids[s] continues sequence s, every weight is read once for the
 * batch, attention state and caches are per sequence. All sequences must hold the same number of
 * positions. logits: [S][vocab] or NULL, argmax: [S] or NULL. */
int g5b_engine_use_sequence(g5b_engine *e, int seq);
int g5b_engine_decode_batch(g5b_engine *e, const int *ids, float *logits, int *argmax);

/* Expert-parallel wiring for ep_size > 1 (no counterpart in the reference, whose device list is a
 * layer pipeline, src/gpu/glm53f_gpu.c:758-790): after finalize every rank exports a handle to its
 * exchange region (ep_handle_bytes() bytes, a CUDA IPC handle), the caller gathers all handles in
 * rank order over any transport and gives each rank the full table. From then on every MoE layer
 * ends in one kernel that stores this rank's contribution rows into every rank's region through
 * the peer mappings, waits (bounded; a wait that runs out makes the call return -1) for the other
 * ranks' rows and combines in top-k order. All ranks must make the same sequence of calls.
 * Option "sequence_split" = 1 (ep_size > 1, before the ranks exchange anything) changes what is
 * replicated: every rank then owns its OWN sequences (option "sequences" counts the rank's own) and
 * runs attention, mHC, norms and the head for its own tokens only; a MoE layer gathers the ranks'
 * tokens on every rank (peer stores: the dispatch), every rank routes them and multiplies them by
 * the experts it owns, and the contribution rows travel to the rank the token lives on, which
 * combines in top-k order (the combine). All ranks must call with the same number of tokens per
 * call (lockstep decode steps, prompts of equal length). The KDA head split is off in this mode.
 * Option "ep_loopback" (g5b_engine_set_option) wires stand-in peers in local memory that never
 * answer: it exists to exercise the time-out report on one GPU.
 * The wait is limited in wall-clock time (option "ep_wait_ms", default 5000): the ranks are separate
 * host processes, so ordinary host skew must not look like a lost peer. A wait that does run out
 * poisons the group: the rank that gave up has counted the step while a slower peer may still
 * finish it, so from then on the ranks would pair different steps. After a failed call, bring all
 * ranks to a barrier of your own, call g5b_engine_ep_resync on every rank (it forgets the step
 * words and restarts the count), reset the engines, and pass another barrier before the next step. */
size_t g5b_engine_ep_handle_bytes(void);
int    g5b_engine_ep_export(g5b_engine *e, void *handle_out);
int    g5b_engine_ep_connect(g5b_engine *e, const void *all_handles /* ep_size entries */);
int    g5b_engine_ep_resync(g5b_engine *e);
/* The same wiring for ranks living in one process (one engine per device, engines[r] = rank r of n;
 * this is how the adapter serves the reference's multi-device backend call,
 * src/gpu/glm53f_gpu.h:44-46): no handles, peer access between the devices. Every step must then be
 * run on all engines at the same time, one host thread each. */
int    g5b_engine_ep_connect_local(g5b_engine *const *engines, int n);

/* ---------------------------------------------------------------- LAYER OPS ---- */
/* Host buffers in and out. Activations are FP32 like the reference's. `layer` indexes the
 * engine's loaded layers; ops that carry state read and advance the engine's session state of
 * that layer exactly as the forward pass would. */

/* y[T][rows] = W x[T][cols] for any loaded matrix, by tensor name (glm53f_mm / _mm_batch,
 * glm53f.h:137,142). */
int g5b_op_matvec(g5b_engine *e, const char *name, const float *x, int T, float *y);

/* A matrix that is not part of a model: upload, multiply, discard. */
int g5b_matvec_host(const g5b_tensor *w, int br, int bc, const float *x, int T, float *y,
                    int device);

/* glm53f_rmsnorm (glm53f.h:165); w may be NULL. */
int g5b_rmsnorm_host(float *y, const float *x, const float *w, int n, int rows, float eps,
                     int device);
/* glm53f_swiglu_clamp (glm53f.h:168) over rows of [gate | up]. */
int g5b_swiglu_host(float *y, const float *gu, int n, int rows, float limit, int device);
/* glm53f_shortconv (glm53f.h:171). state [channels][k-1] is read and updated. */
int g5b_shortconv_host(float *y, const float *x, const float *w, float *state, int channels,
                       int k, int T, int device);

/* site 0 = attention, 1 = feed-forward. glm53f_hc_pre / glm53f_hc_post (glm53f.h:300-304):
 * h is [T][M][hidden]; x [T][hidden], post [T][M], comb [T][M*M]. */
int g5b_op_hc_pre(g5b_engine *e, int layer, int site, const float *h, int T, float *x,
                  float *post, float *comb);
int g5b_op_hc_post(g5b_engine *e, float *h, const float *y, const float *post,
                   const float *comb, int T);

/* glm53f_kda_layer (glm53f.h:309): x [T][hidden] -> out [T][hidden], state advanced. */
int g5b_op_kda(g5b_engine *e, int layer, const float *x, int T, float *out);
/* glm53f_mla with the latent cache plus glm53f_dsa_append / _select (glm53f.h:318-337):
 * appends T positions at the engine's cached position and attends. sel_out (may be NULL)
 * receives, for the LAST query, the selected positions; n_sel_out their count or -1 when the
 * query attended densely. Advances nothing but the layer's caches. */
int g5b_op_mla(g5b_engine *e, int layer, const float *x, int T, int cached, float *out,
               int *sel_out, int *n_sel_out);
/* glm53f_router (glm53f.h:340): idx/w [T][topk]. */
int g5b_op_router(g5b_engine *e, int layer, const float *x, int T, int *idx, float *w);
/* Expert indices and weights [T][topk] of the most recent MoE pass on this engine (the last chunk of
 * T <= 64 positions), whichever entry point ran it: lets a caller of a whole-layer op see the
 * routing the reference exposes through glm53f_router. Either output may be NULL. */
int g5b_engine_last_picks(g5b_engine *e, int T, int *idx, float *w);
/* glm53f_moe (glm53f.h:348); with_shared = 0 gives glm53f_moe_routed (glm53f.h:344). Any host
 * memory is accepted; when `out` is pinned and mapped (cudaHostAlloc / cudaHostRegister) the layer's
 * last kernel writes it directly and the device-to-host copy is skipped. */
int g5b_op_moe(g5b_engine *e, int layer, const float *x, int T, float *out, int with_shared);
/* glm53f_mlp on a dense layer's gate/up/down (glm53f.h:352). */
int g5b_op_mlp(g5b_engine *e, int layer, const float *x, int T, float *out);
/* glm53f_decoder_layer (glm53f.h:358): h [T][M][hidden] in place at position `cached`. */
int g5b_op_decoder_layer(g5b_engine *e, int layer, float *h, int T, int cached);

/* Session state access, to seed a layer without replaying a context (the reference's tests
 * fill Glm53fModel.state / ckv / idx directly). kind: 0 KDA state [H*D*D + 3*H*D*(k-1)],
 * 1 MLA latent cache [cap][kv_lora], 2 DSA state (k | gate | pool keys, glm53f_dsa.c:44-53).
 * Values cross as FP32; `count` floats starting at float offset `offset`. */
int g5b_state_write(g5b_engine *e, int layer, int kind, size_t offset, const float *src,
                    size_t count);
int g5b_state_read(g5b_engine *e, int layer, int kind, size_t offset, float *dst,
                   size_t count);

/* The checkpoint's multi-token-prediction layer (layer n_layers; reference src/model/glm53f_mtp.h).
 * g5b_engine_enable_mtp (before loading) makes the engine expect "layers.<n_layers>.*": an MLA + MoE
 * layer of the model's shapes without mHC tensors, plus enorm.weight, hnorm.weight,
 * shared_head.norm.weight and eh_proj.weight [hidden][2 hidden] (glm53f_bind.c:208-249), with its
 * own latent cache, indexer state and routed experts; every forward call then keeps the mean of
 * the residual streams of each of its positions (row t = position t of the call,
 * glm53f_model.c:460-468). g5b_mtp_feed is glm53f_mtp_feed (glm53f_mtp.c:100-144): h holds T hidden
 * states (NULL = the rows the last forward call kept), next_ids[t] the token that follows position
 * t; the layer advances its own position count by T and *draft (may be NULL) receives the token
 * predicted after the last one. x_out (may be NULL) receives the layer's output rows
 * [T][hidden]. g5b_engine_reset forgets the fed positions. The reference only scores drafts
 * against the tokens the model produces (glm53f_mtp_score); so do the tests here. */
int g5b_engine_enable_mtp(g5b_engine *e);
int g5b_mtp_feed(g5b_engine *e, const float *h, const int *next_ids, int T, int *draft, float *x_out);
int g5b_mtp_hidden(g5b_engine *e, int first, int T, float *dst);
/* Speculative greedy decode on top of it (the use glm53f_mtp.h:11-14 describes; the reference stops
 * at counting right drafts): every pass feeds the model the current token and the MTP layer's draft
 * of the next one; the draft is kept only when the model's own arg-max is the same token, otherwise
 * the KDA states fall back to what they were after the first position (every KDA layer writes that
 * to a second buffer during such a pass) and only the first position's token stands.
 * The tokens are those of greedy decode. Needs the MTP layer fed up to, not including, the last
 * cached position (after a prompt: g5b_mtp_feed with the kept hidden states but the last and the
 * prompt's tokens but the first) and no forward call since the one that produced `first`.
 * stats (may be NULL): drafts made, drafts accepted, model passes. */
int g5b_engine_decode_speculative(g5b_engine *e, int first, int n, int *out, long *stats);

/* Measurement aid (no counterpart in the reference): SM cycles per tcgen05.mma instruction, M = 128,
 * N = n (a multiple of 16 up to 256), kind::f16 (K = 16) or, with fp8 != 0, kind::f8f6f4 (K = 32),
 * issued back to back by one thread of each of `ctas` CTAs on shared-memory tiles that never
 * change, rotating over `accs` accumulators. cycles[0]: until issued, cycles[1]: until complete. */
int g5b_debug_mma_rate(int n, int fp8, int accs, int ctas, int reps, double *cycles);

/* RMSNorm of `rows` rows of n floats on DEVICE buffers of the current CUDA device, enqueued on
 * `stream` (a cudaStream_t, NULL for the default stream) without waiting: y = w * x / sqrt(mean(x^2)
 * + eps), w may be NULL. This entry point has no counterpart in the reference. It exists for
 * callers that must not allocate: it calls no cudaMalloc / cudaFree and no allocating library
 * routine, because its per-row scratch (the normalisation factors) is a fixed array built into
 * the library. Limits and rules that follow from that:
 *   - rows <= 4096; more is refused with -1 and a message (split the call);
 *   - every GPU that loads the library holds the 16 KB array until the process exits;
 *   - the first call on each device resolves the array's address (once per device, with that
 *     device current): make that first call before any stream capture begins, from one thread
 *     (two first calls must not race), and not across a cudaDeviceReset (the address is kept);
 *   - all calls on a device share the array: two calls that may overlap on the GPU (different
 *     streams, or different threads) race on it and must be ordered by the caller. Nothing in it
 *     has to start at zero; each call overwrites every factor it reads.
 * Same arithmetic and same kernels as g5b_rmsnorm_host. */
int g5b_rmsnorm_noalloc(float *y_dev, const float *x_dev, const float *w_dev, int n, int rows,
                        float eps, void *stream);

/* --------------------------------------------------------------- DEVICE OPS ---- */
/* Device pointers on the engine's GPU, launched on the engine's stream, no host copies and
 * no synchronisation (call g5b_engine_sync to wait). */
int   g5b_dev_moe(g5b_engine *e, int layer, const float *x_dev, int T, float *out_dev);
int   g5b_dev_kda(g5b_engine *e, int layer, const float *x_dev, int T, float *out_dev);
int   g5b_dev_mla(g5b_engine *e, int layer, const float *x_dev, int T, int cached,
                  float *out_dev);
int   g5b_dev_decoder_layer(g5b_engine *e, int layer, float *h_dev, int T, int cached);
int   g5b_engine_sync(g5b_engine *e);
void *g5b_engine_stream(g5b_engine *e);            /* the cudaStream_t ops are launched on */
/* Kernels this library has launched since it was loaded (benchmark bookkeeping). */
uint64_t g5b_launch_count(void);
/* Time `iters` launches of one op ("moe", "kda", "mla", "layer") between CUDA events recorded on
 * the engine's stream. Before each launch `flush_bytes` of scratch memory are overwritten (0 =
 * no flush) so that the weights come from HBM and not from L2. ms_total receives the sum of the
 * per-launch times, ms_each (may be NULL, `iters` floats) each of them. For "layer", out_dev is
 * the residual stream h, updated in place. */
int g5b_time_op(g5b_engine *e, const char *op, int layer, const float *x_dev, int T, int cached,
                float *out_dev, int iters, size_t flush_bytes, float *ms_total, float *ms_each);
/* The same for one product y[T][rows] = W x[T][cols] of a loaded matrix, on the path the forward pass
 * takes for T positions (x_dev, y_dev: device buffers of T * cols and T * rows floats). */
int g5b_time_matvec(g5b_engine *e, const char *name, const float *x_dev, int T, float *y_dev, int iters,
                    size_t flush_bytes, float *ms_each);
/* With the "profile" option on, every MoE op also records events between its phases; this
 * reads the accumulated milliseconds of [router+plan, gate/up, down, combine] and the number of
 * ops they cover, and optionally clears them. */
int g5b_engine_profile_read(g5b_engine *e, float *ms, int n, long *count, int reset);

#ifdef __cplusplus
}
#endif

#endif /* GLM53F_B200_H */
