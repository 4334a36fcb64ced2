/*
 * crabml_meresun.h -- creation of the host driver of the Meresun decoder family (crabml_b200/csrc/host/meresun_runner.cpp); the
 * runner it returns is served through crabml_seqrunner.h (slots, step, greedy generation) like every multi-sequence runner.
 *
 * The stack: x = embed[token] (the table arrives already multiplied by the embedding scale).  A layer reads ONE norm of the residual
 * stream, h = norm(x) (RMS norm in groups), hands it to its mixer and to its feed-forward side by side, multiplies each result by
 * sigmoid(W_g h + b_g) and adds their sum to x; then a per-layer token input is added:
 *   g = gelu_tanh(W_sg x) * e_layer[token] ; y = W_sp g ; x += y / rms(y) * w_s.
 * Layers loop_start .. loop_stop-1 run loop_times times with the same weights; every run has its own cache, and before each run of
 * the block but the first the embedding output is added to x.
 * Mixer: latent attention.  Queries go through a normed latent; a cache row is [c | r] (cc_latent_ring_append); sliding window,
 * softmax with a per-head sink (cc_window_attention_sink).  A pass of few rows (decoding) folds the per-head key up-projection into
 * the query and applies the value up-projection to the attention result (cc_head_project), so scores and sums run over the cached
 * rows themselves; a pass of many rows (prompts) expands the cached rows into per-head keys and values with two dense products and
 * runs the same attention per head.
 * Feed-forward: dense with PolyNorm (cc_poly_norm), or routed (cc_moe_route_ex: sigmoid scores, group score = sum of the two
 * largest, renormalised weights; cc_moe_experts_glu: clamped gate and up, swish(1.702), up + 1), or none.
 */
#ifndef CRABML_MERESUN_H
#define CRABML_MERESUN_H

#include "crabml_seqops.h"
#include "crabml_seqrunner.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CMR_FF_NONE 0
#define CMR_FF_DENSE 1
#define CMR_FF_ROUTED 2

typedef struct cmr_layer_config {
    int32_t heads, dim, rot_dim, vdim, q_rank, kv_rank;
    int32_t window;                 /* position i sees j with 0 <= i - j < window; <= 0: every j <= i (the cache then holds max_seq rows) */
    float scale;                    /* score scale */
    float rot_mag;                  /* factor on cos and sin */
    int32_t ff_kind;                /* CMR_FF_* */
    int32_t ff;                     /* dense: hidden width; routed: an expert's hidden width */
    int32_t experts, top, groups, keep_groups;
    float limit;                    /* routed: clamp of the gated unit */
} cmr_layer_config;

typedef struct cmr_config {
    int32_t n_layers, width, vocab;
    float norm_eps;
    int32_t norm_groups;
    int32_t loop_start, loop_stop, loop_times;      /* loop_times <= 1: every layer runs once */
    int32_t side_dim;               /* width of the per-layer token input; 0: none */
    int32_t chunk;                  /* longest run of tokens one pass takes; sizes the caches.  <= 0: 256 */
    int32_t max_seq;                /* rows of the cache of a layer without a window.  <= 0: 4096 */
} cmr_config;

/* every pointer is a tensor uploaded by the caller; unused ones are NULL.  Matrices of dense products: F32 or BF16; uk_t, uv_f32,
 * router and everything else: F32. */
typedef struct cmr_layer_weights {
    cc_buf *norm1;                                  /* [width] */
    /* everything that multiplies the layer's normed input h, stacked one under the other so that it is ONE product: mix.dkv
     * [kv_rank + rot_dim, width], mix.dq [q_rank, width], then rg1 [width, width] if rg1_b is given, rg2 [width, width] if rg2_b is
     * given, mlp.up [ff, width] if the feed-forward is dense */
    cc_buf *h_stack;
    cc_buf *dq_norm, *uq;                           /* [q_rank], [heads * (dim + rot_dim), q_rank] */
    cc_buf *dkv_norm;                               /* [kv_rank] */
    cc_buf *uk, *uv;                                /* [heads * dim, kv_rank], [heads * vdim, kv_rank]: dense products of the many-row pass */
    cc_buf *uk_t, *uv_f32;                          /* few-row pass, F32: [heads * kv_rank, dim] (every head's block of uk transposed), uv itself */
    cc_buf *sink, *rot_freq, *o;                    /* [heads] or NULL, [P] frequencies of the rotated pairs (2 P <= rot_dim), [width, heads * vdim] */
    cc_buf *rg1_b, *rg2_b;                          /* biases of the gates of the two results: [width]; NULL = that result is not gated */
    cc_buf *down, *act;                             /* dense: [width, ff], [4] */
    cc_buf *router, *correction;                    /* routed: [experts, width], [experts] */
    cc_buf *e_gate, *e_up, *e_down;                 /* routed: expert-major stacks [experts * ff, width] x 2, [experts * width, ff] */
    cc_buf *side_table, *side_gate, *side_proj, *side_norm;   /* [vocab, side_dim] (this layer's part), [side_dim, width], [width, side_dim], [width] */
} cmr_layer_weights;

CC_API int cmr_runner_create(cc_device* dev, const cmr_config* conf, const cmr_layer_config* layers, const cmr_layer_weights* weights, cc_buf* embed,
                             cc_buf* final_norm, cc_buf* head, csr_runner** out);

#ifdef __cplusplus
}
#endif
#endif
