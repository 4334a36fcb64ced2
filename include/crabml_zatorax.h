/*
 * crabml_zatorax.h -- C entry points of the host driver of the Zatorax decoder family (crabml_b200/csrc/host/zatorax_runner.cpp):
 * a stack of layers, each a token mixer (gated delta rule with short convolutions, or sliding-window attention with a
 * logarithmic distance penalty, optionally reading another layer's keys and values) and an optional routed feed-forward with a
 * shared expert, every sublayer's OUTPUT normalised (one-number RMS gain) before it is added to the 32-bit residual stream.
 *
 * Like the llama runner (crabml_runner.h) it is a replay of tensor ops over the C ABI (crabml_cuda.h + crabml_seqops.h) and holds
 * no arithmetic of its own.  Unlike it, it serves several sequences: a sequence owns a SLOT of per-layer state (key/value rings of
 * the attention layers, recurrent matrix and convolution tails of the delta layers) from czr_seq_open to czr_seq_close; closed
 * slots are reused.  A step feeds any number of a sequence's next tokens; how a prompt is cut into steps does not change a
 * position's logits beyond rounding.
 */
#ifndef CRABML_ZATORAX_H
#define CRABML_ZATORAX_H

#include "crabml_seqops.h"
#include "crabml_seqrunner.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CZR_MIXER_DELTA 0
#define CZR_MIXER_ATTENTION 1

typedef struct czr_layer_config {
    int32_t mixer;                  /* CZR_MIXER_* */
    int32_t heads, kv_heads, dim, vdim;
    int32_t conv;                   /* delta: taps of the short convolutions */
    int32_t window;                 /* attention: position i sees j with 0 <= i - j < window */
    int32_t kv_from;                /* attention: -1 = projections of its own; else the layer whose keys / values it reads */
    float scale;                    /* attention: score scale */
    int32_t has_mlp;                /* 0: the layer is its mixer only */
    int32_t experts, top, groups, keep_groups, expert_ff;
    int32_t shared_ff;              /* 0: no shared expert */
} czr_layer_config;

typedef struct czr_config {
    int32_t n_layers, width, vocab;
    float norm_eps;
    int32_t chunk;                  /* longest run of tokens one pass takes (longer steps are cut); sizes the key/value rings. <= 0: 256 */
} czr_config;

/* every pointer is a tensor uploaded by the caller; unused ones are NULL.  Matrices: F32 or BF16; everything else F32. */
typedef struct czr_layer_weights {
    cc_buf *norm1, *norm2;                                            /* [1] */
    cc_buf *q, *k, *v, *o;                                            /* mixer projections [out, in] */
    cc_buf *q_conv, *k_conv, *v_conv;                                 /* delta: [channels, taps] */
    cc_buf *b, *a, *a_log, *dt_bias, *out_norm, *g;                   /* delta: beta / decay projections [heads, width], [heads], [vdim], gate [heads*vdim, width] */
    cc_buf *q_norm, *k_norm, *r1, *r2;                                /* attention: [dim], [dim], [heads], [heads] */
    cc_buf *router, *correction;                                      /* [experts, width] F32, [experts] */
    cc_buf *e_gate, *e_up, *e_down;                                   /* expert-major stacks [experts*ff, width], [experts*ff, width], [experts*width, ff] */
    cc_buf *s_gate, *s_up, *s_down;                                   /* shared expert */
} czr_layer_weights;

/* a Zatorax runner is a sequence runner (crabml_seqrunner.h); the czr_ functions below the creation are the csr_ ones under their older names */
typedef csr_runner czr_runner;

CC_API int czr_runner_create(cc_device* dev, const czr_config* conf, const czr_layer_config* layers, const czr_layer_weights* weights, cc_buf* embed,
                             cc_buf* final_norm, cc_buf* head, czr_runner** out);
/* why the last czr_runner_create of this thread failed */
CC_API const char* czr_last_create_error(void);
CC_API void czr_runner_destroy(czr_runner* r);
CC_API const char* czr_runner_last_error(czr_runner* r);

/* sequence state: open takes a free slot (or makes a new one), zeroes its recurrent state and sets its length to 0 */
CC_API int czr_seq_open(czr_runner* r, int32_t* slot_out);
CC_API int czr_seq_close(czr_runner* r, int32_t slot);
CC_API int64_t czr_seq_len(czr_runner* r, int32_t slot);
/* {slots allocated, slots live, bytes of state per slot} */
CC_API int czr_runner_stats(czr_runner* r, int64_t* out3);

/* feed the sequence's next n_tokens tokens; logits of the positions want[0..n_want) (indices into this step's tokens, ascending) are
 * written to logits_out as [n_want, vocab] floats.  n_want may be 0 (then logits_out may be NULL and nothing is copied to the host). */
CC_API int czr_runner_step(czr_runner* r, int32_t slot, const int64_t* tokens, int32_t n_tokens, const int32_t* want, int32_t n_want, float* logits_out);
/* greedy generation: feeds the prompt, then generates up to `steps` tokens; sampling runs on the device (the LAST maximum, as the
 * llama runner's sampler) and the sampled id feeds the next step from a device slot.  eos < 0: no step waits for the host. */
CC_API int czr_runner_generate_greedy(czr_runner* r, int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos,
                                      int64_t* out_tokens, int32_t* n_out);

#ifdef __cplusplus
}
#endif
#endif
