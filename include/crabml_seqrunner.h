/*
 * crabml_seqrunner.h -- what every multi-sequence model runner of this library offers, whatever its family (crabml_zatorax.h,
 * crabml_meresun.h create them): sequence slots, the step function, greedy generation.
 *
 * A sequence owns a SLOT of per-layer state (caches, recurrent state) from csr_seq_open to csr_seq_close; closed slots are reused,
 * lowest first.  A step feeds any number of a sequence's next tokens; how a prompt is cut into steps does not change a position's
 * logits beyond rounding.  Steps longer than the runner's chunk are cut into passes.
 */
#ifndef CRABML_SEQRUNNER_H
#define CRABML_SEQRUNNER_H

#include "crabml_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct csr_runner csr_runner;

CC_API void csr_runner_destroy(csr_runner* r);
CC_API const char* csr_runner_last_error(csr_runner* r);
/* why the last runner creation of this thread failed (any family) */
CC_API const char* csr_last_create_error(void);

/* open takes a free slot (or makes a new one), resets its state and sets its length to 0 */
CC_API int csr_seq_open(csr_runner* r, int32_t* slot_out);
CC_API int csr_seq_close(csr_runner* r, int32_t slot);
CC_API int64_t csr_seq_len(csr_runner* r, int32_t slot);
/* {slots allocated, slots live, bytes of state per slot} */
CC_API int csr_runner_stats(csr_runner* r, int64_t* out3);

/* feed the sequence's next n_tokens tokens; logits of the positions want[0..n_want) (indices into this step's tokens, ascending) are
 * written to logits_out as [n_want, vocab] floats.  n_want may be 0 (then logits_out may be NULL and nothing is copied to the host). */
CC_API int csr_runner_step(csr_runner* r, int32_t slot, const int64_t* tokens, int32_t n_tokens, const int32_t* want, int32_t n_want, float* logits_out);
/* greedy generation: feeds the prompt, then generates up to `steps` tokens; sampling runs on the device (the LAST maximum, as the
 * llama runner's sampler) and the sampled id feeds the next step from a device slot.  eos < 0: no step waits for the host. */
CC_API int csr_runner_generate_greedy(csr_runner* r, int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos,
                                      int64_t* out_tokens, int32_t* n_out);

#ifdef __cplusplus
}
#endif
#endif
