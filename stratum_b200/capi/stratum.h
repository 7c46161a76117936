/* stratum.h - the C interface of stratum_b200.
 *
 * The reference has no library interface (everything is static in one translation unit,
 * CONTRIBUTING.md:52); these names are this library's own.  The host of this library is Python (its parts
 * are Python classes that a user can add to); this interface is a thin layer in front of that host for callers
 * written in C: libstratum_c.so starts an interpreter inside the calling process if there is none (or uses the
 * one that is running), imports the package and forwards every call.  One model, step function, cache and set of
 * kernels serve both interfaces; nothing is computed in this layer.
 *
 * Every function returns 0 on success and a negative STRATUM_E_* code otherwise; stratum_last_error gives the
 * message of the last failure (of the context, or of stratum_open when it returned no context).  Calls on one
 * context must not overlap; the layer takes the interpreter's lock around every call.
 */
#ifndef STRATUM_C_H
#define STRATUM_C_H

#ifdef __cplusplus
extern "C" {
#endif

#define STRATUM_OK 0
#define STRATUM_E_ARGUMENT (-1)     /* a null pointer, a negative count */
#define STRATUM_E_ENGINE (-2)       /* the library raised: bad slot, token id outside the vocabulary, cache full,
                                       weights that do not match, a kernel that gave up a wait, ... */
#define STRATUM_E_INTERPRETER (-3)  /* the interpreter or the package could not be brought up */

typedef struct stratum_ctx stratum_ctx;

/* Open a model folder (config.json + model.safetensors; the model class is chosen by config.json).
 * dtype: "bfloat16" (the serving kernels) or "float32" (true 32-bit).  max_tokens: what live sequences may hold
 * together, each rounded up to 64.  max_seqs: sequences that may be live at once (0: as many as pages). */
int stratum_open(const char* model_dir, const char* dtype, long long max_tokens, int max_seqs, stratum_ctx** out);
void stratum_close(stratum_ctx* ctx);
int stratum_vocab(stratum_ctx* ctx, int* vocab);

/* A slot holds one sequence's keys, values and state; released slots are used again. */
int stratum_slot_acquire(stratum_ctx* ctx, int* slot);
int stratum_slot_release(stratum_ctx* ctx, int slot);
int stratum_slot_length(stratum_ctx* ctx, int slot, int* length);

/* One step: sequence i brings n_tok[i] new tokens (packed one after another in `tokens`) and asks for the logits
 * at n_want[i] places among them (packed in `want`, each < n_tok[i]).  Either every sequence starts (prompts of
 * unequal lengths) or every one goes on.  logits receives [sum of n_want][vocab] float32 in the order of the
 * sequences and of their wanted places.  On failure nothing has changed. */
int stratum_step(stratum_ctx* ctx, int n_seq, const int* slots, const int* n_tok, const int* tokens,
                 const int* n_want, const int* want, float* logits);

/* Generate for n_prompts prompts of prompt_len[i] tokens (packed in prompt_tokens): at most max_new tokens each,
 * ending early at any of the n_stop ids.  temperature <= 0: greedy; top_k 0 and top_p 1: no filter.  out_tokens
 * receives [n_prompts][max_new] ids (row i holds out_count[i] of them; a stop id, if met, is the last). */
int stratum_generate(stratum_ctx* ctx, int n_prompts, const int* prompt_len, const int* prompt_tokens, int max_new,
                     const int* stop_ids, int n_stop, float temperature, int top_k, float top_p,
                     unsigned long long seed, int* out_tokens, int* out_count);

/* The message of the last failure; ctx may be null (then: of the last stratum_open that failed). */
const char* stratum_last_error(stratum_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif
