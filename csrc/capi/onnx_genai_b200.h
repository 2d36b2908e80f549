/*
 * C interface of onnx_genai_b200: load a model directory, generate text, plug in a token sampler written
 * in C.  The eight entry points have the names and signatures of the reference's C header
 * (crates/onnx-genai-capi/include/onnx_genai.h:30-106), so a client of that header recompiles against
 * this one unchanged.
 *
 * The library hosts the Python engine.  Inside a Python process it attaches to the running interpreter;
 * in a plain C program it starts one on first use.  Two environment variables steer that start-up:
 *   ONNX_GENAI_B200_PYTHON  interpreter whose environment (site-packages) is used
 *   ONNX_GENAI_B200_ROOT    directory that contains the onnx_genai_b200 package
 * Both default to the values recorded when the library was built.
 *
 * Errors: a failing call returns NULL and leaves a message for oge_last_error() on the calling thread.
 * Thread safety: calls may come from any thread; they are serialised on the interpreter lock.
 */
#ifndef ONNX_GENAI_B200_H
#define ONNX_GENAI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OgeEngine OgeEngine;   /* a loaded model */
typedef struct OgeSampler OgeSampler; /* a token-selection callback with its state */

/*
 * Chooses the next token.  `logits` holds `logits_len` (= vocabulary size) values after the request's
 * logit processors ran; tokens they removed are -inf.  `generated` lists the `generated_len` tokens this
 * request has produced so far and `step` counts decode steps from 0.  Both arrays belong to the library
 * and are valid only during the call.  The return value must be below `logits_len`.
 */
typedef uint32_t (*OgeSampleFn)(void *user_data, const float *logits, size_t logits_len, const uint32_t *generated,
                                size_t generated_len, size_t step);

/* Releases `user_data`; called once, when the sampler is destroyed. */
typedef void (*OgeFreeFn)(void *user_data);

typedef struct OgeSamplerVTable {
  void *user_data;    /* handed to every callback; may be NULL */
  OgeSampleFn sample; /* required */
  const char *name;   /* optional label, copied; NULL means "foreign" */
  OgeFreeFn free;     /* optional; NULL means the library never frees user_data */
} OgeSamplerVTable;

/* Wraps a vtable.  NULL on failure.  Release with oge_sampler_free() unless a generate call consumed it. */
OgeSampler *oge_sampler_new(OgeSamplerVTable vtable);

/* Destroys a sampler that no generate call consumed.  NULL is accepted. */
void oge_sampler_free(OgeSampler *sampler);

/* Loads a flat model directory or a model package.  NULL on failure.  Release with oge_engine_free(). */
OgeEngine *oge_engine_load(const char *model_dir);

/* NULL is accepted. */
void oge_engine_free(OgeEngine *engine);

/*
 * Generates with the built-in samplers (the model's generation defaults decide greedy or categorical).
 * max_new_tokens == 0 keeps the default budget.  The result is heap memory: release it with
 * oge_string_free().  NULL on failure.
 */
char *oge_engine_generate(OgeEngine *engine, const char *prompt, size_t max_new_tokens);

/*
 * Generates with `sampler`, which this call consumes whether it succeeds or fails: do not touch the
 * pointer afterwards.  Result and failure as for oge_engine_generate().
 */
char *oge_engine_generate_with_sampler(OgeEngine *engine, const char *prompt, size_t max_new_tokens, OgeSampler *sampler);

/* Releases a string returned by this library.  NULL is accepted. */
void oge_string_free(char *text);

/*
 * Message of the latest failure on the calling thread, or NULL when its latest call succeeded.  The
 * pointer stays owned by the library and is valid until the thread's next call into it.
 */
const char *oge_last_error(void);

#ifdef __cplusplus
}
#endif

#endif /* ONNX_GENAI_B200_H */
