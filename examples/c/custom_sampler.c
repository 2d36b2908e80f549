/*
 * A sampler written in C, driven by the onnx_genai_b200 engine.
 *
 *   cc custom_sampler.c -I ../../csrc/capi -L ../../onnx_genai_b200/_lib -lonnx_genai_b200 \
 *      -Wl,-rpath,$PWD/../../onnx_genai_b200/_lib -o custom_sampler
 *   ./custom_sampler MODEL_DIR "prompt" 16
 *
 * The sampler takes the most likely token, except that it never repeats the token it chose one step
 * earlier (then it takes the runner-up).  It keeps a call counter in user_data to show that state and the
 * destructor work.  Output: the generated text on stdout and "calls=<n> freed=<0|1>" on stderr.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "onnx_genai_b200.h"

struct state {
  size_t calls;
  int *freed_flag;
};

static uint32_t no_repeat_argmax(void *user_data, const float *logits, size_t n, const uint32_t *generated, size_t generated_len,
                                 size_t step) {
  struct state *st = (struct state *)user_data;
  st->calls++;
  (void)step;
  long banned = generated_len ? (long)generated[generated_len - 1] : -1;
  uint32_t best = 0;
  float best_v = -INFINITY;
  for (size_t i = 0; i < n; ++i) {
    if ((long)i == banned) continue;
    if (logits[i] > best_v) {
      best_v = logits[i];
      best = (uint32_t)i;
    }
  }
  return best;
}

static void release(void *user_data) {
  struct state *st = (struct state *)user_data;
  *st->freed_flag = 1;
  fprintf(stderr, "calls=%zu ", st->calls);
  free(st);
}

int main(int argc, char **argv) {
  if (argc < 3) {
    fprintf(stderr, "usage: %s MODEL_DIR PROMPT [MAX_NEW_TOKENS]\n", argv[0]);
    return 2;
  }
  size_t max_new = argc > 3 ? (size_t)strtoul(argv[3], NULL, 10) : 16;
  OgeEngine *engine = oge_engine_load(argv[1]);
  if (!engine) {
    fprintf(stderr, "load failed: %s\n", oge_last_error());
    return 1;
  }
  int freed = 0;
  struct state *st = (struct state *)calloc(1, sizeof *st);
  st->freed_flag = &freed;
  OgeSamplerVTable vt = {st, no_repeat_argmax, "no-repeat-argmax", release};
  OgeSampler *sampler = oge_sampler_new(vt);
  if (!sampler) {
    fprintf(stderr, "sampler failed: %s\n", oge_last_error());
    return 1;
  }
  char *text = oge_engine_generate_with_sampler(engine, argv[2], max_new, sampler); /* consumes the sampler */
  if (!text) {
    fprintf(stderr, "generate failed: %s\n", oge_last_error());
    oge_engine_free(engine);
    return 1;
  }
  fprintf(stderr, "freed=%d\n", freed);
  printf("%s\n", text);
  oge_string_free(text);
  char *plain = oge_engine_generate(engine, argv[2], max_new);
  if (plain) {
    printf("%s\n", plain);
    oge_string_free(plain);
  }
  oge_engine_free(engine);
  return 0;
}
