/* A caller of the C interface written in C, for tests/test_capi*.py: it links libstratum_c.so only.
 *
 *   capi_client probe MODEL_DIR              open must fail; prints the code and the message
 *   capi_client run MODEL_DIR DTYPE IN OUT   IN: int32 file "n | len[n] | tokens"; writes into folder OUT
 *       prompt_logits.f32   logits at the last place of every prompt (one step for all prompts)
 *       decode_logits.f32   3 further steps, each feeding the best id of the step before: [3][n][vocab]
 *       picked.i32          the best ids fed and found: [4][n]
 *       generated.i32       stratum_generate, greedy, 4 new tokens: count[n] | ids[n][4]
 *       sampled.i32         stratum_generate at temperature 0.8, top-k 5, seed 7: count[n] | ids[n][4]
 *       notes.txt           slots, lengths and the messages of the calls that had to fail
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "stratum.h"

#define CHECK(call)                                                                          \
  do {                                                                                       \
    int rc_ = (call);                                                                        \
    if (rc_ != STRATUM_OK) {                                                                 \
      fprintf(stderr, "%s -> %d: %s\n", #call, rc_, stratum_last_error(ctx));                \
      return 1;                                                                              \
    }                                                                                        \
  } while (0)

static int argmax(const float* row, int n) {
  int best = 0;
  for (int i = 1; i < n; ++i) if (row[i] > row[best]) best = i;
  return best;
}

static int dump(const char* dir, const char* name, const void* data, size_t bytes) {
  char path[4096];
  snprintf(path, sizeof path, "%s/%s", dir, name);
  FILE* f = fopen(path, "wb");
  if (!f) return 1;
  size_t n = fwrite(data, 1, bytes, f);
  fclose(f);
  return n != bytes;
}

int main(int argc, char** argv) {
  stratum_ctx* ctx = NULL;
  if (argc == 3 && !strcmp(argv[1], "probe")) {
    int rc = stratum_open(argv[2], "bfloat16", 256, 0, &ctx);
    printf("open -> %d ctx %s: %s\n", rc, ctx ? "set" : "null", stratum_last_error(NULL));
    int rc2 = stratum_open(NULL, "bfloat16", 256, 0, &ctx);
    printf("open(null) -> %d: %s\n", rc2, stratum_last_error(NULL));
    printf("vocab(null) -> %d\n", stratum_vocab(NULL, NULL));
    stratum_close(NULL);
    return (rc == STRATUM_E_ENGINE && !ctx && rc2 == STRATUM_E_ARGUMENT) ? 0 : 1;
  }
  if (argc != 6 || strcmp(argv[1], "run")) {
    fprintf(stderr, "usage: capi_client probe MODEL_DIR | run MODEL_DIR DTYPE IN OUT\n");
    return 2;
  }
  const char* out_dir = argv[5];
  FILE* in = fopen(argv[4], "rb");
  if (!in) return 2;
  int n = 0;
  if (fread(&n, 4, 1, in) != 1 || n < 1 || n > 64) return 2;
  int lens[64], total = 0;
  if (fread(lens, 4, n, in) != (size_t)n) return 2;
  for (int i = 0; i < n; ++i) total += lens[i];
  int* tokens = malloc(4 * (size_t)total);
  if (fread(tokens, 4, total, in) != (size_t)total) return 2;
  fclose(in);

  char notes[8192];
  size_t at = 0;
  CHECK(stratum_open(argv[2], argv[3], 2048, 0, &ctx));
  int vocab = 0;
  CHECK(stratum_vocab(ctx, &vocab));
  int slots[64], wants_n[64], wants[64], ones[64], zeros[64], picked[4][64];
  for (int i = 0; i < n; ++i) {
    CHECK(stratum_slot_acquire(ctx, &slots[i]));
    wants_n[i] = 1; wants[i] = lens[i] - 1; ones[i] = 1; zeros[i] = 0;
    at += snprintf(notes + at, sizeof notes - at, "slot %d\n", slots[i]);
  }
  float* logits = malloc(4 * (size_t)n * vocab);
  float* decode = malloc(4 * (size_t)3 * n * vocab);
  CHECK(stratum_step(ctx, n, slots, lens, tokens, wants_n, wants, logits));
  if (dump(out_dir, "prompt_logits.f32", logits, 4 * (size_t)n * vocab)) return 3;
  for (int i = 0; i < n; ++i) picked[0][i] = argmax(logits + (size_t)i * vocab, vocab);
  for (int k = 0; k < 3; ++k) {
    float* dst = decode + (size_t)k * n * vocab;
    CHECK(stratum_step(ctx, n, slots, ones, picked[k], wants_n, zeros, dst));
    for (int i = 0; i < n; ++i) picked[k + 1][i] = argmax(dst + (size_t)i * vocab, vocab);
  }
  if (dump(out_dir, "decode_logits.f32", decode, 4 * (size_t)3 * n * vocab)) return 3;
  if (dump(out_dir, "picked.i32", picked, sizeof picked)) return 3;
  for (int i = 0; i < n; ++i) {
    int len = -1;
    CHECK(stratum_slot_length(ctx, slots[i], &len));
    at += snprintf(notes + at, sizeof notes - at, "length %d\n", len);
  }
  /* calls that must fail, and leave everything as it was */
  int bad = vocab, len_after = -1, rc;
  rc = stratum_step(ctx, 1, slots, ones, &bad, wants_n, zeros, logits);
  at += snprintf(notes + at, sizeof notes - at, "bad token -> %d: %s\n", rc, stratum_last_error(ctx));
  CHECK(stratum_slot_length(ctx, slots[0], &len_after));
  at += snprintf(notes + at, sizeof notes - at, "length after %d\n", len_after);
  rc = stratum_slot_release(ctx, 9999);
  at += snprintf(notes + at, sizeof notes - at, "bad slot -> %d: %s\n", rc, stratum_last_error(ctx));
  rc = stratum_step(ctx, 1, slots, ones, NULL, wants_n, zeros, logits);
  at += snprintf(notes + at, sizeof notes - at, "null tokens -> %d: %s\n", rc, stratum_last_error(ctx));
  for (int i = 0; i < n; ++i) CHECK(stratum_slot_release(ctx, slots[i]));
  rc = stratum_slot_release(ctx, slots[0]);
  at += snprintf(notes + at, sizeof notes - at, "released twice -> %d: %s\n", rc, stratum_last_error(ctx));
  int again = -1;
  CHECK(stratum_slot_acquire(ctx, &again));
  at += snprintf(notes + at, sizeof notes - at, "slot again %d\n", again);
  CHECK(stratum_slot_release(ctx, again));

  int gen[64 + 64 * 4];
  memset(gen, 0xff, sizeof gen);
  CHECK(stratum_generate(ctx, n, lens, tokens, 4, NULL, 0, 0.0f, 0, 1.0f, 0ull, gen + n, gen));
  if (dump(out_dir, "generated.i32", gen, 4 * (size_t)(n + 4 * n))) return 3;
  memset(gen, 0xff, sizeof gen);
  CHECK(stratum_generate(ctx, n, lens, tokens, 4, NULL, 0, 0.8f, 5, 1.0f, 7ull, gen + n, gen));
  if (dump(out_dir, "sampled.i32", gen, 4 * (size_t)(n + 4 * n))) return 3;
  int stop = picked[1][0];                      /* the second token of the first prompt ends it */
  memset(gen, 0xff, sizeof gen);
  CHECK(stratum_generate(ctx, 1, lens, tokens, 4, &stop, 1, 0.0f, 0, 1.0f, 0ull, gen + 1, gen));
  at += snprintf(notes + at, sizeof notes - at, "stopped after %d\n", gen[0]);
  if (dump(out_dir, "notes.txt", notes, at)) return 3;
  stratum_close(ctx);
  free(tokens); free(logits); free(decode);
  printf("ok\n");
  return 0;
}
