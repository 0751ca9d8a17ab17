/* A caller of libluminal_b200.so that is neither Python nor C++: plain C99 over include/luminal_b200.h, the
 * way a Julia `ccall` shim sees the library (handles, plain pointers, int32 status codes).  It creates the
 * small Llama of examples/llama.jl's shape family, fills it from the counter-based generator, runs a prompt
 * and a greedy loop (src/Decoding.jl:91-130), and prints the produced tokens as one JSON line.  The tests
 * compile it with gcc, run it, and compare the line with the Python host mirror and with the CPU oracle.
 *
 *   cabi_driver <dtype 0|1> <batch> <prompt_len> <steps> <seed>
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "luminal_b200.h"

#define CHECK(call)                                                                      \
  do {                                                                                   \
    int32_t rc_ = (call);                                                                \
    if (rc_ != LMB200_OK) {                                                              \
      fprintf(stderr, "%s -> %d: %s\n", #call, (int)rc_, lmb200_last_error());           \
      return 2;                                                                          \
    }                                                                                    \
  } while (0)

int main(int argc, char** argv) {
  if (argc != 6) {
    fprintf(stderr, "usage: %s dtype batch prompt_len steps seed\n", argv[0]);
    return 64;
  }
  const int dtype = atoi(argv[1]), batch = atoi(argv[2]), prompt = atoi(argv[3]), steps = atoi(argv[4]);
  const uint64_t seed = strtoull(argv[5], NULL, 10);
  if (batch < 1 || prompt < 1 || steps < 1) return 64;

  lmb200_model_config cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.n_layers = 4; cfg.hidden = 256; cfg.n_heads = 8; cfg.n_kv_heads = 8; cfg.head_dim = 32;
  cfg.intermediate = 688; cfg.vocab = 1024; cfg.rms_eps = 1e-5f; cfg.rope_base = 10000.0f;
  cfg.dtype = dtype; cfg.tp_size = 1; cfg.tp_rank = 0; cfg.arch = LMB200_ARCH_LLAMA;

  lmb200_ctx ctx = 0;
  lmb200_model model = 0;
  lmb200_session sess = 0;
  CHECK(lmb200_init(0, &ctx));
  CHECK(lmb200_model_create(ctx, &cfg, &model));
  CHECK(lmb200_model_init_random(model, seed, 0.02f));
  CHECK(lmb200_session_create(model, batch, prompt + steps + 1, &sess));

  int32_t* toks = (int32_t*)malloc(sizeof(int32_t) * (size_t)batch * (size_t)prompt);
  float* logits = (float*)malloc(sizeof(float) * (size_t)batch * (size_t)cfg.vocab);
  int32_t* first = (int32_t*)malloc(sizeof(int32_t) * (size_t)batch);
  int32_t* out = (int32_t*)malloc(sizeof(int32_t) * (size_t)batch * (size_t)steps);
  if (!toks || !logits || !first || !out) return 3;
  for (int b = 0; b < batch; ++b)
    for (int i = 0; i < prompt; ++i) toks[b * prompt + i] = (7 * i + 3 + 11 * b) % cfg.vocab;

  CHECK(lmb200_prefill(sess, toks, prompt, logits));
  for (int b = 0; b < batch; ++b) {          /* first index of the maximum, as argmax does */
    int best = 0;
    for (int v = 1; v < cfg.vocab; ++v)
      if (logits[b * cfg.vocab + v] > logits[b * cfg.vocab + best]) best = v;
    first[b] = best;
  }
  /* one step through the host-buffer call, the rest through the device-resident loop */
  CHECK(lmb200_decode_step(sess, first, out, NULL));
  if (steps > 1) CHECK(lmb200_decode_n(sess, out, steps - 1, out + batch));
  int32_t pos = -1;
  CHECK(lmb200_session_position(sess, &pos));

  printf("{\"position\": %d, \"first\": [", (int)pos);
  for (int b = 0; b < batch; ++b) printf("%s%d", b ? ", " : "", (int)first[b]);
  printf("], \"tokens\": [");
  for (int i = 0; i < batch * steps; ++i) printf("%s%d", i ? ", " : "", (int)out[i]);
  printf("]}\n");

  free(toks); free(logits); free(first); free(out);
  CHECK(lmb200_session_destroy(sess));
  CHECK(lmb200_model_destroy(model));
  CHECK(lmb200_shutdown(ctx));
  return 0;
}
