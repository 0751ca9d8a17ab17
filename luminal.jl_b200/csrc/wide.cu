// A session of more than 32 sequences.  The GEMV kernels hold one batch tile of at most 32 columns in tensor memory,
// so a wider batch runs as a row of sub-sessions of at most 32 sequences each over the same model (weights, embedding
// and head are shared; every sub-session has its own cache, scratch and CUDA graphs).  A step streams the weights once
// per sub-session: the reference's Llama / Phi-3 accept any batch (src/NN.jl:448-455), and so does this entry, at the
// cost of one weight pass per 32 sequences.  Llama / Phi-3 on one GPU only.
#include <cstring>
#include <vector>

#include "model.cuh"

namespace lmb {
namespace {

constexpr int kPart = 32;

// f(sub-session handle, its first sequence, its sequence count) for every sub-session, stopping at the first error
template <class F>
int32_t each_part(Session* S, F f) {
  int b0 = 0;
  for (uint64_t h : S->parts) {
    Session* P = session_from(h);
    if (!P) return LMB200_EINVAL;
    const int32_t rc = f(h, b0, P->B);
    if (rc != LMB200_OK) return rc;
    b0 += P->B;
  }
  return LMB200_OK;
}

}  // namespace

int32_t wide_create(Model* M, int batch, int max_ctx, lmb200_session* out) {
  LMB_REQUIRE(M->cfg.arch != LMB200_ARCH_WHISPER_DECODER, "session_create: batch %d above 32 is built for Llama / Phi-3 only", batch);
  LMB_REQUIRE(M->ctx->tp_size == 1, "session_create: batch %d above 32 is not built for tensor parallelism", batch);
  LMB_REQUIRE(batch <= 4096, "session_create: batch %d above 4096", batch);
  Session* S = new Session();
  S->m = M; S->B = batch; S->max_ctx = max_ctx;
  for (int b0 = 0; b0 < batch; b0 += kPart) {
    lmb200_session p = 0;
    const int32_t rc = lmb200_session_create(reinterpret_cast<lmb200_model>(M), batch - b0 < kPart ? batch - b0 : kPart, max_ctx, &p);
    if (rc != LMB200_OK) { wide_destroy(S); return rc; }
    S->parts.push_back(p);
  }
  *out = reinterpret_cast<lmb200_session>(S);
  return LMB200_OK;
}

int32_t wide_destroy(Session* S) {
  for (uint64_t h : S->parts) lmb200_session_destroy(h);
  S->parts.clear();
  S->magic = 0;
  delete S;
  return LMB200_OK;
}

int32_t wide_reset(Session* S) {
  return each_part(S, [](uint64_t h, int, int) { return lmb200_session_reset(h); });
}

int32_t wide_position(Session* S, int32_t* pos) {
  *pos = 0;
  return each_part(S, [&](uint64_t h, int, int) {
    int32_t p = 0;
    const int32_t rc = lmb200_session_position(h, &p);
    if (p > *pos) *pos = p;
    return rc;
  });
}

int32_t wide_set_position(Session* S, int32_t pos) {
  return each_part(S, [&](uint64_t h, int, int) { return lmb200_session_set_position(h, pos); });
}

int32_t wide_set_positions(Session* S, const int32_t* pos) {
  return each_part(S, [&](uint64_t h, int b0, int) { return lmb200_session_set_positions(h, pos + b0); });
}

int32_t wide_positions(Session* S, int32_t* pos_out) {
  return each_part(S, [&](uint64_t h, int b0, int) { return lmb200_session_positions(h, pos_out + b0); });
}

int32_t wide_fill_kv_random(Session* S, int32_t n_pos, uint64_t seed) {
  return each_part(S, [&](uint64_t h, int b0, int) { return lmb200_session_fill_kv_random(h, n_pos, seed + (uint64_t)b0); });
}

int32_t wide_set_capture(Session* S, int32_t enable) {
  return each_part(S, [&](uint64_t h, int, int) { return lmb200_session_set_capture(h, enable); });
}

int32_t wide_read_layer_output(Session* S, int32_t layer, float* host) {
  const int64_t hidden = S->m->cfg.hidden;
  return each_part(S, [&](uint64_t h, int b0, int) { return lmb200_session_read_layer_output(h, layer, host ? host + b0 * hidden : nullptr); });
}

int32_t wide_prefill(Session* S, const int32_t* tokens, int32_t n, float* logits_out) {
  const int64_t vocab = S->m->cfg.vocab;
  return each_part(S, [&](uint64_t h, int b0, int) {
    return lmb200_prefill(h, tokens + (int64_t)b0 * n, n, logits_out ? logits_out + b0 * vocab : nullptr);
  });
}

int32_t wide_prefill_ragged(Session* S, const int32_t* tokens, const int32_t* lengths, int32_t n_max, float* logits_out) {
  const int64_t vocab = S->m->cfg.vocab;
  return each_part(S, [&](uint64_t h, int b0, int) {
    return lmb200_prefill_ragged(h, tokens + (int64_t)b0 * n_max, lengths + b0, n_max, logits_out ? logits_out + b0 * vocab : nullptr);
  });
}

int32_t wide_decode_step(Session* S, const int32_t* tokens_in, int32_t* next_tokens_out, float* logits_out) {
  const int64_t vocab = S->m->cfg.vocab;
  return each_part(S, [&](uint64_t h, int b0, int) {
    return lmb200_decode_step(h, tokens_in ? tokens_in + b0 : nullptr, next_tokens_out ? next_tokens_out + b0 : nullptr,
                              logits_out ? logits_out + b0 * vocab : nullptr);
  });
}

// tokens_out is [n_steps][batch]: every sub-session fills its columns
int32_t wide_decode_n(Session* S, const int32_t* first_tokens, int32_t n_steps, int32_t* tokens_out) {
  LMB_REQUIRE(n_steps >= 1, "decode_n: n_steps %d", n_steps);
  const int B = S->B;
  std::vector<int32_t> part((size_t)n_steps * kPart);
  return each_part(S, [&](uint64_t h, int b0, int nb) {
    const int32_t rc = lmb200_decode_n(h, first_tokens ? first_tokens + b0 : nullptr, n_steps, tokens_out ? part.data() : nullptr);
    if (rc == LMB200_OK && tokens_out)
      for (int s = 0; s < n_steps; ++s)
        for (int b = 0; b < nb; ++b) tokens_out[(size_t)s * B + b0 + b] = part[(size_t)s * nb + b];
    return rc;
  });
}

// Every sub-session runs the loop to its own end; the whole batch ends with the step in which its last sequence
// finished (or at the caps), and the rows a sub-session did not reach hold the end-of-text id, as they would in
// one session.
int32_t wide_decode_until(Session* S, const int32_t* first_tokens, int32_t max_steps, int32_t eot_token, int32_t* tokens_out,
                          int32_t* steps_done) {
  LMB_REQUIRE(steps_done && max_steps >= 1, "decode_until: bad argument");
  const int B = S->B;
  std::vector<int32_t> all((size_t)max_steps * B, eot_token), part((size_t)max_steps * kPart);
  int longest = 0;
  *steps_done = 0;
  const int32_t rc = each_part(S, [&](uint64_t h, int b0, int nb) {
    int32_t done = 0;
    const int32_t r = lmb200_decode_until(h, first_tokens ? first_tokens + b0 : nullptr, max_steps, eot_token, part.data(), &done);
    if (r != LMB200_OK) return r;
    for (int s = 0; s < done; ++s)
      for (int b = 0; b < nb; ++b) all[(size_t)s * B + b0 + b] = part[(size_t)s * nb + b];
    if (done > longest) longest = done;
    return r;
  });
  if (rc != LMB200_OK) return rc;
  if (tokens_out) memcpy(tokens_out, all.data(), (size_t)longest * B * 4);
  *steps_done = longest;
  return LMB200_OK;
}

int32_t wide_step_bytes(Session* S, int32_t T, int64_t* bytes) {
  *bytes = 0;
  return each_part(S, [&](uint64_t h, int, int) {
    int64_t b = 0;
    const int32_t rc = lmb200_session_step_bytes(h, T, &b);
    *bytes += b;
    return rc;
  });
}

}  // namespace lmb
