// Split-KV decode attention over the tiled GQA cache (one new query per sequence).
// Replaces the S = 1 case of SelfAttention's QK^T -> softmax -> PV (src/NN.jl:369-386, with
// repeat_kv's mapping q head = kv + KV*g, src/NN.jl:305-317) and whisper_self_attn_cached's
// attention over [0, step_pos] (src/Whisper.jl:606-617).
#pragma once
#include "common.cuh"

namespace lmb {

struct AttnParams {
  const void* q = nullptr;        // [B, q_pitch]; local q head (kvl*G + g) at column (kvl*G+g)*D
  int q_pitch = 0;
  const void* kv_layer = nullptr; // tiled cache of one layer: [B, KVl, blocks, 32*D]
  int64_t kv_batch_stride = 0;
  int64_t kv_head_stride = 0;
  int B = 0, KVl = 0, G = 0, D = 0;
  const int* pos = nullptr;       // device [B]; context length of sequence b is pos[b] + 1 (NULL -> T_fixed for all)
  int T_fixed = 0;
  int keys_per_cta = 0;           // multiple of 64
  int nsplit = 0;                 // gridDim.y, covers the cache capacity
  float scale = 1.f;              // 1/sqrt(D)
  float* part_o = nullptr;        // scratch [B*KVl, nsplit, G, D]
  float* part_ml = nullptr;       // scratch [B*KVl, nsplit, G, 2]  (max, sum)
  void* out = nullptr;            // [B, out_pitch], same head-major order as q ...
  int out_pitch = 0;
  int out_tiled_bp = 0;           // ... or, when > 0, a GEMV activation buffer (Layout<T>::x_offset) of that padding
  unsigned* counters = nullptr;   // [B*KVl] zeros: the last CTA of a (sequence, kv head) merges the splits (bf16); NULL: separate kernel
};

int32_t attn_configure();
// scratch floats needed: part_o, part_ml
void attn_plan(const Ctx* ctx, int B, int KVl, int G, int D, int ctx_capacity, int* keys_per_cta,
               int* nsplit, int64_t* part_o_floats, int64_t* part_ml_floats);
int32_t attn_decode_launch(Ctx* ctx, int dtype, const AttnParams& p, cudaStream_t stream);

}  // namespace lmb
