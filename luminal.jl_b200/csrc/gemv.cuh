// Decode-time Linear layers: y[b, o] = sum_i x[b, i] * W[o, i] for a handful of rows b (the
// batch), i.e. a GEMV / skinny GEMM that is bound by streaming W from HBM once.
// Replaces NN.Linear -> MatMul for S = 1 (src/NN.jl:22-35, src/Execution.jl:56-90).
#pragma once
#include "common.cuh"

namespace lmb {

enum GemvEpilogue {
  EPI_STORE_F32 = 0,   // out[b, row] = acc                       (o_proj, down_proj, lm_head)
  EPI_SILU_GATE = 1,   // act[b, i] = silu(gate_i) * up_i         (rows interleaved 8 gate / 8 up)
  EPI_QKV_ROPE = 2     // RoPE on q and k, q -> q_out, k/v appended to the cache at *pos
};

struct GemvParams {
  const void* W = nullptr;   // tiled weights (wtile_offset)
  const void* x = nullptr;   // tiled activations (xtile_offset), same element type as W
  int B = 0;
  int rows = 0;              // valid logical rows (<= 16*RB)
  int RB = 0;                // 16-row blocks
  int KC = 0;                // 32-wide k chunks
  // work split, filled by gemv_plan
  int ksplit = 1;            // ring kernel: k-splits (gridDim.y)
  int kc_per_split = 0;
  int grid = 0;              // stream kernel: number of CTAs
  float* partials = nullptr;     // split-K scratch
  unsigned* counters = nullptr;  // one per row group, zero between launches
  int epi = EPI_STORE_F32;
  // EPI_STORE_F32
  float* out = nullptr;
  int out_pitch = 0;
  // EPI_SILU_GATE: act is a tiled activation buffer of the same batch padding as x
  void* act = nullptr;
  int n_act = 0;
  // EPI_QKV_ROPE
  void* q_out = nullptr;     // [B, q_pitch], head-major (local head * D + d)
  int q_pitch = 0;
  void* kv_layer = nullptr;  // this layer's cache: [B, KVl, blocks, 32*D]
  int64_t kv_batch_stride = 0;
  int64_t kv_head_stride = 0;
  const float* inv_freq = nullptr;   // [D/2]
  const int* pos = nullptr;          // device scalar: position the new key is written at
  int Hl = 0, KVl = 0, D = 0;
};

struct GemvPlan {
  int ksplit = 1, kc_per_split = 0, grid = 0;
  int64_t partial_floats = 0;
  int n_counters = 0;
};

int32_t gemv_configure();
// bf16 kernel choice: true = bulk-TMA stream-K kernel (default), false = register-ring kernel
void gemv_set_stream_kernel(bool on);
GemvPlan gemv_plan(const Ctx* ctx, int dtype, int B, int RB, int KC);
// dtype: LMB200_F32 or LMB200_BF16
int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream);

}  // namespace lmb
