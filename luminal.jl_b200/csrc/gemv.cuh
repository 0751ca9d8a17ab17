// Decode-time Linear layers: y[b, o] = sum_i x[b, i] * W[o, i] for a handful of rows b (the
// batch), i.e. a GEMV / skinny GEMM that is bound by streaming W from HBM once.
// Replaces NN.Linear -> MatMul for S = 1 (src/NN.jl:22-35, src/Execution.jl:56-90).
#pragma once
#include "common.cuh"

namespace lmb {

enum GemvEpilogue {
  EPI_STORE_F32 = 0,   // out[b, row] = acc                       (o_proj, down_proj, lm_head)
  EPI_SILU_GATE = 1,   // act[b, i] = silu(gate_i) * up_i         (rows interleaved 8 gate / 8 up)
  EPI_QKV_ROPE = 2,    // RoPE on q and k (if `rope`), q -> q_out, k/v appended to the cache at *pos
  EPI_GELU_ACT = 3     // act[b, row] = gelu(acc)                  (Whisper fc1)
};

// bf16 kernel variants (float32 always runs the register-ring kernel)
enum GemvVariant {
  GEMV_TCGEN05 = 0,    // tcgen05.mma, accumulators in TMEM (default)
  GEMV_MMA_SYNC = 1    // mma.sync m16n8k16 from ldmatrix
};

struct GemvParams {
  const void* W = nullptr;   // weights in Layout<WT>::w_offset order
  const void* x = nullptr;   // activations in Layout<WT>::x_offset order, same element type as W
  int B = 0;
  int rows = 0;              // valid internal rows
  int K = 0;                 // valid reduction length
  int RB = 0;                // float32 ring kernel: 16-row blocks
  int KC = 0;                //                      32-wide k chunks
  // work split, filled from gemv_plan
  int ksplit = 1;            // ring: k-splits (gridDim.y); bf16: contributors reserved per row group
  int kc_per_split = 0;
  int grid = 0;              // bf16 kernels: number of CTAs
  int cluster = 0;           // > 1: one thread-block cluster of this size per 128-row group (small matrices)
  float* partials = nullptr;     // split-K scratch
  unsigned* counters = nullptr;  // zero between launches
  int epi = EPI_STORE_F32;
  // EPI_STORE_F32
  float* out = nullptr;
  int out_pitch = 0;
  // EPI_SILU_GATE: act is a GEMV activation buffer of the same batch padding as x
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
  int rope = 1;                      // 0: no rotation (Whisper), q and k rows are only scaled
  float qk_scale = 1.f;              // multiplies q and k rows (Whisper: head_dim^-0.25, src/Whisper.jl:257)
  // every epilogue: added to the accumulator first, one value per internal row (NULL: none)
  const float* bias = nullptr;
  // L2 prefetch for the GEMV that runs next (bf16 tensor-core kernels): once a CTA's producer has issued
  // its last copy, HBM would idle through this kernel's fold, epilogue and drain; instead it pulls the
  // head of every next-kernel CTA's weight range into L2.  The next matrix has pf_units 32 KB units;
  // CTA i of its pf_parts CTAs starts at unit i * pf_units / pf_parts; pf_chunk units are fetched per part.
  const void* pf_base = nullptr;
  int pf_units = 0, pf_parts = 0, pf_chunk = 0;
};


struct GemvPlan {
  int ksplit = 1, kc_per_split = 0, grid = 0, cluster = 0;
  int64_t partial_floats = 0;
  int n_counters = 0;
};

int32_t gemv_configure();
void gemv_set_variant(int variant);
int gemv_variant();
GemvPlan gemv_plan(const Ctx* ctx, int dtype, int B, int rows, int K);
// Fills the prefetch fields of `p` from the matrix (and plan) of the GEMV that follows it.
void gemv_prefetch_next(GemvParams& p, const Ctx* ctx, int dtype, const void* next_W, int next_rows, int next_K,
                        const GemvPlan& next_plan);
// dtype: LMB200_F32 or LMB200_BF16
int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream);

}  // namespace lmb
