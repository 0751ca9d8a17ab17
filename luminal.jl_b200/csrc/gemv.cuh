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
  EPI_GELU_ACT = 3,    // act[b, row] = gelu(acc)                  (Whisper fc1)
  EPI_RESID_NORM = 4   // row-parallel projection + all-reduce + residual add + RMSNorm preparation (ResidNorm below)
};

// Exchange of a row-parallel projection's partial results between the tensor-parallel ranks, done by
// the projection's own CTAs.  The CTA that finalises a tile of rows stores its partial (bf16) into the
// same place of EVERY rank's exchange region with plain peer stores, and then reads the peers' partials
// of its tile from its OWN region, where every element starts as bf16 -0.0 ("not written yet", a value
// the senders never send): a thread simply re-reads its 16 bytes per peer until none of the eight
// elements is that pattern (bounded).  No flag and no fence sit between a partial and its use, so the
// exchange costs one NVLink transit.  The n partials are added in rank order -- every rank adds the
// same bf16 values in the same order, so the replicated residual stream stays bit-identical across
// ranks -- and the thread puts the "not written yet" pattern back.  Two buffers alternate: a peer
// writes a buffer again only two reductions later, and it can start that reduction only after it has
// this rank's partial of the one in between, which a later kernel than the one that cleared sends.
// A flag per (source rank, CTA) still travels beside the data, unordered with it, as a validity
// channel: the epoch, marked when the sender had a wait run out earlier.  It is checked after the sum,
// so that a rank that ran a step the others never saw cannot feed them its leftovers silently.
constexpr int kPushMaxCtas = 256;      // flag slots per source rank
struct PeerPush {
  int n = 0, rank = 0;
  __nv_bfloat16* part[8];                  // rank r's buffer of this reduction: [src rank][row][Bp] bf16
  unsigned long long* flag[8];             // rank r's flag array: [src rank][kPushMaxCtas]
  const unsigned long long* step = nullptr;
  unsigned phase = 0;
  int* dev_err = nullptr;
  int* broken = nullptr;
  long long wait_cycles = 0;
};

// EPI_RESID_NORM: the residual stream and what the next Linear needs of its RMSNorm.
//   x[row][b] += sum over ranks of acc                          (x: float32 [rows][Bp], batch fastest)
//   xg[b, row] = bf16(x * gain[row])                            (the next GEMV's activation buffer)
//   ssq[cta][b] = sum over this CTA's rows of x^2               (one slot per CTA, summed by the consumer)
// RMSNorm's scale recip(sqrt(mean(x*x) + eps)) is one number per sequence, so it commutes with the
// next Linear: W ((x inv) g) = inv (W (x g)); the consumer multiplies its accumulators by it (InvScale).
// src/HighLevelOps.jl:299-304, src/NN.jl:149-161, 406-414.
struct ResidNorm {
  float* x = nullptr;
  const float* gain = nullptr;
  void* xg = nullptr;
  float* ssq = nullptr;
  float* sum = nullptr;                    // LayerNorm: sum over this CTA's rows of x, slots like ssq (NULL: RMSNorm)
  float* capture = nullptr;                // [B][rows] float32 copy of the new residual rows (parity tests) or NULL
};

// Consumer side: inv[b] = 1 / sqrt(sum_t ssq[t][b] * (1/n) + eps) multiplies every accumulator of batch
// column b before the rest of the epilogue.  ssq == NULL: no scaling.
// LayerNorm (sum != NULL; src/NN.jl:138-173, src/HighLevelOps.jl:292-304): with mu = mean(x) and inv = 1 / sqrt(mean(x*x)
// - mu*mu + eps), W ((x - mu) inv g + b) = inv (W (x g)) - inv mu (W g) + W b: the consumer multiplies its accumulators
// by inv, subtracts inv mu wg[row] (GemvParams::ln_wg = W g) and adds a bias that already holds W b.
struct InvScale {
  const float* ssq = nullptr;
  const float* sum = nullptr;
  int tiles = 0;                           // slots written by the producer (its CTA count)
  int n = 0;                               // row length of the norm (hidden)
  float eps = 0.f;
};

// bf16 kernel (float32 always runs the register-ring kernel): tcgen05.mma, accumulators in TMEM
enum GemvVariant { GEMV_TCGEN05 = 0 };

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
  const int* pos = nullptr;          // device [B]: the position each sequence's new key is written at
  int pos_uniform = 1;               // the host knows all B positions are equal (one sine / cosine per row)
  int Hl = 0, KVl = 0, D = 0;
  int rope = 1;                      // 0: no rotation (Whisper), q and k rows are only scaled
  float qk_scale = 1.f;              // multiplies q and k rows (Whisper: head_dim^-0.25, src/Whisper.jl:257)
  // every epilogue: added to the accumulator first, one value per internal row (NULL: none)
  const float* bias = nullptr;
  InvScale inv;              // per-sequence RMSNorm scale applied to the accumulators (before the bias)
  const float* ln_wg = nullptr;  // LayerNorm input: W g per internal row (see InvScale)
  ResidNorm rn;              // EPI_RESID_NORM
  PeerPush push;             // EPI_RESID_NORM under tensor parallelism (n > 1)
  // L2 prefetch for the GEMV that runs next (bf16 tensor-core kernels): once a CTA's producer has issued
  // its last copy, HBM would idle through this kernel's fold, epilogue and drain; instead it pulls the
  // head of every next-kernel CTA's weight range into L2.  The next matrix has pf_units 32 KB units;
  // CTA i of its pf_parts CTAs starts at unit i * pf_units / pf_parts; pf_chunk units are fetched per part.
  const void* pf_base = nullptr;
  int pf_units = 0, pf_parts = 0, pf_chunk = 0;
};


struct GemvPlan {
  int ksplit = 1, kc_per_split = 0, grid = 0, cluster = 0;      // cluster == 1 is valid for EPI_RESID_NORM (one CTA per row group)
  int64_t partial_floats = 0;
  int n_counters = 0;
};

int32_t gemv_configure();
void gemv_set_variant(int variant);
int gemv_variant();
GemvPlan gemv_plan(const Ctx* ctx, int dtype, int B, int rows, int K);
// Plan for a projection that runs EPI_RESID_NORM: always the cluster kernel (a cluster of 1 when no larger one fits);
// cluster == 0 in the result means the shape cannot run it (more than one wave of row groups).
GemvPlan gemv_plan_resid(const Ctx* ctx, int B, int rows, int K);
// CTAs the planned launch has (the number of ssq slots an EPI_RESID_NORM launch writes)
int gemv_plan_ctas(const GemvPlan& pl, int rows);
// Fills the prefetch fields of `p` from the matrix (and plan) of the GEMV that follows it.
void gemv_prefetch_next(GemvParams& p, const Ctx* ctx, int dtype, const void* next_W, int next_rows, int next_K,
                        const GemvPlan& next_plan);
// dtype: LMB200_F32 or LMB200_BF16
int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream);

}  // namespace lmb
