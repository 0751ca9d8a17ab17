// Prompt phase of the Llama / Phi-3 path (bf16): all positions of all sequences at once.
//
// The reference runs the model over the whole prompt as one graph -- Linear on [B, S, hidden]
// through batch_matmul (src/Execution.jl:12-54), SelfAttention with a materialised [B, H, S, S]
// score tensor and a -1e9 mask (src/NN.jl:343-387).  Here the Linears are one tensor-core GEMM
// each (tcgen05.mma, accumulators in TMEM) and attention is the tensor-core flash kernel with
// grouped kv heads; K and V are also appended to the decode cache.
//
// gemm_tc_kernel: acc[row, token] = sum_k W[row, k] * X[token, k]
//   one CTA = 128 weight rows x 128 tokens, k in steps of 64 through a 6-stage ring:
//   warp 5      : one thread issues, per step, a bulk copy of half a weight unit (16 KB, already in
//                 the tensor core's layout) and a 3-D TMA box of the row-major activations that lands
//                 in the same layout,
//   warp 4      : one thread issues tcgen05.mma 128 x 128 x 16,
//   warps 0..3  : epilogue, one weight row per thread, tcgen05.ld 32 tokens at a time:
//                 store float32 / SiLU(gate) * up / RoPE + q, k, v (and the cache).
#include <cuda.h>
#include <math_constants.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include "model.cuh"
#include "tc.cuh"

namespace lmb {

int32_t flash_tc_launch_view(Ctx* ctx, void* out, const void* q, const void* k, const void* v, const FlashView& fv, int64_t B,
                             int64_t S, int64_t D, float scale, int causal, cudaStream_t stream);
bool flash_tc_supported(int64_t D);

namespace {

constexpr int kGemmThreads = 6 * 32;
constexpr int kUnitBytes = 32768;
constexpr int kEpiStageBytes = 32 * 80;        // per epilogue warp: 32 tokens x 32 bf16 outputs, rows of 80 bytes
constexpr float kInvLn2 = 1.4426950408889634f;
constexpr float kHalfPi = 1.5707963267948966f;

enum GemmEpilogue { GEMM_STORE_F32 = 0, GEMM_SILU_GATE = 1, GEMM_QKV_ROPE = 2, GEMM_AFFINE = 3, GEMM_CROSS_KV = 4 };

struct GemmParams {
  const __nv_bfloat16* W = nullptr;     // canonical 128 x 128 units, unit (row group, k step) at (rg * KS + ks) * 16384
  const __nv_bfloat16* X = nullptr;     // [T, ldx] row-major
  int ldx = 0, T = 0, rows = 0, K = 0;
  int epi = GEMM_STORE_F32;
  float* out = nullptr;                 // GEMM_STORE_F32: out[token * ldo + row]
  int ldo = 0;
  __nv_bfloat16* act = nullptr;         // GEMM_SILU_GATE: act[token * ld_act + i], rows interleaved 8 gate / 8 up
  int ld_act = 0, n_act = 0;
  // GEMM_QKV_ROPE: token t = b * n_seq + s sits at position pos0 + s of sequence b
  __nv_bfloat16* q = nullptr;           // [T, ldq]: local head * D + d
  __nv_bfloat16* kbuf = nullptr;        // [T, ldkv]: local kv head * D + d
  __nv_bfloat16* vbuf = nullptr;
  int ldq = 0, ldkv = 0;
  __nv_bfloat16* kv_layer = nullptr;    // the decode cache of this layer
  int64_t kv_batch_stride = 0, kv_head_stride = 0;
  // GEMM_AFFINE: y = (acc + bias[row]) -> gelu? -> * out_scale, stored float32 or bf16 at out_any[token * ldo + row]
  // GEMM_CROSS_KV: the same y as bf16 into a tiled cache layer: row = head * D + d, token = b * n_seq + position
  const float* bias = nullptr;
  float out_scale = 1.f;
  int gelu = 0, out_bf16 = 0, is_v = 0;
  void* out_any = nullptr;
  const float2* rope = nullptr;         // [n_seq, D/2]: (sin, cos) of position pos0 + s times inv_freq[d0]
  int pos0 = 0, n_seq = 1, Hl = 0, KVl = 0, D = 0;
  // Implicit 1-D convolution (conv_taps > 0; src/NN.jl:55-104 without the unfolded buffer): X is the token-major input
  // [conv_B][conv_rows_in][ldx] (channels contiguous, conv_rows_in a multiple of the stride conv_P, rows past the valid
  // input zero), output position o of batch b reads input rows o * conv_P + tap - conv_pad (rows outside the tensor read
  // as zeros: the padding), K = conv_taps * conv_cpad with W's column tap * conv_cpad + c the weight of (c, tap).  The
  // accumulator of (b, o) is stored at token index b * conv_out_rpb + o.
  int conv_taps = 0, conv_P = 1, conv_pad = 0, conv_C = 0, conv_cpad = 0, conv_B = 0, conv_rows_in = 0, conv_Lout = 0, conv_out_rpb = 0;
};

// GELU with the reference's tanh (src/HighLevelOps.jl:162-168): tanh z = sigmoid(2z) * 2 - 1
__device__ __forceinline__ float gelu_ref(float a) {
  const float inner = (0.7978845608f * a) * (1.0f + (0.044715f * a) * a);
  const float z = inner * 2.0f;
  const float sg = 1.0f / (1.0f + exp2f((z * -1.0f) * kInvLn2));
  const float th = sg * 2.0f + -1.0f;
  return (a * 0.5f) * (1.0f + th);
}

// v[i] = accumulator of (row, token t0 + i).  Rows g and g+8 of a 16-row block, which the fused
// epilogues combine, are 8 lanes apart.
__device__ __forceinline__ void gemm_epilogue(const GemmParams& p, float (&v)[32], int row, int t0, int t_end, unsigned char* stage) {
  const int rb = row >> 4, rr = row & 15, g = rr & 7, hi = rr >> 3;
  if (p.epi == GEMM_STORE_F32) {
    if (row < p.rows) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (t0 + i < t_end) p.out[(int64_t)(t0 + i) * p.ldo + row] = v[i];
    }
    return;
  }
  if (p.epi == GEMM_AFFINE || p.epi == GEMM_CROSS_KV) {
    if (row >= p.rows) return;
    const float bias = p.bias ? p.bias[row] : 0.f;
    const int h = p.epi == GEMM_CROSS_KV ? row / p.D : 0, d = p.epi == GEMM_CROSS_KV ? row - h * p.D : 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int t = t0 + i;
      if (t >= t_end) continue;
      float y = v[i] + bias;
      if (p.gelu) y = gelu_ref(y);
      y *= p.out_scale;
      if (p.epi == GEMM_CROSS_KV) {
        const int b = t / p.n_seq, pos = t - b * p.n_seq;
        p.kv_layer[b * p.kv_batch_stride + h * p.kv_head_stride + (p.is_v ? vcache_offset(pos, d, p.D) : kcache_offset(pos, d, p.D))] =
            __float2bfloat16_rn(y);
      } else if (p.out_bf16) {
        reinterpret_cast<__nv_bfloat16*>(p.out_any)[(int64_t)t * p.ldo + row] = __float2bfloat16_rn(y);
      } else {
        reinterpret_cast<float*>(p.out_any)[(int64_t)t * p.ldo + row] = y;
      }
    }
    return;
  }
  // The fused epilogues below give every thread (one row) 32 tokens of one column of the output: stored directly,
  // a warp's store instruction would write 16-byte pieces of 32 different token rows.  Instead the warp turns its
  // 32 x 32 block round through its own 2.5 KB of shared memory (rows of 80 bytes: conflict-free both ways), after
  // which lane L holds token t0 + L's 32 outputs and writes them as 16-byte vectors.
  float w[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i] = __shfl_xor_sync(0xffffffffu, v[i], 8);
  const int lane = threadIdx.x & 31;
  const int rbl = (row >> 4) & 1;                      // which of the warp's two 16-row blocks
  const int row0 = row & ~31;                          // the warp's first row: rows row0 .. row0 + 31 (a multiple of 32)
  __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(stage);
  constexpr int kPitch = 40;                           // bf16 elements per staged token row (80 bytes)
  const int tL = t0 + lane;                            // the token this lane stores after the turn
  if (p.epi == GEMM_SILU_GATE) {
    // column of (rb, g): rbl * 8 + g, 16 outputs per token = act[t, (row0 / 16) * 8 .. + 16)
    if (hi == 0) {
      const int col = rbl * 8 + g;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float a = v[i], u = w[i];
        const float ex = exp2f((a * -1.0f) * kInvLn2);          // src/HighLevelOps.jl:153-160
        const float sg = 1.0f / (1.0f + ex);
        st[i * kPitch + col] = __float2bfloat16_rn((a * sg) * u);
      }
    }
    __syncwarp();
    const int o0 = (row0 >> 4) * 8;
    if (tL < t_end && o0 < p.n_act) {
      __nv_bfloat16* dst = p.act + (int64_t)tL * p.ld_act + o0;
      const uint4* src = reinterpret_cast<const uint4*>(st + lane * kPitch);
      if (o0 + 16 <= p.n_act && (p.ld_act & 7) == 0) {
        reinterpret_cast<uint4*>(dst)[0] = src[0];
        reinterpret_cast<uint4*>(dst)[1] = src[1];
      } else {
        for (int c = 0; c < 16 && o0 + c < p.n_act; ++c) dst[c] = st[lane * kPitch + c];
      }
    }
    __syncwarp();
    return;
  }
  // GEMM_QKV_ROPE
  const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
  const int hs = rb / tiles_per_head, jj = rb - hs * tiles_per_head;
  const int jj0 = jj - rbl;                            // the warp's first 16-row block inside the head (even)
  const bool live = row0 < p.rows;                     // uniform over the warp (rows is a multiple of 32 here)
  if (hs < p.Hl + p.KVl) {
    const int d0 = 8 * jj + g;                         // rows g / g+8 are the pair (d0, d0 + D/2), src/NN.jl:253-303
    // staged columns: [0, 16) = d 8*jj0 .. + 15, [16, 32) = D/2 + the same
    const int col = rbl * 8 + g + (hi ? 16 : 0);
    if (live) {
      // all table reads of the chunk first: between stores the compiler could not move them
      float2 sc[32];
      int sq = t0 % p.n_seq;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        sc[i] = (t0 + i < t_end) ? __ldg(p.rope + (int64_t)sq * half + d0) : make_float2(0.f, 1.f);
        if (++sq == p.n_seq) sq = 0;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float sn = sc[i].x, cs = sc[i].y;
        const float o = hi ? (w[i] * sn + v[i] * cs) : (v[i] * cs + (w[i] * sn) * -1.0f);
        st[i * kPitch + col] = __float2bfloat16_rn(o);
      }
    }
    __syncwarp();
    if (live && tL < t_end) {
      __nv_bfloat16* base = hs < p.Hl ? p.q + (int64_t)tL * p.ldq + hs * D : p.kbuf + (int64_t)tL * p.ldkv + (hs - p.Hl) * D;
      const uint4* src = reinterpret_cast<const uint4*>(st + lane * kPitch);
      uint4* lo = reinterpret_cast<uint4*>(base + 8 * jj0);
      uint4* up = reinterpret_cast<uint4*>(base + half + 8 * jj0);
      lo[0] = src[0]; lo[1] = src[1];
      up[0] = src[2]; up[1] = src[3];
    }
  } else {
    const int kvh = hs - p.Hl - p.KVl;
    const int col = rbl * 16 + rr;                     // d = 16 * jj0 + col
    if (live) {
#pragma unroll
      for (int i = 0; i < 32; ++i) st[i * kPitch + col] = __float2bfloat16_rn(v[i]);
    }
    __syncwarp();
    if (live && tL < t_end) {
      uint4* dst = reinterpret_cast<uint4*>(p.vbuf + (int64_t)tL * p.ldkv + kvh * D + 16 * jj0);
      const uint4* src = reinterpret_cast<const uint4*>(st + lane * kPitch);
#pragma unroll
      for (int c = 0; c < 4; ++c) dst[c] = src[c];
    }
  }
  __syncwarp();
}

// Tile order: groups of `gt` token tiles (their activations, about 64 MB, stay in L2); inside a
// group the row groups follow one another and the token tile is the fast index, so the CTAs running
// at one time share a few weight row groups and the weights stream from HBM once per group.
struct TileOrder {
  int n_tt, n_rg, gt;
  __device__ __forceinline__ void decode(int tile, int* rg, int* tt) const {
    const int per_group = gt * n_rg;
    const int grp = tile / per_group, within = tile - grp * per_group;
    const int tt0 = grp * gt;
    const int width = min(gt, n_tt - tt0);          // the last group may be narrower
    // tiles of the last group are numbered with its own width
    const int w_rg = within / width;
    *rg = w_rg;
    *tt = tt0 + (within - w_rg * width);
  }
};

// Shared-memory descriptor of a K-major operand tile whose rows are 128 bytes (64 bf16) in the 128-byte
// swizzle a tensor map with CU_TENSOR_MAP_SWIZZLE_128B writes: groups of 8 rows are 1024 bytes apart
// (stride byte offset), the leading byte offset is not used (1), layout type 2.  The tile starts on a
// 1024-byte boundary; a K = 16 step inside the row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// BN tokens per tile (128 or 256).  256 halves the number of MMA instructions and barrier round trips
// per flop and doubles the reuse of each weight byte read from shared memory; its two accumulators
// take all 512 TMEM columns.
template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap,
                                                                  int* err) {
  using namespace tc;
  constexpr int kGemmBN = BN;
  constexpr int kGemmStages = BN == 256 ? 4 : 6;
  constexpr int kABytes = kUnitBytes / 2;                 // 128 rows x 64 k: half a weight unit (its first / last 8 k-groups)
  constexpr int kBBytes = kGemmBN * 128;                  // BN tokens x 64 k, bf16: one 128-byte swizzled row per token
  constexpr int kStage = kABytes + kBBytes;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kGemmStages], empty[kGemmStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int KS = (p.K + 127) >> 7;                        // weight units along k
  const int NS = (p.K + 63) >> 6;                         // pipeline steps of 64 k per tile
  // Persistent CTAs walk the tiles with the token tile as the fast index: the CTAs running at one
  // time share a few weight row groups (L2 hits) and the activations fit L2 as a whole.
  const bool conv = p.conv_taps > 0;
  const int tpb = conv ? (p.conv_Lout + kGemmBN - 1) / kGemmBN : 0;      // convolution: token tiles per batch element
  const int n_tt = conv ? p.conv_B * tpb : (p.T + kGemmBN - 1) / kGemmBN, n_rg = (p.rows + 127) >> 7;
  const int n_tiles = n_tt * n_rg;
  TileOrder order;
  order.n_tt = n_tt; order.n_rg = n_rg;
  order.gt = max(8, min(n_tt, (64 << 20) / (kGemmBN * p.K * 2)));
  if (tid == 0) {
    for (int s = 0; s < kGemmStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    mbar_init_fence();
  }
  if (warp == 4) tmem_alloc(&tmem_slot, 2 * kGemmBN);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  bool dead = false;

  if (warp == 5) {
    // producer: per step half a weight unit (bulk copy, already in the tensor core's layout) and the
    // activations of BN tokens x 64 k through a 2-D tensor map over the row-major [T, K] matrix: the box
    // {64, BN} lands as BN rows of 128 bytes in the 128-byte swizzle (one request per row instead of one
    // per 16 bytes); rows past T and columns past K arrive as zeros
    int g = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      int rg, tt_;
      order.decode(tile, &rg, &tt_);
      for (int st = 0; st < NS; ++st, ++g) {
        const int s = g % kGemmStages;
        mbar_wait(&empty[s], ((g / kGemmStages) & 1) ^ 1, dead, err);
        if (lane == 0 && conv) {
          // tap k of output rows [o0, o0 + BN): input rows o * P + k - pad = (o + shift) * P + par, i.e. the box
          // {64 channels, parity par, BN row pairs from o0 + shift, batch b} of the [B][rows / P][P][C] view
          const int b = tt_ / tpb, o0 = (tt_ - b * tpb) * kGemmBN;
          const int spt = p.conv_cpad >> 6, tap = st / spt, c0 = (st - tap * spt) << 6;
          const int j = tap - p.conv_pad;
          const int shift = j >= 0 ? j / p.conv_P : -((-j + p.conv_P - 1) / p.conv_P), par = j - shift * p.conv_P;
          mbar_expect_tx(&full[s], (uint32_t)kStage);
          bulk_g2s(smem + s * kStage, p.W + ((int64_t)rg * KS + (st >> 1)) * 16384 + (st & 1) * 8192, (uint32_t)kABytes, &full[s]);
          asm volatile(
              "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::"r"(
                  smem_u32(smem + s * kStage + kABytes)),
              "l"(reinterpret_cast<uint64_t>(&xmap)), "r"(c0), "r"(par), "r"(o0 + shift), "r"(b), "r"(smem_u32(&full[s]))
              : "memory");
        } else if (lane == 0) {
          mbar_expect_tx(&full[s], (uint32_t)kStage);
          bulk_g2s(smem + s * kStage, p.W + ((int64_t)rg * KS + (st >> 1)) * 16384 + (st & 1) * 8192, (uint32_t)kABytes, &full[s]);
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                  smem_u32(smem + s * kStage + kABytes)),
              "l"(reinterpret_cast<uint64_t>(&xmap)), "r"(st * 64), "r"(tt_ * kGemmBN), "r"(smem_u32(&full[s]))
              : "memory");
        }
        __syncwarp();
      }
    }
  } else if (warp == 4) {
    constexpr uint32_t kIdesc = idesc_bf16(128, kGemmBN, false, false);
    int g = 0, n = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n) {
      const int buf = n & 1;
      mbar_wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1, dead, err);        // the epilogue has drained this accumulator
      fence_after();
      for (int st = 0; st < NS; ++st, ++g) {
        const int s = g % kGemmStages;
        mbar_wait(&full[s], (g / kGemmStages) & 1, dead, err);
        fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + s * kStage);
          const uint64_t adesc = smem_desc(sa, 2048, 128);
          const uint64_t bdesc = smem_desc_sw128(sa + kABytes);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mma_f16(tmem + buf * kGemmBN, adesc + (uint64_t)(j * (4096 >> 4)), bdesc + (uint64_t)(j * (32 >> 4)),
                    kIdesc, (st == 0 && j == 0) ? 0u : 1u);
          commit(&empty[s]);
          if (st == NS - 1) commit(&acc_full[buf]);
        }
        __syncwarp();
      }
    }
  } else {
    // epilogue of tile n while the MMAs of tile n + 1 fill the other accumulator
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    int n = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n) {
      const int buf = n & 1;
      int rg_, tt_;
      order.decode(tile, &rg_, &tt_);
      int t0 = tt_ * kGemmBN, t_end = p.T;
      if (conv) {
        const int b = tt_ / tpb, o0 = (tt_ - b * tpb) * kGemmBN;
        t0 = b * p.conv_out_rpb + o0;
        t_end = b * p.conv_out_rpb + p.conv_Lout;
      }
      const int row = rg_ * 128 + 32 * warp + lane;
      mbar_wait(&acc_full[buf], (n >> 1) & 1, dead, err);
      fence_after();
#pragma unroll 1
      for (int ch = 0; ch < kGemmBN / 32; ++ch) {
        float v[32];
        tmem_ld32(v, tmem + lane_base + buf * kGemmBN + ch * 32);
        if (ch == kGemmBN / 32 - 1) {                  // the whole accumulator is in registers or done with
          fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        gemm_epilogue(p, v, row, t0 + ch * 32, t_end, smem + kGemmStages * kStage + warp * kEpiStageBytes);
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 4) {
    fence_after();
    tmem_dealloc(tmem, 2 * kGemmBN);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same product with two CTAs (a cluster of 2 on one TPC) on one 256-row x 256-token tile: tcgen05.mma
// cta_group::2, M = 256.  CTA r of the pair stages ITS row group's weights and ITS half of the tokens (plain TMA
// boxes, no multicast); the tensor core of each SM reads both halves of the token tile, so every byte staged in
// shared memory is used for twice the flops: 32 KB per CTA per 64-k step instead of 48 KB, and six stages instead of
// four.  One thread of CTA 0 issues the MMAs for both.  Signals: both CTAs' loads complete on CTA 0's `full`
// barrier (a cta_group::2 TMA load may count on the partner's barrier); the MMA thread's commits arrive on the
// `empty` / `acc_full` barriers of both CTAs (multicast commit); CTA 1's epilogue warps hand its accumulator back with
// a remote arrive on CTA 0's `acc_empty`.  (A first version forwarded CTA 1's "stage landed" through a thread doing
// remote release-arrives: about a microsecond each, in series -- 518 TFLOP/s instead of 890.)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;\n" ::: "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(
                   tc::smem_u32(bar)),
               "h"((uint16_t)3)
               : "memory");
}

// TMA tile load whose completion is counted on a barrier given by its shared::cluster address: with cta_group::2 that
// may be the partner CTA's barrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}

constexpr int kPairStages = 6;
constexpr int kPairStage = 32768;       // 128 rows x 64 k of weights + 128 tokens x 64 k of activations

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_tc2_kernel(const GemmParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, int* err) {
  using namespace tc;
  constexpr int kBN = 256, kABytes = 16384;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kPairStages], empty[kPairStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t rank = cluster_rank();
  const int KS = (p.K + 127) >> 7, NS = (p.K + 63) >> 6;
  const int n_tt = (p.T + kBN - 1) / kBN, n_rgp = (p.rows + 255) >> 8;
  const int n_tiles = n_tt * n_rgp;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  TileOrder order;
  order.n_tt = n_tt; order.n_rg = n_rgp;
  order.gt = max(8, min(n_tt, (64 << 20) / (kBN * p.K * 2)));
  if (tid == 0) {
    for (int s = 0; s < kPairStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    mbar_init_fence();
  }
  if (warp == 4) tmem_alloc(&tmem_slot, 512);          // all columns in both CTAs: the same base address in both
  fence_before();
  __syncthreads();
  cluster_barrier();                                     // both CTAs' barriers exist before anything arrives on them
  fence_after();
  const uint32_t tmem = tmem_slot;
  bool dead = false;

  if (warp == 5) {
    int g = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs) {
      int rgp, tt_;
      order.decode(tile, &rgp, &tt_);
      const int rg = 2 * rgp + (int)rank;
      for (int st = 0; st < NS; ++st, ++g) {
        const int s = g % kPairStages;
        mbar_wait(&empty[s], ((g / kPairStages) & 1) ^ 1, dead, err);
        if (lane == 0) {
          // both CTAs' loads complete on CTA 0's barrier (cta_group::2 lets a TMA load signal the partner's
          // barrier): the MMA thread waits for one barrier per stage and nothing has to be forwarded
          const uint32_t bar0 = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2u * (uint32_t)kPairStage);
          tma_load_2d_pair(smem_u32(smem + s * kPairStage), &wmap, 0, (int)((((int64_t)rg * KS + (st >> 1)) * 2 + (st & 1)) * 128), bar0);
          tma_load_2d_pair(smem_u32(smem + s * kPairStage + kABytes), &xmap, st * 64, tt_ * kBN + (int)rank * 128, bar0);
        }
        __syncwarp();
      }
    }
  } else if (warp == 4 && rank == 1) {
    // CTA 1 issues no MMAs: CTA 0's thread drives both tensor cores
  } else if (warp == 4) {
    constexpr uint32_t kIdesc = idesc_bf16(256, kBN, false, false);
    int g = 0, n = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++n) {
      const int buf = n & 1;
      mbar_wait(&acc_empty[buf], ((n >> 1) & 1) ^ 1, dead, err);        // both CTAs' epilogues have drained this accumulator
      fence_after();
      for (int st = 0; st < NS; ++st, ++g) {
        const int s = g % kPairStages;
        mbar_wait(&full[s], (g / kPairStages) & 1, dead, err);
        fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(smem + s * kPairStage);
          const uint64_t adesc = smem_desc(sa, 2048, 128);
          const uint64_t bdesc = smem_desc_sw128(sa + kABytes);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mma_f16_pair(tmem + buf * kBN, adesc + (uint64_t)(j * (4096 >> 4)), bdesc + (uint64_t)(j * (32 >> 4)), kIdesc,
                         (st == 0 && j == 0) ? 0u : 1u);
          commit_pair(&empty[s]);
          if (st == NS - 1) commit_pair(&acc_full[buf]);
        }
        __syncwarp();
      }
    }
  } else {
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    const uint32_t acc_empty_remote[2] = {map_to_cta(smem_u32(&acc_empty[0]), 0), map_to_cta(smem_u32(&acc_empty[1]), 0)};
    int n = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++n) {
      const int buf = n & 1;
      int rgp, tt_;
      order.decode(tile, &rgp, &tt_);
      const int t0 = tt_ * kBN, row = (2 * rgp + (int)rank) * 128 + 32 * warp + lane;
      mbar_wait(&acc_full[buf], (n >> 1) & 1, dead, err);
      fence_after();
#pragma unroll 1
      for (int ch = 0; ch < kBN / 32; ++ch) {
        float v[32];
        tmem_ld32(v, tmem + lane_base + buf * kBN + ch * 32);
        if (ch == kBN / 32 - 1) {
          fence_before();
          __syncwarp();
          if (lane == 0) {
            if (rank == 0) mbar_arrive(&acc_empty[buf]);
            else mbar_arrive_cluster(acc_empty_remote[buf]);
          }
        }
        gemm_epilogue(p, v, row, t0 + ch * 32, p.T, smem + kPairStages * kPairStage + warp * kEpiStageBytes);
      }
    }
  }
  fence_before();
  __syncthreads();
  cluster_barrier();            // no CTA leaves while its partner may still arrive on its barriers or read its shared memory
  if (warp == 4) {
    fence_after();
    tmem_dealloc(tmem, 512);
  }
}

constexpr size_t gemm_pair_smem() { return (size_t)kPairStages * kPairStage + 4 * kEpiStageBytes + 1024; }

template <int BN>
constexpr size_t gemm_smem() { return (size_t)(BN == 256 ? 4 : 6) * (kUnitBytes / 2 + BN * 128) + 4 * kEpiStageBytes + 1024; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, resolved through the runtime so the library does not link libcuda
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      cudaGetLastError();
  }
  return fn;
}

int32_t gemm_launch(Ctx* ctx, const GemmParams& p, cudaStream_t st) {
  LMB_REQUIRE(p.K % 8 == 0 && p.ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(p.X) & 15) == 0, "prefill gemm: K %d, row pitch %d", p.K, p.ldx);
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(LMB200_ECUDA, "prefill gemm: cuTensorMapEncodeTiled is not available");
  // 256-token tiles once there are enough tokens to fill them (LMB200_GEMM_BN=128 keeps the narrow tile for A/B runs)
  static const int forced_bn = [] { const char* e = getenv("LMB200_GEMM_BN"); return e ? atoi(e) : 0; }();
  const bool conv = p.conv_taps > 0;
  const int n_tok = conv ? p.conv_Lout : p.T;
  const int BN = forced_bn == 128 || forced_bn == 256 ? forced_bn : (n_tok >= 256 ? 256 : 128);
  CUtensorMap xmap;
  CUresult r;
  if (conv) {
    LMB_REQUIRE(p.conv_P >= 1 && p.conv_rows_in % p.conv_P == 0 && p.conv_cpad % 64 == 0 && p.K == p.conv_taps * p.conv_cpad &&
                    p.conv_C <= p.conv_cpad && p.conv_C <= p.ldx,
                "implicit convolution: stride %d, rows %d, channels %d padded to %d, K %d", p.conv_P, p.conv_rows_in, p.conv_C,
                p.conv_cpad, p.K);
    // the input seen as [B][rows / P][P][C]: a tap of a strided convolution is one parity of consecutive row groups
    const cuuint64_t dims[4] = {(cuuint64_t)p.conv_C, (cuuint64_t)p.conv_P, (cuuint64_t)(p.conv_rows_in / p.conv_P), (cuuint64_t)p.conv_B};
    const cuuint64_t strides[3] = {(cuuint64_t)p.ldx * 2, (cuuint64_t)p.ldx * 2 * p.conv_P, (cuuint64_t)p.ldx * 2 * p.conv_rows_in};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)BN, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<__nv_bfloat16*>(p.X), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.T};
    const cuuint64_t strides[1] = {(cuuint64_t)p.ldx * 2};               // bytes, dim 1
    const cuuint32_t box[2] = {64, (cuuint32_t)BN};
    const cuuint32_t estr[2] = {1, 1};
    r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.X), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) return fail(LMB200_ECUDA, "prefill gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
  // CTA pairs where the tile grid allows them (LMB200_GEMM_PAIR=0 keeps the single-CTA kernel for A/B runs)
  static const bool pair_on = [] { const char* e = getenv("LMB200_GEMM_PAIR"); return !(e && atoi(e) == 0); }();
  if (pair_on && !conv && BN == 256 && p.rows % 256 == 0) {
    CUtensorMap hmap;                                       // each CTA's half of a token tile: a box of 128 tokens
    const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.T};
    const cuuint64_t strides[1] = {(cuuint64_t)p.ldx * 2};
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t estr[2] = {1, 1};
    r = enc(&hmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.X), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LMB200_ECUDA, "prefill gemm: cuTensorMapEncodeTiled failed (%d)", (int)r);
    // the weights as rows of 128 bytes: half a canonical unit (128 rows x 64 k) is 128 consecutive rows, copied as it lies
    CUtensorMap wmap;
    const int64_t w_rows = (int64_t)(p.rows / 128) * ceil_div(p.K, 128) * 2 * 128;
    const cuuint64_t wdims[2] = {64, (cuuint64_t)w_rows};
    const cuuint64_t wstrides[1] = {128};
    r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(p.W), wdims, wstrides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LMB200_ECUDA, "prefill gemm: cuTensorMapEncodeTiled (weights) failed (%d)", (int)r);
    const int64_t pair_tiles = (int64_t)(p.rows / 256) * ceil_div(p.T, 256);
    // a persistent grid: as many pairs as can be resident at once (SMs whose TPC partner is fused off take none)
    static int max_pairs = 0;
    if (!max_pairs) {
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3((unsigned)(ctx->sm_count / 2 * 2));
      qc.blockDim = dim3(kGemmThreads);
      qc.dynamicSmemBytes = gemm_pair_smem();
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel, &qc) != cudaSuccess || n < 1) { cudaGetLastError(); n = ctx->sm_count / 2; }
      max_pairs = n;
      if (getenv("LMB200_DEBUG_GEMM")) fprintf(stderr, "gemm_tc2_kernel: %d pairs resident on %d SMs\n", n, ctx->sm_count);
    }
    const unsigned pairs = (unsigned)std::min<int64_t>(pair_tiles, max_pairs);
    gemm_tc2_kernel<<<2 * pairs, kGemmThreads, gemm_pair_smem(), st>>>(p, wmap, hmap, ctx->dev_err);
    ctx->launches++;
    LMB_CUDA(cudaGetLastError());
    return LMB200_OK;
  }
  const int64_t tiles = ceil_div(p.rows, 128) * (conv ? (int64_t)p.conv_B * ceil_div(p.conv_Lout, BN) : ceil_div(p.T, BN));
  const unsigned grid = (unsigned)std::min<int64_t>(tiles, ctx->sm_count);
  if (BN == 256) gemm_tc_kernel<256><<<grid, kGemmThreads, gemm_smem<256>(), st>>>(p, xmap, ctx->dev_err);
  else gemm_tc_kernel<128><<<grid, kGemmThreads, gemm_smem<128>(), st>>>(p, xmap, ctx->dev_err);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

// K and V of the prompt, token-major [B * n_seq, KVl * D], into the decode cache of one layer: one CTA
// per (sequence, kv head, 16-key block) reads 16 rows of D elements and writes the block's 32 * D
// contiguous elements (K units then V units, the layout of kcache_offset / vcache_offset).
__global__ void __launch_bounds__(256) cache_fill_kernel(__nv_bfloat16* __restrict__ kv_layer, int64_t batch_stride, int64_t head_stride,
                                                         const __nv_bfloat16* __restrict__ kbuf, const __nv_bfloat16* __restrict__ vbuf,
                                                         int ldkv, int n_seq, int pos0, int KVl, int D) {
  const int blk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  __nv_bfloat16* base = kv_layer + b * batch_stride + kvh * head_stride;
  for (int i = threadIdx.x; i < 16 * D; i += 256) {
    const int key = i / D, d = i - key * D;
    const int sq = blk * 16 + key - (pos0 & 15);                 // position pos0 + sq sits in block (pos0 >> 4) + blk
    if (sq < 0 || sq >= n_seq) continue;
    const int pos = pos0 + sq;
    const int64_t src = ((int64_t)b * n_seq + sq) * ldkv + kvh * D + d;
    base[kcache_offset(pos, d, D)] = kbuf[src];
    base[vcache_offset(pos, d, D)] = vbuf[src];
  }
}

// (sin, cos) of every prompt position, with the decode step's expressions (src/NN.jl:253-303)
__global__ void rope_table_kernel(float2* __restrict__ tab, const float* __restrict__ inv_freq, int pos0, int n_seq, int half) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= (int64_t)n_seq * half) return;
  const int sq = (int)(i / half), d0 = (int)(i - (int64_t)sq * half);
  const float ang = (float)(pos0 + sq) * inv_freq[d0];
  tab[i] = make_float2(sinf(ang), sinf(kHalfPi + ang * -1.0f));
}

// x[t, :] = embedding row of token t (zeros when the id is out of range, as _gather_kernel! does)
__global__ void embed_rows_kernel(float* __restrict__ x, const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed,
                                  int vocab, int n) {
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  const __nv_bfloat16* er = embed + (int64_t)(ok ? tok : 0) * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) x[(int64_t)t * n + i] = ok ? __bfloat162float(er[i]) : 0.f;
}

// x[t, :] += delta[t, :] (if given); xn[t, :] = bf16((x * recip(sqrt(mean(x*x) + eps))) * w)
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                           const float* __restrict__ w, __nv_bfloat16* __restrict__ xn, int n,
                                                           float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  float* xr = x + (int64_t)t * n;
  float ss = 0.f;
  for (int i = tid; i < n; i += 256) {
    float v = xr[i];
    if (delta) { v += delta[(int64_t)t * n + i]; xr[i] = v; }
    row[i] = v;
    ss += v * v;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = 1.0f / sqrtf(tot * (1.0f / (float)n) + eps);
  if (xn)
    for (int i = tid; i < n; i += 256) xn[(int64_t)t * n + i] = __float2bfloat16_rn((row[i] * inv) * w[i]);
}

// the residual rows of each sequence's last prompt position -> the decode step's [B, n] buffer
__global__ void last_rows_kernel(float* __restrict__ dst, const float* __restrict__ x, const float* __restrict__ delta, int n_seq,
                                 int n, const int* __restrict__ lens) {
  const int b = blockIdx.x;
  const int64_t t = (int64_t)b * n_seq + (lens ? lens[b] : n_seq) - 1;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[(int64_t)b * n + i] = x[t * n + i] + (delta ? delta[t * n + i] : 0.f);
}

struct Scratch {
  void* p[12] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n = 0;
  ~Scratch() { for (int i = 0; i < n; ++i) cudaFree(p[i]); }
  template <typename T>
  int32_t get(T** out, int64_t elems) {
    void* q = nullptr;
    if (cudaMalloc(&q, (size_t)elems * sizeof(T)) != cudaSuccess) {
      cudaGetLastError();
      return fail(LMB200_ENOMEM, "prefill: scratch allocation of %lld bytes failed", (long long)(elems * (int64_t)sizeof(T)));
    }
    p[n++] = q;
    *out = reinterpret_cast<T*>(q);
    return LMB200_OK;
  }
};

}  // namespace

namespace {
__global__ void f32_to_bf16_kernel(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
}  // namespace

// out[t, row] = sum_k x[t, k] * W[row, k]: W in the bf16 weight layout, x float32 row-major on the
// device (rounded to bf16 here), out float32 [T, rows].
int32_t prefill_linear(Ctx* ctx, const void* W, const float* x_dev, int T, int rows, int K, float* out_dev, cudaStream_t st) {
  LMB_REQUIRE(K % 8 == 0, "prefill_gemm: K %d must be a multiple of 8", K);
  Scratch sc;
  __nv_bfloat16* xb = nullptr;
  LMB_TRY(sc.get(&xb, (int64_t)T * K));
  const int64_t n = (int64_t)T * K;
  f32_to_bf16_kernel<<<(unsigned)std::min<int64_t>(ceil_div(n, 256), 4096), 256, 0, st>>>(xb, x_dev, n);
  ctx->launches++;
  GemmParams p;
  p.W = reinterpret_cast<const __nv_bfloat16*>(W); p.X = xb; p.ldx = K; p.T = T; p.rows = rows; p.K = K;
  p.epi = GEMM_STORE_F32; p.out = out_dev; p.ldo = rows;
  LMB_TRY(gemm_launch(ctx, p, st));
  LMB_CUDA(cudaStreamSynchronize(st));
  return LMB200_OK;
}

// y[t, row] = ((sum_k x[t, k] W[row, k]) + bias[row]) -> gelu? -> * scale, float32 or bf16 at out[t * ldo + row]
int32_t gemm_affine(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int T, int rows, int K, const float* bias, float scale,
                    int gelu, void* out, int ldo, int out_bf16, cudaStream_t st) {
  GemmParams p;
  p.W = reinterpret_cast<const __nv_bfloat16*>(W); p.X = X; p.ldx = ldx; p.T = T; p.rows = rows; p.K = K;
  p.epi = GEMM_AFFINE; p.bias = bias; p.out_scale = scale; p.gelu = gelu; p.out_bf16 = out_bf16; p.out_any = out; p.ldo = ldo;
  return gemm_launch(ctx, p, st);
}

// y[b, o, row] = act(sum_{tap, c} W[row, tap * cpad + c] * x[b, o * stride + tap - pad, c] + bias[row]) stored as bf16 at
// out[(b * out_rpb + o) * ldo + row]: NN.Conv1D (src/NN.jl:55-104) as a GEMM whose activation tiles come straight from the
// token-major input through a 4-D tensor map, one tap of 64 channels per pipeline step; nothing is unfolded in memory.
int32_t gemm_conv1d(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int batch, int rows_in, int C, int cpad, int taps,
                    int stride, int pad, int Lout, int out_rpb, int rows, const float* bias, int gelu, void* out, int ldo,
                    int out_bf16, cudaStream_t st) {
  GemmParams p;
  p.W = reinterpret_cast<const __nv_bfloat16*>(W); p.X = X; p.ldx = ldx; p.T = batch * out_rpb; p.rows = rows; p.K = taps * cpad;
  p.epi = GEMM_AFFINE; p.bias = bias; p.out_scale = 1.0f; p.gelu = gelu; p.out_bf16 = out_bf16; p.out_any = out; p.ldo = ldo;
  p.conv_taps = taps; p.conv_P = stride; p.conv_pad = pad; p.conv_C = C; p.conv_cpad = cpad; p.conv_B = batch;
  p.conv_rows_in = rows_in; p.conv_Lout = Lout; p.conv_out_rpb = out_rpb;
  return gemm_launch(ctx, p, st);
}

// the same product written as bf16 into a tiled cache layer (rows = heads * D in head-major order)
int32_t gemm_cross_kv(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int T, int rows, int K, const float* bias, float scale,
                      void* kv_layer, int64_t batch_stride, int64_t head_stride, int n_seq, int D, int is_v, cudaStream_t st) {
  GemmParams p;
  p.W = reinterpret_cast<const __nv_bfloat16*>(W); p.X = X; p.ldx = ldx; p.T = T; p.rows = rows; p.K = K;
  p.epi = GEMM_CROSS_KV; p.bias = bias; p.out_scale = scale; p.is_v = is_v;
  p.kv_layer = reinterpret_cast<__nv_bfloat16*>(kv_layer); p.kv_batch_stride = batch_stride; p.kv_head_stride = head_stride;
  p.n_seq = n_seq; p.D = D;
  return gemm_launch(ctx, p, st);
}

int32_t prefill_configure() {
  LMB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem<128>()));
  LMB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem<256>()));
  LMB_CUDA(cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_pair_smem()));
  return LMB200_OK;
}

bool prefill_gemm_ok(const Session* S, int n) {
  const Model* M = S->m;
  const lmb200_model_config& c = M->cfg;
  const char* e = getenv("LMB200_PREFILL");          // "steps": feed the prompt through the decode step
  if (e && strcmp(e, "steps") == 0) return false;
  return c.arch == LMB200_ARCH_LLAMA && c.dtype == LMB200_BF16 && S->host_pos == 0 && !S->capture_on && n >= 8 && flash_tc_supported(M->D) &&
         c.hidden % 8 == 0 && M->inter_l % 8 == 0;
}

// tokens_dev: [B, n] int32, sequence-major.  On return the cache holds positions 0..n-1 of every
// sequence and S->x the residual rows of the last position (the caller runs the final norm + head).
int32_t prefill_gemm(Session* S, const int* tokens_dev, int n, const int* lens_dev, cudaStream_t st) {
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int B = S->B, hid = c.hidden, L = c.n_layers, D = M->D;
  const int T = B * n;
  const int qw = M->Hl * D, kvw = M->KVl * D;
  // one scratch block per session, kept for the next prompt of the same or a smaller size
  const int64_t sizes[9] = {(int64_t)T * hid * 4, (int64_t)T * hid * 4, (int64_t)T * hid * 2, (int64_t)T * qw * 2, (int64_t)T * kvw * 2,
                            (int64_t)T * kvw * 2, (int64_t)T * qw * 2, (int64_t)T * M->inter_l * 2, (int64_t)n * (D / 2) * 8};
  int64_t offs[9], total = 0;
  for (int i = 0; i < 9; ++i) { offs[i] = total; total += round_up(sizes[i], 256); }
  if (total > S->prefill_bytes) {
    cudaFree(S->prefill_buf);
    S->prefill_buf = nullptr;
    S->prefill_bytes = 0;
    if (cudaMalloc(&S->prefill_buf, (size_t)total) != cudaSuccess) {
      cudaGetLastError();
      return fail(LMB200_ENOMEM, "prefill: scratch allocation of %lld bytes failed", (long long)total);
    }
    S->prefill_bytes = total;
  }
  char* base = reinterpret_cast<char*>(S->prefill_buf);
  float* x = reinterpret_cast<float*>(base + offs[0]);
  float* delta = reinterpret_cast<float*>(base + offs[1]);
  __nv_bfloat16* xn = reinterpret_cast<__nv_bfloat16*>(base + offs[2]);
  __nv_bfloat16* q = reinterpret_cast<__nv_bfloat16*>(base + offs[3]);
  __nv_bfloat16* kb = reinterpret_cast<__nv_bfloat16*>(base + offs[4]);
  __nv_bfloat16* vb = reinterpret_cast<__nv_bfloat16*>(base + offs[5]);
  __nv_bfloat16* attn = reinterpret_cast<__nv_bfloat16*>(base + offs[6]);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(base + offs[7]);
  float2* rope = reinterpret_cast<float2*>(base + offs[8]);
  rope_table_kernel<<<(unsigned)ceil_div((int64_t)n * (D / 2), 256), 256, 0, st>>>(rope, M->inv_freq, 0, n, D / 2);
  ctx->launches++;
  embed_rows_kernel<<<T, 256, 0, st>>>(x, tokens_dev, reinterpret_cast<const __nv_bfloat16*>(M->embed), c.vocab, hid);
  ctx->launches++;
  const size_t norm_smem = (size_t)hid * sizeof(float);
  auto reduce = [&](float* buf) -> int32_t {          // row-parallel projection under tensor parallelism
    if (c.tp_size > 1 && !M->tp_solo) return nccl_allreduce_f32(ctx, buf, (int64_t)T * hid, st);
    return LMB200_OK;
  };
  FlashView fv;
  fv.H = M->Hl; fv.G = M->G;
  fv.q_b = (int64_t)n * qw; fv.q_h = D; fv.q_s = qw;
  fv.k_b = (int64_t)n * kvw; fv.k_h = D; fv.k_s = kvw;
  for (int l = 0; l < L; ++l) {
    LayerWeights& W = M->layers[l];
    rmsnorm_rows_kernel<<<T, 256, norm_smem, st>>>(x, l == 0 ? nullptr : delta, (const float*)W.attn_norm, xn, hid, c.rms_eps);
    ctx->launches++;
    {
      GemmParams p;
      p.W = reinterpret_cast<const __nv_bfloat16*>(W.wqkv); p.X = xn; p.ldx = hid; p.T = T; p.rows = M->m_qkv.rows; p.K = hid;
      p.epi = GEMM_QKV_ROPE;
      p.q = q; p.kbuf = kb; p.vbuf = vb; p.ldq = qw; p.ldkv = kvw;
      p.kv_layer = reinterpret_cast<__nv_bfloat16*>(S->kv) + (int64_t)l * S->kv_layer_stride;
      p.kv_batch_stride = S->kv_batch_stride; p.kv_head_stride = S->kv_head_stride;
      p.rope = rope; p.pos0 = 0; p.n_seq = n; p.Hl = M->Hl; p.KVl = M->KVl; p.D = D;
      LMB_TRY(gemm_launch(ctx, p, st));
      cache_fill_kernel<<<dim3((unsigned)ceil_div(n, 16), (unsigned)M->KVl, (unsigned)B), 256, 0, st>>>(
          p.kv_layer, p.kv_batch_stride, p.kv_head_stride, kb, vb, kvw, n, 0, M->KVl, D);
      ctx->launches++;
    }
    LMB_TRY(flash_tc_launch_view(ctx, attn, q, kb, vb, fv, B, n, D, 1.0f / sqrtf((float)D), 1, st));
    {
      GemmParams p;
      p.W = reinterpret_cast<const __nv_bfloat16*>(W.wo); p.X = attn; p.ldx = qw; p.T = T; p.rows = hid; p.K = qw;
      p.epi = GEMM_STORE_F32; p.out = delta; p.ldo = hid;
      LMB_TRY(gemm_launch(ctx, p, st));
      LMB_TRY(reduce(delta));
    }
    rmsnorm_rows_kernel<<<T, 256, norm_smem, st>>>(x, delta, (const float*)W.ffn_norm, xn, hid, c.rms_eps);
    ctx->launches++;
    {
      GemmParams p;
      p.W = reinterpret_cast<const __nv_bfloat16*>(W.wgu); p.X = xn; p.ldx = hid; p.T = T; p.rows = M->m_gu.rows; p.K = hid;
      p.epi = GEMM_SILU_GATE; p.act = act; p.ld_act = M->inter_l; p.n_act = M->inter_l;
      LMB_TRY(gemm_launch(ctx, p, st));
    }
    {
      GemmParams p;
      p.W = reinterpret_cast<const __nv_bfloat16*>(W.wdown); p.X = act; p.ldx = M->inter_l; p.T = T; p.rows = hid; p.K = M->inter_l;
      p.epi = GEMM_STORE_F32; p.out = delta; p.ldo = hid;
      LMB_TRY(gemm_launch(ctx, p, st));
      LMB_TRY(reduce(delta));
    }
  }
  last_rows_kernel<<<B, 256, 0, st>>>(S->x, x, delta, n, hid, lens_dev);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  LMB_CUDA(cudaStreamSynchronize(st));
  return LMB200_OK;
}

}  // namespace lmb
