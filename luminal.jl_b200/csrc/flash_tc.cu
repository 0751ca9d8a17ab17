// FlashAttentionOp on the tensor cores (bf16): out = softmax(scale * Q K^T [+ causal]) V.
// Replaces flash_attn_fwd_kernel (src/Execution.jl:374-450, one query row per block, keys in
// series, no tensor cores) for bf16 tensors of head_dim 64, 96 or 128.
//
// One CTA = two tiles of 128 query rows of one (batch, head) sharing the key/value stream, keys in
// tiles of 128:
//   2 loader warps : Q by cp.async 16-byte chunks into the canonical core-matrix layout (8 rows x 16
//                    bytes); then one warp streams K and the other V by TMA (cp.async.bulk.tensor over
//                    a 4-D map d / key / kv head / batch, 2 stages each): a key tile lands as D / W
//                    sub-tiles of [128 keys][W head dims] in the 128-byte (W = 64) or 64-byte (W = 32,
//                    head_dim 96) swizzle, which the tensor core reads K-major for Q K^T and MN-major
//                    for P V;
//   1 MMA warp     : one thread issues tcgen05.mma for both query tiles -- S = Q K^T (M 128, N 128,
//                    K = D) into the tile's 128 columns of tensor memory, and O += P V (M 128, N = D,
//                    K 128) with P read FROM TENSOR MEMORY (the A operand), accumulating O in tensor
//                    memory over all key tiles; tcgen05.commit signals mbarriers;
//   16 softmax warps, two threads per query row (warps w and w + 8 reach the same 32 lanes; each takes
//                    64 of the tile's 128 keys): tcgen05.ld the scores twice (row maximum, then
//                    exp2 with the scale folded in), exchange the halves' maxima through shared
//                    memory, and tcgen05.st P as bf16 pairs over the columns of S.  The running maximum
//                    is only raised -- and O rescaled in place -- when it grows by more than 2^8 (p
//                    stays <= 256, exact in the final O / l).
// S and P of a tile share their columns, so a tile runs S -> softmax -> P V strictly in turn and the
// two query tiles alternate on the tensor core.  Tensor memory: S / P 2 x 128 columns, O 2 x D.
// (Earlier forms: keys in tiles of 64 with P through shared memory -- 16 + 8 small MMAs per 64 keys,
// all operands from shared memory, 160 KB of operand reads per 128 keys and tile -- ran at 709
// TFLOP/s on [4, 32, 4096, 128]; 128-key tiles with P in tensor memory 729; two softmax threads
// per row 948; packed float32 pairs and three-input maxima in the softmax 959.)
// Causal: key tiles beyond a query tile's diagonal are never computed; inside the diagonal tile
// keys j > i are masked -- the reference's `if causal && j > i continue`.
#include <cuda.h>
#include <math_constants.h>

#include "common.cuh"
#include "tc.cuh"

namespace lmb {
namespace {

constexpr int kBM = 128;
constexpr int kLoaders = 2 * 32;          // loader threads
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.0f;     // log2 units the maximum may lag behind before O is rescaled

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// chunk (row, d8) of a [rows x D] row-major tile -> canonical offset [d8][row/8][row%8][16 B]
__device__ __forceinline__ uint32_t canon(int row, int c8, int rows) {
  return (uint32_t)(c8 * (rows * 16) + (row >> 3) * 128 + (row & 7) * 16);
}

// Shared-memory descriptor of a tile in the 128-byte (layout type 2) or 64-byte (type 4) swizzle a
// tensor map writes.  K-major: lbo unused (1), sbo = bytes between groups of 8 rows.  MN-major: lbo =
// bytes between swizzle-wide blocks along N, sbo = bytes between groups of 8 rows along K.
__device__ __forceinline__ uint64_t smem_desc_swz(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t type) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | ((uint64_t)type << 61);
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::"r"(
          tc::smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(tc::smem_u32(bar))
      : "memory");
}

// packed float32 pairs (two lanes of one 64-bit register) and the three-input maximum of this architecture: fewer
// instructions per score in the softmax threads, whose issue slots are as scarce as the exp2 unit
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

constexpr int kBN = 128, kStages = 2;
constexpr int kMmaWarp = 16;                       // warps 0-15 softmax (two per query row), 16 MMA issue, 17-18 loaders
constexpr int kThreads = (kMmaWarp + 1) * 32 + kLoaders;

template <int D>
struct Smem {
  static constexpr int kQ = kBM * D * 2;
  static constexpr int kKV = kBN * D * 2;
  static constexpr int offQ = 0;                              // two query tiles
  static constexpr int offK = offQ + 2 * kQ;
  static constexpr int offV = offK + kStages * kKV;
  static constexpr int total = offV + kStages * kKV;
};

__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_tc_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q, const __grid_constant__ CUtensorMap kmap,
                   const __grid_constant__ CUtensorMap vmap, const FlashView fv, int S, float scale, int causal, int* err) {
  constexpr int W = D % 64 == 0 ? 64 : 32;            // head dims per swizzled sub-tile
  constexpr int kSub = kBN * W * 2;                  // bytes of one sub-tile [128 keys][W]
  constexpr uint32_t kSwz = W == 64 ? 2u : 4u;
  using namespace tc;
  typedef Smem<D> SM;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  __shared__ __align__(8) uint64_t s_full[2], p_full[2], o_done[2];
  __shared__ float xch[2][2][kBM];                    // [tile][column half][row]: the halves' row maxima, later their sums
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;          // S / P: [tile] x 128 columns, O: [tile] x D columns

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qp = (int)gridDim.x - 1 - (int)blockIdx.x;        // heavy (late) causal tiles first
  const int q0 = qp * 2 * kBM;
  const int bi = (int)blockIdx.y / fv.H, hi = (int)blockIdx.y - bi * fv.H;
  const __nv_bfloat16* qb = q + bi * fv.q_b + hi * fv.q_h;
  const int kvh = hi / fv.G;
  __nv_bfloat16* ob_base = out + bi * fv.q_b + hi * fv.q_h;
  const int64_t q_s = fv.q_s;
  int n_tiles[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt0 = q0 + t * kBM;
    const int k_stop = qt0 >= S ? 0 : (causal ? min(S, qt0 + kBM) : S);
    n_tiles[t] = (k_stop + kBN - 1) / kBN;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

  if (tid == 0) {
    mbar_init(&q_full, kLoaders / 32);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 8); mbar_init(&o_done[t], 1); }
    mbar_init_fence();
  }
  if (warp == kMmaWarp) tmem_alloc(&tmem_slot, kTmemCols);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  bool dead = false;

  if (warp > kMmaWarp) {
    // ------------------------------ loaders: Q by both warps, then K by one and V by the other ------------------------------
    const int lw = warp - kMmaWarp - 1, lt = tid - (kMmaWarp + 1) * 32;
    const uint32_t sQ = smem_u32(smem + SM::offQ);
    for (int i = lt; i < 2 * kBM * (D / 8); i += kLoaders) {
      const int row = i / (D / 8), c8 = i - row * (D / 8);
      const int qi = q0 + row;
      cp_async16(sQ + (row >> 7) * SM::kQ + canon(row & 127, c8, kBM), qb + (int64_t)min(qi, S - 1) * q_s + c8 * 8, qi < S ? 16u : 0u);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_full);
    uint64_t* full = lw == 0 ? k_full : v_full;
    uint64_t* empty = lw == 0 ? k_empty : v_empty;
    const CUtensorMap* map = lw == 0 ? &kmap : &vmap;
    const int off = lw == 0 ? SM::offK : SM::offV;
    for (int j = 0; j < n_max; ++j) {
      const int s = j % kStages;
      mbar_wait(&empty[s], ((j / kStages) & 1) ^ 1, dead, err);
      if (lane == 0) {
        mbar_expect_tx(&full[s], (uint32_t)SM::kKV);
#pragma unroll
        for (int sub = 0; sub < D / W; ++sub) tma_load_4d(smem + off + s * SM::kKV + sub * kSub, map, sub * W, j * kBN, kvh, bi, &full[s]);
      }
      __syncwarp();
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issue ------------------------------
    constexpr uint32_t kIdescS = idesc_bf16(kBM, kBN, false, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, D, false, true);          // V is read MN-major
    mbar_wait(&q_full, 0, dead, err);
    auto issue_s = [&](int j, int t) {                // S[t] = Q[t] K(j)^T
      if (lane == 0) {
        const uint64_t adesc = smem_desc(smem_u32(smem + SM::offQ + t * SM::kQ), kBM * 16, 128);
        const uint32_t sK = smem_u32(smem + SM::offK + (j % kStages) * SM::kKV);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t bdesc = smem_desc_swz(sK + ((16 * ks) / W) * kSub + ((16 * ks) % W) * 2, 16, 16 * W, kSwz);
          mma_f16(tmem + kColS + t * kBN, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)), bdesc, kIdescS, ks ? 1u : 0u);
        }
        commit(&s_full[t]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int j, int t) {               // O[t] += P[t] V(j), P read from tensor memory
      if (lane == 0) {
        const uint64_t bdesc = smem_desc_swz(smem_u32(smem + SM::offV + (j % kStages) * SM::kKV), kSub, 16 * W, kSwz);
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks)
          mma_f16_ts(tmem + kColO + t * D, tmem + kColS + t * kBN + ks * 8, bdesc + (uint64_t)(ks * ((32 * W) >> 4)), kIdescPV,
                     (j > 0 || ks > 0) ? 1u : 0u);
        if (j == n_tiles[t] - 1) commit(&o_done[t]);
      }
      __syncwarp();
    };
    if (n_max >= 1) {
      mbar_wait(&k_full[0], 0, dead, err);
      fence_after();
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (n_tiles[t] >= 1) issue_s(0, t);
      if (lane == 0) commit(&k_empty[0]);
      __syncwarp();
    }
    for (int j = 0; j < n_max; ++j) {
      const int s = j % kStages, s1 = (j + 1) % kStages;
      mbar_wait(&v_full[s], (j / kStages) & 1, dead, err);
      if (j + 1 < n_max) mbar_wait(&k_full[s1], ((j + 1) / kStages) & 1, dead, err);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j >= n_tiles[t]) continue;
        mbar_wait(&p_full[t], j & 1, dead, err);
        fence_after();
        issue_pv(j, t);
        if (j + 1 < n_tiles[t]) issue_s(j + 1, t);       // runs after P V(j) in the tensor pipe: S overwrites P's columns
      }
      if (lane == 0) {
        commit(&v_empty[s]);
        if (j + 1 < n_max) commit(&k_empty[s1]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ softmax + output ------------------------------
    // Two threads per query row: warps 0-7 take keys 0-63 of a tile, warps 8-15 keys 64-127 (a warp reaches the 32
    // tensor-memory lanes of its index modulo 4, so warp w and w + 8 see the same rows).  The two halves exchange
    // their row maxima through shared memory and a 64-thread barrier, keep their own partial sums, and each writes
    // its half of P -- after a second barrier, because P's columns lie over the other half's scores.
    const int h = warp >> 3, t = (warp >> 2) & 1, wq = warp & 3;
    const int r = 32 * wq + lane;
    const int qi = q0 + t * kBM + r;
    const uint32_t lane_base = (uint32_t)(32 * wq) << 16;
    const uint32_t colS = kColS + t * kBN + h * 64, colP = kColS + t * kBN + h * 32, colO = kColO + t * D + h * (D / 2);
    const int pair_bar = 1 + t * 4 + wq;              // named barrier of the two warps that share these rows
    const float c = scale * kLog2e;
    const int nt = n_tiles[t];
    float m = -CUDART_INF_F, l = 0.f;
    for (int j = 0; j < nt; ++j) {
      mbar_wait(&s_full[t], j & 1, dead, err);          // S(j) is complete, and with it (pipe order) P V(j - 1): O is at rest
      fence_after();
      const int key0 = j * kBN + h * 64;
      const bool inside = (j + 1) * kBN <= S && (!causal || (j + 1) * kBN - 1 <= q0 + t * kBM);   // no key of the tile is masked
      // pass 1: the maximum of this thread's 64 scores
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int qd = 0; qd < 2; ++qd) {
        float sv[32];
        tmem_ld32(sv, tmem + lane_base + colS + qd * 32);
        if (inside) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], sv[i], sv[i + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + qd * 32 + i;
            if (!(key >= S || (causal && key > qi))) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
          }
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      xch[t][h][r] = mx;
      asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
      mx = fmaxf(mx, xch[t][h ^ 1][r]);
      mx *= c;
      const bool first = m == -CUDART_INF_F && mx > -CUDART_INF_F;
      const bool raise = m > -CUDART_INF_F && mx > m + kRescaleStep;
      if (__any_sync(0xffffffffu, raise) && j > 0) {      // both halves decide alike; each rescales its half of O's columns
        const float alpha = raise ? exp2f(m - mx) : 1.0f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          float o[16];
          tmem_ld16(o, tmem + lane_base + colO + ch * 16);
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] *= alpha;
          uint32_t ou[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) ou[i] = __float_as_uint(o[i]);
          tmem_st16_nowait(tmem + lane_base + colO + ch * 16, ou);
        }
      }
      if (raise) { l *= exp2f(m - mx); m = mx; }
      if (first) m = mx;
      const float neg_m = m == -CUDART_INF_F ? 0.f : -m;
      // pass 2: p = exp2(s c - m) as bf16 pairs, kept in registers until the other half has read its scores too
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};           // four chains of (even, odd) partial sums
      const uint64_t c2 = pack2(c, c), negm2 = pack2(neg_m, neg_m);
      uint32_t packed[32];
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        float sv[16];
        tmem_ld16(sv, tmem + lane_base + colS + qd * 16);
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float a0 = sv[i], a1 = sv[i + 1];
          if (!inside) {
            const int key = key0 + qd * 16 + i;
            if (key >= S || (causal && key > qi)) a0 = -CUDART_INF_F;
            if (key + 1 >= S || (causal && key + 1 > qi)) a1 = -CUDART_INF_F;
          }
          float x0, x1;
          unpack2(fma2(pack2(a0, a1), c2, negm2), x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          sum2[(i >> 1) & 3] = add2(sum2[(i >> 1) & 3], pack2(p0, p1));
          const __nv_bfloat162 pb2 = __floats2bfloat162_rn(p0, p1);
          packed[qd * 8 + i / 2] = *reinterpret_cast<const uint32_t*>(&pb2);
        }
      }
      {
        float e, o;
        unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), e, o);
        l += e + o;
      }
      asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
      {
        uint32_t lo[16], hi2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = packed[i]; hi2[i] = packed[16 + i]; }
        tmem_st16_nowait(tmem + lane_base + colP, lo);
        tmem_st16_nowait(tmem + lane_base + colP + 16, hi2);
      }
      tmem_st_wait();
      fence_before();                    // orders the stores (P, a rescaled O) before the MMA that the arrive releases
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    if (nt >= 1) {
      xch[t][h][r] = l;
      asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory");
      l += xch[t][h ^ 1][r];
      mbar_wait(&o_done[t], 0, dead, err);            // the last P V has landed
      fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* ob = ob_base + (int64_t)qi * q_s + h * (D / 2);
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        float o[16];
        tmem_ld16(o, tmem + lane_base + colO + ch * 16);
        if (qi < S) {
#pragma unroll
          for (int i = 0; i < 16; i += 8) {
            uint4 w;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv), a1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv), a3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
            w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
            w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
            *reinterpret_cast<uint4*>(ob + ch * 16 + i) = w;
          }
        }
      }
      fence_before();
    }
  }
  fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

int32_t flash_tc_configure() {
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::total + 1024));
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_kernel<96>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<96>::total + 1024));
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::total + 1024));
  return LMB200_OK;
}

bool flash_tc_supported(int64_t D) { return D == 64 || D == 96 || D == 128; }

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn flash_encode_fn() {
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
// 4-D map over K or V: dims {d, key, kv head, batch}; a box is [box_keys keys][W head dims], swizzled over its W * 2 bytes.
// Keys past S arrive as zeros (the softmax masks them).
int32_t kv_tensor_map(CUtensorMap* map, const void* base, const FlashView& fv, int64_t B, int64_t S, int64_t D, int box_keys) {
  EncodeTiledFn enc = flash_encode_fn();
  if (!enc) return fail(LMB200_ECUDA, "flash attention: cuTensorMapEncodeTiled is not available");
  const int W = D % 64 == 0 ? 64 : 32;
  const int64_t n_kv = fv.H / fv.G;
  const int64_t head_stride = n_kv > 1 ? fv.k_h : S * fv.k_s;           // a dimension of extent 1 still needs a valid stride
  const int64_t batch_stride = B > 1 ? fv.k_b : S * fv.k_s * n_kv;
  LMB_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0 && fv.k_s % 8 == 0 && head_stride % 8 == 0 && batch_stride % 8 == 0,
              "flash attention: K / V base and strides must be multiples of 16 bytes");
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)n_kv, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)fv.k_s * 2, (cuuint64_t)head_stride * 2, (cuuint64_t)batch_stride * 2};
  const cuuint32_t box[4] = {(cuuint32_t)W, (cuuint32_t)box_keys, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, W == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LMB200_ECUDA, "flash attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return LMB200_OK;
}
}  // namespace

// q, out: element (b, h, s, d) at b * q_b + h * q_h + s * q_s + d; k, v likewise with the k strides
int32_t flash_tc_launch_view(Ctx* ctx, void* out, const void* q, const void* k, const void* v, const FlashView& fv, int64_t B,
                             int64_t S, int64_t D, float scale, int causal, cudaStream_t stream) {
  dim3 grid((unsigned)ceil_div(S, 2 * kBM), (unsigned)(B * fv.H));
  CUtensorMap kmap, vmap;
  LMB_TRY(kv_tensor_map(&kmap, k, fv, B, S, D, kBN));
  LMB_TRY(kv_tensor_map(&vmap, v, fv, B, S, D, kBN));
#define LMB_FLASH(DD)                                                                                                   \
  flash_tc_kernel<DD><<<grid, kThreads, Smem<DD>::total + 1024, stream>>>(                                        \
      (__nv_bfloat16*)out, (const __nv_bfloat16*)q, kmap, vmap, fv, (int)S, scale, causal, ctx->dev_err)
  if (D == 128) LMB_FLASH(128);
  else if (D == 96) LMB_FLASH(96);
  else if (D == 64) LMB_FLASH(64);
  else return fail(LMB200_EINVAL, "flash attention: head_dim %lld has no tensor-core kernel", (long long)D);
#undef LMB_FLASH
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

int32_t flash_tc_launch(Ctx* ctx, void* out, const void* q, const void* k, const void* v, int64_t BH, int64_t S, int64_t D,
                        float scale, int causal) {
  FlashView fv;                       // [B*H, S, D] contiguous, as the op's tensors are
  fv.H = 1; fv.G = 1;
  fv.q_b = fv.k_b = S * D; fv.q_h = fv.k_h = 0; fv.q_s = fv.k_s = D;
  return flash_tc_launch_view(ctx, out, q, k, v, fv, BH, S, D, scale, causal, ctx->stream);
}

}  // namespace lmb
