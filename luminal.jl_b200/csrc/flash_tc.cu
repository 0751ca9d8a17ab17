// FlashAttentionOp on the tensor cores (bf16): out = softmax(scale * Q K^T [+ causal]) V.
// Replaces flash_attn_fwd_kernel (src/Execution.jl:374-450, one query row per block, keys in
// series, no tensor cores) for bf16 tensors of head_dim 64, 96 or 128.
//
// One CTA = two tiles of 128 query rows of one (batch, head) sharing the key/value stream, keys in
// tiles of 64:
//   2 loader warps : cp.async 16-byte chunks of Q / K / V from row-major global memory into the
//                    canonical core-matrix layout (8 rows x 16 bytes) the tensor core reads, 3 K/V
//                    stages in flight;
//   1 MMA warp     : one thread issues tcgen05.mma for both query tiles -- S = Q K^T (M 128, N 64,
//                    K = D) into a double-buffered TMEM tile, then O += P V (M 128, N = D, K 64; V
//                    read MN-major from the same tile layout as K) accumulating in TMEM over all
//                    key tiles; tcgen05.commit signals mbarriers;
//   2 x 4 softmax warps, one group per query tile, one query row per thread: tcgen05.ld the S row,
//                    exp2 with the scale folded in, write P as bf16 straight into the A-operand
//                    layout.  The running maximum is only raised -- and O in TMEM rescaled -- when
//                    it grows by more than 2^8 (p stays <= 256, exact in the final O / l), so in the
//                    steady state a softmax thread never touches O and the two groups keep the
//                    tensor core busy in turn.
// Causal: key tiles beyond a query tile's diagonal are never computed; inside the diagonal tile
// keys j > i are masked -- the reference's `if causal && j > i continue`.
#include <math_constants.h>

#include "common.cuh"
#include "tc.cuh"

namespace lmb {
namespace {

constexpr int kBM = 128, kBN = 64, kKvStages = 3;
constexpr int kLoaders = 2 * 32;          // loader threads
constexpr int kThreads = 9 * 32 + kLoaders;   // warps 0-3 / 4-7 softmax of query tile 0 / 1, 8 MMA, 9.. loaders
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.0f;     // log2 units the maximum may lag behind before O is rescaled

// Optional phase stamps (SM clock) of CTA (0, 0) for tuning; compiled in only with -DLMB_FLASH_TRACE.
#ifdef LMB_FLASH_TRACE
}  // namespace
__device__ long long g_flash_trace[64 * 16];
namespace {
#define FL_TRACE(tile, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (tile) < 64) g_flash_trace[(tile) * 16 + (slot)] = clock64(); } while (0)
#else
#define FL_TRACE(tile, slot) ((void)0)
#endif

template <int D>
struct Smem {
  static constexpr int kQ = kBM * D * 2;
  static constexpr int kKV = kBN * D * 2;
  static constexpr int kP = kBM * kBN * 2;
  static constexpr int offQ = 0;                              // two query tiles
  static constexpr int offK = offQ + 2 * kQ;
  static constexpr int offV = offK + kKvStages * kKV;
  static constexpr int offP = offV + kKvStages * kKV;          // [tile][buffer]
  static constexpr int total = offP + 4 * kP;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// chunk (row, d8) of a [rows x D] row-major tile -> canonical offset [d8][row/8][row%8][16 B]
__device__ __forceinline__ uint32_t canon(int row, int c8, int rows) {
  return (uint32_t)(c8 * (rows * 16) + (row >> 3) * 128 + (row & 7) * 16);
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_tc_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                const __nv_bfloat16* __restrict__ v, const FlashView fv, int S, float scale, int causal, int* err) {
  using namespace tc;
  typedef Smem<D> SM;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, kv_full[kKvStages], kv_empty[kKvStages];
  __shared__ __align__(8) uint64_t s_full[2][2], s_empty[2][2], p_full[2][2], p_empty[2][2], pv_done[2];
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;                 // S: [tile][buffer] x 64 columns, O: [tile] x D columns

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qp = (int)gridDim.x - 1 - (int)blockIdx.x;        // heavy (late) causal tiles first
  const int q0 = qp * 2 * kBM;
  // blockIdx.y = batch * H + head; query head h reads kv head h / G (G = 1: an op with H kv heads)
  const int bi = (int)blockIdx.y / fv.H, hi = (int)blockIdx.y - bi * fv.H;
  const __nv_bfloat16* qb = q + bi * fv.q_b + hi * fv.q_h;
  const __nv_bfloat16* kb = k + bi * fv.k_b + (hi / fv.G) * fv.k_h;
  const __nv_bfloat16* vb = v + bi * fv.k_b + (hi / fv.G) * fv.k_h;
  __nv_bfloat16* ob_base = out + bi * fv.q_b + hi * fv.q_h;
  const int64_t q_s = fv.q_s, k_s = fv.k_s;
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
    for (int s = 0; s < kKvStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int t = 0; t < 2; ++t) {
      for (int i = 0; i < 2; ++i) {
        mbar_init(&s_full[t][i], 1); mbar_init(&s_empty[t][i], 4);
        mbar_init(&p_full[t][i], 4); mbar_init(&p_empty[t][i], 1);
      }
      mbar_init(&pv_done[t], 1);
    }
    mbar_init_fence();
  }
  if (warp == 8) tmem_alloc(&tmem_slot, kTmemCols);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  bool dead = false;

  if (warp >= 9) {
    // ------------------------------ loaders ------------------------------
    // The loader warps take the key tiles in turn (warp w: tiles w, w + 2, ...), each waiting for
    // its own tile to land before it signals it, so one warp's wait never holds back the other's
    // next issue.
    const int lw = warp - 9, lt = tid - 9 * 32;     // lt: 0..kLoaders-1
    constexpr int kLw = kLoaders / 32;
    const uint32_t sQ = smem_u32(smem + SM::offQ);
    for (int i = lt; i < 2 * kBM * (D / 8); i += kLoaders) {
      const int row = i / (D / 8), c8 = i - row * (D / 8);      // row 0..255 over both tiles
      const int qi = q0 + row;
      cp_async16(sQ + (row >> 7) * SM::kQ + canon(row & 127, c8, kBM), qb + (int64_t)min(qi, S - 1) * q_s + c8 * 8, qi < S ? 16u : 0u);
    }
    cp_async_commit();
    bool q_signalled = false;
    for (int j = lw; j < n_max; j += kLw) {
      const int s = j % kKvStages;
      mbar_wait(&kv_empty[s], ((j / kKvStages) & 1) ^ 1, dead, err);
      const uint32_t sK = smem_u32(smem + SM::offK + s * SM::kKV), sV = smem_u32(smem + SM::offV + s * SM::kKV);
      if ((32 % (D / 8)) == 0 && (j + 1) * kBN <= S) {
        // tile inside the sequence, and a lane keeps its 16-byte column: rows advance by 32 / (D/8)
        constexpr int kCols = D / 8, kRowStep = 32 / kCols;
        const int c8 = lane % kCols, row0 = lane / kCols;
        const __nv_bfloat16* ks = kb + (int64_t)(j * kBN + row0) * k_s + c8 * 8;
        const __nv_bfloat16* vs = vb + (int64_t)(j * kBN + row0) * k_s + c8 * 8;
#pragma unroll 8
        for (int it = 0; it < kBN / kRowStep; ++it) {
          const uint32_t off = canon(row0 + it * kRowStep, c8, kBN);
          cp_async16(sK + off, ks + (int64_t)it * kRowStep * k_s, 16u);
          cp_async16(sV + off, vs + (int64_t)it * kRowStep * k_s, 16u);
        }
      } else {
        for (int i = lane; i < kBN * (D / 8); i += 32) {
          const int row = i / (D / 8), c8 = i - row * (D / 8);
          const int key = j * kBN + row;
          const int64_t src = (int64_t)min(key, S - 1) * k_s + c8 * 8;
          const uint32_t nb = key < S ? 16u : 0u;
          cp_async16(sK + canon(row, c8, kBN), kb + src, nb);
          cp_async16(sV + canon(row, c8, kBN), vb + src, nb);
        }
      }
      cp_async_commit();
      if (!q_signalled) {
        cp_async_wait<1>();                          // this warp's share of Q has landed
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&q_full);
        q_signalled = true;
      }
      cp_async_wait<0>();                            // tile j has landed
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[s]);
    }
    if (!q_signalled) {
      cp_async_wait<0>();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full);
    }
  } else if (warp == 8) {
    // ------------------------------ MMA issue ------------------------------
    constexpr uint32_t kIdescS = idesc_bf16(kBM, kBN, false, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, D, false, true);          // V is read MN-major
    mbar_wait(&q_full, 0, dead, err);
    auto issue_pv = [&](int j) {                     // O[t] += P[t](j) V(j) for the tiles that reach key tile j
      const int pb = j & 1, s = j % kKvStages;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j >= n_tiles[t]) continue;
        mbar_wait(&p_full[t][pb], (j >> 1) & 1, dead, err);
        fence_after();
        if (lane == 0) FL_TRACE(j, 8 + t);
        if (lane == 0) {
          // A = P [128 x 64] K-major: lbo (between key groups of 8) = 128*16, sbo = 128
          // B = V tile [64 keys x D] read as N = d (contiguous), K = key: sbo (between d groups) =
          //     64*16 = 1024, lbo (between key groups) = 128
          const uint64_t adesc = smem_desc(smem_u32(smem + SM::offP + (t * 2 + pb) * SM::kP), kBM * 16, 128);
          const uint64_t bdesc = smem_desc(smem_u32(smem + SM::offV + s * SM::kKV), 128, kBN * 16);
#pragma unroll
          for (int ks = 0; ks < kBN / 16; ++ks)
            mma_f16(tmem + kColO + t * D, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)), bdesc + (uint64_t)(ks * (256 >> 4)),
                    kIdescPV, (j > 0 || ks > 0) ? 1u : 0u);
          commit(&pv_done[t]);
          commit(&p_empty[t][pb]);
        }
        __syncwarp();
      }
      if (lane == 0) commit(&kv_empty[s]);
      __syncwarp();
    };
    for (int j = 0; j < n_max; ++j) {
      const int sb = j & 1, s = j % kKvStages;
      mbar_wait(&kv_full[s], (j / kKvStages) & 1, dead, err);
      if (lane == 0) FL_TRACE(j, 10);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (j >= n_tiles[t]) continue;
        mbar_wait(&s_empty[t][sb], ((j >> 1) & 1) ^ 1, dead, err);
        fence_after();
        if (lane == 0) FL_TRACE(j, 11 + t);
        if (lane == 0) {
          // A = Q [128 x D] K-major: lbo = 128*16, sbo = 128;  B = K tile [64 x D] K-major: lbo = 64*16
          const uint64_t adesc = smem_desc(smem_u32(smem + SM::offQ + t * SM::kQ), kBM * 16, 128);
          const uint64_t bdesc = smem_desc(smem_u32(smem + SM::offK + s * SM::kKV), kBN * 16, 128);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks)
            mma_f16(tmem + kColS + (t * 2 + sb) * kBN, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)),
                    bdesc + (uint64_t)(ks * ((2 * kBN * 16) >> 4)), kIdescS, ks ? 1u : 0u);
          commit(&s_full[t][sb]);
        }
        __syncwarp();
      }
      if (j >= 1) issue_pv(j - 1);
    }
    if (n_max >= 1) issue_pv(n_max - 1);
  } else {
    // ------------------------------ softmax + output: one query row per thread ------------------------------
    const int t = warp >> 2, wq = warp & 3;
    const int r = 32 * wq + lane;
    const int qi = q0 + t * kBM + r;
    const uint32_t lane_base = (uint32_t)(32 * wq) << 16;
    const uint32_t colO = kColO + t * D;
    const float c = scale * kLog2e;
    const int nt = n_tiles[t];
    float m = -CUDART_INF_F, l = 0.f;
    for (int j = 0; j < nt; ++j) {
      const int sb = j & 1;
      if (wq == 0 && lane == 0) FL_TRACE(j, 0 + 4 * t);
      mbar_wait(&s_full[t][sb], (j >> 1) & 1, dead, err);
      fence_after();
      if (wq == 0 && lane == 0) FL_TRACE(j, 1 + 4 * t);
      float sv[kBN];
      tmem_ld64(sv, tmem + lane_base + kColS + (t * 2 + sb) * kBN);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[t][sb]);
      // scores stay unscaled in registers; the scale (c > 0) enters through the exp2 argument
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};     // four chains, not one of 64
      const bool inside = (j + 1) * kBN <= S && (!causal || (j + 1) * kBN - 1 <= q0 + t * kBM);   // no key of the tile is masked
      if (inside) {
#pragma unroll
        for (int i = 0; i < kBN; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
      } else {
#pragma unroll
        for (int i = 0; i < kBN; ++i) {
          const int key = j * kBN + i;
          if (key >= S || (causal && key > qi)) sv[i] = -CUDART_INF_F;
          mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
        }
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= c;
      // raise the reference maximum only when it lags by more than kRescaleStep; O and l follow it
      const bool first = m == -CUDART_INF_F && mx > -CUDART_INF_F;
      const bool raise = m > -CUDART_INF_F && mx > m + kRescaleStep;
      if (__any_sync(0xffffffffu, raise) && j > 0) {
        const float alpha = raise ? exp2f(m - mx) : 1.0f;
        mbar_wait(&pv_done[t], (j - 1) & 1, dead, err);          // every P V issued so far has landed in O
        fence_after();
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          float o[32];
          tmem_ld32(o, tmem + lane_base + colO + ch * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(tmem + lane_base + colO + ch * 32, o);
        }
        fence_before();
      }
      if (raise) { l *= exp2f(m - mx); m = mx; }
      if (first) m = mx;
      const float neg_m = m == -CUDART_INF_F ? 0.f : -m;             // row fully masked so far: p = exp2(-inf) = 0
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN; i += 2) {
        const float p0 = ex2_approx(fmaf(sv[i], c, neg_m)), p1 = ex2_approx(fmaf(sv[i + 1], c, neg_m));
        sum4[(i >> 1) & 3] += p0 + p1;
        const __nv_bfloat162 pb2 = __floats2bfloat162_rn(p0, p1);
        packed[i / 2] = *reinterpret_cast<const uint32_t*>(&pb2);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (wq == 0 && lane == 0) FL_TRACE(j, 2 + 4 * t);
      mbar_wait(&p_empty[t][sb], ((j >> 1) & 1) ^ 1, dead, err);
      unsigned char* pt = smem + SM::offP + (t * 2 + sb) * SM::kP;
#pragma unroll
      for (int c8 = 0; c8 < kBN / 8; ++c8)
        *reinterpret_cast<uint4*>(pt + canon(r, c8, kBM)) =
            make_uint4(packed[4 * c8], packed[4 * c8 + 1], packed[4 * c8 + 2], packed[4 * c8 + 3]);
      fence_async_smem();
      fence_before();                    // orders a rescale's tcgen05.st before the MMA that the arrive releases
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t][sb]);
      if (wq == 0 && lane == 0) FL_TRACE(j, 3 + 4 * t);
    }
    if (nt >= 1) {
      mbar_wait(&pv_done[t], (nt - 1) & 1, dead, err);
      fence_after();
      const float inv = 1.0f / l;
      __nv_bfloat16* ob = ob_base + (int64_t)qi * q_s;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        float o[32];
        tmem_ld32(o, tmem + lane_base + colO + ch * 32);
        if (qi < S) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            __nv_bfloat162 a0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv), a1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
            __nv_bfloat162 a2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv), a3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
            w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
            w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
            *reinterpret_cast<uint4*>(ob + ch * 32 + i) = w;
          }
        }
      }
      fence_before();
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 8) {
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

// q, out: element (b, h, s, d) at b * q_b + h * q_h + s * q_s + d; k, v likewise with the k strides
int32_t flash_tc_launch_view(Ctx* ctx, void* out, const void* q, const void* k, const void* v, const FlashView& fv, int64_t B,
                             int64_t S, int64_t D, float scale, int causal, cudaStream_t stream) {
  dim3 grid((unsigned)ceil_div(S, 2 * kBM), (unsigned)(B * fv.H));
#define LMB_FLASH(DD)                                                                                                   \
  flash_tc_kernel<DD><<<grid, kThreads, Smem<DD>::total + 1024, stream>>>(                                             \
      (__nv_bfloat16*)out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, fv, (int)S, scale, causal, \
      ctx->dev_err)
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

#ifdef LMB_FLASH_TRACE
extern "C" int32_t lmb200_debug_flash_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, lmb::g_flash_trace, sizeof(lmb::g_flash_trace)) == cudaSuccess ? 0 : -3;
}
#endif
