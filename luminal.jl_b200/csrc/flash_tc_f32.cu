// FlashAttentionOp with float32 tensors on the tensor cores.
//
// The reference's flash attention is float32 throughout (src/Execution.jl:374-479, 565-578; its numeric pin
// is rtol 1e-4 against the materialised softmax, tests/test_flash_attention_verification.jl:24-50).  The
// tensor cores multiply bf16, so every float32 operand x is split into hi = bf16(x) and lo = bf16(x - hi)
// (x = hi + lo to about 2^-17 |x|) and every product a b is taken as a_hi b_hi + a_hi b_lo + a_lo b_hi with
// float32 accumulation in TMEM: three MMAs per product, relative error about 2^-16 per term -- the split that
// turns bf16 tensor cores into a float32-class product.  P = exp2(...) is split the same way before P V.
//
// One CTA = one tile of 128 query rows of one (batch, head); keys in tiles of 64, two stages of
// (K_hi, K_lo, V_hi, V_lo) in flight through TMA (swizzled sub-tiles, as in flash_tc.cu); one MMA warp;
// four softmax warps, one query row per thread; S double-buffered in TMEM, P single-buffered in shared
// memory; the running maximum is raised lazily as in the bf16 kernel.
#include <cuda.h>
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"
#include "tc.cuh"

namespace lmb {
namespace {

constexpr int kBM = 128, kBN = 64, kStages = 2;
constexpr int kLoaders = 2 * 32;
constexpr int kThreads = 5 * 32 + kLoaders;      // warps 0-3 softmax, 4 MMA, 5-6 loaders
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.0f;

template <int D>
struct SmemF {
  static constexpr int kQ = kBM * D * 2;          // one of Q_hi / Q_lo
  static constexpr int kKV = kBN * D * 2;         // one of K_hi / K_lo / V_hi / V_lo
  static constexpr int kP = kBM * kBN * 2;        // one of P_hi / P_lo
  static constexpr int offQ = 0;                  // [hi, lo]
  static constexpr int offKV = offQ + 2 * kQ;     // [stage][K_hi, K_lo, V_hi, V_lo]
  static constexpr int offP = offKV + kStages * 4 * kKV;
  static constexpr int total = offP + 2 * kP;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t canon(int row, int c8, int rows) {
  return (uint32_t)(c8 * (rows * 16) + (row >> 3) * 128 + (row & 7) * 16);
}
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
__device__ __forceinline__ void split2(float a, float b, uint32_t* hi, uint32_t* lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const float2 hf = __bfloat1622float2(h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - hf.x, b - hf.y);
  *hi = *reinterpret_cast<const uint32_t*>(&h);
  *lo = *reinterpret_cast<const uint32_t*>(&l);
}

// x (float32) -> hl[0][i] = bf16(x), hl[1][i] = bf16(x - hl[0][i]);  n a multiple of 4
__global__ void split_hi_lo_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hl, int64_t n) {
  for (int64_t i = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    uint2 h, l;
    split2(v.x, v.y, &h.x, &l.x);
    split2(v.z, v.w, &h.y, &l.y);
    *reinterpret_cast<uint2*>(hl + i) = h;
    *reinterpret_cast<uint2*>(hl + n + i) = l;
  }
}

// qhl: [2][BH][S][D] bf16 (hi, lo); kmap / vmap: 4-D maps over [2][BH][S][D] (d, key, batch-head, hi/lo)
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
flash_tc_f32_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ qhl, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap, int64_t BH, int S, float scale, int causal, int* err) {
  using namespace tc;
  typedef SmemF<D> SM;
  constexpr int W = D % 64 == 0 ? 64 : 32;
  constexpr int kSub = kBN * W * 2;
  constexpr uint32_t kSwz = W == 64 ? 2u : 4u;
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[2], s_empty[2], p_full, p_empty;
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kColS = 0, kColO = 128;                  // S: two buffers of 64 columns; O: D columns

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qp = (int)gridDim.x - 1 - (int)blockIdx.x;         // heavy (late) causal tiles first
  const int q0 = qp * kBM;
  const int bh = (int)blockIdx.y;
  const int k_stop = causal ? min(S, q0 + kBM) : S;
  const int nt = (k_stop + kBN - 1) / kBN;

  if (tid == 0) {
    mbar_init(&q_full, kLoaders / 32);
    for (int s = 0; s < kStages; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); }
    mbar_init(&p_full, 4);
    mbar_init(&p_empty, 1);
    mbar_init_fence();
  }
  if (warp == 4) tmem_alloc(&tmem_slot, kTmemCols);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  bool dead = false;

  if (warp >= 5) {
    // ------------------------------ loaders ------------------------------
    const int lw = warp - 5, lt = tid - 5 * 32;
    const uint32_t sQ = smem_u32(smem + SM::offQ);
    for (int i = lt; i < 2 * kBM * (D / 8); i += kLoaders) {
      const int part = i / (kBM * (D / 8)), rem = i - part * (kBM * (D / 8));      // 0: hi, 1: lo
      const int row = rem / (D / 8), c8 = rem - row * (D / 8);
      const int qi = q0 + row;
      const __nv_bfloat16* src = qhl + ((int64_t)part * BH + bh) * (int64_t)S * D + (int64_t)min(qi, S - 1) * D + c8 * 8;
      cp_async16(sQ + part * SM::kQ + canon(row, c8, kBM), src, qi < S ? 16u : 0u);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_full);
    if (lw == 0) {
      for (int j = 0; j < nt; ++j) {
        const int s = j % kStages;
        mbar_wait(&kv_empty[s], ((j / kStages) & 1) ^ 1, dead, err);
        if (lane == 0) {
          mbar_expect_tx(&kv_full[s], (uint32_t)(4 * SM::kKV));
          unsigned char* st = smem + SM::offKV + s * 4 * SM::kKV;
#pragma unroll
          for (int part = 0; part < 2; ++part) {
#pragma unroll
            for (int sub = 0; sub < D / W; ++sub) {
              tma_load_4d(st + part * SM::kKV + sub * kSub, &kmap, sub * W, j * kBN, bh, part, &kv_full[s]);
              tma_load_4d(st + (2 + part) * SM::kKV + sub * kSub, &vmap, sub * W, j * kBN, bh, part, &kv_full[s]);
            }
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 4) {
    // ------------------------------ MMA issue ------------------------------
    constexpr uint32_t kIdescS = idesc_bf16(kBM, kBN, false, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, D, false, true);          // V is read MN-major
    mbar_wait(&q_full, 0, dead, err);
    // the three partial products of one float32-class product: (hi, hi), (hi, lo), (lo, hi)
    const int a_part[3] = {0, 0, 1}, b_part[3] = {0, 1, 0};
    auto issue_pv = [&](int j) {
      const int s = j % kStages;
      mbar_wait(&p_full, j & 1, dead, err);
      fence_after();
      if (lane == 0) {
        unsigned char* st = smem + SM::offKV + s * 4 * SM::kKV;
#pragma unroll
        for (int t3 = 0; t3 < 3; ++t3) {
          const uint64_t adesc = smem_desc(smem_u32(smem + SM::offP + a_part[t3] * SM::kP), kBM * 16, 128);
          const uint64_t bdesc = smem_desc_swz(smem_u32(st + (2 + b_part[t3]) * SM::kKV), kSub, 16 * W, kSwz);
#pragma unroll
          for (int ks = 0; ks < kBN / 16; ++ks)
            mma_f16(tmem + kColO, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)), bdesc + (uint64_t)(ks * ((32 * W) >> 4)),
                    kIdescPV, (j > 0 || ks > 0 || t3 > 0) ? 1u : 0u);
        }
        commit(&p_empty);
        commit(&kv_empty[s]);
      }
      __syncwarp();
    };
    for (int j = 0; j < nt; ++j) {
      const int sb = j & 1, s = j % kStages;
      mbar_wait(&kv_full[s], (j / kStages) & 1, dead, err);
      mbar_wait(&s_empty[sb], ((j >> 1) & 1) ^ 1, dead, err);
      fence_after();
      if (lane == 0) {
        unsigned char* st = smem + SM::offKV + s * 4 * SM::kKV;
#pragma unroll
        for (int t3 = 0; t3 < 3; ++t3) {
          const uint64_t adesc = smem_desc(smem_u32(smem + SM::offQ + a_part[t3] * SM::kQ), kBM * 16, 128);
          const uint32_t sK = smem_u32(st + b_part[t3] * SM::kKV);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t bdesc = smem_desc_swz(sK + ((16 * ks) / W) * kSub + ((16 * ks) % W) * 2, 16, 16 * W, kSwz);
            mma_f16(tmem + kColS + sb * kBN, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)), bdesc, kIdescS, (ks || t3) ? 1u : 0u);
          }
        }
        commit(&s_full[sb]);
      }
      __syncwarp();
      if (j >= 1) issue_pv(j - 1);
    }
    if (nt >= 1) issue_pv(nt - 1);
  } else {
    // ------------------------------ softmax + output: one query row per thread ------------------------------
    const int r = 32 * warp + lane;
    const int qi = q0 + r;
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    const float c = scale * kLog2e;
    float m = -CUDART_INF_F, l = 0.f;
    for (int j = 0; j < nt; ++j) {
      const int sb = j & 1;
      mbar_wait(&s_full[sb], (j >> 1) & 1, dead, err);
      fence_after();
      float sv[kBN];
      tmem_ld64(sv, tmem + lane_base + kColS + sb * kBN);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      const bool inside = (j + 1) * kBN <= S && (!causal || (j + 1) * kBN - 1 <= q0);
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
      const bool first = m == -CUDART_INF_F && mx > -CUDART_INF_F;
      const bool raise = m > -CUDART_INF_F && mx > m + kRescaleStep;
      // P V of the previous key tile has landed: the single P buffer is free again and O may be rescaled.  This
      // thread waits every phase of the barrier in turn, so the parity is never that of an older phase.
      if (j > 0) {
        mbar_wait(&p_empty, (j - 1) & 1, dead, err);
        fence_after();
      }
      if (__any_sync(0xffffffffu, raise) && j > 0) {
        const float alpha = raise ? exp2f(m - mx) : 1.0f;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          float o[32];
          tmem_ld32(o, tmem + lane_base + kColO + ch * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(tmem + lane_base + kColO + ch * 32, o);
        }
        fence_before();
      }
      if (raise) { l *= exp2f(m - mx); m = mx; }
      if (first) m = mx;
      const float neg_m = m == -CUDART_INF_F ? 0.f : -m;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* ph = smem + SM::offP;
      unsigned char* pl = ph + SM::kP;
#pragma unroll
      for (int c8 = 0; c8 < kBN / 8; ++c8) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = 8 * c8 + 2 * e;
          const float p0 = ex2_approx(fmaf(sv[i], c, neg_m)), p1 = ex2_approx(fmaf(sv[i + 1], c, neg_m));
          sum4[e] += p0 + p1;
          split2(p0, p1, &hi[e], &lo[e]);
        }
        *reinterpret_cast<uint4*>(ph + canon(r, c8, kBM)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(pl + canon(r, c8, kBM)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      fence_async_smem();
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    if (nt >= 1) {
      mbar_wait(&p_empty, (nt - 1) & 1, dead, err);
      fence_after();
      const float inv = 1.0f / l;
      float* ob = out + ((int64_t)bh * S + qi) * D;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        float o[32];
        tmem_ld32(o, tmem + lane_base + kColO + ch * 32);
        if (qi < S) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(ob + ch * 32 + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        }
      }
      fence_before();
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 4) {
    fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
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

// map over a [2][BH][S][D] bf16 tensor: dims {d, key, batch-head, hi/lo}; box [64 keys][W head dims]
int32_t hl_tensor_map(CUtensorMap* map, const void* base, int64_t BH, int64_t S, int64_t D) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fail(LMB200_ECUDA, "flash attention: cuTensorMapEncodeTiled is not available");
  const int W = D % 64 == 0 ? 64 : 32;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH, 2};
  const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)S * D * 2, (cuuint64_t)BH * S * D * 2};
  const cuuint32_t box[4] = {(cuuint32_t)W, (cuuint32_t)kBN, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, W == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LMB200_ECUDA, "flash attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return LMB200_OK;
}

}  // namespace

int32_t flash_tc_f32_configure() {
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_f32_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemF<128>::total + 1024));
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_f32_kernel<96>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemF<96>::total + 1024));
  LMB_CUDA(cudaFuncSetAttribute(flash_tc_f32_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemF<64>::total + 1024));
  return LMB200_OK;
}

// out, q, k, v: float32 [BH, S, D] contiguous on the device.  Scratch: the six bf16 halves (3 x 2 x BH x S x D x 2 bytes),
// kept in the context between calls.  Asynchronous on the context's stream like the bf16 kernel.
int32_t flash_tc_f32_launch(Ctx* ctx, float* out, const float* q, const float* k, const float* v, int64_t BH, int64_t S, int64_t D,
                            float scale, int causal) {
  const int64_t n = BH * S * D;
  LMB_REQUIRE(n % 4 == 0, "flash attention: element count must be a multiple of 4");
  const size_t need = (size_t)n * 2 * 3 * sizeof(__nv_bfloat16);
  if (ctx->scratch_bytes < need) {
    if (ctx->capturing)
      return fail(LMB200_ESTATE, "flash attention: the scratch must grow to %lld bytes, which a capture cannot record: run the call once before capture_begin",
                  (long long)need);
    // work queued on the stream may still use the smaller block
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch_in_graph) {                // a recorded graph reads it on every replay: keep it
      ctx->retired_scratch.push_back(ctx->scratch);
      ctx->scratch_in_graph = false;
    } else {
      cudaFree(ctx->scratch);
    }
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    if (cudaMalloc(&ctx->scratch, need) != cudaSuccess) {
      cudaGetLastError();
      return fail(LMB200_ENOMEM, "flash attention: scratch allocation of %lld bytes failed", (long long)need);
    }
    ctx->scratch_bytes = need;
  }
  if (ctx->capturing) ctx->scratch_in_graph = true;
  __nv_bfloat16* hl = reinterpret_cast<__nv_bfloat16*>(ctx->scratch);
  __nv_bfloat16 *qhl = hl, *khl = hl + 2 * n, *vhl = hl + 4 * n;
  const unsigned grid1 = (unsigned)std::min<int64_t>(ceil_div(n / 4, 256), 148 * 16);
  split_hi_lo_kernel<<<grid1, 256, 0, ctx->stream>>>(q, qhl, n);
  split_hi_lo_kernel<<<grid1, 256, 0, ctx->stream>>>(k, khl, n);
  split_hi_lo_kernel<<<grid1, 256, 0, ctx->stream>>>(v, vhl, n);
  ctx->launches += 3;
  CUtensorMap kmap, vmap;
  int32_t rc = hl_tensor_map(&kmap, khl, BH, S, D);
  if (rc == LMB200_OK) rc = hl_tensor_map(&vmap, vhl, BH, S, D);
  if (rc == LMB200_OK) {
    dim3 grid((unsigned)ceil_div(S, kBM), (unsigned)BH);
#define LMB_FLASH(DD) \
  flash_tc_f32_kernel<DD><<<grid, kThreads, SmemF<DD>::total + 1024, ctx->stream>>>(out, qhl, kmap, vmap, BH, (int)S, scale, causal, ctx->dev_err)
    if (D == 128) LMB_FLASH(128);
    else if (D == 96) LMB_FLASH(96);
    else if (D == 64) LMB_FLASH(64);
    else rc = fail(LMB200_EINVAL, "flash attention: head_dim %lld has no tensor-core kernel", (long long)D);
#undef LMB_FLASH
    if (rc == LMB200_OK) {
      ctx->launches++;
      if (cudaGetLastError() != cudaSuccess) rc = fail(LMB200_ECUDA, "flash attention: launch failed");
    }
  }
  return rc;
}

}  // namespace lmb
