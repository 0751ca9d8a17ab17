// FlashAttentionOp: out = softmax(scale * Q K^T [+ causal]) V on [B, H, S, D].
// Replaces flash_attn_fwd_kernel / flash_attn_cpu (src/Execution.jl:374-479, 565-578).
//
// CUDA-core kernel: a CTA owns 64 query rows of one (batch, head), 4 threads per row, each
// holding a quarter of the row's q and output accumulators in registers.  K/V tiles of 32 keys
// are staged in shared memory as float32 and every key updates the running (max, sum, output)
// exactly like the reference's scalar online softmax; causal skips keys j > i.
#include <math_constants.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace lmb {
// tensor-core kernel (flash_tc.cu)
bool flash_tc_supported(int64_t D);
int32_t flash_tc_f32_launch(Ctx* ctx, float* out, const float* q, const float* k, const float* v, int64_t BH, int64_t S, int64_t D,
                            float scale, int causal);
int32_t flash_tc_launch(Ctx* ctx, void* out, const void* q, const void* k, const void* v, int64_t BH, int64_t S, int64_t D,
                        float scale, int causal);
namespace {

constexpr int kBQ = 64, kBK = 32, kThreads = 256;

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) flash_simple_kernel(T* out, const T* q, const T* k, const T* v, int S,
                                                                float scale, int causal) {
  constexpr int NV = D / 16;                 // float4 chunks per thread
  __shared__ __align__(16) float ks[kBK][D];
  __shared__ __align__(16) float vs[kBK][D];
  const int tid = threadIdx.x, sub = tid & 3, row = tid >> 2;
  const int64_t bh = blockIdx.y;
  const int qi = blockIdx.x * kBQ + row;
  const T* qb = q + bh * (int64_t)S * D;
  const T* kb = k + bh * (int64_t)S * D;
  const T* vb = v + bh * (int64_t)S * D;
  float4 qr[NV], o[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = (i * 4 + sub) * 4;
    if (qi < S) {
      qr[i] = make_float4(to_f32(qb[(int64_t)qi * D + d]), to_f32(qb[(int64_t)qi * D + d + 1]),
                          to_f32(qb[(int64_t)qi * D + d + 2]), to_f32(qb[(int64_t)qi * D + d + 3]));
    } else {
      qr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float m = -CUDART_INF_F, l = 0.f;
  const int q_last = min(S, (int)(blockIdx.x + 1) * kBQ) - 1;
  const int k_stop = causal ? q_last + 1 : S;
  for (int k0 = 0; k0 < k_stop; k0 += kBK) {
    __syncthreads();
    for (int i = tid; i < kBK * D; i += kThreads) {
      const int kk = i / D, d = i - kk * D;
      const bool ok = k0 + kk < S;
      ks[kk][d] = ok ? to_f32(kb[(int64_t)(k0 + kk) * D + d]) : 0.f;
      vs[kk][d] = ok ? to_f32(vb[(int64_t)(k0 + kk) * D + d]) : 0.f;
    }
    __syncthreads();
    const int kmax = min(kBK, S - k0);
    for (int kk = 0; kk < kmax; ++kk) {
      const int j = k0 + kk;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const float4 kv4 = *reinterpret_cast<const float4*>(&ks[kk][(i * 4 + sub) * 4]);
        dot = fmaf(qr[i].x, kv4.x, dot); dot = fmaf(qr[i].y, kv4.y, dot);
        dot = fmaf(qr[i].z, kv4.z, dot); dot = fmaf(qr[i].w, kv4.w, dot);
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      if (causal && j > qi) continue;           // `if causal && j > i continue`
      dot *= scale;
      const float m_next = fmaxf(m, dot);
      const float p = expf(dot - m_next);
      const float so = (m == -CUDART_INF_F) ? 0.f : expf(m - m_next);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const float4 vv = *reinterpret_cast<const float4*>(&vs[kk][(i * 4 + sub) * 4]);
        o[i].x = fmaf(p, vv.x, o[i].x * so); o[i].y = fmaf(p, vv.y, o[i].y * so);
        o[i].z = fmaf(p, vv.z, o[i].z * so); o[i].w = fmaf(p, vv.w, o[i].w * so);
      }
      l = l * so + p;
      m = m_next;
    }
  }
  if (qi < S) {
    T* ob = out + bh * (int64_t)S * D + (int64_t)qi * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (i * 4 + sub) * 4;
      ob[d] = from_f32<T>(o[i].x * inv); ob[d + 1] = from_f32<T>(o[i].y * inv);
      ob[d + 2] = from_f32<T>(o[i].z * inv); ob[d + 3] = from_f32<T>(o[i].w * inv);
    }
  }
}

template <typename T>
int32_t launch(Ctx* ctx, void* out, const void* q, const void* k, const void* v, int64_t BH, int64_t S, int64_t D,
               float scale, int causal) {
  dim3 grid((unsigned)ceil_div(S, kBQ), (unsigned)BH);
#define LMB_FLASH(DD)                                                                               \
  flash_simple_kernel<T, DD><<<grid, kThreads, 0, ctx->stream>>>((T*)out, (const T*)q, (const T*)k, \
                                                                 (const T*)v, (int)S, scale, causal)
  switch (D) {
    case 16: LMB_FLASH(16); break;
    case 32: LMB_FLASH(32); break;
    case 64: LMB_FLASH(64); break;
    case 96: LMB_FLASH(96); break;
    case 128: LMB_FLASH(128); break;
    default: return fail(LMB200_EINVAL, "flash_attention: head_dim %lld not built (16/32/64/96/128)", (long long)D);
  }
#undef LMB_FLASH
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

}  // namespace
}  // namespace lmb

using namespace lmb;

extern "C" int32_t lmb200_flash_attention(lmb200_ctx h, void* out, const void* q, const void* k, const void* v,
                                          int32_t dtype, int64_t B, int64_t H, int64_t S, int64_t D, float scale,
                                          int32_t causal) {
  Ctx* ctx = ctx_from(h);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(out && q && k && v, "flash_attention: null pointer");
  LMB_REQUIRE(B >= 1 && H >= 1 && S >= 1 && B * H <= 65535, "flash_attention: bad shape");
  LMB_CUDA(cudaSetDevice(ctx->device));
  // LMB200_FLASH_KERNEL=simple keeps the CUDA-core kernel (comparison runs)
  const char* sel = getenv("LMB200_FLASH_KERNEL");
  if (dtype == LMB200_F32) {
    // float32 on the tensor cores: operands split into bf16 hi + lo, three MMAs per product (flash_tc_f32.cu)
    if (flash_tc_supported(D) && !(sel && strcmp(sel, "simple") == 0))
      return flash_tc_f32_launch(ctx, (float*)out, (const float*)q, (const float*)k, (const float*)v, B * H, S, D, scale, causal);
    return launch<float>(ctx, out, q, k, v, B * H, S, D, scale, causal);
  }
  if (dtype == LMB200_BF16) {
    if (flash_tc_supported(D) && !(sel && strcmp(sel, "simple") == 0))
      return flash_tc_launch(ctx, out, q, k, v, B * H, S, D, scale, causal);
    return launch<__nv_bfloat16>(ctx, out, q, k, v, B * H, S, D, scale, causal);
  }
  return fail(LMB200_EINVAL, "flash_attention: dtype %d", dtype);
}
