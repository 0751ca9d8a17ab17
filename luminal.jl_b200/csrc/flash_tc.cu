// FlashAttentionOp on the tensor cores (bf16): out = softmax(scale * Q K^T [+ causal]) V.
// Replaces flash_attn_fwd_kernel (src/Execution.jl:374-450, one query row per block, keys in
// series, no tensor cores) for bf16 tensors of head_dim 64 or 128.
//
// One CTA = 128 query rows of one (batch, head), keys in tiles of 64:
//   4 loader warps : cp.async 16-byte chunks of Q / K / V from row-major global memory into the
//                    canonical core-matrix layout (8 rows x 16 bytes) the tensor core reads, 3 K/V
//                    stages in flight;
//   1 MMA warp     : one thread issues tcgen05.mma -- S = Q K^T (M 128, N 64, K = D) into a
//                    double-buffered TMEM tile, then PV = P V (M 128, N = D, K 64; V read MN-major
//                    from the same tile layout as K) into another; tcgen05.commit signals mbarriers;
//   4 softmax warps: one query row per thread: tcgen05.ld the S row, online softmax (exp2 with the
//                    scale folded in), write P as bf16 straight into the A-operand layout, and fold
//                    the previous tile's PV into the row's float32 output registers
//                    (O = O * alpha + PV), so the softmax of tile j+1 overlaps the PV MMA of tile j.
// Causal: key tiles beyond the diagonal are never loaded; inside the diagonal tile keys j > i are
// masked -- the reference's `if causal && j > i continue`.
#include <math_constants.h>

#include "common.cuh"
#include "tc.cuh"

namespace lmb {
namespace {

constexpr int kBM = 128, kBN = 64, kKvStages = 3;
constexpr int kThreads = 9 * 32;         // warps 0-3 softmax, 4 MMA, 5-8 loaders
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct Smem {
  static constexpr int kQ = kBM * D * 2;
  static constexpr int kKV = kBN * D * 2;
  static constexpr int kP = kBM * kBN * 2;
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + kQ;
  static constexpr int offV = offK + kKvStages * kKV;
  static constexpr int offP = offV + kKvStages * kKV;
  static constexpr int total = offP + 2 * kP;
};

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
  __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], pv_full[2], pv_empty[2];
  __shared__ uint32_t tmem_slot;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColPV = 128;               // S: 2 x 64 columns, PV: 2 x D columns

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;      // heavy (late) causal tiles first
  const int q0 = qt * kBM;
  // blockIdx.y = batch * H + head; query head h reads kv head h / G (G = 1: an op with H kv heads)
  const int bi = (int)blockIdx.y / fv.H, hi = (int)blockIdx.y - bi * fv.H;
  const __nv_bfloat16* qb = q + bi * fv.q_b + hi * fv.q_h;
  const __nv_bfloat16* kb = k + bi * fv.k_b + (hi / fv.G) * fv.k_h;
  const __nv_bfloat16* vb = v + bi * fv.k_b + (hi / fv.G) * fv.k_h;
  __nv_bfloat16* ob_base = out + bi * fv.q_b + hi * fv.q_h;
  const int64_t q_s = fv.q_s, k_s = fv.k_s;
  const int k_stop = causal ? min(S, q0 + kBM) : S;
  const int n_tiles = (k_stop + kBN - 1) / kBN;

  if (tid == 0) {
    mbar_init(&q_full, 4);
    for (int s = 0; s < kKvStages; ++s) { mbar_init(&kv_full[s], 4); mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1);
      mbar_init(&pv_full[i], 1); mbar_init(&pv_empty[i], 4);
    }
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
    const int lt = tid - 5 * 32;                    // 0..127
    const uint32_t sQ = smem_u32(smem + SM::offQ);
    for (int i = lt; i < kBM * (D / 8); i += 128) {
      const int row = i / (D / 8), c8 = i - row * (D / 8);
      const int qi = q0 + row;
      cp_async16(sQ + canon(row, c8, kBM), qb + (int64_t)min(qi, S - 1) * q_s + c8 * 8, qi < S ? 16u : 0u);
    }
    cp_async_commit();
    auto signal_oldest = [&](int j) {               // tile j has landed in its stage
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&kv_full[j % kKvStages]);
    };
    bool q_signalled = false;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % kKvStages;
      mbar_wait(&kv_empty[s], ((j / kKvStages) & 1) ^ 1, dead, err);
      const uint32_t sK = smem_u32(smem + SM::offK + s * SM::kKV), sV = smem_u32(smem + SM::offV + s * SM::kKV);
      for (int i = lt; i < kBN * (D / 8); i += 128) {
        const int row = i / (D / 8), c8 = i - row * (D / 8);
        const int key = j * kBN + row;
        const int64_t src = (int64_t)min(key, S - 1) * k_s + c8 * 8;
        const uint32_t nb = key < S ? 16u : 0u;
        cp_async16(sK + canon(row, c8, kBN), kb + src, nb);
        cp_async16(sV + canon(row, c8, kBN), vb + src, nb);
      }
      cp_async_commit();
      // groups in flight: Q (until signalled), tiles j-1 and j at most
      if (!q_signalled) {
        cp_async_wait<1>();                          // Q (and everything before tile j) has landed
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&q_full);
        q_signalled = true;
      }
      if (j >= 1) {
        cp_async_wait<1>();                          // tile j-1 has landed
        signal_oldest(j - 1);
      }
    }
    cp_async_wait<0>();
    if (!q_signalled) {
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full);
    }
    if (n_tiles >= 1) signal_oldest(n_tiles - 1);
  } else if (warp == 4) {
    // ------------------------------ MMA issue ------------------------------
    constexpr uint32_t kIdescS = idesc_bf16(kBM, kBN, false, false);
    constexpr uint32_t kIdescPV = idesc_bf16(kBM, D, false, true);          // V is read MN-major
    const uint32_t sQ = smem_u32(smem + SM::offQ);
    mbar_wait(&q_full, 0, dead, err);
    auto issue_pv = [&](int j) {
      const int pb = j & 1, s = j % kKvStages;
      mbar_wait(&p_full[pb], (j >> 1) & 1, dead, err);
      mbar_wait(&pv_empty[pb], ((j >> 1) & 1) ^ 1, dead, err);
      fence_after();
      if (lane == 0) {
        // A = P [128 x 64] K-major: lbo (between key groups of 8) = 128*16, sbo = 128
        // B = V tile [64 keys x D] read as N = d (contiguous), K = key: sbo (between d groups) =
        //     64*16 = 1024, lbo (between key groups) = 128
        const uint64_t adesc = smem_desc(smem_u32(smem + SM::offP + pb * SM::kP), kBM * 16, 128);
        const uint64_t bdesc = smem_desc(smem_u32(smem + SM::offV + s * SM::kKV), 128, kBN * 16);
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks)
          mma_f16(tmem + kColPV + pb * D, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)), bdesc + (uint64_t)(ks * (256 >> 4)),
                  kIdescPV, ks ? 1u : 0u);
        commit(&pv_full[pb]);
        commit(&p_empty[pb]);
        commit(&kv_empty[s]);
      }
      __syncwarp();
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1, s = j % kKvStages;
      mbar_wait(&kv_full[s], (j / kKvStages) & 1, dead, err);
      mbar_wait(&s_empty[sb], ((j >> 1) & 1) ^ 1, dead, err);
      fence_after();
      if (lane == 0) {
        // A = Q [128 x D] K-major: lbo = 128*16, sbo = 128;  B = K tile [64 x D] K-major: lbo = 64*16
        const uint64_t adesc = smem_desc(sQ, kBM * 16, 128);
        const uint64_t bdesc = smem_desc(smem_u32(smem + SM::offK + s * SM::kKV), kBN * 16, 128);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          mma_f16(tmem + kColS + sb * kBN, adesc + (uint64_t)(ks * ((2 * kBM * 16) >> 4)),
                  bdesc + (uint64_t)(ks * ((2 * kBN * 16) >> 4)), kIdescS, ks ? 1u : 0u);
        commit(&s_full[sb]);
      }
      __syncwarp();
      if (j >= 1) issue_pv(j - 1);
    }
    if (n_tiles >= 1) issue_pv(n_tiles - 1);
  } else {
    // ------------------------------ softmax + output: one query row per thread ------------------------------
    const int r = 32 * warp + lane;
    const int qi = q0 + r;
    const uint32_t lane_base = (uint32_t)(32 * warp) << 16;
    const float c = scale * kLog2e;
    float m = -CUDART_INF_F, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    float alpha_pending = 1.f;
    auto accumulate = [&](int j, float alpha) {       // O = O * alpha + P_j V_j
      const int pb = j & 1;
      mbar_wait(&pv_full[pb], (j >> 1) & 1, dead, err);
      fence_after();
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        float t[32];
        tmem_ld32(t, tmem + lane_base + kColPV + pb * D + ch * 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[ch * 32 + i] = fmaf(o[ch * 32 + i], alpha, t[i]);
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pv_empty[pb]);
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      mbar_wait(&s_full[sb], (j >> 1) & 1, dead, err);
      fence_after();
      float sv[2][32];
      tmem_ld32(sv[0], tmem + lane_base + kColS + sb * kBN);
      tmem_ld32(sv[1], tmem + lane_base + kColS + sb * kBN + 32);
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);
      float mx = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < kBN; ++i) {
        const int key = j * kBN + i;
        const bool masked = key >= S || (causal && key > qi);
        sv[i >> 5][i & 31] = masked ? -CUDART_INF_F : sv[i >> 5][i & 31] * c;
        mx = fmaxf(mx, sv[i >> 5][i & 31]);
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;     // row fully masked so far
      const float alpha = exp2f(m - m_use);
      float sum = 0.f;
      uint32_t packed[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN; i += 2) {
        const float p0 = exp2f(sv[i >> 5][i & 31] - m_use), p1 = exp2f(sv[i >> 5][(i & 31) + 1] - m_use);
        // the row sum uses the same bf16-rounded values the tensor core multiplies with V
        const __nv_bfloat162 pb2 = __floats2bfloat162_rn(p0, p1);
        sum += __low2float(pb2) + __high2float(pb2);
        packed[i / 2] = *reinterpret_cast<const uint32_t*>(&pb2);
      }
      l = l * alpha + sum;
      m = m_new;
      mbar_wait(&p_empty[sb], ((j >> 1) & 1) ^ 1, dead, err);
      unsigned char* pt = smem + SM::offP + sb * SM::kP;
#pragma unroll
      for (int c8 = 0; c8 < kBN / 8; ++c8)
        *reinterpret_cast<uint4*>(pt + canon(r, c8, kBM)) =
            make_uint4(packed[4 * c8], packed[4 * c8 + 1], packed[4 * c8 + 2], packed[4 * c8 + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
      if (j >= 1) accumulate(j - 1, alpha_pending);
      alpha_pending = alpha;
    }
    if (n_tiles >= 1) accumulate(n_tiles - 1, alpha_pending);
    if (qi < S) {
      const float inv = 1.0f / l;
      __nv_bfloat16* ob = ob_base + (int64_t)qi * q_s;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        uint4 w;
        __nv_bfloat162 a0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv), a1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
        __nv_bfloat162 a2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv), a3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
        w.x = *reinterpret_cast<uint32_t*>(&a0); w.y = *reinterpret_cast<uint32_t*>(&a1);
        w.z = *reinterpret_cast<uint32_t*>(&a2); w.w = *reinterpret_cast<uint32_t*>(&a3);
        *reinterpret_cast<uint4*>(ob + i) = w;
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 4) {
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
  dim3 grid((unsigned)ceil_div(S, kBM), (unsigned)(B * fv.H));
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
