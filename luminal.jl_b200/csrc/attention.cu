// Split-KV decode attention.
//
// bf16 path: one CTA = 4 warps owns `keys_per_cta` consecutive keys of one (sequence, kv head);
// every warp streams 16-key blocks of the tiled cache (8 KB per block at D = 128, contiguous,
// 16 bytes per lane per MMA operand) straight into registers, double buffered, and computes
//   S[key, head]  = K[key, :] . Q[head, :]       mma m16n8k16, M = keys, N = the <= 8 q heads
//   O^T[d, head] += V^T[d, key] * P[key, head]    mma m16n8k16, M = d,    N = heads
// so the G query heads that share a kv head read its keys once.  P goes from the accumulator
// layout of the first MMA to the B-operand layout of the second with one movmatrix per 8 keys;
// the online-softmax maxima are reduced over keys with warp shuffles.  Warps, then CTAs
// (through global scratch), are merged with the usual (max, sum, weighted O) rule.
//
// float32 path (parity configs): same cache layout and the same scratch format, CUDA cores.
#include <math_constants.h>
#include <stdlib.h>

#include "attention.cuh"
#include "pdl.cuh"

namespace lmb {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kAttnThreads = 128;

// Keys per CTA for a context of T keys: the launch has nsplit CTAs per (sequence, kv head), planned
// for the cache capacity; a shorter context is divided evenly among the same CTAs (multiples of 64).
__device__ __forceinline__ int keys_per_cta_for(const AttnParams& p, int T) {
  const int even = (((T + p.nsplit - 1) / p.nsplit + 63) >> 6) << 6;
  return even < p.keys_per_cta ? even : p.keys_per_cta;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_bf16_kernel(const AttnParams p) {
  constexpr int DK = D / 16;
  __shared__ float sm_o[4][8][D];
  __shared__ float sm_m[4][8];
  __shared__ float sm_l[4][8];

  pdl_launch_dependents();
  pdl_wait();
  const int bk = blockIdx.x;
  const int b = bk / p.KVl, kvl = bk - b * p.KVl;
  const int T = p.pos ? (p.pos[b] + 1) : p.T_fixed;        // every sequence has its own context length
  const int kpc = keys_per_cta_for(p, T);
  const int k_begin = blockIdx.y * kpc;
  if (k_begin >= T) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int G = p.G;
  const float c = p.scale * kLog2e;

  // Q as the B operand of S = K Q^T: lane (g,t) holds Q[head g][d 2t,2t+1] and [d 2t+8,2t+9]
  uint32_t qf[DK][2];
  {
    const __nv_bfloat16* qrow =
        reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t)b * p.q_pitch + (kvl * G + g) * D;
#pragma unroll
    for (int dk = 0; dk < DK; ++dk) {
      qf[dk][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + 16 * dk + 2 * t) : 0u;
      qf[dk][1] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + 16 * dk + 2 * t + 8) : 0u;
    }
  }

  const int kpw = kpc / 4;
  const int wb = k_begin + warp * kpw;
  const int we = min(T, wb + kpw);
  const int kb_begin = wb >> 4, kb_end = (we + 15) >> 4;     // empty when wb >= T

  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  float o[DK][4];
#pragma unroll
  for (int i = 0; i < DK; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const uint4* base = reinterpret_cast<const uint4*>(
      reinterpret_cast<const __nv_bfloat16*>(p.kv_layer) + b * p.kv_batch_stride + kvl * p.kv_head_stride);
  auto load_block = [&](uint4 (&kf)[DK], uint4 (&vf)[DK], int kb) {
    const uint4* blk = base + (int64_t)kb * (4 * D) + lane;   // 32*D elements = 4*D uint4 per block
#pragma unroll
    for (int i = 0; i < DK; ++i) kf[i] = __ldcs(blk + i * 32);
#pragma unroll
    for (int i = 0; i < DK; ++i) vf[i] = __ldcs(blk + (DK + i) * 32);
  };
  auto process = [&](const uint4 (&kf)[DK], const uint4 (&vf)[DK], int kb) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int dk = 0; dk < DK; ++dk) mma_bf16(s, kf[dk].x, kf[dk].y, kf[dk].z, kf[dk].w, qf[dk][0], qf[dk][1]);
    const int key0 = kb * 16 + g;
    if (key0 >= T) s[0] = s[1] = -CUDART_INF_F;
    if (key0 + 8 >= T) s[2] = s[3] = -CUDART_INF_F;
    float bm0 = fmaxf(s[0], s[2]), bm1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      bm0 = fmaxf(bm0, __shfl_xor_sync(0xffffffffu, bm0, off));
      bm1 = fmaxf(bm1, __shfl_xor_sync(0xffffffffu, bm1, off));
    }
    const float mn0 = fmaxf(m0, bm0), mn1 = fmaxf(m1, bm1);
    const float a0 = exp2f((m0 - mn0) * c), a1 = exp2f((m1 - mn1) * c);
    const float p00 = exp2f((s[0] - mn0) * c), p01 = exp2f((s[1] - mn1) * c);
    const float p10 = exp2f((s[2] - mn0) * c), p11 = exp2f((s[3] - mn1) * c);
    l0 = l0 * a0 + (p00 + p10);
    l1 = l1 * a1 + (p01 + p11);
    m0 = mn0;
    m1 = mn1;
    const uint32_t pb0 = movmatrix_trans(pack_bf16(p00, p01));   // P[key 2t,2t+1][head g]
    const uint32_t pb1 = movmatrix_trans(pack_bf16(p10, p11));   // P[key 2t+8,2t+9][head g]
#pragma unroll
    for (int dm = 0; dm < DK; ++dm) {
      o[dm][0] *= a0; o[dm][1] *= a1; o[dm][2] *= a0; o[dm][3] *= a1;
      mma_bf16(o[dm], vf[dm].x, vf[dm].y, vf[dm].z, vf[dm].w, pb0, pb1);
    }
  };

  if (kb_begin < kb_end) {
    uint4 kf0[DK], vf0[DK], kf1[DK], vf1[DK];
    load_block(kf0, vf0, kb_begin);
    for (int kb = kb_begin; kb < kb_end; kb += 2) {
      const bool has1 = kb + 1 < kb_end;
      if (has1) load_block(kf1, vf1, kb + 1);
      process(kf0, vf0, kb);
      if (has1) {
        if (kb + 2 < kb_end) load_block(kf0, vf0, kb + 2);
        process(kf1, vf1, kb + 1);
      }
    }
  }
  // the row sums were kept per lane; finish them over the 8 key lanes
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, off);
    l1 += __shfl_xor_sync(0xffffffffu, l1, off);
  }
  // lane (g,t) holds O^T[d = 16dm+g (+8)][head 2t, 2t+1]
  if (2 * t < G) {
    if (g == 0) { sm_m[warp][2 * t] = m0; sm_l[warp][2 * t] = l0; }
#pragma unroll
    for (int dm = 0; dm < DK; ++dm) { sm_o[warp][2 * t][16 * dm + g] = o[dm][0]; sm_o[warp][2 * t][16 * dm + g + 8] = o[dm][2]; }
  }
  if (2 * t + 1 < G) {
    if (g == 0) { sm_m[warp][2 * t + 1] = m1; sm_l[warp][2 * t + 1] = l1; }
#pragma unroll
    for (int dm = 0; dm < DK; ++dm) { sm_o[warp][2 * t + 1][16 * dm + g] = o[dm][1]; sm_o[warp][2 * t + 1][16 * dm + g + 8] = o[dm][3]; }
  }
  __syncthreads();
  const int64_t slot = (int64_t)bk * p.nsplit + blockIdx.y;
  for (int i = tid; i < G * D; i += kAttnThreads) {
    const int h = i / D, d = i - h * D;
    const float M = fmaxf(fmaxf(sm_m[0][h], sm_m[1][h]), fmaxf(sm_m[2][h], sm_m[3][h]));
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = exp2f((sm_m[w][h] - M) * c);
      acc += wgt * sm_o[w][h][d];
      lsum += wgt * sm_l[w][h];
    }
    p.part_o[(slot * G + h) * D + d] = acc;
    if (d == 0) {
      p.part_ml[(slot * G + h) * 2] = M * c;        // stored in log2 units
      p.part_ml[(slot * G + h) * 2 + 1] = lsum;
    }
  }
  if (!p.counters) return;          // the splits are merged by attn_combine_kernel
  // The CTA that finishes last for this (sequence, kv head) merges the splits itself: same
  // arithmetic and order as attn_combine_kernel, without another launch.
  __shared__ int is_last;
  const int nvalid = (T + kpc - 1) / kpc;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(&p.counters[bk], 1u);
    is_last = prev == (unsigned)nvalid - 1u;
    if (is_last) p.counters[bk] = 0u;          // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* w_m = &sm_o[0][0][0];                  // [nvalid][G] maxima, then [nvalid][G] sums
  float* w_l = w_m + p.nsplit * G;
  const int64_t slot0 = (int64_t)bk * p.nsplit;
  for (int i = tid; i < nvalid * G; i += kAttnThreads) {
    w_m[i] = __ldcg(p.part_ml + (slot0 * G + i) * 2);
    w_l[i] = __ldcg(p.part_ml + (slot0 * G + i) * 2 + 1);
  }
  __syncthreads();
  __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
  for (int i = tid; i < G * D; i += kAttnThreads) {
    const int h = i / D, d = i - h * D;
    float Mx = -CUDART_INF_F;
    for (int sp = 0; sp < nvalid; ++sp) Mx = fmaxf(Mx, w_m[sp * G + h]);
    float denom = 0.f;
    for (int sp = 0; sp < nvalid; ++sp) denom += exp2f(w_m[sp * G + h] - Mx) * w_l[sp * G + h];
    const float inv = 1.0f / denom;
    float acc = 0.f;
    const float* po = p.part_o + (slot0 * G + h) * D + d;
#pragma unroll 8
    for (int sp = 0; sp < nvalid; ++sp) acc += exp2f(w_m[sp * G + h] - Mx) * __ldcg(po + (int64_t)sp * G * D);
    const int hl = kvl * G + h;
    const int64_t o = p.out_tiled_bp > 0 ? Layout<__nv_bfloat16>::x_offset(b, hl * D + d, p.out_tiled_bp)
                                         : (int64_t)b * p.out_pitch + hl * D + d;
    out[o] = __float2bfloat16_rn(acc * inv);
  }
}

// float32 path: one CTA per (sequence, kv head, split, q head of the group).
template <typename T>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_simple_kernel(const AttnParams p) {
  extern __shared__ float sm[];       // q[D] | p[keys_per_cta] | red[kAttnThreads]
  const int D = p.D;
  float* qs = sm;
  float* ps = sm + D;
  float* red = ps + p.keys_per_cta;
  pdl_launch_dependents();
  pdl_wait();
  const int bk = blockIdx.x, h = blockIdx.z;
  const int b = bk / p.KVl, kvl = bk - b * p.KVl;
  const int Tctx = p.pos ? (p.pos[b] + 1) : p.T_fixed;
  const int kpc = keys_per_cta_for(p, Tctx);
  const int k_begin = blockIdx.y * kpc;
  if (k_begin >= Tctx) return;
  const int k_end = min(Tctx, k_begin + kpc);
  const int n = k_end - k_begin;
  const int tid = threadIdx.x;
  const T* q = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_pitch + (kvl * p.G + h) * D;
  const T* kv = reinterpret_cast<const T*>(p.kv_layer) + b * p.kv_batch_stride + kvl * p.kv_head_stride;
  for (int d = tid; d < D; d += kAttnThreads) qs[d] = to_f32(q[d]);
  __syncthreads();
  // scores: (q.k) * scale, as src/NN.jl:369
  float lmax = -CUDART_INF_F;
  for (int i = tid; i < n; i += kAttnThreads) {
    const int key = k_begin + i;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(qs[d], to_f32(kv[kcache_offset(key, d, D)]), s);
    s *= p.scale;
    ps[i] = s;
    lmax = fmaxf(lmax, s);
  }
  red[tid] = lmax;
  __syncthreads();
  for (int off = kAttnThreads / 2; off > 0; off >>= 1) {
    if (tid < off) red[tid] = fmaxf(red[tid], red[tid + off]);
    __syncthreads();
  }
  const float M = red[0];
  __syncthreads();
  // exp(x) = exp2(x * 1/ln2), src/HighLevelOps.jl:127-129
  float lsum = 0.f;
  for (int i = tid; i < n; i += kAttnThreads) {
    const float e = exp2f((ps[i] - M) * kLog2e);
    ps[i] = e;
    lsum += e;
  }
  red[tid] = lsum;
  __syncthreads();
  for (int off = kAttnThreads / 2; off > 0; off >>= 1) {
    if (tid < off) red[tid] += red[tid + off];
    __syncthreads();
  }
  const float L = red[0];
  const int64_t slot = (int64_t)bk * p.nsplit + blockIdx.y;
  for (int d = tid; d < D; d += kAttnThreads) {
    float acc = 0.f;
    for (int i = 0; i < n; ++i) acc = fmaf(ps[i], to_f32(kv[vcache_offset(k_begin + i, d, D)]), acc);
    p.part_o[(slot * p.G + h) * D + d] = acc;
  }
  if (tid == 0) {
    p.part_ml[(slot * p.G + h) * 2] = M * kLog2e;    // log2 units, like the bf16 kernel
    p.part_ml[(slot * p.G + h) * 2 + 1] = L;
  }
}

// merge the splits of one (sequence, local q head) and normalise: out = sum_s w_s O_s / sum_s w_s l_s
template <typename T>
__global__ void attn_combine_kernel(const AttnParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x / (p.KVl * p.G);
  const int Tctx = p.pos ? (p.pos[b] + 1) : p.T_fixed;
  const int kpc = keys_per_cta_for(p, Tctx);
  const int nvalid = (Tctx + kpc - 1) / kpc;
  const int hl = blockIdx.x - b * (p.KVl * p.G);
  const int kvl = hl / p.G, h = hl - kvl * p.G;
  const int64_t slot0 = (int64_t)(b * p.KVl + kvl) * p.nsplit;
  float M = -CUDART_INF_F;
  for (int s = 0; s < nvalid; ++s) M = fmaxf(M, p.part_ml[((slot0 + s) * p.G + h) * 2]);
  float denom = 0.f;
  for (int s = 0; s < nvalid; ++s) {
    const float* ml = p.part_ml + ((slot0 + s) * p.G + h) * 2;
    denom += exp2f(ml[0] - M) * ml[1];
  }
  const float inv = 1.0f / denom;
  T* out = reinterpret_cast<T*>(p.out);
  for (int d = threadIdx.x; d < p.D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nvalid; ++s) {
      const float w = exp2f(p.part_ml[((slot0 + s) * p.G + h) * 2] - M);
      acc += w * p.part_o[((slot0 + s) * p.G + h) * p.D + d];
    }
    const int64_t o = p.out_tiled_bp > 0 ? Layout<T>::x_offset(b, hl * p.D + d, p.out_tiled_bp)
                                         : (int64_t)b * p.out_pitch + hl * p.D + d;
    out[o] = from_f32<T>(acc * inv);
  }
}

}  // namespace

// The decode-attention kernels keep their operands in flight through L1 (streaming loads), so
// they want the largest L1 split; the tiny combine kernel follows the GEMV's split instead.
int32_t attn_configure() {
  LMB_CUDA(cudaFuncSetAttribute(attn_combine_kernel<float>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                cudaSharedmemCarveoutMaxShared));
  LMB_CUDA(cudaFuncSetAttribute(attn_combine_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                cudaSharedmemCarveoutMaxShared));
  return LMB200_OK;
}

void attn_plan(const Ctx* ctx, int B, int KVl, int G, int D, int ctx_capacity, int* keys_per_cta,
               int* nsplit, int64_t* part_o_floats, int64_t* part_ml_floats) {
  // Two CTAs are resident per SM (registers).  Pick the split whose CTAs fill whole waves of
  // 2 x #SMs: cost = waves x (keys per CTA + a fixed per-CTA cost, about 96 keys' worth of q load,
  // merge and partial store).  Few (sequence, kv head) pairs -- tensor-parallel shards -- want few,
  // long splits in a single wave; many pairs want about 1024 keys per CTA.
  const int64_t pairs = (int64_t)B * KVl, resident = (int64_t)ctx->sm_count * 2;
  int64_t best_k = 64, best_cost = -1;
  for (int64_t k = 64; k <= 2048; k += 64) {
    const int64_t ns = ceil_div(ctx_capacity, k);
    if (k > 64 && ceil_div(ctx_capacity, k - 64) == ns) continue;      // same split count with shorter CTAs exists
    const int64_t cost = ceil_div(pairs * ns, resident) * (k + 96);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_k = k; }
  }
  const int64_t want = best_k;
  *keys_per_cta = (int)want;
  *nsplit = (int)ceil_div(ctx_capacity, want);
  *part_o_floats = (int64_t)B * KVl * (*nsplit) * G * D;
  *part_ml_floats = (int64_t)B * KVl * (*nsplit) * G * 2;
}

int32_t attn_decode_launch(Ctx* ctx, int dtype, const AttnParams& p_in, cudaStream_t stream) {
  AttnParams p = p_in;
  // the in-kernel merge keeps the splits' (max, sum) pairs in the shared memory of the O tiles
  if (dtype != LMB200_BF16 || 2 * p.nsplit * p.G > 32 * p.D) p.counters = nullptr;
  LMB_REQUIRE(p.keys_per_cta >= 64 && p.keys_per_cta % 64 == 0, "attention: keys_per_cta %d", p.keys_per_cta);
  LMB_REQUIRE(p.D % 16 == 0 && p.D >= 16 && p.D <= 256, "attention: head_dim %d", p.D);
  dim3 grid((unsigned)(p.B * p.KVl), (unsigned)p.nsplit, 1);
  // The attention kernels are launched in plain stream order: they keep their loads in flight
  // through L1, and a CTA that became resident next to a GEMV CTA (programmatic launch) would run
  // with that kernel's small-L1 / large-shared split (measured: 0.79 instead of 0.99 of the HBM rate).
  // LMB200_ATTN_PDL=1 launches it programmatically after all (A/B runs: with few (sequence, kv head) pairs per
  // GPU the launch gap weighs more than the L1 split).
  static const bool attn_pdl = [] { const char* e = getenv("LMB200_ATTN_PDL"); return e && atoi(e) == 1; }();
  if (dtype == LMB200_BF16) {
    LMB_REQUIRE(p.G <= 8, "attention: %d query heads per kv head (max 8 on the bf16 path)", p.G);
    switch (p.D) {
      case 32: LMB_CUDA(launch_k_opt(attn_pdl, attn_decode_bf16_kernel<32>, grid, dim3(kAttnThreads), 0, stream, p)); break;
      case 64: LMB_CUDA(launch_k_opt(attn_pdl, attn_decode_bf16_kernel<64>, grid, dim3(kAttnThreads), 0, stream, p)); break;
      case 96: LMB_CUDA(launch_k_opt(attn_pdl, attn_decode_bf16_kernel<96>, grid, dim3(kAttnThreads), 0, stream, p)); break;
      case 128: LMB_CUDA(launch_k_opt(attn_pdl, attn_decode_bf16_kernel<128>, grid, dim3(kAttnThreads), 0, stream, p)); break;
      default: return fail(LMB200_EINVAL, "attention: head_dim %d not built for bf16", p.D);
    }
    ctx->launches++;
    LMB_CUDA(cudaGetLastError());
    if (p.counters) return LMB200_OK;        // merged by the last CTA of each (sequence, kv head)
    LMB_CUDA(launch_k(attn_combine_kernel<__nv_bfloat16>, dim3(p.B * p.KVl * p.G), dim3(128), 0, stream, p));
  } else {
    grid.z = (unsigned)p.G;
    const size_t smem = (size_t)(p.D + p.keys_per_cta + kAttnThreads) * sizeof(float);
    LMB_CUDA(launch_k(attn_decode_simple_kernel<float>, grid, dim3(kAttnThreads), smem, stream, p));
    ctx->launches++;
    LMB_CUDA(cudaGetLastError());
    LMB_CUDA(launch_k(attn_combine_kernel<float>, dim3(p.B * p.KVl * p.G), dim3(128), 0, stream, p));
  }
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

}  // namespace lmb
