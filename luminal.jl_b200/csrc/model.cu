// Model weights (tiled, sharded), the decode session and its CUDA graph.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <type_traits>

#include "model.cuh"
#include "pdl.cuh"

namespace lmb {

// ---------------------------------------------------------------------------------------------
// logical <-> internal index maps
// ---------------------------------------------------------------------------------------------
// Internal element (row i, col k) of a tiled matrix -> (slot, logical row, logical col) of the
// reference tensor it comes from; false for padding.
__host__ __device__ inline bool wmap_resolve(const WMap& m, int i, int k, int* slot, int* lrow, int* lcol) {
  if (i >= m.rows || k >= m.K) return false;
  switch (m.kind) {
    case MAP_PLAIN:
      *slot = 0; *lrow = i; *lcol = k;
      return true;
    case MAP_QKV: {
      const int tile = i >> 4, r = i & 15;
      const int tph = m.D >> 4;
      const int hs = tile / tph, j = tile - hs * tph;
      *lcol = k;
      if (hs < m.Hl) {           // q head: local order (kv-local, group) -> global h = kv + KV*g
        const int kvl = hs / m.G, g = hs - kvl * m.G;
        const int h = (m.kv_off + kvl) + m.KV * g;
        const int d = 8 * j + (r & 7) + (r >> 3) * (m.D >> 1);
        *slot = 0; *lrow = h + m.H * d;           // feature f = h + H*d
      } else if (hs < m.Hl + m.KVl) {
        const int kvh = m.kv_off + (hs - m.Hl);
        const int d = 8 * j + (r & 7) + (r >> 3) * (m.D >> 1);
        *slot = 1; *lrow = kvh + m.KV * d;
      } else {
        const int kvh = m.kv_off + (hs - m.Hl - m.KVl);
        const int d = 16 * j + r;
        *slot = 2; *lrow = kvh + m.KV * d;
      }
      return true;
    }
    case MAP_O: {                // columns follow the attention output order (local head, d)
      const int hl = k / m.D, d = k - hl * m.D;
      const int kvl = hl / m.G, g = hl - kvl * m.G;
      const int h = (m.kv_off + kvl) + m.KV * g;
      *slot = 0; *lrow = i; *lcol = h + m.H * d;
      return true;
    }
    case MAP_GATEUP: {           // 16-row tiles: 8 gate rows then the 8 matching up rows
      const int tile = i >> 4, r = i & 15;
      const int idx = 8 * tile + (r & 7);
      if (idx >= m.inter_l) return false;
      *slot = r >> 3; *lrow = m.inter_off + idx; *lcol = k;
      return true;
    }
    case MAP_DOWN:
      *slot = 0; *lrow = i; *lcol = m.inter_off + k;
      return true;
  }
  return false;
}

struct FillSrc {
  uint64_t key[3];
  const float* src[3];     // staged logical tensors (NULL -> generator)
  int colmajor;
  int only_slot;           // -1: all
  float scale;             // sigma / 131072
};

template <typename WT>
__global__ void fill_tiled_kernel(WT* dst, WMap m, FillSrc f) {
  // every valid (internal row, k); the padding of the layout stays zero from the allocation
  const int64_t total = (int64_t)m.rows * m.K;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total;
       o += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(o / m.K);
    const int k = (int)(o - (int64_t)i * m.K);
    int slot, lrow, lcol;
    const int64_t at = Layout<WT>::w_offset(i, k, m.K);
    if (!wmap_resolve(m, i, k, &slot, &lrow, &lcol)) {
      if (f.only_slot < 0) dst[at] = from_f32<WT>(0.f);
      continue;
    }
    if (f.only_slot >= 0 && slot != f.only_slot) continue;
    float v;
    if (f.src[slot]) {
      const int64_t idx = f.colmajor ? (int64_t)lrow + (int64_t)m.src_rows[slot] * lcol
                                     : (int64_t)lrow * m.src_cols[slot] + lcol;
      v = f.src[slot][idx];
    } else {
      v = synth_value(f.key[slot], (uint64_t)lrow * m.src_cols[slot] + lcol, f.scale, 0.f);
    }
    dst[at] = from_f32<WT>(v);
  }
}

// plain row-major tensors (embedding table, norm gains)
template <typename WT>
__global__ void fill_plain_kernel(WT* dst, int64_t rows, int64_t cols, uint64_t key, const float* src,
                                  int colmajor, float scale, float offset) {
  const int64_t total = rows * cols;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total;
       o += (int64_t)gridDim.x * blockDim.x) {
    float v;
    if (src) {
      const int64_t r = o / cols, c = o - r * cols;
      v = src[colmajor ? r + rows * c : o];
    } else {
      v = synth_value(key, (uint64_t)o, scale, offset);
    }
    dst[o] = from_f32<WT>(v);
  }
}

template <typename WT>
__global__ void fill_kv_kernel(WT* kv, int64_t batch_stride, int64_t head_stride, int B, int KVl,
                               int KV, int kv_off, int D, int n_pos, int max_ctx, uint64_t key_k,
                               uint64_t key_v) {
  const int64_t total = (int64_t)B * KVl * n_pos * D;
  const float scale = 1.0f / 131072.0f;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total;
       o += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(o % D);
    const int pos = (int)((o / D) % n_pos);
    const int kvl = (int)((o / ((int64_t)D * n_pos)) % KVl);
    const int b = (int)(o / ((int64_t)D * n_pos * KVl));
    // logical index in a [B, KV, max_ctx, D] tensor
    const uint64_t li = (((uint64_t)b * KV + (kv_off + kvl)) * max_ctx + pos) * D + d;
    WT* base = kv + b * batch_stride + kvl * head_stride;
    base[kcache_offset(pos, d, D)] = from_f32<WT>(synth_value(key_k, li, scale, 0.f));
    base[vcache_offset(pos, d, D)] = from_f32<WT>(synth_value(key_v, li, scale, 0.f));
  }
}

// ---------------------------------------------------------------------------------------------
// small fused kernels of the decode step
// ---------------------------------------------------------------------------------------------
// x <- embedding row (first layer) or x + delta (residual add of the previous projection), then
// xn = (x * recip(sqrt(mean(x*x) + eps))) * w          src/HighLevelOps.jl:299-304, NN.jl:149-161
// One CTA per sequence; the row stays in shared memory between the two passes and all global
// accesses are independent float4s, so the kernel costs a couple of memory round trips.
// xn is a GEMV activation buffer (Layout<WT>::x_offset) of batch padding Bp.  n % 4 == 0.
constexpr int kNormThreads = 512;
// four consecutive activation elements (inside one 8-k group, so 8- or 16-byte aligned) in one store
__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(__nv_bfloat16* o, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&lo);
  u.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(o) = u;
}
template <typename WT>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                                   const int* __restrict__ tokens,
                                                                   const WT* __restrict__ embed, int vocab,
                                                                   const float* __restrict__ w, WT* __restrict__ xn,
                                                                   int Bp, int n, float eps,
                                                                   float* __restrict__ capture, PeerReduce pr) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[kNormThreads / 32];
  const int b = blockIdx.x, tid = threadIdx.x;
  const int n4 = n >> 2;
  // the gains never change: they are fetched before this kernel waits for its producer
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
  if (xn) {
    if (tid < n4) g0 = w4[tid];
    if (tid + kNormThreads < n4) g1 = w4[tid + kNormThreads];
  }
  pdl_launch_dependents();
  pdl_wait();
  // tensor parallel: delta is the sum of every rank's partial projection, read from the ranks'
  // exchange regions once all of them have signalled (all-reduce folded into this kernel)
  const bool peers = pr.n > 1 && !tokens;
  if (peers) peer_exchange_wait(pr);
  float4* xr = reinterpret_cast<float4*>(x + (int64_t)b * n);
  float4* rs = reinterpret_cast<float4*>(row);
  float ss = 0.f;
  if (tokens) {
    const int tok = tokens[b];
    const bool ok = tok >= 0 && tok < vocab;     // out of range -> zeros, as _gather_kernel! does
    const WT* er = embed + (int64_t)(ok ? tok : 0) * n;
#pragma unroll 4
    for (int i = tid; i < n4; i += kNormThreads) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ok) v = make_float4(to_f32(er[4 * i]), to_f32(er[4 * i + 1]), to_f32(er[4 * i + 2]), to_f32(er[4 * i + 3]));
      xr[i] = v;
      rs[i] = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + (int64_t)b * n) : nullptr;
    float4* cr = capture ? reinterpret_cast<float4*>(capture + (int64_t)b * n) : nullptr;
    if (peers) {
      // two row elements per pass, every rank's partial of both in flight at once (one NVLink round
      // trip for a row of up to 2 x kNormThreads float4s), summed in rank order
      for (int i0 = tid; i0 < n4; i0 += 2 * kNormThreads) {
        const int i1 = i0 + kNormThreads;
        const bool two = i1 < n4;
        float4 e0[8], e1[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < pr.n) {
            e0[r] = peer_load4(pr.part[r] + (int64_t)b * n + 4 * i0);
            if (two) e1[r] = peer_load4(pr.part[r] + (int64_t)b * n + 4 * i1);
          }
        }
        float4 v0 = xr[i0], v1 = two ? xr[i1] : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 d0 = e0[0], d1 = two ? e1[0] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 1; r < 8; ++r) {
          if (r < pr.n) {
            d0.x += e0[r].x; d0.y += e0[r].y; d0.z += e0[r].z; d0.w += e0[r].w;
            if (two) { d1.x += e1[r].x; d1.y += e1[r].y; d1.z += e1[r].z; d1.w += e1[r].w; }
          }
        }
        v0.x += d0.x; v0.y += d0.y; v0.z += d0.z; v0.w += d0.w;
        xr[i0] = v0; rs[i0] = v0;
        if (cr) cr[i0] = v0;
        ss += v0.x * v0.x + v0.y * v0.y + v0.z * v0.z + v0.w * v0.w;
        if (two) {
          v1.x += d1.x; v1.y += d1.y; v1.z += d1.z; v1.w += d1.w;
          xr[i1] = v1; rs[i1] = v1;
          if (cr) cr[i1] = v1;
          ss += v1.x * v1.x + v1.y * v1.y + v1.z * v1.z + v1.w * v1.w;
        }
      }
    } else {
#pragma unroll 4
      for (int i = tid; i < n4; i += kNormThreads) {
        float4 v = xr[i];
        if (dr) { const float4 d = dr[i]; v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w; }
        xr[i] = v;
        rs[i] = v;
        if (cr) cr[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float var = tot * (1.0f / (float)n);
  const float inv = 1.0f / sqrtf(var + eps);
  if (xn) {
#pragma unroll 4
    for (int i = tid; i < n4; i += kNormThreads) {
      const float4 v = rs[i];
      const float4 g = i == tid ? g0 : (i == tid + kNormThreads ? g1 : w4[i]);
      WT* o = xn + Layout<WT>::x_offset(b, 4 * i, Bp);   // 4 consecutive k stay inside one 8-k group
      store4(o, (v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
    }
  }
}

// Tensor-parallel form of the residual add + RMSNorm: a cluster of kTpSplit CTAs per sequence, each
// summing one slice of the row over every rank's partial (peer loads issued from four times as
// many SMs as one CTA per row would use), the slices' sums of squares exchanged through
// distributed shared memory and added in CTA order, so every rank still gets the same bits.
constexpr int kTpSplit = 4, kTpThreads = 256;
template <typename WT>
__global__ void __launch_bounds__(kTpThreads) add_rmsnorm_tp_kernel(float* __restrict__ x, const float* __restrict__ w,
                                                                    WT* __restrict__ xn, int Bp, int n, float eps,
                                                                    float* __restrict__ capture, PeerReduce pr) {
  extern __shared__ __align__(16) float row[];          // this CTA's slice
  __shared__ float red[kTpThreads / 32];
  __shared__ float ss_part[kTpSplit];
  uint32_t c;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(c));
  const int b = blockIdx.x / kTpSplit, tid = threadIdx.x;
  const int q4 = (n >> 2) / kTpSplit, col0 = (int)c * q4;      // float4s per slice, first float4 of this slice
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (xn && tid < q4) g0 = w4[col0 + tid];                     // the gains never change: before the wait
  pdl_launch_dependents();
  pdl_wait();
  peer_exchange_wait(pr);
  float4* xr = reinterpret_cast<float4*>(x + (int64_t)b * n);
  float4* rs = reinterpret_cast<float4*>(row);
  float4* cr = capture ? reinterpret_cast<float4*>(capture + (int64_t)b * n) : nullptr;
  float ss = 0.f;
  for (int i = tid; i < q4; i += kTpThreads) {
    const int idx = col0 + i;
    float4 e[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < pr.n) e[r] = peer_load4(pr.part[r] + (int64_t)b * n + 4 * idx);
    float4 v = xr[idx];
    float4 d = e[0];
#pragma unroll
    for (int r = 1; r < 8; ++r)
      if (r < pr.n) { d.x += e[r].x; d.y += e[r].y; d.z += e[r].z; d.w += e[r].w; }
    v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    xr[idx] = v;
    rs[i] = v;
    if (cr) cr[idx] = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float mine = 0.f;
#pragma unroll
  for (int i = 0; i < kTpThreads / 32; ++i) mine += red[i];
  if (tid < kTpSplit) {                                        // this slice's sum into slot c of every CTA of the cluster
    uint32_t local = (uint32_t)__cvta_generic_to_shared(&ss_part[c]), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"((uint32_t)tid));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(mine) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
  const float tot = ((ss_part[0] + ss_part[1]) + ss_part[2]) + ss_part[3];
  const float inv = 1.0f / sqrtf(tot * (1.0f / (float)n) + eps);
  if (xn) {
    for (int i = tid; i < q4; i += kTpThreads) {
      const float4 v = rs[i];
      const float4 g = i == tid ? g0 : w4[col0 + i];
      WT* o = xn + Layout<WT>::x_offset(b, 4 * (col0 + i), Bp);
      store4(o, (v.x * inv) * g.x, (v.y * inv) * g.y, (v.z * inv) * g.z, (v.w * inv) * g.w);
    }
  }
}

// Whisper decoder: x <- embedding row + positional row (first layer) or x + delta, then LayerNorm
// with mean-centering, gain and bias:  xc = x + mean*(-1);  y = (xc * recip(sqrt(mean(xc*xc) + eps))) * w + b
// (src/NN.jl:138-173, src/HighLevelOps.jl:292-304; positions src/Whisper.jl:699-701).
template <typename WT>
__global__ void __launch_bounds__(kNormThreads) add_layernorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                                     const float* __restrict__ delta_bias,
                                                                     const int* __restrict__ tokens,
                                                                     const WT* __restrict__ embed, int vocab,
                                                                     const float* __restrict__ pos_emb,
                                                                     const int* __restrict__ pos,
                                                                     const float* __restrict__ w,
                                                                     const float* __restrict__ bias, WT* __restrict__ xn,
                                                                     int Bp, int n, float eps, float* __restrict__ capture) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[kNormThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  float* xr = x + (int64_t)b * n;
  auto block_sum = [&](float v) -> float {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) t += red[i];
    return t;
  };
  float s1 = 0.f;
  if (tokens) {
    const int tok = tokens[b];
    const bool ok = tok >= 0 && tok < vocab;
    const WT* er = embed + (int64_t)(ok ? tok : 0) * n;
    const float* pr = pos_emb + (int64_t)pos[b] * n;
    for (int i = tid; i < n; i += kNormThreads) {
      const float v = (ok ? to_f32(er[i]) : 0.f) + pr[i];
      xr[i] = v; row[i] = v; s1 += v;
    }
  } else {
    const float* dr = delta ? delta + (int64_t)b * n : nullptr;
    for (int i = tid; i < n; i += kNormThreads) {
      float v = xr[i];
      if (dr) v += dr[i];
      (void)delta_bias;
      xr[i] = v; row[i] = v; s1 += v;
      if (capture) capture[(int64_t)b * n + i] = v;
    }
  }
  const float mean = block_sum(s1) * (1.0f / (float)n);
  float s2 = 0.f;
  for (int i = tid; i < n; i += kNormThreads) { const float c = row[i] + mean * -1.0f; row[i] = c; s2 += c * c; }
  const float var = block_sum(s2) * (1.0f / (float)n);
  const float inv = 1.0f / sqrtf(var + eps);
  if (xn)
    for (int i = tid; i < n; i += kNormThreads)
      xn[Layout<WT>::x_offset(b, i, Bp)] = from_f32<WT>((row[i] * inv) * w[i] + bias[i]);
}

// bias of a fused matrix in internal row order: dst[i] = src[logical row] for rows of `slot`
__global__ void fill_bias_kernel(float* dst, WMap m, const float* src, int slot) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m.rows; i += gridDim.x * blockDim.x) {
    int s, lrow, lcol;
    if (wmap_resolve(m, i, 0, &s, &lrow, &lcol) && s == slot) dst[i] = src[lrow];
  }
}

// scatter a logical [B, H, T, D] float32 tensor pair into a tiled cache layer
template <typename WT>
__global__ void scatter_kv_kernel(WT* kv, int64_t batch_stride, int64_t head_stride, int B, int H, int T, int D,
                                  const float* ksrc, const float* vsrc, int colmajor) {
  const int64_t total = (int64_t)B * H * T * D;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(o % D);
    const int t = (int)((o / D) % T);
    const int h = (int)((o / ((int64_t)D * T)) % H);
    const int b = (int)(o / ((int64_t)D * T * H));
    const int64_t src = colmajor ? (int64_t)b + (int64_t)B * (h + (int64_t)H * (t + (int64_t)T * d)) : o;
    WT* base = kv + b * batch_stride + h * head_stride;
    base[kcache_offset(t, d, D)] = from_f32<WT>(ksrc[src]);
    base[vcache_offset(t, d, D)] = from_f32<WT>(vsrc[src]);
  }
}

// greedy token: first maximum of the logits row; also logs it for the device-resident loop
constexpr int kArgmaxThreads = 1024;
// `stop` (device: [0] the end-of-text id or -1, [1] how many sequences have produced it, [2 + b] whether
// sequence b has): once a sequence has produced the end-of-text token it keeps emitting it, the batch
// form of the reference's `break` at EOT (src/Decoding.jl:126-129).
__global__ void __launch_bounds__(kArgmaxThreads) argmax_step_kernel(const float* logits, int pitch, int n, int* tokens,
                                                                     int* hist, const int* step_ctr, int B, int* stop) {
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ int si[kArgmaxThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)b * pitch;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  };
  if ((pitch & 3) == 0) {              // rows are 16-byte aligned: four logits per load
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = n >> 2;
#pragma unroll 4
    for (int i = tid; i < n4; i += kArgmaxThreads) {
      const float4 v = row4[i];
      take(v.x, 4 * i); take(v.y, 4 * i + 1); take(v.z, 4 * i + 2); take(v.w, 4 * i + 3);
    }
    for (int i = 4 * n4 + tid; i < n; i += kArgmaxThreads) take(row[i], i);
  } else {
    for (int i = tid; i < n; i += kArgmaxThreads) take(row[i], i);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, best, off);
    const int i = __shfl_xor_sync(0xffffffffu, bi, off);
    take(v, i);
  }
  if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    best = sv[tid];
    bi = si[tid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float v = __shfl_xor_sync(0xffffffffu, best, off);
      const int i = __shfl_xor_sync(0xffffffffu, bi, off);
      take(v, i);
    }
    if (tid == 0) {
      const int eot = stop ? stop[0] : -1;
      if (eot >= 0) {
        if (stop[2 + b]) bi = eot;
        else if (bi == eot) { stop[2 + b] = 1; atomicAdd(&stop[1], 1); }
      }
      tokens[b] = bi;
      if (hist) hist[(int64_t)(*step_ctr) * B + b] = bi;
    }
  }
}

// End of a step: every sequence whose position is below its limit moves on by one.  The limit is "never"
// during decoding; while a ragged prompt is fed step by step it is the sequence's prompt end, so a sequence
// whose prompt is over stays where it is (its lane of the batch then recomputes the same slot, harmlessly).
__global__ void advance_kernel(int* pos, const int* limit, int B, int* step_ctr, unsigned long long* peer_step) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = threadIdx.x;
  if (b < B && pos[b] < limit[b]) pos[b] += 1;
  if (b == 0) {
    *step_ctr += 1;
    if (peer_step) *peer_step += 1;     // epoch base of the next step's in-kernel all-reduces
  }
}


// Tensor-parallel head: the best (logit, id) of this rank's slice of the vocabulary, per sequence, written where the
// peers can read it (this rank's exchange buffer): pairs[2 b] = value, pairs[2 b + 1] = the id's bits.
__global__ void __launch_bounds__(kArgmaxThreads) argmax_pairs_kernel(const float* logits, int pitch, int n, int id0, float* pairs) {
  __shared__ float sv[kArgmaxThreads / 32];
  __shared__ int si[kArgmaxThreads / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (int64_t)b * pitch;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  };
  for (int i = tid; i < n; i += kArgmaxThreads) take(row[i], i);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float v = __shfl_xor_sync(0xffffffffu, best, off);
    const int i = __shfl_xor_sync(0xffffffffu, bi, off);
    take(v, i);
  }
  if ((tid & 31) == 0) { sv[tid >> 5] = best; si[tid >> 5] = bi; }
  __syncthreads();
  if (tid < 32) {
    best = sv[tid];
    bi = si[tid];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float v = __shfl_xor_sync(0xffffffffu, best, off);
      const int i = __shfl_xor_sync(0xffffffffu, bi, off);
      take(v, i);
    }
    if (tid == 0) {
      pairs[2 * b] = best;
      pairs[2 * b + 1] = __int_as_float(bi == 0x7fffffff ? bi : bi + id0);
    }
  }
}

// ... and the choice among the ranks' pairs: the flag exchange of the float32 all-reduce (every rank announces the epoch,
// waits -- bounded -- for the others', then reads their pairs with peer loads), the largest logit wins and the lowest id
// among equals, exactly what argmax_step_kernel does over the whole row; then the same bookkeeping.  One block.
__global__ void __launch_bounds__(256) argmax_tp_select_kernel(const PeerReduce pr, int B, int* tokens, int* hist, const int* step_ctr,
                                                               int* stop) {
  pdl_launch_dependents();
  pdl_wait();
  peer_exchange_wait(pr);
  const int b = threadIdx.x;
  if (b >= B) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int r = 0; r < pr.n; ++r) {
    float v, f;
    asm volatile("ld.relaxed.sys.global.v2.f32 {%0,%1}, [%2];" : "=f"(v), "=f"(f) : "l"(pr.part[r] + 2 * b) : "memory");
    const int i = __float_as_int(f);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  const int eot = stop ? stop[0] : -1;
  if (eot >= 0) {
    if (stop[2 + b]) bi = eot;
    else if (bi == eot) { stop[2 + b] = 1; atomicAdd(&stop[1], 1); }
  }
  tokens[b] = bi;
  if (hist) hist[(int64_t)(*step_ctr) * B + b] = bi;
}

// First kernel of the fused step: x <- embedding rows (out-of-range ids -> zeros, as _gather_kernel! does,
// src/Execution.jl:580-595), laid out [hidden][Bp]; xg <- bf16(x * gain) in the GEMV activation layout; one
// slot of per-sequence sums of squares per CTA.  What add_rmsnorm_kernel does for the first layer, minus
// the scale, which the q/k/v projection applies to its accumulators.  128 threads: thread e owns rows
// (e >> 2) + 32 j of the CTA's rows and batch columns 8 (e & 3) .. + 7.
template <int N>
__global__ void __launch_bounds__(128) embed_prep_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed,
                                                         int vocab, int hidden, int B, const float* __restrict__ gain,
                                                         float* __restrict__ x, __nv_bfloat16* __restrict__ xg,
                                                         float* __restrict__ ssq_out, int rows_per_cta) {
  __shared__ float s_red[128];
  pdl_launch_dependents();
  pdl_wait();
  const int e = threadIdx.x, lane = e & 31, we = e >> 5;
  const int bg = e & 3, rl0 = e >> 2;
  int tok[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int b = 8 * bg + i;
    const int t = (b < B && bg < N / 8) ? tokens[b] : -1;
    tok[i] = (t >= 0 && t < vocab) ? t : -1;
  }
  float ssq[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) ssq[i] = 0.f;
  for (int rl = rl0; rl < rows_per_cta; rl += 32) {
    const int k = blockIdx.x * rows_per_cta + rl;
    if (k >= hidden || bg >= N / 8) continue;
    float xv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) xv[i] = tok[i] >= 0 ? __bfloat162float(embed[(int64_t)tok[i] * hidden + k]) : 0.f;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)k * N + 8 * bg);
    xr[0] = make_float4(xv[0], xv[1], xv[2], xv[3]);
    xr[1] = make_float4(xv[4], xv[5], xv[6], xv[7]);
    const float g = gain[k];
    __nv_bfloat16* o = xg + (size_t)(k >> 3) * (N * 8) + bg * 64 + (k & 7);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o[8 * i] = __float2bfloat16_rn(xv[i] * g);
      ssq[i] += xv[i] * xv[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 4);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 8);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 16);
  }
  if (lane < 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_red[we * 32 + 8 * lane + i] = ssq[i];
  }
  __syncthreads();
  if (e < 32) ssq_out[(size_t)blockIdx.x * 32 + e] = ((s_red[e] + s_red[32 + e]) + s_red[64 + e]) + s_red[96 + e];
}

// The same for the Whisper decoder: x <- embedding row + position row (src/Whisper.jl:704-707), the first
// LayerNorm's x * gain, and per-CTA sums of x and of x^2 (mean and variance for the consumer, InvScale).
template <int N>
__global__ void __launch_bounds__(128) embed_prep_ln_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ embed,
                                                            int vocab, int hidden, int B, const float* __restrict__ pos_emb,
                                                            const int* __restrict__ pos, const float* __restrict__ gain,
                                                            float* __restrict__ x, __nv_bfloat16* __restrict__ xg,
                                                            float* __restrict__ ssq_out, float* __restrict__ sum_out, int rows_per_cta) {
  __shared__ float s_red[2][128];
  pdl_launch_dependents();
  pdl_wait();
  const int e = threadIdx.x, lane = e & 31, we = e >> 5;
  const int bg = e & 3, rl0 = e >> 2;
  int tok[8], ps[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int b = 8 * bg + i;
    const bool live = b < B && bg < N / 8;
    const int t = live ? tokens[b] : -1;
    tok[i] = (t >= 0 && t < vocab) ? t : -1;
    ps[i] = live ? pos[b] : 0;
  }
  float ssq[8], sx[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { ssq[i] = 0.f; sx[i] = 0.f; }
  for (int rl = rl0; rl < rows_per_cta; rl += 32) {
    const int k = blockIdx.x * rows_per_cta + rl;
    if (k >= hidden || bg >= N / 8) continue;
    float xv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float ev = tok[i] >= 0 ? __bfloat162float(embed[(int64_t)tok[i] * hidden + k]) : 0.f;
      xv[i] = 8 * bg + i < B ? ev + pos_emb[(int64_t)ps[i] * hidden + k] : 0.f;
    }
    float4* xr = reinterpret_cast<float4*>(x + (size_t)k * N + 8 * bg);
    xr[0] = make_float4(xv[0], xv[1], xv[2], xv[3]);
    xr[1] = make_float4(xv[4], xv[5], xv[6], xv[7]);
    const float g = gain[k];
    __nv_bfloat16* o = xg + (size_t)(k >> 3) * (N * 8) + bg * 64 + (k & 7);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o[8 * i] = __float2bfloat16_rn(xv[i] * g);
      ssq[i] += xv[i] * xv[i];
      sx[i] += xv[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 4);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 8);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 16);
    sx[i] += __shfl_xor_sync(0xffffffffu, sx[i], 4);
    sx[i] += __shfl_xor_sync(0xffffffffu, sx[i], 8);
    sx[i] += __shfl_xor_sync(0xffffffffu, sx[i], 16);
  }
  if (lane < 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { s_red[0][we * 32 + 8 * lane + i] = ssq[i]; s_red[1][we * 32 + 8 * lane + i] = sx[i]; }
  }
  __syncthreads();
  if (e < 32) {
    ssq_out[(size_t)blockIdx.x * 32 + e] = ((s_red[0][e] + s_red[0][32 + e]) + s_red[0][64 + e]) + s_red[0][96 + e];
    sum_out[(size_t)blockIdx.x * 32 + e] = ((s_red[1][e] + s_red[1][32 + e]) + s_red[1][64 + e]) + s_red[1][96 + e];
  }
}

// wg[r] = sum_k W[r, k] g[k];  bf[r] = sum_k W[r, k] b[k] + bias[r]: the two vectors that fold a LayerNorm (gain g,
// bias b) into the Linear W that follows it.  W in the tiled bf16 layout, one block per internal row.
__global__ void __launch_bounds__(128) ln_fold_kernel(const __nv_bfloat16* __restrict__ W, int rows, int K, const float* __restrict__ g,
                                                      const float* __restrict__ b, const float* __restrict__ bias,
                                                      float* __restrict__ wg, float* __restrict__ bf) {
  __shared__ float red[2][4];
  const int r = blockIdx.x, KS = (K + 127) >> 7;
  float sg = 0.f, sb = 0.f;
  for (int k = threadIdx.x; k < K; k += 128) {
    const float w = __bfloat162float(W[wcanon_offset(r, k, KS)]);
    sg += w * g[k];
    sb += w * b[k];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    sg += __shfl_xor_sync(0xffffffffu, sg, off);
    sb += __shfl_xor_sync(0xffffffffu, sb, off);
  }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = sg; red[1][threadIdx.x >> 5] = sb; }
  __syncthreads();
  if (threadIdx.x == 0 && r < rows) {
    wg[r] = (red[0][0] + red[0][1]) + (red[0][2] + red[0][3]);
    bf[r] = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]) + (bias ? bias[r] : 0.f);
  }
}

int32_t step_kernels_configure() {
#define LMB_CARVE(KERN) \
  LMB_CUDA(cudaFuncSetAttribute(KERN, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared))
  LMB_CARVE(add_layernorm_kernel<float>);
  LMB_CARVE(add_layernorm_kernel<__nv_bfloat16>);
  LMB_CARVE(add_rmsnorm_kernel<float>);
  LMB_CARVE(add_rmsnorm_kernel<__nv_bfloat16>);
  LMB_CARVE(argmax_step_kernel);
  LMB_CARVE(advance_kernel);
#undef LMB_CARVE
  return LMB200_OK;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
Model* model_from(lmb200_model h) {
  Model* m = reinterpret_cast<Model*>(h);
  if (!m || m->magic != 0x4D4F444C) { set_error("invalid model handle"); return nullptr; }
  if (m->ctx && m->ctx->capturing) { set_error("model and session calls cannot be recorded between capture_begin and capture_end"); return nullptr; }
  return m;
}
Session* session_from(lmb200_session h) {
  Session* s = reinterpret_cast<Session*>(h);
  if (!s || s->magic != 0x53455353) { set_error("invalid session handle"); return nullptr; }
  if (s->m && s->m->ctx && s->m->ctx->capturing) { set_error("model and session calls cannot be recorded between capture_begin and capture_end"); return nullptr; }
  return s;
}

namespace {

int fill_grid(int64_t total) {
  int64_t g = ceil_div(total, 256);
  if (g > 148 * 32) g = 148 * 32;
  if (g < 1) g = 1;
  return (int)g;
}

uint64_t layer_tensor_id(int layer, int slot) { return (uint64_t)16 * layer + slot; }
enum Slot { S_ATTN_NORM = 0, S_Q = 1, S_K = 2, S_V = 3, S_O = 4, S_FFN_NORM = 5, S_GATE = 6, S_UP = 7, S_DOWN = 8 };
constexpr uint64_t kIdEmbed = 0xFFFF0, kIdFinalNorm = 0xFFFF1, kIdHead = 0xFFFF2;
constexpr uint64_t kIdKvBase = 0x100000;

int64_t tiled_elems(const WMap& m, int dtype) {
  return dtype == LMB200_BF16 ? Layout<__nv_bfloat16>::w_elems(m.rows, m.K) : Layout<float>::w_elems(m.rows, m.K);
}

template <typename WT>
int32_t fill_tiled(Ctx* ctx, void* dst, const WMap& m, const FillSrc& f) {
  fill_tiled_kernel<WT><<<fill_grid((int64_t)m.rows * m.K), 256, 0, ctx->stream>>>(reinterpret_cast<WT*>(dst), m, f);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}
int32_t fill_tiled_dt(Model* M, void* dst, const WMap& m, const FillSrc& f) {
  return M->cfg.dtype == LMB200_BF16 ? fill_tiled<__nv_bfloat16>(M->ctx, dst, m, f)
                                     : fill_tiled<float>(M->ctx, dst, m, f);
}
template <typename WT>
int32_t fill_plain(Ctx* ctx, void* dst, int64_t rows, int64_t cols, uint64_t key, const float* src,
                   int colmajor, float scale, float offset) {
  fill_plain_kernel<WT><<<fill_grid(rows * cols), 256, 0, ctx->stream>>>(reinterpret_cast<WT*>(dst), rows, cols, key,
                                                                         src, colmajor, scale, offset);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

void finish_map(WMap& m) {
  m.RB = (int)ceil_div(m.rows, 16);
  m.KC = (int)ceil_div(m.K, 32);
}

int32_t dmalloc(void** p, int64_t bytes, bool zero, cudaStream_t st) {
  *p = nullptr;
  if (bytes <= 0) bytes = 16;
  cudaError_t e = cudaMalloc(p, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LMB200_ENOMEM, "cudaMalloc of %lld bytes failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  if (zero) LMB_CUDA(cudaMemsetAsync(*p, 0, (size_t)bytes, st));
  return LMB200_OK;
}

}  // namespace
}  // namespace lmb

using namespace lmb;

// =============================================================================================
// model
// =============================================================================================
// Validates a configuration and derives this rank's shard extents and index maps.  Host
// arithmetic only (no CUDA call), so the sharding can be checked without a GPU.
static int32_t derive_model(const lmb200_model_config& c, Model* M) {
  LMB_REQUIRE(c.n_layers >= 1 && c.hidden >= 16 && c.n_heads >= 1 && c.n_kv_heads >= 1 && c.vocab >= 1 &&
                  c.intermediate >= 8, "model_create: non-positive dimension");
  LMB_REQUIRE(c.head_dim * c.n_heads == c.hidden, "model_create: head_dim %d * n_heads %d != hidden %d",
              c.head_dim, c.n_heads, c.hidden);
  LMB_REQUIRE(c.head_dim % 16 == 0, "model_create: head_dim %d must be a multiple of 16", c.head_dim);
  LMB_REQUIRE(c.n_heads % c.n_kv_heads == 0, "model_create: n_heads %d not a multiple of n_kv_heads %d",
              c.n_heads, c.n_kv_heads);
  LMB_REQUIRE(c.dtype == LMB200_F32 || c.dtype == LMB200_BF16, "model_create: dtype %d", c.dtype);
  LMB_REQUIRE(c.tp_size >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_size, "model_create: tp rank %d of %d",
              c.tp_rank, c.tp_size);
  LMB_REQUIRE(c.n_kv_heads % c.tp_size == 0, "model_create: tp_size %d does not divide the %d kv heads",
              c.tp_size, c.n_kv_heads);
  LMB_REQUIRE(c.intermediate % c.tp_size == 0 && (c.intermediate / c.tp_size) % 8 == 0,
              "model_create: intermediate %d / tp %d must be a multiple of 8", c.intermediate, c.tp_size);
  LMB_REQUIRE(c.hidden % 4 == 0, "model_create: hidden %d must be a multiple of 4", c.hidden);
  LMB_REQUIRE(c.arch == LMB200_ARCH_LLAMA || c.arch == LMB200_ARCH_WHISPER_DECODER, "model_create: arch %d", c.arch);
  if (c.arch == LMB200_ARCH_WHISPER_DECODER) {
    LMB_REQUIRE(c.n_kv_heads == c.n_heads && c.tp_size == 1, "model_create: the Whisper decoder has no GQA and no tensor parallelism");
    LMB_REQUIRE(c.max_positions >= 1 && c.cross_len >= 1, "model_create: Whisper needs max_positions and cross_len");
  }
  M->cfg = c;
  M->esz = c.dtype == LMB200_BF16 ? 2 : 4;
  M->D = c.head_dim;
  M->G = c.n_heads / c.n_kv_heads;
  M->KVl = c.n_kv_heads / c.tp_size;
  M->Hl = M->KVl * M->G;
  M->kv_off = c.tp_rank * M->KVl;
  M->inter_l = c.intermediate / c.tp_size;
  M->inter_off = c.tp_rank * M->inter_l;

  auto base = [&](WMap& m, int kind) {
    m.kind = kind;
    m.H = c.n_heads; m.KV = c.n_kv_heads; m.D = M->D; m.G = M->G; m.Hl = M->Hl; m.KVl = M->KVl;
    m.kv_off = M->kv_off; m.inter_l = M->inter_l; m.inter_off = M->inter_off;
  };
  base(M->m_qkv, MAP_QKV);
  M->m_qkv.rows = (M->Hl + 2 * M->KVl) * M->D; M->m_qkv.K = c.hidden;
  M->m_qkv.src_rows[0] = c.hidden; M->m_qkv.src_rows[1] = M->m_qkv.src_rows[2] = c.n_kv_heads * M->D;
  M->m_qkv.src_cols[0] = M->m_qkv.src_cols[1] = M->m_qkv.src_cols[2] = c.hidden;
  finish_map(M->m_qkv);
  base(M->m_o, MAP_O);
  M->m_o.rows = c.hidden; M->m_o.K = M->Hl * M->D;
  M->m_o.src_rows[0] = c.hidden; M->m_o.src_cols[0] = c.n_heads * M->D;
  finish_map(M->m_o);
  base(M->m_gu, MAP_GATEUP);
  M->m_gu.rows = 2 * M->inter_l; M->m_gu.K = c.hidden;
  M->m_gu.src_rows[0] = M->m_gu.src_rows[1] = c.intermediate;
  M->m_gu.src_cols[0] = M->m_gu.src_cols[1] = c.hidden;
  finish_map(M->m_gu);
  base(M->m_down, MAP_DOWN);
  M->m_down.rows = c.hidden; M->m_down.K = M->inter_l;
  M->m_down.src_rows[0] = c.hidden; M->m_down.src_cols[0] = c.intermediate;
  finish_map(M->m_down);
  base(M->m_head, MAP_PLAIN);
  M->m_head.rows = c.vocab; M->m_head.K = c.hidden;
  M->m_head.src_rows[0] = c.vocab; M->m_head.src_cols[0] = c.hidden;
  finish_map(M->m_head);
  if (c.arch == LMB200_ARCH_WHISPER_DECODER) {
    // fc1 / fc2 are plain matrices; the cross-attention q projection is a q-only head-ordered matrix
    M->m_gu.kind = MAP_PLAIN; M->m_gu.rows = c.intermediate; M->m_gu.K = c.hidden;
    M->m_gu.src_rows[0] = c.intermediate; M->m_gu.src_cols[0] = c.hidden;
    finish_map(M->m_gu);
    M->m_down.kind = MAP_PLAIN; M->m_down.rows = c.hidden; M->m_down.K = c.intermediate;
    M->m_down.src_rows[0] = c.hidden; M->m_down.src_cols[0] = c.intermediate;
    finish_map(M->m_down);
    M->m_qc = M->m_qkv;
    M->m_qc.KVl = 0; M->m_qc.rows = M->Hl * M->D;
    finish_map(M->m_qc);
  }
  return LMB200_OK;
}

extern "C" int32_t lmb200_shard_extent(const lmb200_model_config* cfg, int32_t matrix, int32_t* rows, int32_t* cols) {
  LMB_REQUIRE(cfg && rows && cols, "shard_extent: null argument");
  Model M;
  LMB_TRY(derive_model(*cfg, &M));
  const WMap* maps[5] = {&M.m_qkv, &M.m_o, &M.m_gu, &M.m_down, &M.m_head};
  LMB_REQUIRE(matrix >= 0 && matrix < 5, "shard_extent: matrix %d", matrix);
  *rows = maps[matrix]->rows;
  *cols = maps[matrix]->K;
  return LMB200_OK;
}

extern "C" int32_t lmb200_shard_map(const lmb200_model_config* cfg, int32_t matrix, int32_t row, int32_t col,
                                    int32_t* slot, int32_t* logical_row, int32_t* logical_col) {
  LMB_REQUIRE(cfg && slot && logical_row && logical_col, "shard_map: null argument");
  Model M;
  LMB_TRY(derive_model(*cfg, &M));
  const WMap* maps[5] = {&M.m_qkv, &M.m_o, &M.m_gu, &M.m_down, &M.m_head};
  LMB_REQUIRE(matrix >= 0 && matrix < 5, "shard_map: matrix %d", matrix);
  int s = -1, r = -1, c = -1;
  if (!wmap_resolve(*maps[matrix], row, col, &s, &r, &c)) { s = -1; r = -1; c = -1; }   // padding
  *slot = s; *logical_row = r; *logical_col = c;
  return LMB200_OK;
}

extern "C" int32_t lmb200_model_create(lmb200_ctx hctx, const lmb200_model_config* cfg, lmb200_model* out) {
  Ctx* ctx = ctx_from(hctx);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(cfg && out, "model_create: null argument");
  const lmb200_model_config& c = *cfg;
  Model* M = new Model();
  M->ctx = ctx;
  {
    const int32_t rc0 = derive_model(c, M);
    if (rc0 != LMB200_OK) { delete M; return rc0; }
  }
  // LMB200_TP_SOLO=1 (profiling aid): one rank's shard without its peers.  The partial sums are
  // never reduced, so the results are not the model's; the kernels and their sizes are the rank's.
  const char* solo = getenv("LMB200_TP_SOLO");
  M->tp_solo = c.tp_size > 1 && !ctx->nccl_comm && solo && atoi(solo) == 1;
  if (c.tp_size > 1 && !M->tp_solo && !(ctx->nccl_comm && ctx->tp_size == c.tp_size && ctx->tp_rank == c.tp_rank)) {
    delete M;
    return fail(LMB200_EINVAL, "model_create: tp_size %d needs lmb200_comm_init with the same ranks first", c.tp_size);
  }
  if (cudaSetDevice(ctx->device) != cudaSuccess) { delete M; return fail(LMB200_ECUDA, "model_create: cudaSetDevice failed"); }

  int32_t rc = LMB200_OK;
  auto alloc = [&](void** p, int64_t bytes) {
    if (rc != LMB200_OK) return;
    rc = dmalloc(p, bytes, true, ctx->stream);
    if (rc == LMB200_OK) M->weight_bytes += bytes;
  };
  M->layers.resize(c.n_layers);
  for (auto& L : M->layers) {
    alloc(&L.wqkv, tiled_elems(M->m_qkv, c.dtype) * M->esz);
    alloc(&L.wo, tiled_elems(M->m_o, c.dtype) * M->esz);
    alloc(&L.wgu, tiled_elems(M->m_gu, c.dtype) * M->esz);
    alloc(&L.wdown, tiled_elems(M->m_down, c.dtype) * M->esz);
    alloc((void**)&L.attn_norm, (int64_t)c.hidden * 4);
    alloc((void**)&L.ffn_norm, (int64_t)c.hidden * 4);
  }
  if (c.arch == LMB200_ARCH_WHISPER_DECODER) {
    for (auto& L : M->layers) {
      alloc(&L.wq_cross, tiled_elems(M->m_qc, c.dtype) * M->esz);
      alloc(&L.wo_cross, tiled_elems(M->m_o, c.dtype) * M->esz);
      alloc((void**)&L.attn_norm_b, (int64_t)c.hidden * 4);
      alloc((void**)&L.ffn_norm_b, (int64_t)c.hidden * 4);
      alloc((void**)&L.cross_norm, (int64_t)c.hidden * 4);
      alloc((void**)&L.cross_norm_b, (int64_t)c.hidden * 4);
      alloc((void**)&L.b_qkv, (int64_t)M->m_qkv.rows * 4);
      alloc((void**)&L.b_o, (int64_t)c.hidden * 4);
      alloc((void**)&L.b_q_cross, (int64_t)M->m_qc.rows * 4);
      alloc((void**)&L.b_o_cross, (int64_t)c.hidden * 4);
      alloc((void**)&L.b_fc1, (int64_t)c.intermediate * 4);
      alloc((void**)&L.b_fc2, (int64_t)c.hidden * 4);
    }
    alloc((void**)&M->final_norm_b, (int64_t)c.hidden * 4);
    alloc((void**)&M->pos_emb, (int64_t)c.max_positions * c.hidden * 4);
    alloc(&M->embed_tiled, tiled_elems(M->m_head, c.dtype) * M->esz);
  }
  alloc(&M->embed, (int64_t)c.vocab * c.hidden * M->esz);
  alloc((void**)&M->final_norm, (int64_t)c.hidden * 4);
  if (c.arch == LMB200_ARCH_LLAMA) alloc(&M->lm_head, tiled_elems(M->m_head, c.dtype) * M->esz);
  alloc((void**)&M->inv_freq, (int64_t)(M->D / 2) * 4);
  if (rc != LMB200_OK) { lmb200_model_destroy(reinterpret_cast<lmb200_model>(M)); return rc; }

  // inv_freq[i] = recip(exp2((i*2*(1/D)) * log2(base)))              src/NN.jl:261-263
  std::vector<float> inv(M->D / 2);
  const float l2b = log2f(c.rope_base);
  for (int i = 0; i < M->D / 2; ++i) {
    volatile float f = (float)i * 2.0f;
    f = f * (1.0f / (float)M->D);
    f = f * l2b;
    inv[i] = 1.0f / exp2f(f);
  }
  LMB_CUDA(cudaMemcpyAsync(M->inv_freq, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  *out = reinterpret_cast<lmb200_model>(M);
  return LMB200_OK;
}

extern "C" int32_t lmb200_model_destroy(lmb200_model h) {
  Model* M = model_from(h);
  if (!M) return LMB200_EINVAL;
  cudaSetDevice(M->ctx->device);
  for (auto& L : M->layers) {
    cudaFree(L.wqkv); cudaFree(L.wo); cudaFree(L.wgu); cudaFree(L.wdown);
    cudaFree(L.attn_norm); cudaFree(L.ffn_norm);
    cudaFree(L.wq_cross); cudaFree(L.wo_cross); cudaFree(L.attn_norm_b); cudaFree(L.ffn_norm_b);
    cudaFree(L.cross_norm); cudaFree(L.cross_norm_b); cudaFree(L.b_qkv); cudaFree(L.b_o); cudaFree(L.b_q_cross);
    cudaFree(L.b_o_cross); cudaFree(L.b_fc1); cudaFree(L.b_fc2);
    cudaFree(L.wg_qkv); cudaFree(L.bf_qkv); cudaFree(L.wg_qc); cudaFree(L.bf_qc); cudaFree(L.wg_fc1); cudaFree(L.bf_fc1);
  }
  cudaFree(M->final_norm_b); cudaFree(M->pos_emb); cudaFree(M->embed_tiled); cudaFree(M->wg_head); cudaFree(M->bf_head);
  cudaFree(M->embed); cudaFree(M->final_norm); cudaFree(M->lm_head); cudaFree(M->inv_freq);
  M->magic = 0;
  delete M;
  return LMB200_OK;
}

extern "C" int32_t lmb200_model_weight_bytes(lmb200_model h, int64_t* bytes) {
  Model* M = model_from(h);
  if (!M || !bytes) return LMB200_EINVAL;
  *bytes = M->weight_bytes;
  return LMB200_OK;
}

extern "C" int32_t lmb200_model_init_random(lmb200_model h, uint64_t seed, float sigma) {
  Model* M = model_from(h);
  if (!M) return LMB200_EINVAL;
  LMB_REQUIRE(M->cfg.arch == LMB200_ARCH_LLAMA, "init_random: only for Llama-shaped models; set Whisper weights by name");
  Ctx* ctx = M->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const float scale = sigma / 131072.0f;
  const int hid = M->cfg.hidden;
  for (int l = 0; l < M->cfg.n_layers; ++l) {
    LayerWeights& L = M->layers[l];
    FillSrc f{};
    f.only_slot = -1; f.scale = scale; f.colmajor = 0;
    f.src[0] = f.src[1] = f.src[2] = nullptr;
    f.key[0] = stream_key(seed, layer_tensor_id(l, S_Q));
    f.key[1] = stream_key(seed, layer_tensor_id(l, S_K));
    f.key[2] = stream_key(seed, layer_tensor_id(l, S_V));
    LMB_TRY(fill_tiled_dt(M, L.wqkv, M->m_qkv, f));
    f.key[0] = stream_key(seed, layer_tensor_id(l, S_O));
    LMB_TRY(fill_tiled_dt(M, L.wo, M->m_o, f));
    f.key[0] = stream_key(seed, layer_tensor_id(l, S_GATE));
    f.key[1] = stream_key(seed, layer_tensor_id(l, S_UP));
    LMB_TRY(fill_tiled_dt(M, L.wgu, M->m_gu, f));
    f.key[0] = stream_key(seed, layer_tensor_id(l, S_DOWN));
    LMB_TRY(fill_tiled_dt(M, L.wdown, M->m_down, f));
    LMB_TRY(fill_plain<float>(ctx, L.attn_norm, 1, hid, stream_key(seed, layer_tensor_id(l, S_ATTN_NORM)), nullptr, 0, scale, 1.0f));
    LMB_TRY(fill_plain<float>(ctx, L.ffn_norm, 1, hid, stream_key(seed, layer_tensor_id(l, S_FFN_NORM)), nullptr, 0, scale, 1.0f));
  }
  if (M->cfg.dtype == LMB200_BF16)
    LMB_TRY(fill_plain<__nv_bfloat16>(ctx, M->embed, M->cfg.vocab, hid, stream_key(seed, kIdEmbed), nullptr, 0, scale, 0.f));
  else
    LMB_TRY(fill_plain<float>(ctx, M->embed, M->cfg.vocab, hid, stream_key(seed, kIdEmbed), nullptr, 0, scale, 0.f));
  LMB_TRY(fill_plain<float>(ctx, M->final_norm, 1, hid, stream_key(seed, kIdFinalNorm), nullptr, 0, scale, 1.0f));
  FillSrc f{};
  f.only_slot = -1; f.scale = scale;
  f.key[0] = stream_key(seed, kIdHead);
  LMB_TRY(fill_tiled_dt(M, M->lm_head, M->m_head, f));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  M->all_weights_set = true;
  M->fold_valid = false;
  return LMB200_OK;
}

// The caller states the shape of what `host` points to; it must be the logical shape the model's
// configuration gives the tensor (matrices [out, in]; vectors [n], [1, n] or [n, 1]), so that a
// checkpoint of another width is refused instead of being read out of bounds.
static int32_t check_weight_shape(const char* name, int32_t rank, const int64_t* dims, int64_t rows, int64_t cols) {
  LMB_REQUIRE(rank >= 1 && rank <= 2 && dims, "set_weight: '%s': rank %d (expected 1 or 2 with the dimensions given)", name, rank);
  const int64_t d0 = dims[0], d1 = rank == 2 ? dims[1] : 1;
  bool ok;
  if (rows == 1) ok = (rank == 1 && d0 == cols) || (rank == 2 && ((d0 == 1 && d1 == cols) || (d0 == cols && d1 == 1)));
  else ok = rank == 2 && d0 == rows && d1 == cols;
  if (!ok) {
    if (rows == 1)
      return fail(LMB200_EINVAL, "set_weight: '%s' has shape [%lld%s%lld], the model expects [%lld]", name, (long long)d0,
                  rank == 2 ? ", " : "; rank 1, ", (long long)d1, (long long)cols);
    return fail(LMB200_EINVAL, "set_weight: '%s' has shape [%lld, %lld] (rank %d), the model expects [%lld, %lld]", name,
                (long long)d0, (long long)d1, rank, (long long)rows, (long long)cols);
  }
  return LMB200_OK;
}

extern "C" int32_t lmb200_model_set_weight(lmb200_model h, const char* name, const float* host, int32_t rank,
                                           const int64_t* dims, int32_t layout) {
  Model* M = model_from(h);
  if (!M) return LMB200_EINVAL;
  LMB_REQUIRE(name && host, "set_weight: null argument");
  LMB_REQUIRE(layout == LMB200_ROWMAJOR || layout == LMB200_COLMAJOR, "set_weight: layout %d", layout);
  Ctx* ctx = M->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const lmb200_model_config& c = M->cfg;
  const std::string n(name);
  // resolve the name
  void* dst = nullptr;
  const WMap* map = nullptr;
  int slot = 0;
  int64_t rows = 0, cols = 0;
  bool plain_f32 = false, plain_embed = false, is_bias = false;
  void* also_tiled = nullptr;          // Whisper: the embedding doubles as the head matrix
  if (c.arch == LMB200_ARCH_WHISPER_DECODER) {
    // registry names of TextDecoder (src/Whisper.jl:464-481, 423-431)
    const int hid = c.hidden;
    if (n.rfind("model.encoder.", 0) == 0) return LMB200_OK;            // the encoder is not part of this model
    if (n == "model.decoder.embed_tokens.weight") { dst = M->embed; rows = c.vocab; cols = hid; plain_embed = true; also_tiled = M->embed_tiled; }
    else if (n == "model.decoder.embed_positions.weight") { dst = M->pos_emb; rows = c.max_positions; cols = hid; plain_f32 = true; }
    else if (n == "model.decoder.layer_norm.weight") { dst = M->final_norm; rows = 1; cols = hid; plain_f32 = true; }
    else if (n == "model.decoder.layer_norm.bias") { dst = M->final_norm_b; rows = 1; cols = hid; plain_f32 = true; }
    else {
      int layer = -1, used = 0;
      if (sscanf(name, "model.decoder.layers.%d.%n", &layer, &used) < 1 || layer < 0 || layer >= c.n_layers)
        return fail(LMB200_ENOTFOUND, "set_weight: unknown tensor '%s'", name);
      const std::string tail(name + used);
      LayerWeights& L = M->layers[layer];
      auto vec = [&](float* d, int len) { dst = d; rows = 1; cols = len; plain_f32 = true; };
      auto mat = [&](void* d, const WMap* m, int sl, int r_, int c_) { dst = d; map = m; slot = sl; rows = r_; cols = c_; };
      auto bia = [&](float* d, const WMap* m, int sl, int len) { dst = d; map = m; slot = sl; rows = 1; cols = len; is_bias = true; };
      if (tail == "self_attn.q_proj.weight") mat(L.wqkv, &M->m_qkv, 0, hid, hid);
      else if (tail == "self_attn.k_proj.weight") mat(L.wqkv, &M->m_qkv, 1, hid, hid);
      else if (tail == "self_attn.v_proj.weight") mat(L.wqkv, &M->m_qkv, 2, hid, hid);
      else if (tail == "self_attn.q_proj.bias") bia(L.b_qkv, &M->m_qkv, 0, hid);
      else if (tail == "self_attn.v_proj.bias") bia(L.b_qkv, &M->m_qkv, 2, hid);
      else if (tail == "self_attn.out_proj.weight") mat(L.wo, &M->m_o, 0, hid, hid);
      else if (tail == "self_attn.out_proj.bias") vec(L.b_o, hid);
      else if (tail == "self_attn_layer_norm.weight") vec(L.attn_norm, hid);
      else if (tail == "self_attn_layer_norm.bias") vec(L.attn_norm_b, hid);
      else if (tail == "encoder_attn.q_proj.weight") mat(L.wq_cross, &M->m_qc, 0, hid, hid);
      else if (tail == "encoder_attn.q_proj.bias") bia(L.b_q_cross, &M->m_qc, 0, hid);
      else if (tail == "encoder_attn.out_proj.weight") mat(L.wo_cross, &M->m_o, 0, hid, hid);
      else if (tail == "encoder_attn.out_proj.bias") vec(L.b_o_cross, hid);
      // k_proj / v_proj of the cross attention act on the encoder output once (project_cross_kv);
      // their result is handed to the session with lmb200_session_set_cross_kv
      else if (tail.rfind("encoder_attn.k_proj", 0) == 0 || tail.rfind("encoder_attn.v_proj", 0) == 0) return LMB200_OK;
      else if (tail == "encoder_attn_layer_norm.weight") vec(L.cross_norm, hid);
      else if (tail == "encoder_attn_layer_norm.bias") vec(L.cross_norm_b, hid);
      else if (tail == "fc1.weight") mat(L.wgu, &M->m_gu, 0, c.intermediate, hid);
      else if (tail == "fc1.bias") vec(L.b_fc1, c.intermediate);
      else if (tail == "fc2.weight") mat(L.wdown, &M->m_down, 0, hid, c.intermediate);
      else if (tail == "fc2.bias") vec(L.b_fc2, hid);
      else if (tail == "final_layer_norm.weight") vec(L.ffn_norm, hid);
      else if (tail == "final_layer_norm.bias") vec(L.ffn_norm_b, hid);
      else return fail(LMB200_ENOTFOUND, "set_weight: unknown tensor '%s'", name);
    }
  } else if (n == "model.embed_tokens.weight") { dst = M->embed; rows = c.vocab; cols = c.hidden; plain_embed = true; }
  else if (n == "model.norm.weight") { dst = M->final_norm; rows = 1; cols = c.hidden; plain_f32 = true; }
  else if (n == "lm_head.weight") { dst = M->lm_head; map = &M->m_head; rows = c.vocab; cols = c.hidden; }
  else {
    int layer = -1, used = 0;
    if (sscanf(name, "model.layers.%d.%n", &layer, &used) < 1 || layer < 0 || layer >= c.n_layers)
      return fail(LMB200_ENOTFOUND, "set_weight: unknown tensor '%s'", name);
    const std::string tail(name + used);
    LayerWeights& L = M->layers[layer];
    const int kvd = c.n_kv_heads * M->D;
    if (tail == "input_layernorm.weight") { dst = L.attn_norm; rows = 1; cols = c.hidden; plain_f32 = true; }
    else if (tail == "post_attention_layernorm.weight") { dst = L.ffn_norm; rows = 1; cols = c.hidden; plain_f32 = true; }
    else if (tail == "self_attn.q_proj.weight") { dst = L.wqkv; map = &M->m_qkv; slot = 0; rows = c.hidden; cols = c.hidden; }
    else if (tail == "self_attn.k_proj.weight") { dst = L.wqkv; map = &M->m_qkv; slot = 1; rows = kvd; cols = c.hidden; }
    else if (tail == "self_attn.v_proj.weight") { dst = L.wqkv; map = &M->m_qkv; slot = 2; rows = kvd; cols = c.hidden; }
    else if (tail == "self_attn.o_proj.weight") { dst = L.wo; map = &M->m_o; rows = c.hidden; cols = c.hidden; }
    else if (tail == "mlp.gate_proj.weight") { dst = L.wgu; map = &M->m_gu; slot = 0; rows = c.intermediate; cols = c.hidden; }
    else if (tail == "mlp.up_proj.weight") { dst = L.wgu; map = &M->m_gu; slot = 1; rows = c.intermediate; cols = c.hidden; }
    else if (tail == "mlp.down_proj.weight") { dst = L.wdown; map = &M->m_down; rows = c.hidden; cols = c.intermediate; }
    else return fail(LMB200_ENOTFOUND, "set_weight: unknown tensor '%s'", name);
  }
  LMB_TRY(check_weight_shape(name, rank, dims, rows, cols));
  float* stage = nullptr;
  const int64_t bytes = rows * cols * 4;
  LMB_TRY(dmalloc((void**)&stage, bytes, false, ctx->stream));
  int32_t rc = LMB200_OK;
  do {
    if (cudaMemcpyAsync(stage, host, (size_t)bytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "set_weight: upload failed"); break;
    }
    if (is_bias) {
      fill_bias_kernel<<<fill_grid(map->rows), 256, 0, ctx->stream>>>(reinterpret_cast<float*>(dst), *map, stage, slot);
      ctx->launches++;
      if (cudaGetLastError() != cudaSuccess) rc = fail(LMB200_ECUDA, "set_weight: bias fill failed");
    } else if (plain_f32) {
      rc = fill_plain<float>(ctx, dst, rows, cols, 0, stage, rows > 1 ? layout : 0, 0.f, 0.f);
    } else if (plain_embed) {
      rc = c.dtype == LMB200_BF16 ? fill_plain<__nv_bfloat16>(ctx, dst, rows, cols, 0, stage, layout, 0.f, 0.f)
                                  : fill_plain<float>(ctx, dst, rows, cols, 0, stage, layout, 0.f, 0.f);
      if (rc == LMB200_OK && also_tiled) {
        FillSrc f{};
        f.only_slot = 0; f.colmajor = layout; f.scale = 0.f;
        f.src[0] = stage; f.src[1] = f.src[2] = nullptr;
        rc = fill_tiled_dt(M, also_tiled, M->m_head, f);
      }
    } else {
      FillSrc f{};
      f.only_slot = slot; f.colmajor = layout; f.scale = 0.f;
      f.src[0] = f.src[1] = f.src[2] = nullptr;
      f.src[slot] = stage;
      rc = fill_tiled_dt(M, dst, *map, f);
    }
  } while (0);
  cudaStreamSynchronize(ctx->stream);
  cudaFree(stage);
  if (rc == LMB200_OK) M->weights_set.insert(n);
  M->fold_valid = false;
  return rc;
}

// Registry names of every tensor this model reads (src/NN.jl:180-225, 433-445; src/Whisper.jl:423-481).
static std::vector<std::string> expected_weight_names(const Model* M) {
  std::vector<std::string> v;
  const lmb200_model_config& c = M->cfg;
  char buf[160];
  if (c.arch == LMB200_ARCH_WHISPER_DECODER) {
    v = {"model.decoder.embed_tokens.weight", "model.decoder.embed_positions.weight", "model.decoder.layer_norm.weight",
         "model.decoder.layer_norm.bias"};
    static const char* tails[] = {"self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                                  "self_attn.q_proj.bias", "self_attn.v_proj.bias", "self_attn.out_proj.weight",
                                  "self_attn.out_proj.bias", "self_attn_layer_norm.weight", "self_attn_layer_norm.bias",
                                  "encoder_attn.q_proj.weight", "encoder_attn.q_proj.bias", "encoder_attn.out_proj.weight",
                                  "encoder_attn.out_proj.bias", "encoder_attn_layer_norm.weight", "encoder_attn_layer_norm.bias",
                                  "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias", "final_layer_norm.weight",
                                  "final_layer_norm.bias"};
    for (int l = 0; l < c.n_layers; ++l)
      for (const char* t : tails) { snprintf(buf, sizeof(buf), "model.decoder.layers.%d.%s", l, t); v.push_back(buf); }
    return v;
  }
  v = {"model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"};
  static const char* tails[] = {"input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                                "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"};
  for (int l = 0; l < c.n_layers; ++l)
    for (const char* t : tails) { snprintf(buf, sizeof(buf), "model.layers.%d.%s", l, t); v.push_back(buf); }
  return v;
}

extern "C" int32_t lmb200_model_missing_weights(lmb200_model h, char* names_out, int64_t capacity, int32_t* n_missing) {
  Model* M = model_from(h);
  if (!M) return LMB200_EINVAL;
  LMB_REQUIRE(n_missing && (names_out || capacity == 0) && capacity >= 0, "missing_weights: bad argument");
  int32_t n = 0;
  int64_t used = 0;
  if (capacity > 0) names_out[0] = 0;
  if (!M->all_weights_set) {
    for (const std::string& name : expected_weight_names(M)) {
      if (M->weights_set.count(name)) continue;
      ++n;
      const int64_t need = (int64_t)name.size() + 1;
      if (used + need < capacity) {
        memcpy(names_out + used, name.c_str(), name.size());
        names_out[used + name.size()] = '\n';
        used += need;
        names_out[used] = 0;
      }
    }
  }
  *n_missing = n;
  return LMB200_OK;
}

// =============================================================================================
// session
// =============================================================================================
namespace lmb {
namespace {

GemvParams gemv_params(Session* S, const void* W, const WMap& m, const GemvPlan& pl, const void* x) {
  GemvParams p;
  p.W = W; p.x = x; p.B = S->B;
  p.rows = m.rows; p.K = m.K; p.RB = m.RB; p.KC = m.KC;
  p.ksplit = pl.ksplit; p.kc_per_split = pl.kc_per_split; p.grid = pl.grid; p.cluster = pl.cluster;
  p.partials = S->gemv_partials; p.counters = S->gemv_counters;
  return p;
}

// Partial-sum exchange of the two row-parallel projections of a layer (index 2l: o_proj, 2l + 1:
// down_proj).  With the peer regions mapped, the projection writes this rank's partial into its
// region (buffers alternate, so a buffer is rewritten only after every peer has passed the next
// reduction) and the following norm kernel sums all ranks' partials itself; otherwise the partial
// goes through ncclAllReduce in place.
struct RowParallelOut {
  float* out;          // where the GEMV stores its [B, hidden] result
  bool nccl;           // all-reduce `out` in place afterwards
  PeerReduce pr;       // for the consuming norm kernel (n == 0: read `out` as is)
};

RowParallelOut row_parallel_out(Session* S, int index) {
  Ctx* ctx = S->m->ctx;
  RowParallelOut r;
  r.out = S->delta;
  r.nccl = false;
  const int n = S->m->cfg.tp_size;
  if (n <= 1 || S->m->tp_solo) return r;
  if (ctx->peer_n != n || (int64_t)S->B * S->m->cfg.hidden > kPeerBufFloats || (unsigned long long)index + 1 >= kPeerEpochStride) {
    r.nccl = true;
    return r;
  }
  const int64_t buf = (int64_t)(index & 1) * kPeerBufFloats;
  r.out = reinterpret_cast<float*>(ctx->peer_base[ctx->tp_rank]) + buf;
  r.pr.n = n;
  r.pr.rank = ctx->tp_rank;
  for (int k = 0; k < n; ++k) {
    r.pr.part[k] = reinterpret_cast<const float*>(ctx->peer_base[k]) + buf;
    r.pr.remote_flag[k] = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(ctx->peer_base[k]) + kPeerFlagsOffset) + ctx->tp_rank;
  }
  r.pr.local_flag = reinterpret_cast<const unsigned long long*>(reinterpret_cast<char*>(ctx->peer_base[ctx->tp_rank]) + kPeerFlagsOffset);
  r.pr.step = ctx->peer_step;
  r.pr.phase = (unsigned)index + 1;
  r.pr.dev_err = ctx->dev_err;
  r.pr.broken = ctx->dev_broken;
  r.pr.wait_cycles = ctx->peer_wait_cycles > 0 ? ctx->peer_wait_cycles : kPeerWaitCycles;
  return r;
}

template <typename WT>
int32_t enqueue_step_t(Session* S, cudaStream_t st, bool with_head) {
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int dt = c.dtype;
  const int B = S->B, hid = c.hidden;
  const int L = c.n_layers;
  const size_t norm_smem = (size_t)hid * sizeof(float);
  RowParallelOut prev;             // the down_proj of the previous layer
  prev.out = S->delta; prev.nccl = false;
  // residual add + RMSNorm; with the ranks' partials in peer regions the clustered kernel does the all-reduce
  auto launch_norm = [&](const float* delta, const int* tokens, const float* w, WT* xn, float* capture, const PeerReduce& pr) -> int32_t {
    if (pr.n > 1 && !tokens && hid % (16 * kTpSplit) == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(B * kTpSplit));
      cfg.blockDim = dim3(kTpThreads);
      cfg.dynamicSmemBytes = norm_smem / kTpSplit;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = kTpSplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      LMB_CUDA(cudaLaunchKernelEx(&cfg, add_rmsnorm_tp_kernel<WT>, S->x, w, xn, S->Bp, hid, c.rms_eps, capture, pr));
    } else {
      LMB_CUDA(launch_k(add_rmsnorm_kernel<WT>, dim3(B), dim3(kNormThreads), norm_smem, st, S->x, delta, tokens,
                        reinterpret_cast<const WT*>(M->embed), c.vocab, w, xn, S->Bp, hid, c.rms_eps, capture, pr));
    }
    ctx->launches++;
    return LMB200_OK;
  };
  for (int l = 0; l < L; ++l) {
    LayerWeights& W = M->layers[l];
    // residual add of the previous MLP (or the embedding gather) + attention RMSNorm
    LMB_TRY(launch_norm(l == 0 ? (const float*)nullptr : (const float*)prev.out, l == 0 ? (const int*)S->tokens : (const int*)nullptr,
                        (const float*)W.attn_norm, reinterpret_cast<WT*>(S->xn),
                        (S->capture_on && l > 0) ? S->capture + (int64_t)(l - 1) * B * hid : (float*)nullptr,
                        l == 0 ? PeerReduce() : prev.pr));
    void* kv_layer = reinterpret_cast<char*>(S->kv) + (int64_t)l * S->kv_layer_stride * M->esz;
    {  // q/k/v projections + RoPE + KV append
      GemvParams p = gemv_params(S, W.wqkv, M->m_qkv, S->p_qkv, S->xn);
      p.epi = EPI_QKV_ROPE;
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = kv_layer; p.kv_batch_stride = S->kv_batch_stride; p.kv_head_stride = S->kv_head_stride;
      p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = M->KVl; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {  // attention over the cache; the result is the tiled input of o_proj
      AttnParams a;
      a.q = S->qbuf; a.q_pitch = S->q_pitch; a.kv_layer = kv_layer;
      a.kv_batch_stride = S->kv_batch_stride; a.kv_head_stride = S->kv_head_stride;
      a.B = B; a.KVl = M->KVl; a.G = M->G; a.D = M->D; a.pos = S->pos;
      a.keys_per_cta = S->keys_per_cta; a.nsplit = S->nsplit;
      a.scale = 1.0f / sqrtf((float)M->D);
      a.part_o = S->part_o; a.part_ml = S->part_ml; a.out = S->attn_out; a.out_tiled_bp = S->Bp;
      a.counters = S->attn_counters;
      LMB_TRY(attn_decode_launch(ctx, dt, a, st));
    }
    RowParallelOut ro = row_parallel_out(S, 2 * l);
    {  // o_proj (row-parallel under TP)
      GemvParams p = gemv_params(S, W.wo, M->m_o, S->p_o, S->attn_out);
      p.epi = EPI_STORE_F32; p.out = ro.out; p.out_pitch = hid;
      gemv_prefetch_next(p, ctx, dt, W.wgu, M->m_gu.rows, M->m_gu.K, S->p_gu);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
      if (ro.nccl) LMB_TRY(nccl_allreduce_f32(ctx, ro.out, (int64_t)B * hid, st));
    }
    LMB_TRY(launch_norm((const float*)ro.out, (const int*)nullptr, (const float*)W.ffn_norm, reinterpret_cast<WT*>(S->xn),
                        (float*)nullptr, ro.pr));
    {  // gate/up + SiLU gate
      GemvParams p = gemv_params(S, W.wgu, M->m_gu, S->p_gu, S->xn);
      p.epi = EPI_SILU_GATE; p.act = S->act; p.n_act = M->inter_l;
      gemv_prefetch_next(p, ctx, dt, W.wdown, M->m_down.rows, M->m_down.K, S->p_down);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    prev = row_parallel_out(S, 2 * l + 1);
    {  // down_proj (row-parallel under TP)
      GemvParams p = gemv_params(S, W.wdown, M->m_down, S->p_down, S->act);
      p.epi = EPI_STORE_F32; p.out = prev.out; p.out_pitch = hid;
      if (l + 1 < L) gemv_prefetch_next(p, ctx, dt, M->layers[l + 1].wqkv, M->m_qkv.rows, M->m_qkv.K, S->p_qkv);
      else if (with_head) gemv_prefetch_next(p, ctx, dt, M->lm_head, M->m_head.rows, M->m_head.K, S->p_head);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
      if (prev.nccl) LMB_TRY(nccl_allreduce_f32(ctx, prev.out, (int64_t)B * hid, st));
    }
  }
  // last residual add (+ final norm); without the head only the add is needed for the capture
  LMB_TRY(launch_norm((const float*)prev.out, (const int*)nullptr, (const float*)M->final_norm,
                      with_head ? reinterpret_cast<WT*>(S->xn) : (WT*)nullptr,
                      S->capture_on ? S->capture + (int64_t)(L - 1) * B * hid : (float*)nullptr, prev.pr));
  if (with_head) {
    GemvParams p = gemv_params(S, M->lm_head, M->m_head, S->p_head, S->xn);
    p.epi = EPI_STORE_F32; p.out = S->logits; p.out_pitch = S->logits_pitch;
    LMB_TRY(gemv_launch(ctx, dt, p, st));
    LMB_CUDA(launch_k(argmax_step_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits, S->logits_pitch, c.vocab,
                      S->tokens, S->tok_hist, (const int*)S->step_ctr, B, S->stop));
    ctx->launches++;
  }
  LMB_CUDA(launch_k(advance_kernel, dim3(1), dim3(32), 0, st, S->pos, (const int*)S->limit, S->B, S->step_ctr, ctx->peer_n > 1 ? ctx->peer_step : (unsigned long long*)nullptr));
  ctx->launches++;
  return LMB200_OK;
}

// Exchange parameters of the projection that carries reduction `index` of the step (2l: o_proj, 2l + 1:
// down_proj) when it runs EPI_RESID_NORM under tensor parallelism.
PeerPush peer_push(Session* S, int index) {
  Ctx* ctx = S->m->ctx;
  PeerPush pp;
  const int n = S->m->cfg.tp_size;
  if (n <= 1 || S->m->tp_solo) return pp;
  const int64_t buf = kPeerPushOffset + (int64_t)(index & 1) * kPeerBufFloats * 4;
  pp.n = n;
  pp.rank = ctx->tp_rank;
  for (int k = 0; k < n; ++k) {
    pp.part[k] = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(ctx->peer_base[k]) + buf);
    pp.flag[k] = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(ctx->peer_base[k]) + kPeerPushFlagsOffset);
  }
  pp.step = ctx->peer_step;
  pp.phase = (unsigned)index + 1;
  pp.dev_err = ctx->dev_err;
  pp.broken = ctx->dev_broken;
  pp.wait_cycles = ctx->peer_wait_cycles > 0 ? ctx->peer_wait_cycles : kPeerWaitCycles;
  return pp;
}

// The fused decode step of a bf16 Llama / Phi-3: five launches per layer.  The residual add and the
// RMSNorm around every Linear (src/NN.jl:406-414, 149-161) are carried by the projections themselves:
// o_proj and down_proj finish with EPI_RESID_NORM (under tensor parallelism including the all-reduce of
// their partial sums), q/k/v, gate/up and the head multiply their accumulators by the norm's
// per-sequence scale (InvScale).
// head: 0 no head, 1 head with the full logits, 2 tokens only (the sliced head, where the session has one)
int32_t enqueue_step_fused(Session* S, cudaStream_t st, int head) {
  const bool with_head = head != 0;
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int dt = LMB200_BF16;
  const int B = S->B, hid = c.hidden, L = c.n_layers;
  {
    const int rows_per = S->embed_rows_per_cta;
    const int grid = (int)ceil_div(hid, rows_per);
    if (S->Bp == 16)
      LMB_CUDA(launch_k(embed_prep_kernel<16>, dim3(grid), dim3(128), 0, st, (const int*)S->tokens,
                        reinterpret_cast<const __nv_bfloat16*>(M->embed), c.vocab, hid, B, (const float*)M->layers[0].attn_norm,
                        S->xT, reinterpret_cast<__nv_bfloat16*>(S->xn), S->ssq, rows_per));
    else
      LMB_CUDA(launch_k(embed_prep_kernel<32>, dim3(grid), dim3(128), 0, st, (const int*)S->tokens,
                        reinterpret_cast<const __nv_bfloat16*>(M->embed), c.vocab, hid, B, (const float*)M->layers[0].attn_norm,
                        S->xT, reinterpret_cast<__nv_bfloat16*>(S->xn), S->ssq, rows_per));
    ctx->launches++;
  }
  int tiles = (int)ceil_div(hid, S->embed_rows_per_cta);        // slots of S->ssq the last producer wrote
  auto inv_scale = [&]() { InvScale iv; iv.ssq = S->ssq; iv.tiles = tiles; iv.n = hid; iv.eps = c.rms_eps; return iv; };
  for (int l = 0; l < L; ++l) {
    LayerWeights& W = M->layers[l];
    void* kv_layer = reinterpret_cast<char*>(S->kv) + (int64_t)l * S->kv_layer_stride * M->esz;
    {  // q/k/v projections (norm scale on the accumulators) + RoPE + KV append
      GemvParams p = gemv_params(S, W.wqkv, M->m_qkv, S->p_qkv, S->xn);
      p.epi = EPI_QKV_ROPE; p.inv = inv_scale();
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = kv_layer; p.kv_batch_stride = S->kv_batch_stride; p.kv_head_stride = S->kv_head_stride;
      p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = M->KVl; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {
      AttnParams a;
      a.q = S->qbuf; a.q_pitch = S->q_pitch; a.kv_layer = kv_layer;
      a.kv_batch_stride = S->kv_batch_stride; a.kv_head_stride = S->kv_head_stride;
      a.B = B; a.KVl = M->KVl; a.G = M->G; a.D = M->D; a.pos = S->pos;
      a.keys_per_cta = S->keys_per_cta; a.nsplit = S->nsplit;
      a.scale = 1.0f / sqrtf((float)M->D);
      a.part_o = S->part_o; a.part_ml = S->part_ml; a.out = S->attn_out; a.out_tiled_bp = S->Bp;
      a.counters = S->attn_counters;
      LMB_TRY(attn_decode_launch(ctx, dt, a, st));
    }
    {  // o_proj + all-reduce + residual add + what the MLP's norm needs
      GemvParams p = gemv_params(S, W.wo, M->m_o, S->p_o, S->attn_out);
      p.epi = EPI_RESID_NORM;
      p.rn.x = S->xT; p.rn.gain = W.ffn_norm; p.rn.xg = S->xn; p.rn.ssq = S->ssq;
      p.push = peer_push(S, 2 * l);
      gemv_prefetch_next(p, ctx, dt, W.wgu, M->m_gu.rows, M->m_gu.K, S->p_gu);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
      tiles = gemv_plan_ctas(S->p_o, M->m_o.rows);
    }
    {  // gate/up (norm scale on the accumulators) + SiLU gate
      GemvParams p = gemv_params(S, W.wgu, M->m_gu, S->p_gu, S->xn);
      p.epi = EPI_SILU_GATE; p.inv = inv_scale(); p.act = S->act; p.n_act = M->inter_l;
      gemv_prefetch_next(p, ctx, dt, W.wdown, M->m_down.rows, M->m_down.K, S->p_down);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {  // down_proj + all-reduce + residual add + what the next norm (next layer's, or the final one) needs
      GemvParams p = gemv_params(S, W.wdown, M->m_down, S->p_down, S->act);
      p.epi = EPI_RESID_NORM;
      p.rn.x = S->xT; p.rn.gain = l + 1 < L ? M->layers[l + 1].attn_norm : M->final_norm; p.rn.xg = S->xn; p.rn.ssq = S->ssq;
      p.rn.capture = S->capture_on ? S->capture + (int64_t)l * B * hid : nullptr;
      p.push = peer_push(S, 2 * l + 1);
      if (l + 1 < L) gemv_prefetch_next(p, ctx, dt, M->layers[l + 1].wqkv, M->m_qkv.rows, M->m_qkv.K, S->p_qkv);
      else if (with_head) gemv_prefetch_next(p, ctx, dt, M->lm_head, M->m_head.rows, M->m_head.K, S->p_head);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
      tiles = gemv_plan_ctas(S->p_down, M->m_down.rows);
    }
  }
  if (with_head && S->head_sliced) {
    // this rank's rows of the head, its best (logit, id) per sequence, the exchange; the full logits only on request
    {
      WMap ms = M->m_head;
      ms.rows = S->head_rows;
      ms.RB = (int)ceil_div(S->head_rows, 16);
      const int64_t KS = ceil_div(M->m_head.K, 128);
      const __nv_bfloat16* Ws = reinterpret_cast<const __nv_bfloat16*>(M->lm_head) + (int64_t)S->head_rg0 * KS * 16384;
      GemvParams p = gemv_params(S, Ws, ms, S->p_head_slice, S->xn);
      p.epi = EPI_STORE_F32; p.inv = inv_scale(); p.out = S->logits_slice; p.out_pitch = S->head_pitch;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    RowParallelOut ex = row_parallel_out(S, 2 * L);       // the buffers and flags of the float32 exchange, phase 2 L + 1
    LMB_CUDA(launch_k(argmax_pairs_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits_slice, S->head_pitch,
                      S->head_rows, S->head_rg0 * 128, ex.out));
    LMB_CUDA(launch_k(argmax_tp_select_kernel, dim3(1), dim3(256), 0, st, ex.pr, B, S->tokens, S->tok_hist, (const int*)S->step_ctr,
                      S->stop));
    ctx->launches += 2;
    if (head == 1) {
      GemvParams p = gemv_params(S, M->lm_head, M->m_head, S->p_head, S->xn);
      p.epi = EPI_STORE_F32; p.inv = inv_scale(); p.out = S->logits; p.out_pitch = S->logits_pitch;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
  } else if (with_head) {
    GemvParams p = gemv_params(S, M->lm_head, M->m_head, S->p_head, S->xn);
    p.epi = EPI_STORE_F32; p.inv = inv_scale(); p.out = S->logits; p.out_pitch = S->logits_pitch;
    LMB_TRY(gemv_launch(ctx, dt, p, st));
    LMB_CUDA(launch_k(argmax_step_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits, S->logits_pitch, c.vocab,
                      S->tokens, S->tok_hist, (const int*)S->step_ctr, B, S->stop));
    ctx->launches++;
  }
  LMB_CUDA(launch_k(advance_kernel, dim3(1), dim3(32), 0, st, S->pos, (const int*)S->limit, S->B, S->step_ctr, ctx->peer_n > 1 ? ctx->peer_step : (unsigned long long*)nullptr));
  ctx->launches++;
  return LMB200_OK;
}

// One decode step of the Whisper TextDecoder with cached self attention and cross attention
// (build_decode_step!, src/Whisper.jl:679-742): per layer LayerNorm -> q/k/v (bias, head_dim^-0.25
// on q and k, no RoPE) + cache append -> attention over [0, pos] -> out_proj -> LayerNorm ->
// cross q -> attention over the fixed cross K/V -> out_proj -> LayerNorm -> fc1 + GELU -> fc2;
// then the final LayerNorm and the tied-embedding head.
template <typename WT>
int32_t enqueue_whisper_step_t(Session* S, cudaStream_t st, bool with_head) {
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int dt = c.dtype;
  const int B = S->B, hid = c.hidden, L = c.n_layers;
  const size_t norm_smem = (size_t)hid * sizeof(float);
  const float qk_scale = powf((float)hid / (float)c.n_heads, -0.25f);
  auto norm = [&](const float* delta, bool first, const float* w, const float* b, bool write_xn, float* cap) -> int32_t {
    LMB_CUDA(launch_k(add_layernorm_kernel<WT>, dim3(B), dim3(kNormThreads), norm_smem, st, S->x, delta,
                      (const float*)nullptr, first ? (const int*)S->tokens : (const int*)nullptr,
                      reinterpret_cast<const WT*>(M->embed), c.vocab, (const float*)M->pos_emb, (const int*)S->pos, w, b,
                      write_xn ? reinterpret_cast<WT*>(S->xn) : (WT*)nullptr, S->Bp, hid, c.rms_eps, cap));
    ctx->launches++;
    return LMB200_OK;
  };
  auto attention = [&](void* kv_layer, int64_t bs, int64_t hs, const int* pos, int T_fixed, int kpc, int nsplit) -> int32_t {
    AttnParams a;
    a.q = S->qbuf; a.q_pitch = S->q_pitch; a.kv_layer = kv_layer; a.kv_batch_stride = bs; a.kv_head_stride = hs;
    a.B = B; a.KVl = M->KVl; a.G = 1; a.D = M->D; a.pos = pos; a.T_fixed = T_fixed;
    a.keys_per_cta = kpc; a.nsplit = nsplit;
    a.scale = 1.0f;                      // the scale is already in q and k
    a.part_o = S->part_o; a.part_ml = S->part_ml; a.out = S->attn_out; a.out_tiled_bp = S->Bp;
      a.counters = S->attn_counters;
    return attn_decode_launch(ctx, dt, a, st);
  };
  for (int l = 0; l < L; ++l) {
    LayerWeights& W = M->layers[l];
    LMB_TRY(norm(l == 0 ? nullptr : S->delta, l == 0, W.attn_norm, W.attn_norm_b, true,
                 (S->capture_on && l > 0) ? S->capture + (int64_t)(l - 1) * B * hid : nullptr));
    void* kv_layer = reinterpret_cast<char*>(S->kv) + (int64_t)l * S->kv_layer_stride * M->esz;
    {
      GemvParams p = gemv_params(S, W.wqkv, M->m_qkv, S->p_qkv, S->xn);
      p.epi = EPI_QKV_ROPE; p.rope = 0; p.qk_scale = qk_scale; p.bias = W.b_qkv;
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = kv_layer; p.kv_batch_stride = S->kv_batch_stride; p.kv_head_stride = S->kv_head_stride;
      p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = M->KVl; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    LMB_TRY(attention(kv_layer, S->kv_batch_stride, S->kv_head_stride, S->pos, 0, S->keys_per_cta, S->nsplit));
    {
      GemvParams p = gemv_params(S, W.wo, M->m_o, S->p_o, S->attn_out);
      p.epi = EPI_STORE_F32; p.out = S->delta; p.out_pitch = hid; p.bias = W.b_o;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    LMB_TRY(norm(S->delta, false, W.cross_norm, W.cross_norm_b, true, nullptr));
    {  // cross-attention query: q rows only, nothing is appended to a cache
      GemvParams p = gemv_params(S, W.wq_cross, M->m_qc, S->p_qc, S->xn);
      p.epi = EPI_QKV_ROPE; p.rope = 0; p.qk_scale = qk_scale; p.bias = W.b_q_cross;
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = nullptr; p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = 0; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    void* cross_layer = reinterpret_cast<char*>(S->cross_kv) + (int64_t)l * S->cross_layer_stride * M->esz;
    LMB_TRY(attention(cross_layer, S->cross_batch_stride, S->cross_head_stride, nullptr, c.cross_len,
                      S->cross_keys_per_cta, S->cross_nsplit));
    {
      GemvParams p = gemv_params(S, W.wo_cross, M->m_o, S->p_o, S->attn_out);
      p.epi = EPI_STORE_F32; p.out = S->delta; p.out_pitch = hid; p.bias = W.b_o_cross;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    LMB_TRY(norm(S->delta, false, W.ffn_norm, W.ffn_norm_b, true, nullptr));
    {
      GemvParams p = gemv_params(S, W.wgu, M->m_gu, S->p_gu, S->xn);
      p.epi = EPI_GELU_ACT; p.act = S->act; p.n_act = c.intermediate; p.bias = W.b_fc1;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {
      GemvParams p = gemv_params(S, W.wdown, M->m_down, S->p_down, S->act);
      p.epi = EPI_STORE_F32; p.out = S->delta; p.out_pitch = hid; p.bias = W.b_fc2;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
  }
  LMB_TRY(norm(S->delta, false, M->final_norm, M->final_norm_b, with_head,
               S->capture_on ? S->capture + (int64_t)(L - 1) * B * hid : nullptr));
  if (with_head) {
    GemvParams p = gemv_params(S, M->embed_tiled, M->m_head, S->p_head, S->xn);     // logits = out * E^T
    p.epi = EPI_STORE_F32; p.out = S->logits; p.out_pitch = S->logits_pitch;
    LMB_TRY(gemv_launch(ctx, dt, p, st));
    LMB_CUDA(launch_k(argmax_step_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits, S->logits_pitch, c.vocab,
                      S->tokens, S->tok_hist, (const int*)S->step_ctr, B, S->stop));
    ctx->launches++;
  }
  LMB_CUDA(launch_k(advance_kernel, dim3(1), dim3(32), 0, st, S->pos, (const int*)S->limit, S->B, S->step_ctr, (unsigned long long*)nullptr));
  ctx->launches++;
  return LMB200_OK;
}

// The vectors that fold every LayerNorm of the Whisper decoder into the Linear after it (LayerWeights::wg_*, bf_*):
// computed from the bf16 weights the step multiplies with, once per set of weights.
int32_t whisper_fold(Model* M) {
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  auto fold = [&](const void* W, const WMap& m, const float* g, const float* b, const float* bias, float** wg, float** bf) -> int32_t {
    const int rows_pad = (int)round_up(m.rows, 128);
    if (!*wg) LMB_TRY(dmalloc((void**)wg, (int64_t)rows_pad * 4, true, ctx->stream));
    if (!*bf) LMB_TRY(dmalloc((void**)bf, (int64_t)rows_pad * 4, true, ctx->stream));
    ln_fold_kernel<<<m.rows, 128, 0, ctx->stream>>>(reinterpret_cast<const __nv_bfloat16*>(W), m.rows, m.K, g, b, bias, *wg, *bf);
    ctx->launches++;
    return LMB200_OK;
  };
  for (LayerWeights& W : M->layers) {
    LMB_TRY(fold(W.wqkv, M->m_qkv, W.attn_norm, W.attn_norm_b, W.b_qkv, &W.wg_qkv, &W.bf_qkv));
    LMB_TRY(fold(W.wq_cross, M->m_qc, W.cross_norm, W.cross_norm_b, W.b_q_cross, &W.wg_qc, &W.bf_qc));
    LMB_TRY(fold(W.wgu, M->m_gu, W.ffn_norm, W.ffn_norm_b, W.b_fc1, &W.wg_fc1, &W.bf_fc1));
  }
  LMB_TRY(fold(M->embed_tiled, M->m_head, M->final_norm, M->final_norm_b, nullptr, &M->wg_head, &M->bf_head));
  LMB_CUDA(cudaGetLastError());
  (void)c;
  M->fold_valid = true;
  return LMB200_OK;
}

// The fused decode step of the bf16 Whisper decoder: eight launches per layer instead of eleven.  As in the Llama
// step the residual add and the norm around every Linear ride on the projections: out_proj (self and cross) and fc2
// finish with EPI_RESID_NORM (their own bias added on the way), which leaves x * gain and the per-sequence sums of x
// and x^2; q/k/v, the cross q projection, fc1 and the tied head apply the LayerNorm to their accumulators
// (InvScale with a mean, GemvParams::ln_wg, a bias that already holds W b).  src/Whisper.jl:584-742.
int32_t enqueue_whisper_step_fused(Session* S, cudaStream_t st, bool with_head) {
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int dt = c.dtype;
  const int B = S->B, hid = c.hidden, L = c.n_layers;
  const float qk_scale = powf((float)hid / (float)c.n_heads, -0.25f);
  {
    const int rows_per = S->embed_rows_per_cta;
    const int grid = (int)ceil_div(hid, rows_per);
    if (S->Bp == 16)
      LMB_CUDA(launch_k(embed_prep_ln_kernel<16>, dim3(grid), dim3(128), 0, st, (const int*)S->tokens,
                        reinterpret_cast<const __nv_bfloat16*>(M->embed), c.vocab, hid, B, (const float*)M->pos_emb, (const int*)S->pos,
                        (const float*)M->layers[0].attn_norm, S->xT, reinterpret_cast<__nv_bfloat16*>(S->xn), S->ssq, S->sum_slots,
                        rows_per));
    else
      LMB_CUDA(launch_k(embed_prep_ln_kernel<32>, dim3(grid), dim3(128), 0, st, (const int*)S->tokens,
                        reinterpret_cast<const __nv_bfloat16*>(M->embed), c.vocab, hid, B, (const float*)M->pos_emb, (const int*)S->pos,
                        (const float*)M->layers[0].attn_norm, S->xT, reinterpret_cast<__nv_bfloat16*>(S->xn), S->ssq, S->sum_slots,
                        rows_per));
    ctx->launches++;
  }
  int tiles = (int)ceil_div(hid, S->embed_rows_per_cta);
  auto layer_norm = [&](GemvParams& p, const float* wg, const float* bf) {
    p.inv.ssq = S->ssq; p.inv.sum = S->sum_slots; p.inv.tiles = tiles; p.inv.n = hid; p.inv.eps = c.rms_eps;
    p.ln_wg = wg; p.bias = bf;
  };
  auto resid = [&](GemvParams& p, const float* bias, const float* next_gain, const GemvPlan& plan, int rows) {
    p.epi = EPI_RESID_NORM; p.bias = bias;
    p.rn.x = S->xT; p.rn.gain = next_gain; p.rn.xg = S->xn; p.rn.ssq = S->ssq; p.rn.sum = S->sum_slots;
    tiles = gemv_plan_ctas(plan, rows);
  };
  auto attention = [&](void* kv_layer, int64_t bs, int64_t hs, const int* pos, int T_fixed, int kpc, int nsplit) -> int32_t {
    AttnParams a;
    a.q = S->qbuf; a.q_pitch = S->q_pitch; a.kv_layer = kv_layer; a.kv_batch_stride = bs; a.kv_head_stride = hs;
    a.B = B; a.KVl = M->KVl; a.G = 1; a.D = M->D; a.pos = pos; a.T_fixed = T_fixed;
    a.keys_per_cta = kpc; a.nsplit = nsplit;
    a.scale = 1.0f;                      // the scale is already in q and k
    a.part_o = S->part_o; a.part_ml = S->part_ml; a.out = S->attn_out; a.out_tiled_bp = S->Bp;
    a.counters = S->attn_counters;
    return attn_decode_launch(ctx, dt, a, st);
  };
  for (int l = 0; l < L; ++l) {
    LayerWeights& W = M->layers[l];
    void* kv_layer = reinterpret_cast<char*>(S->kv) + (int64_t)l * S->kv_layer_stride * M->esz;
    {
      GemvParams p = gemv_params(S, W.wqkv, M->m_qkv, S->p_qkv, S->xn);
      p.epi = EPI_QKV_ROPE; p.rope = 0; p.qk_scale = qk_scale;
      layer_norm(p, W.wg_qkv, W.bf_qkv);
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = kv_layer; p.kv_batch_stride = S->kv_batch_stride; p.kv_head_stride = S->kv_head_stride;
      p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = M->KVl; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    LMB_TRY(attention(kv_layer, S->kv_batch_stride, S->kv_head_stride, S->pos, 0, S->keys_per_cta, S->nsplit));
    {
      GemvParams p = gemv_params(S, W.wo, M->m_o, S->p_o, S->attn_out);
      resid(p, W.b_o, W.cross_norm, S->p_o, M->m_o.rows);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {  // cross-attention query: q rows only, nothing is appended to a cache
      GemvParams p = gemv_params(S, W.wq_cross, M->m_qc, S->p_qc, S->xn);
      p.epi = EPI_QKV_ROPE; p.rope = 0; p.qk_scale = qk_scale;
      layer_norm(p, W.wg_qc, W.bf_qc);
      p.q_out = S->qbuf; p.q_pitch = S->q_pitch;
      p.kv_layer = nullptr; p.inv_freq = M->inv_freq; p.pos = S->pos; p.pos_uniform = S->ragged ? 0 : 1; p.Hl = M->Hl; p.KVl = 0; p.D = M->D;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    void* cross_layer = reinterpret_cast<char*>(S->cross_kv) + (int64_t)l * S->cross_layer_stride * M->esz;
    LMB_TRY(attention(cross_layer, S->cross_batch_stride, S->cross_head_stride, nullptr, c.cross_len, S->cross_keys_per_cta,
                      S->cross_nsplit));
    {
      GemvParams p = gemv_params(S, W.wo_cross, M->m_o, S->p_o, S->attn_out);
      resid(p, W.b_o_cross, W.ffn_norm, S->p_o, M->m_o.rows);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {
      GemvParams p = gemv_params(S, W.wgu, M->m_gu, S->p_gu, S->xn);
      p.epi = EPI_GELU_ACT; p.act = S->act; p.n_act = c.intermediate;
      layer_norm(p, W.wg_fc1, W.bf_fc1);
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
    {
      GemvParams p = gemv_params(S, W.wdown, M->m_down, S->p_down, S->act);
      resid(p, W.b_fc2, l + 1 < L ? M->layers[l + 1].attn_norm : M->final_norm, S->p_down, M->m_down.rows);
      p.rn.capture = S->capture_on ? S->capture + (int64_t)l * B * hid : nullptr;
      LMB_TRY(gemv_launch(ctx, dt, p, st));
    }
  }
  if (with_head) {
    GemvParams p = gemv_params(S, M->embed_tiled, M->m_head, S->p_head, S->xn);     // logits = LayerNorm(x) * E^T
    p.epi = EPI_STORE_F32; p.out = S->logits; p.out_pitch = S->logits_pitch;
    layer_norm(p, M->wg_head, M->bf_head);
    LMB_TRY(gemv_launch(ctx, dt, p, st));
    LMB_CUDA(launch_k(argmax_step_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits, S->logits_pitch, c.vocab,
                      S->tokens, S->tok_hist, (const int*)S->step_ctr, B, S->stop));
    ctx->launches++;
  }
  LMB_CUDA(launch_k(advance_kernel, dim3(1), dim3(32), 0, st, S->pos, (const int*)S->limit, S->B, S->step_ctr, (unsigned long long*)nullptr));
  ctx->launches++;
  return LMB200_OK;
}

int32_t enqueue_step(Session* S, cudaStream_t st, int head) {
  const bool with_head = head != 0;
  if (S->fused && S->m->cfg.arch == LMB200_ARCH_WHISPER_DECODER) return enqueue_whisper_step_fused(S, st, with_head);
  if (S->fused) return enqueue_step_fused(S, st, head);
  if (S->m->cfg.arch == LMB200_ARCH_WHISPER_DECODER)
    return S->m->cfg.dtype == LMB200_BF16 ? enqueue_whisper_step_t<__nv_bfloat16>(S, st, with_head)
                                          : enqueue_whisper_step_t<float>(S, st, with_head);
  return S->m->cfg.dtype == LMB200_BF16 ? enqueue_step_t<__nv_bfloat16>(S, st, with_head)
                                        : enqueue_step_t<float>(S, st, with_head);
}

// Final norm + head + greedy token on the residual rows already in S->x (after the GEMM prefill).
int32_t enqueue_head_bf16(Session* S, cudaStream_t st) {
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  const lmb200_model_config& c = M->cfg;
  const int B = S->B, hid = c.hidden;
  LMB_CUDA(launch_k(add_rmsnorm_kernel<__nv_bfloat16>, dim3(B), dim3(kNormThreads), (size_t)hid * sizeof(float), st, S->x,
                    (const float*)nullptr, (const int*)nullptr, (const __nv_bfloat16*)nullptr, 0, (const float*)M->final_norm,
                    reinterpret_cast<__nv_bfloat16*>(S->xn), S->Bp, hid, c.rms_eps, (float*)nullptr, PeerReduce()));
  ctx->launches++;
  GemvParams p = gemv_params(S, M->lm_head, M->m_head, S->p_head, S->xn);
  p.epi = EPI_STORE_F32; p.out = S->logits; p.out_pitch = S->logits_pitch;
  LMB_TRY(gemv_launch(ctx, c.dtype, p, st));
  LMB_CUDA(launch_k(argmax_step_kernel, dim3(B), dim3(kArgmaxThreads), 0, st, (const float*)S->logits, S->logits_pitch, c.vocab,
                    S->tokens, S->tok_hist, (const int*)S->step_ctr, B, S->stop));
  ctx->launches++;
  return LMB200_OK;
}

void drop_graphs(Session* S) {
  if (S->graph_full) cudaGraphExecDestroy(S->graph_full);
  if (S->graph_body) cudaGraphExecDestroy(S->graph_body);
  if (S->graph_tok) cudaGraphExecDestroy(S->graph_tok);
  S->graph_full = S->graph_body = S->graph_tok = nullptr;
  S->graph_stream = nullptr;
}

int32_t capture_one(Session* S, cudaStream_t st, int head, cudaGraphExec_t* exec, int* nodes) {
  Ctx* ctx = S->m->ctx;
  const int64_t before = ctx->launches;
  LMB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  int32_t rc = enqueue_step(S, st, head);
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(st, &graph);
  ctx->launches = before;            // captured, not run
  if (rc != LMB200_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
  if (e != cudaSuccess) return fail(LMB200_ECUDA, "graph capture failed: %s", cudaGetErrorString(e));
  size_t n = 0;
  cudaGraphGetNodes(graph, nullptr, &n);
  *nodes = (int)n;
  e = cudaGraphInstantiate(exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(LMB200_ECUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
  return LMB200_OK;
}

// graphs are tied to the stream they were captured on and to the capture flag
int32_t ensure_graphs(Session* S) {
  Ctx* ctx = S->m->ctx;
  if (S->graph_full && S->graph_stream == ctx->stream) return LMB200_OK;
  drop_graphs(S);
  LMB_TRY(capture_one(S, ctx->stream, 1, &S->graph_full, &S->graph_nodes_full));
  LMB_TRY(capture_one(S, ctx->stream, 0, &S->graph_body, &S->graph_nodes_body));
  if (S->head_sliced) LMB_TRY(capture_one(S, ctx->stream, 2, &S->graph_tok, &S->graph_nodes_tok));
  S->graph_stream = ctx->stream;
  return LMB200_OK;
}

// with_head: the step ends in the head and the greedy token; want_logits: a caller will read the full logits after it
// (under tensor parallelism the step otherwise computes only this rank's slice of them)
int32_t run_step(Session* S, bool with_head, bool want_logits = true) {
  Ctx* ctx = S->m->ctx;
  if (S->fused && S->m->cfg.arch == LMB200_ARCH_WHISPER_DECODER && !S->m->fold_valid) LMB_TRY(whisper_fold(S->m));
  LMB_TRY(ensure_graphs(S));
  const bool tok_only = with_head && !want_logits && S->graph_tok;
  LMB_CUDA(cudaGraphLaunch(tok_only ? S->graph_tok : with_head ? S->graph_full : S->graph_body, ctx->stream));
  ctx->launches += tok_only ? S->graph_nodes_tok : with_head ? S->graph_nodes_full : S->graph_nodes_body;
  if (!S->in_ragged_prefill) {
    S->host_pos += 1;
    for (int& v : S->host_pos_v) v += 1;
  }
  return LMB200_OK;
}

}  // namespace
}  // namespace lmb

// Positions live on the device, one per sequence; the host keeps a copy for its bounds checks.  `ragged`
// (the positions differ) selects the per-sequence RoPE path of the kernels, so changing it drops the graphs.
static int32_t push_positions(Session* S) {
  Ctx* ctx = S->m->ctx;
  bool ragged = false;
  int mx = 0;
  for (int b = 0; b < S->B; ++b) {
    ragged = ragged || S->host_pos_v[b] != S->host_pos_v[0];
    if (S->host_pos_v[b] > mx) mx = S->host_pos_v[b];
  }
  LMB_CUDA(cudaMemcpyAsync(S->pos, S->host_pos_v.data(), (size_t)S->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  S->host_pos = mx;
  if (ragged != S->ragged) {
    drop_graphs(S);
    S->ragged = ragged;
  }
  return LMB200_OK;
}
static int32_t set_all_positions(Session* S, int pos) {
  S->host_pos_v.assign(S->B, pos);
  return push_positions(S);
}
// limits == NULL: no limit (decoding)
static int32_t set_limits(Session* S, const int* limits) {
  Ctx* ctx = S->m->ctx;
  std::vector<int> v(S->B, 0x7fffffff);
  if (limits) v.assign(limits, limits + S->B);
  LMB_CUDA(cudaMemcpyAsync(S->limit, v.data(), (size_t)S->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_create(lmb200_model hm, int32_t batch, int32_t max_ctx, lmb200_session* out) {
  Model* M = model_from(hm);
  if (!M) return LMB200_EINVAL;
  LMB_REQUIRE(out, "session_create: null argument");
  LMB_REQUIRE(batch >= 1, "session_create: batch %d", batch);
  LMB_REQUIRE(max_ctx >= 1, "session_create: max_ctx %d", max_ctx);
  if (batch > 32) return wide_create(M, batch, max_ctx, out);
  Ctx* ctx = M->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const lmb200_model_config& c = M->cfg;
  const bool whisper = c.arch == LMB200_ARCH_WHISPER_DECODER;
  if (whisper)
    LMB_REQUIRE(max_ctx <= c.max_positions, "session_create: max_ctx %d exceeds the %d learned positions", max_ctx,
                c.max_positions);
  Session* S = new Session();
  S->m = M; S->B = batch; S->max_ctx = max_ctx;
  S->cap = (int)round_up(max_ctx, 64);
  S->kv_head_stride = (int64_t)(S->cap / 16) * kv_block_elems(M->D);
  S->kv_batch_stride = S->kv_head_stride * M->KVl;
  S->kv_layer_stride = S->kv_batch_stride * batch;
  S->Bp = c.dtype == LMB200_BF16 ? Layout<__nv_bfloat16>::batch_pad(batch) : Layout<float>::batch_pad(batch);
  S->q_pitch = M->Hl * M->D;
  S->logits_pitch = (int)round_up(c.vocab, 16);

  int64_t max_part = 0;
  int max_cnt = 0;
  auto plan = [&](GemvPlan& g, const WMap& m) {
    g = gemv_plan(ctx, c.dtype, batch, m.rows, m.K);
    if (g.partial_floats > max_part) max_part = g.partial_floats;
    if (g.n_counters > max_cnt) max_cnt = g.n_counters;
  };
  plan(S->p_qkv, M->m_qkv); plan(S->p_o, M->m_o); plan(S->p_gu, M->m_gu); plan(S->p_down, M->m_down);
  plan(S->p_head, M->m_head);
  {
    // The fused step (LMB200_FUSED_STEP=0 switches it off for A/B runs): bf16 Llama / Phi-3 / Whisper decoder on the
    // tcgen05 GEMV, every row group of the two row-parallel projections resident at once, and under tensor
    // parallelism the peer regions mapped and large enough for n bf16 partials of [hidden][Bp].
    const char* fe = getenv("LMB200_FUSED_STEP");
    bool fused = !(fe && atoi(fe) == 0) && c.dtype == LMB200_BF16 && gemv_variant() == GEMV_TCGEN05 && c.hidden % 8 == 0 &&
                 ceil_div(c.hidden, 32 * ceil_div(c.hidden, 32 * 256)) <= 256;
    if (fused && c.tp_size > 1 && !M->tp_solo)
      fused = ctx->peer_n == c.tp_size && (int64_t)c.tp_size * c.hidden * S->Bp * 2 <= kPeerBufFloats * 4 &&
              (unsigned long long)2 * c.n_layers + 1 < kPeerEpochStride;
    if (fused) {
      const GemvPlan po = gemv_plan_resid(ctx, batch, M->m_o.rows, M->m_o.K), pd = gemv_plan_resid(ctx, batch, M->m_down.rows, M->m_down.K);
      if (po.cluster >= 1 && pd.cluster >= 1) { S->p_o = po; S->p_down = pd; }
      else fused = false;
    }
    S->fused = fused;
    S->embed_rows_per_cta = 32 * (int)ceil_div(c.hidden, 32 * 256);
    // The head is replicated; under tensor parallelism every rank multiplies only its share of the rows and the ranks
    // exchange their best (logit, id) pairs (LMB200_TP_HEAD=replicated keeps every rank on the whole head, A/B runs).
    const char* he = getenv("LMB200_TP_HEAD");
    if (fused && !whisper && c.tp_size > 1 && !M->tp_solo && ctx->peer_n == c.tp_size && !(he && strcmp(he, "replicated") == 0)) {
      const int n_rg = (int)ceil_div(M->m_head.rows, 128), per = (int)ceil_div(n_rg, c.tp_size);
      const int rg0 = per * c.tp_rank;
      const int rows = (int)std::min<int64_t>((int64_t)per * 128, (int64_t)M->m_head.rows - (int64_t)rg0 * 128);
      if ((int64_t)per * 128 * (c.tp_size - 1) < M->m_head.rows && rows > 0 && (int64_t)batch * c.hidden <= kPeerBufFloats &&
          (unsigned long long)2 * c.n_layers + 2 < kPeerEpochStride) {
        S->head_sliced = true;
        S->head_rg0 = rg0;
        S->head_rows = rows;
        S->head_pitch = per * 128;
        WMap ms = M->m_head;
        ms.rows = rows;
        plan(S->p_head_slice, ms);
      }
    }
  }
  int64_t po, pml;
  attn_plan(ctx, batch, M->KVl, M->G, M->D, S->cap, &S->keys_per_cta, &S->nsplit, &po, &pml);
  if (whisper) {
    plan(S->p_qc, M->m_qc);
    S->cross_cap = (int)round_up(c.cross_len, 64);
    S->cross_head_stride = (int64_t)(S->cross_cap / 16) * kv_block_elems(M->D);
    S->cross_batch_stride = S->cross_head_stride * M->KVl;
    S->cross_layer_stride = S->cross_batch_stride * batch;
    int64_t po2, pml2;
    attn_plan(ctx, batch, M->KVl, M->G, M->D, S->cross_cap, &S->cross_keys_per_cta, &S->cross_nsplit, &po2, &pml2);
    if (po2 > po) po = po2;
    if (pml2 > pml) pml = pml2;
  }

  int32_t rc = LMB200_OK;
  auto alloc = [&](void** p, int64_t bytes) { if (rc == LMB200_OK) rc = dmalloc(p, bytes, true, ctx->stream); };
  alloc(&S->kv, S->kv_layer_stride * c.n_layers * M->esz);
  if (whisper) alloc(&S->cross_kv, S->cross_layer_stride * c.n_layers * M->esz);
  alloc((void**)&S->x, (int64_t)batch * c.hidden * 4);
  alloc((void**)&S->delta, (int64_t)batch * c.hidden * 4);
  alloc((void**)&S->logits, (int64_t)batch * S->logits_pitch * 4);
  // tiled GEMV inputs: [k chunks][Bp][32], zero in the padding rows and columns
  auto x_elems = [&](int K) {
    return c.dtype == LMB200_BF16 ? Layout<__nv_bfloat16>::x_elems(K, S->Bp) : Layout<float>::x_elems(K, S->Bp);
  };
  alloc(&S->xn, x_elems(M->m_qkv.K) * M->esz);
  alloc(&S->qbuf, (int64_t)batch * S->q_pitch * M->esz);
  alloc(&S->attn_out, x_elems(M->m_o.K) * M->esz);
  alloc(&S->act, x_elems(M->m_down.K) * M->esz);
  alloc((void**)&S->tokens, (int64_t)batch * 4);
  alloc((void**)&S->pos, (int64_t)batch * 4);
  alloc((void**)&S->limit, (int64_t)batch * 4);
  alloc((void**)&S->step_ctr, 4);
  alloc((void**)&S->stop, (int64_t)(2 + batch) * 4);
  alloc((void**)&S->tok_hist, (int64_t)(S->cap + 1) * batch * 4);
  alloc((void**)&S->gemv_partials, max_part * 4);
  alloc((void**)&S->gemv_counters, (int64_t)max_cnt * 4);
  alloc((void**)&S->part_o, po * 4);
  alloc((void**)&S->part_ml, pml * 4);
  alloc((void**)&S->attn_counters, (int64_t)S->B * M->KVl * 4);
  if (S->fused) {
    alloc((void**)&S->xT, (int64_t)round_up(c.hidden, 128) * S->Bp * 4);
    alloc((void**)&S->ssq, (int64_t)256 * 32 * 4);
    if (whisper) alloc((void**)&S->sum_slots, (int64_t)256 * 32 * 4);
  }
  if (S->head_sliced) alloc((void**)&S->logits_slice, (int64_t)batch * S->head_pitch * 4);
  S->host_pos_v.assign(batch, 0);
  if (rc == LMB200_OK) rc = set_limits(S, nullptr);
  if (rc == LMB200_OK) {
    const int no_eot = -1;                                  // end-of-text stop disabled until lmb200_decode_until sets it
    if (cudaMemcpyAsync(S->stop, &no_eot, 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) rc = fail(LMB200_ECUDA, "session_create: copy failed");
  }
  if (rc == LMB200_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = fail(LMB200_ECUDA, "session_create: sync failed");
  if (rc != LMB200_OK) { lmb200_session_destroy(reinterpret_cast<lmb200_session>(S)); return rc; }
  *out = reinterpret_cast<lmb200_session>(S);
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_destroy(lmb200_session h) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_destroy(S);
  cudaSetDevice(S->m->ctx->device);
  cudaStreamSynchronize(S->m->ctx->stream);
  drop_graphs(S);
  cudaFree(S->cross_kv);
  cudaFree(S->kv); cudaFree(S->x); cudaFree(S->delta); cudaFree(S->logits); cudaFree(S->xn); cudaFree(S->qbuf);
  cudaFree(S->attn_out); cudaFree(S->act); cudaFree(S->tokens); cudaFree(S->pos); cudaFree(S->limit); cudaFree(S->step_ctr); cudaFree(S->ragged_logits);
  cudaFree(S->tok_hist); cudaFree(S->prompt); cudaFree(S->gemv_partials); cudaFree(S->gemv_counters);
  cudaFree(S->part_o); cudaFree(S->part_ml); cudaFree(S->attn_counters); cudaFree(S->prefill_buf); cudaFree(S->capture);
  cudaFree(S->xT); cudaFree(S->ssq); cudaFree(S->sum_slots); cudaFree(S->logits_slice); cudaFree(S->stop);
  S->magic = 0;
  delete S;
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_reset(lmb200_session h) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_reset(S);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  return set_all_positions(S, 0);
}

extern "C" int32_t lmb200_session_position(lmb200_session h, int32_t* pos) {
  Session* S = session_from(h);
  if (!S || !pos) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_position(S, pos);
  *pos = S->host_pos;
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_set_position(lmb200_session h, int32_t pos) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(pos >= 0 && pos <= S->max_ctx, "set_position: %d outside 0..%d", pos, S->max_ctx);
  if (!S->parts.empty()) return wide_set_position(S, pos);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  return set_all_positions(S, pos);
}

extern "C" int32_t lmb200_session_set_positions(lmb200_session h, const int32_t* pos) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(pos, "set_positions: null argument");
  if (!S->parts.empty()) return wide_set_positions(S, pos);
  for (int b = 0; b < S->B; ++b)
    LMB_REQUIRE(pos[b] >= 0 && pos[b] <= S->max_ctx, "set_positions: sequence %d at %d, outside 0..%d", b, pos[b], S->max_ctx);
  LMB_CUDA(cudaSetDevice(S->m->ctx->device));
  S->host_pos_v.assign(pos, pos + S->B);
  return push_positions(S);
}

extern "C" int32_t lmb200_session_positions(lmb200_session h, int32_t* pos_out) {
  Session* S = session_from(h);
  if (!S || !pos_out) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_positions(S, pos_out);
  for (int b = 0; b < S->B; ++b) pos_out[b] = S->host_pos_v[b];
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_set_cross_kv(lmb200_session h, int32_t layer, const float* k_host, const float* v_host,
                                               int32_t layout) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  Model* M = S->m;
  const lmb200_model_config& c = M->cfg;
  LMB_REQUIRE(c.arch == LMB200_ARCH_WHISPER_DECODER && S->cross_kv, "set_cross_kv: not a Whisper decoder session");
  LMB_REQUIRE(k_host && v_host, "set_cross_kv: null pointer");
  LMB_REQUIRE(layer >= 0 && layer < c.n_layers, "set_cross_kv: layer %d", layer);
  LMB_REQUIRE(layout == LMB200_ROWMAJOR || layout == LMB200_COLMAJOR, "set_cross_kv: layout %d", layout);
  Ctx* ctx = M->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const int64_t n = (int64_t)S->B * M->KVl * c.cross_len * M->D;
  float *ks = nullptr, *vs = nullptr;
  LMB_TRY(dmalloc((void**)&ks, n * 4, false, ctx->stream));
  int32_t rc = dmalloc((void**)&vs, n * 4, false, ctx->stream);
  if (rc == LMB200_OK) {
    cudaMemcpyAsync(ks, k_host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream);
    cudaMemcpyAsync(vs, v_host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream);
    void* dst = reinterpret_cast<char*>(S->cross_kv) + (int64_t)layer * S->cross_layer_stride * M->esz;
    if (c.dtype == LMB200_BF16)
      scatter_kv_kernel<__nv_bfloat16><<<fill_grid(n), 256, 0, ctx->stream>>>(
          reinterpret_cast<__nv_bfloat16*>(dst), S->cross_batch_stride, S->cross_head_stride, S->B, M->KVl, c.cross_len,
          M->D, ks, vs, layout);
    else
      scatter_kv_kernel<float><<<fill_grid(n), 256, 0, ctx->stream>>>(reinterpret_cast<float*>(dst), S->cross_batch_stride,
                                                                      S->cross_head_stride, S->B, M->KVl, c.cross_len,
                                                                      M->D, ks, vs, layout);
    ctx->launches++;
    if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(ctx->stream) != cudaSuccess)
      rc = fail(LMB200_ECUDA, "set_cross_kv: upload failed");
  }
  cudaStreamSynchronize(ctx->stream);
  cudaFree(ks); cudaFree(vs);
  return rc;
}

extern "C" int32_t lmb200_session_fill_kv_random(lmb200_session h, int32_t n_pos, uint64_t seed) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_fill_kv_random(S, n_pos, seed);
  Model* M = S->m;
  Ctx* ctx = M->ctx;
  LMB_REQUIRE(n_pos >= 0 && n_pos <= S->max_ctx, "fill_kv_random: n_pos %d outside 0..%d", n_pos, S->max_ctx);
  LMB_CUDA(cudaSetDevice(ctx->device));
  if (n_pos > 0) {
    for (int l = 0; l < M->cfg.n_layers; ++l) {
      const uint64_t kk = stream_key(seed, kIdKvBase + 2 * l), kvv = stream_key(seed, kIdKvBase + 2 * l + 1);
      const int64_t total = (int64_t)S->B * M->KVl * n_pos * M->D;
      void* layer = reinterpret_cast<char*>(S->kv) + (int64_t)l * S->kv_layer_stride * M->esz;
      if (M->cfg.dtype == LMB200_BF16)
        fill_kv_kernel<__nv_bfloat16><<<fill_grid(total), 256, 0, ctx->stream>>>(
            reinterpret_cast<__nv_bfloat16*>(layer), S->kv_batch_stride, S->kv_head_stride, S->B, M->KVl,
            M->cfg.n_kv_heads, M->kv_off, M->D, n_pos, S->max_ctx, kk, kvv);
      else
        fill_kv_kernel<float><<<fill_grid(total), 256, 0, ctx->stream>>>(
            reinterpret_cast<float*>(layer), S->kv_batch_stride, S->kv_head_stride, S->B, M->KVl,
            M->cfg.n_kv_heads, M->kv_off, M->D, n_pos, S->max_ctx, kk, kvv);
      ctx->launches++;
      LMB_CUDA(cudaGetLastError());
    }
  }
  return set_all_positions(S, n_pos);
}

extern "C" int32_t lmb200_session_set_capture(lmb200_session h, int32_t enable) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_set_capture(S, enable);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  if (enable && !S->capture)
    LMB_TRY(dmalloc((void**)&S->capture, (int64_t)S->m->cfg.n_layers * S->B * S->m->cfg.hidden * 4, true, ctx->stream));
  if ((enable != 0) != S->capture_on) {
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    drop_graphs(S);
    S->capture_on = enable != 0;
  }
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_read_layer_output(lmb200_session h, int32_t layer, float* host) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_read_layer_output(S, layer, host);
  LMB_REQUIRE(S->capture && host, "read_layer_output: capture is not enabled");
  LMB_REQUIRE(layer >= 0 && layer < S->m->cfg.n_layers, "read_layer_output: layer %d", layer);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const int64_t n = (int64_t)S->B * S->m->cfg.hidden;
  LMB_CUDA(cudaMemcpyAsync(host, S->capture + layer * n, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return LMB200_OK;
}

// Tensor-parallel work is refused while the communicator is marked broken (a rank's wait ran out):
// the ranks' counters differ, and a further step would either time out again or sum stale partials.
static int32_t tp_guard(const Session* S, const char* what) {
  const Ctx* ctx = S->m->ctx;
  if (S->m->cfg.tp_size > 1 && !S->m->tp_solo && ctx->comm_broken)
    return fail(LMB200_ESTATE, "%s: a tensor-parallel step failed earlier and the ranks are out of step; every rank must call "
                               "lmb200_comm_resync (and put the session positions back) first", what);
  return LMB200_OK;
}

static int32_t copy_logits_out(Session* S, float* logits_out) {
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaMemcpy2DAsync(logits_out, (size_t)S->m->cfg.vocab * 4, S->logits, (size_t)S->logits_pitch * 4,
                             (size_t)S->m->cfg.vocab * 4, S->B, cudaMemcpyDeviceToHost, ctx->stream));
  return LMB200_OK;
}

extern "C" int32_t lmb200_prefill(lmb200_session h, const int32_t* tokens, int32_t n, float* logits_out) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(tokens && n >= 1, "prefill: null tokens or n < 1");
  if (!S->parts.empty()) return wide_prefill(S, tokens, n, logits_out);
  LMB_REQUIRE(!S->ragged, "prefill: the sequences are at different positions; use lmb200_prefill_ragged");
  LMB_TRY(tp_guard(S, "prefill"));
  if (S->host_pos + n > S->max_ctx)
    return fail(LMB200_ESTATE, "prefill: %d + %d tokens exceed max_ctx %d", S->host_pos, n, S->max_ctx);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const int B = S->B;
  if ((int64_t)n * B > S->prompt_cap) {
    cudaFree(S->prompt);
    S->prompt = nullptr;
    S->prompt_cap = 0;
    LMB_TRY(dmalloc((void**)&S->prompt, (int64_t)n * B * 4, false, ctx->stream));
    S->prompt_cap = (int64_t)n * B;
  }
  if (prefill_gemm_ok(S, n)) {
    // every position at once: GEMMs + flash attention, then the head on the last position
    LMB_CUDA(cudaMemcpyAsync(S->prompt, tokens, (size_t)n * B * 4, cudaMemcpyHostToDevice, ctx->stream));
    LMB_TRY(prefill_gemm(S, S->prompt, n, nullptr, ctx->stream));
    LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
    LMB_TRY(enqueue_head_bf16(S, ctx->stream));
    LMB_TRY(set_all_positions(S, S->host_pos + n));
    if (logits_out) LMB_TRY(copy_logits_out(S, logits_out));
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    return check_device_error(ctx);
  }
  std::vector<int32_t> tr((size_t)n * B);       // [n][B]
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < n; ++i) tr[(size_t)i * B + b] = tokens[(size_t)b * n + i];
  LMB_CUDA(cudaMemcpyAsync(S->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  for (int i = 0; i < n; ++i) {
    LMB_CUDA(cudaMemcpyAsync(S->tokens, S->prompt + (int64_t)i * B, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    LMB_TRY(run_step(S, i == n - 1, logits_out != nullptr));
  }
  if (logits_out) LMB_TRY(copy_logits_out(S, logits_out));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return check_device_error(ctx);
}

// Prompts of different lengths in one batch (the reference's [batch, seq] token tensor, src/NN.jl:448-455, has one
// length; a batch of real prompts does not).  tokens: [batch, n_max] row-major, sequence b uses its first lengths[b]
// ids.  logits_out (NULL or [batch, vocab]): for every sequence the logits of ITS last prompt position.  Afterwards
// sequence b stands at its old position + lengths[b] and decoding goes on with one position per sequence.
// A fresh bf16 Llama / Phi-3 session runs all positions at once through the prompt GEMMs (the padding behind a short
// prompt is computed and never read: attention is causal and later steps overwrite those cache slots); otherwise
// the prompt goes through the decode step, a finished sequence standing still while the longer ones go on.
extern "C" int32_t lmb200_prefill_ragged(lmb200_session h, const int32_t* tokens, const int32_t* lengths, int32_t n_max,
                                         float* logits_out) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(tokens && lengths && n_max >= 1, "prefill_ragged: null argument or n_max < 1");
  if (!S->parts.empty()) return wide_prefill_ragged(S, tokens, lengths, n_max, logits_out);
  LMB_TRY(tp_guard(S, "prefill_ragged"));
  const int B = S->B;
  int longest = 0;
  for (int b = 0; b < B; ++b) {
    LMB_REQUIRE(lengths[b] >= 1 && lengths[b] <= n_max, "prefill_ragged: sequence %d has length %d, outside 1..%d", b, lengths[b], n_max);
    if (S->host_pos_v[b] + lengths[b] > S->max_ctx)
      return fail(LMB200_ESTATE, "prefill_ragged: sequence %d: %d + %d tokens exceed max_ctx %d", b, S->host_pos_v[b], lengths[b], S->max_ctx);
    if (lengths[b] > longest) longest = lengths[b];
  }
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  if ((int64_t)longest * B > S->prompt_cap) {
    cudaFree(S->prompt);
    S->prompt = nullptr;
    S->prompt_cap = 0;
    LMB_TRY(dmalloc((void**)&S->prompt, (int64_t)longest * B * 4, false, ctx->stream));
    S->prompt_cap = (int64_t)longest * B;
  }
  std::vector<int> new_pos(B), limits(B);
  for (int b = 0; b < B; ++b) new_pos[b] = limits[b] = S->host_pos_v[b] + lengths[b];
  if (!S->ragged && prefill_gemm_ok(S, longest)) {
    std::vector<int32_t> tk((size_t)longest * B, 0);            // [B, longest]
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < lengths[b]; ++i) tk[(size_t)b * longest + i] = tokens[(size_t)b * n_max + i];
    int* lens_dev = nullptr;
    LMB_TRY(dmalloc((void**)&lens_dev, (int64_t)B * 4, false, ctx->stream));
    int32_t rc = LMB200_OK;
    if (cudaMemcpyAsync(S->prompt, tk.data(), tk.size() * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(lens_dev, lengths, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
      rc = fail(LMB200_ECUDA, "prefill_ragged: upload failed");
    if (rc == LMB200_OK) rc = prefill_gemm(S, S->prompt, longest, lens_dev, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(lens_dev);
    LMB_TRY(rc);
    LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
    LMB_TRY(enqueue_head_bf16(S, ctx->stream));
    S->host_pos_v = new_pos;
    LMB_TRY(push_positions(S));
    if (logits_out) LMB_TRY(copy_logits_out(S, logits_out));
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    return check_device_error(ctx);
  }
  // step by step: position-major token staging, the per-sequence limits stop a finished sequence
  std::vector<int32_t> tr((size_t)longest * B, 0);              // [longest][B]
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < lengths[b]; ++i) tr[(size_t)i * B + b] = tokens[(size_t)b * n_max + i];
  LMB_CUDA(cudaMemcpyAsync(S->prompt, tr.data(), tr.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  if (logits_out && !S->ragged_logits)
    LMB_TRY(dmalloc((void**)&S->ragged_logits, (int64_t)B * S->logits_pitch * 4, true, ctx->stream));
  if (!S->ragged) {                                             // the steps below run with one position per sequence
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
    drop_graphs(S);
    S->ragged = true;
  }
  LMB_TRY(set_limits(S, limits.data()));
  S->in_ragged_prefill = true;
  int32_t rc = LMB200_OK;
  for (int i = 0; i < longest && rc == LMB200_OK; ++i) {
    bool ends_here = false;
    for (int b = 0; b < B; ++b) ends_here = ends_here || lengths[b] - 1 == i;
    if (cudaMemcpyAsync(S->tokens, S->prompt + (int64_t)i * B, (size_t)B * 4, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "prefill_ragged: token copy failed");
      break;
    }
    rc = run_step(S, ends_here, logits_out != nullptr);
    if (rc == LMB200_OK && ends_here && logits_out) {
      for (int b = 0; b < B; ++b)
        if (lengths[b] - 1 == i &&
            cudaMemcpyAsync(S->ragged_logits + (int64_t)b * S->logits_pitch, S->logits + (int64_t)b * S->logits_pitch,
                            (size_t)S->m->cfg.vocab * 4, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess)
          rc = fail(LMB200_ECUDA, "prefill_ragged: logits copy failed");
    }
  }
  S->in_ragged_prefill = false;
  cudaStreamSynchronize(ctx->stream);
  const int32_t rc2 = set_limits(S, nullptr);
  LMB_TRY(rc);
  LMB_TRY(rc2);
  S->host_pos_v = new_pos;
  LMB_TRY(push_positions(S));
  if (logits_out) {
    LMB_CUDA(cudaMemcpy2DAsync(logits_out, (size_t)S->m->cfg.vocab * 4, S->ragged_logits, (size_t)S->logits_pitch * 4,
                               (size_t)S->m->cfg.vocab * 4, B, cudaMemcpyDeviceToHost, ctx->stream));
    LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return check_device_error(ctx);
}

extern "C" int32_t lmb200_decode_step(lmb200_session h, const int32_t* tokens_in, int32_t* next_tokens_out,
                                      float* logits_out) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(tokens_in, "decode_step: null tokens");
  if (!S->parts.empty()) return wide_decode_step(S, tokens_in, next_tokens_out, logits_out);
  LMB_TRY(tp_guard(S, "decode_step"));
  if (S->host_pos + 1 > S->max_ctx)
    return fail(LMB200_ESTATE, "decode_step: position %d is past max_ctx %d", S->host_pos, S->max_ctx);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  LMB_CUDA(cudaMemcpyAsync(S->tokens, tokens_in, (size_t)S->B * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  LMB_TRY(run_step(S, true, logits_out != nullptr));
  if (next_tokens_out)
    LMB_CUDA(cudaMemcpyAsync(next_tokens_out, S->tokens, (size_t)S->B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  if (logits_out) LMB_TRY(copy_logits_out(S, logits_out));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return check_device_error(ctx);
}

static int32_t decode_n_common(Session* S, const int32_t* first, bool first_on_device, int32_t n_steps) {
  LMB_REQUIRE(n_steps >= 1, "decode_n: n_steps %d", n_steps);
  LMB_TRY(tp_guard(S, "decode_n"));
  if (S->host_pos + n_steps > S->max_ctx)
    return fail(LMB200_ESTATE, "decode_n: %d + %d steps exceed max_ctx %d", S->host_pos, n_steps, S->max_ctx);
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  if (first)
    LMB_CUDA(cudaMemcpyAsync(S->tokens, first, (size_t)S->B * 4,
                             first_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  for (int i = 0; i < n_steps; ++i) LMB_TRY(run_step(S, true, false));
  return LMB200_OK;
}

extern "C" int32_t lmb200_decode_n(lmb200_session h, const int32_t* first_tokens, int32_t n_steps, int32_t* tokens_out) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_decode_n(S, first_tokens, n_steps, tokens_out);
  LMB_TRY(decode_n_common(S, first_tokens, false, n_steps));
  Ctx* ctx = S->m->ctx;
  if (tokens_out)
    LMB_CUDA(cudaMemcpyAsync(tokens_out, S->tok_hist, (size_t)n_steps * S->B * 4, cudaMemcpyDeviceToHost, ctx->stream));
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return check_device_error(ctx);
}

// Greedy steps until every sequence has produced `eot_token` or max_steps (capped by the session's context) have
// run: the generation loop of src/Decoding.jl:91-130 with its two exits (EOT :126-129, the position cap :93-95).
// The steps are CUDA-graph replays issued in short runs; after each run the host reads how many sequences are
// done.  A finished sequence keeps emitting eot_token.  tokens_out: [max_steps, batch], filled for *steps_done rows.
extern "C" int32_t lmb200_decode_until(lmb200_session h, const int32_t* first_tokens, int32_t max_steps, int32_t eot_token,
                                       int32_t* tokens_out, int32_t* steps_done) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(steps_done && max_steps >= 1, "decode_until: bad argument");
  if (!S->parts.empty()) return wide_decode_until(S, first_tokens, max_steps, eot_token, tokens_out, steps_done);
  LMB_REQUIRE(eot_token >= 0 && eot_token < S->m->cfg.vocab, "decode_until: end-of-text id %d outside the vocabulary", eot_token);
  LMB_TRY(tp_guard(S, "decode_until"));
  Ctx* ctx = S->m->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const int B = S->B;
  int budget = S->max_ctx - S->host_pos;                 // the position cap
  if (budget > max_steps) budget = max_steps;
  *steps_done = 0;
  if (budget <= 0) return fail(LMB200_ESTATE, "decode_until: position %d is at max_ctx %d", S->host_pos, S->max_ctx);
  std::vector<int> init(2 + B, 0);
  init[0] = eot_token;
  LMB_CUDA(cudaMemcpyAsync(S->stop, init.data(), init.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
  if (first_tokens) LMB_CUDA(cudaMemcpyAsync(S->tokens, first_tokens, (size_t)B * 4, cudaMemcpyHostToDevice, ctx->stream));
  LMB_CUDA(cudaMemsetAsync(S->step_ctr, 0, 4, ctx->stream));
  int32_t rc = LMB200_OK;
  int done = 0;
  const int kRun = 8;                                     // replays between two looks at the count
  while (done < budget && rc == LMB200_OK) {
    const int n = budget - done < kRun ? budget - done : kRun;
    for (int i = 0; i < n && rc == LMB200_OK; ++i) rc = run_step(S, true, false);
    if (rc != LMB200_OK) break;
    done += n;
    int finished = 0;
    if (cudaMemcpyAsync(&finished, S->stop + 1, 4, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess) { rc = fail(LMB200_ECUDA, "decode_until: readback failed"); break; }
    if (finished >= B) break;
  }
  // the rows past the step in which the last sequence finished hold only end-of-text ids: trim them
  std::vector<int32_t> hist((size_t)done * B);
  if (rc == LMB200_OK && done > 0) {
    if (cudaMemcpyAsync(hist.data(), S->tok_hist, hist.size() * 4, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = fail(LMB200_ECUDA, "decode_until: readback failed");
  }
  const int no_eot = -1;
  cudaMemcpyAsync(S->stop, &no_eot, 4, cudaMemcpyHostToDevice, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  if (rc != LMB200_OK) return rc;
  int keep = done;
  while (keep > 1) {
    bool all_eot = true;
    for (int b = 0; b < B && all_eot; ++b) all_eot = hist[(size_t)(keep - 1) * B + b] == eot_token && hist[(size_t)(keep - 2) * B + b] == eot_token;
    if (!all_eot) break;
    --keep;
  }
  if (keep < done) {                                      // the session goes back to the step after the last useful one
    for (int& v : S->host_pos_v) v -= done - keep;
    LMB_TRY(push_positions(S));
  }
  if (tokens_out) memcpy(tokens_out, hist.data(), (size_t)keep * B * 4);
  *steps_done = keep;
  return check_device_error(ctx);
}

extern "C" int32_t lmb200_decode_n_device(lmb200_session h, const int32_t* first_dptr, int32_t n_steps, int32_t* out_dptr) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(S->parts.empty(), "decode_n_device: not built for a session of more than 32 sequences");
  LMB_TRY(decode_n_common(S, first_dptr, true, n_steps));
  Ctx* ctx = S->m->ctx;
  if (out_dptr)
    LMB_CUDA(cudaMemcpyAsync(out_dptr, S->tok_hist, (size_t)n_steps * S->B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  return LMB200_OK;
}

extern "C" int32_t lmb200_session_step_bytes(lmb200_session h, int32_t T, int64_t* bytes) {
  Session* S = session_from(h);
  if (!S || !bytes) return LMB200_EINVAL;
  if (!S->parts.empty()) return wide_step_bytes(S, T, bytes);
  Model* M = S->m;
  const lmb200_model_config& c = M->cfg;
  const int64_t e = M->esz;
  int64_t per_layer = ((int64_t)M->m_qkv.rows * c.hidden + (int64_t)c.hidden * M->Hl * M->D +
                       (int64_t)2 * M->inter_l * c.hidden + (int64_t)c.hidden * M->inter_l) * e +
                      (int64_t)2 * c.hidden * 4;
  // the head: every row, or under tensor parallelism this rank's slice of the rows (the token-only step)
  const int64_t head_rows = S->head_sliced ? S->head_rows : c.vocab;
  int64_t w = per_layer * c.n_layers + head_rows * c.hidden * e + (int64_t)c.hidden * 4 +
              (int64_t)S->B * c.hidden * e;
  int64_t kv_read = (int64_t)c.n_layers * S->B * M->KVl * T * M->D * 2 * e;
  int64_t kv_write = (int64_t)c.n_layers * S->B * M->KVl * M->D * 2 * e;
  *bytes = w + kv_read + kv_write;
  return LMB200_OK;
}

// ---------------------------------------------------------------------------------------------
// stand-alone Linear for one batch of rows (tests, A/B of the GEMV kernels)
// ---------------------------------------------------------------------------------------------
namespace lmb {
namespace {
template <typename WT>
__global__ void fill_x_kernel(WT* dst, const float* src, int B, int K, int Bp) {
  const int64_t total = (int64_t)B * K;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int b = (int)(o / K), k = (int)(o - (int64_t)b * K);
    dst[Layout<WT>::x_offset(b, k, Bp)] = from_f32<WT>(src[o]);
  }
}
}  // namespace
}  // namespace lmb

extern "C" int32_t lmb200_linear_gemv(lmb200_ctx hctx, int32_t dtype, int32_t variant, int32_t rows, int32_t K,
                                      int32_t batch, const float* w_host, const float* x_host, float* out_host) {
  Ctx* ctx = ctx_from(hctx);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(w_host && x_host && out_host, "linear_gemv: null pointer");
  LMB_REQUIRE(dtype == LMB200_F32 || dtype == LMB200_BF16, "linear_gemv: dtype %d", dtype);
  LMB_REQUIRE(rows >= 1 && K >= 1 && batch >= 1 && batch <= 32, "linear_gemv: rows %d, K %d, batch %d", rows, K, batch);
  LMB_CUDA(cudaSetDevice(ctx->device));
  const bool bf = dtype == LMB200_BF16;
  const int esz = bf ? 2 : 4;
  const int Bp = bf ? Layout<__nv_bfloat16>::batch_pad(batch) : Layout<float>::batch_pad(batch);
  WMap m;
  m.kind = MAP_PLAIN; m.rows = rows; m.K = K; m.src_rows[0] = rows; m.src_cols[0] = K;
  finish_map(m);
  const int saved = gemv_variant();
  if (bf) gemv_set_variant(variant);
  const GemvPlan pl = gemv_plan(ctx, dtype, batch, rows, K);
  void *W = nullptr, *X = nullptr;
  float *ws = nullptr, *xs = nullptr, *out = nullptr, *partials = nullptr;
  unsigned* counters = nullptr;
  int32_t rc = LMB200_OK;
  auto alloc = [&](void** p, int64_t bytes) { if (rc == LMB200_OK) rc = dmalloc(p, bytes, true, ctx->stream); };
  alloc(&W, tiled_elems(m, dtype) * esz);
  alloc(&X, (bf ? Layout<__nv_bfloat16>::x_elems(K, Bp) : Layout<float>::x_elems(K, Bp)) * esz);
  alloc((void**)&ws, (int64_t)rows * K * 4);
  alloc((void**)&xs, (int64_t)batch * K * 4);
  alloc((void**)&out, (int64_t)batch * rows * 4);
  alloc((void**)&partials, pl.partial_floats * 4);
  alloc((void**)&counters, (int64_t)pl.n_counters * 4);
  do {
    if (rc != LMB200_OK) break;
    if (cudaMemcpyAsync(ws, w_host, (size_t)rows * K * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(xs, x_host, (size_t)batch * K * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "linear_gemv: upload failed"); break;
    }
    FillSrc f{};
    f.only_slot = -1; f.src[0] = ws;
    Model tmp; tmp.ctx = ctx; tmp.cfg.dtype = dtype;
    rc = fill_tiled_dt(&tmp, W, m, f);
    if (rc != LMB200_OK) break;
    if (bf) fill_x_kernel<__nv_bfloat16><<<fill_grid((int64_t)batch * K), 256, 0, ctx->stream>>>((__nv_bfloat16*)X, xs, batch, K, Bp);
    else fill_x_kernel<float><<<fill_grid((int64_t)batch * K), 256, 0, ctx->stream>>>((float*)X, xs, batch, K, Bp);
    ctx->launches++;
    GemvParams p;
    p.W = W; p.x = X; p.B = batch; p.rows = rows; p.K = K; p.RB = m.RB; p.KC = m.KC;
    p.ksplit = pl.ksplit; p.kc_per_split = pl.kc_per_split; p.grid = pl.grid; p.cluster = pl.cluster;
    p.partials = partials; p.counters = counters;
    p.epi = EPI_STORE_F32; p.out = out; p.out_pitch = rows;
    rc = gemv_launch(ctx, dtype, p, ctx->stream);
    if (rc != LMB200_OK) break;
    if (cudaMemcpyAsync(out_host, out, (size_t)batch * rows * 4, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "linear_gemv: download failed"); break;
    }
  } while (0);
  cudaError_t se = cudaStreamSynchronize(ctx->stream);
  if (rc == LMB200_OK && se != cudaSuccess) rc = fail(LMB200_ECUDA, "linear_gemv: %s", cudaGetErrorString(se));
  if (rc == LMB200_OK) rc = check_device_error(ctx);
  cudaFree(W); cudaFree(X); cudaFree(ws); cudaFree(xs); cudaFree(out); cudaFree(partials); cudaFree(counters);
  gemv_set_variant(saved);
  return rc;
}

extern "C" int32_t lmb200_prefill_gemm(lmb200_ctx hctx, int32_t rows, int32_t K, int32_t n_tokens, const float* w_host,
                                       const float* x_host, float* out_host) {
  Ctx* ctx = ctx_from(hctx);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(w_host && x_host && out_host, "prefill_gemm: null pointer");
  LMB_REQUIRE(rows >= 1 && K >= 8 && K % 8 == 0 && n_tokens >= 1, "prefill_gemm: rows %d, K %d, tokens %d", rows, K, n_tokens);
  LMB_CUDA(cudaSetDevice(ctx->device));
  WMap m;
  m.kind = MAP_PLAIN; m.rows = rows; m.K = K; m.src_rows[0] = rows; m.src_cols[0] = K;
  finish_map(m);
  void* W = nullptr;
  float *ws = nullptr, *xs = nullptr, *out = nullptr;
  int32_t rc = LMB200_OK;
  auto alloc = [&](void** p, int64_t bytes) { if (rc == LMB200_OK) rc = dmalloc(p, bytes, true, ctx->stream); };
  alloc(&W, tiled_elems(m, LMB200_BF16) * 2);
  alloc((void**)&ws, (int64_t)rows * K * 4);
  alloc((void**)&xs, (int64_t)n_tokens * K * 4);
  alloc((void**)&out, (int64_t)n_tokens * rows * 4);
  do {
    if (rc != LMB200_OK) break;
    if (cudaMemcpyAsync(ws, w_host, (size_t)rows * K * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(xs, x_host, (size_t)n_tokens * K * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "prefill_gemm: upload failed"); break;
    }
    FillSrc f{};
    f.only_slot = -1; f.src[0] = ws;
    Model tmp; tmp.ctx = ctx; tmp.cfg.dtype = LMB200_BF16;
    rc = fill_tiled_dt(&tmp, W, m, f);
    if (rc != LMB200_OK) break;
    rc = prefill_linear(ctx, W, xs, n_tokens, rows, K, out, ctx->stream);
    if (rc != LMB200_OK) break;
    if (cudaMemcpyAsync(out_host, out, (size_t)n_tokens * rows * 4, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) {
      rc = fail(LMB200_ECUDA, "prefill_gemm: download failed"); break;
    }
  } while (0);
  cudaError_t se = cudaStreamSynchronize(ctx->stream);
  if (rc == LMB200_OK && se != cudaSuccess) rc = fail(LMB200_ECUDA, "prefill_gemm: %s", cudaGetErrorString(se));
  if (rc == LMB200_OK) rc = check_device_error(ctx);
  cudaFree(W); cudaFree(ws); cudaFree(xs); cudaFree(out);
  return rc;
}

extern "C" int32_t lmb200_session_kv_layer(lmb200_session h, int32_t layer, void** kv_dptr, int64_t* batch_stride,
                                           int64_t* head_stride) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  LMB_REQUIRE(kv_dptr && batch_stride && head_stride, "session_kv_layer: null argument");
  LMB_REQUIRE(S->parts.empty(), "session_kv_layer: a session of more than 32 sequences has one cache per 32 sequences");
  LMB_REQUIRE(layer >= 0 && layer < S->m->cfg.n_layers, "session_kv_layer: layer %d", layer);
  *kv_dptr = reinterpret_cast<char*>(S->kv) + (int64_t)layer * S->kv_layer_stride * S->m->esz;
  *batch_stride = S->kv_batch_stride;
  *head_stride = S->kv_head_stride;
  return LMB200_OK;
}

extern "C" int32_t lmb200_decode_attention_splitkv(lmb200_session h, int32_t layer, const void* q_dptr,
                                                   void* out_dptr, int32_t T) {
  Session* S = session_from(h);
  if (!S) return LMB200_EINVAL;
  Model* M = S->m;
  LMB_REQUIRE(q_dptr && out_dptr, "decode_attention: null pointer");
  LMB_REQUIRE(S->parts.empty(), "decode_attention: not built for a session of more than 32 sequences");
  LMB_REQUIRE(layer >= 0 && layer < M->cfg.n_layers, "decode_attention: layer %d", layer);
  LMB_REQUIRE(T >= 1 && T <= S->max_ctx, "decode_attention: T %d outside 1..%d", T, S->max_ctx);
  Ctx* ctx = M->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  AttnParams a;
  a.q = q_dptr; a.q_pitch = M->Hl * M->D;
  a.kv_layer = reinterpret_cast<char*>(S->kv) + (int64_t)layer * S->kv_layer_stride * M->esz;
  a.kv_batch_stride = S->kv_batch_stride; a.kv_head_stride = S->kv_head_stride;
  a.B = S->B; a.KVl = M->KVl; a.G = M->G; a.D = M->D; a.pos = nullptr; a.T_fixed = T;
  a.keys_per_cta = S->keys_per_cta; a.nsplit = S->nsplit;
  a.scale = 1.0f / sqrtf((float)M->D);
  a.part_o = S->part_o; a.part_ml = S->part_ml; a.out = out_dptr; a.out_pitch = M->Hl * M->D;
  a.counters = S->attn_counters;
  LMB_TRY(attn_decode_launch(ctx, M->cfg.dtype, a, ctx->stream));
  return LMB200_OK;
}
