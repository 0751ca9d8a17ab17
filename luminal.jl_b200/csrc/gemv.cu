// Bandwidth-bound decode GEMV with fused epilogues (store / SiLU-gate / RoPE + KV append).
//
// bf16 kernels: stream-K over bulk-TMA.  Weights and activations sit in HBM in the tensor-core
// canonical K-major layout (common.cuh), cut into units of 128 rows x 128 k = one contiguous
// 32 KB block; the grid is one CTA per SM and CTA c takes the contiguous unit range
// [c*U/G, (c+1)*U/G), so every SM streams the same number of bytes in a single wave whatever the
// matrix shape.  A producer warp keeps a ring of 5 shared-memory stages full with cp.async.bulk
// copies (one 32 KB copy of weights, evict-first, + the matching activation slice) signalled
// through mbarriers.  One thread issues tcgen05.mma (M = 128 rows, N = batch padding, K = 16)
// straight from the stage through shared-memory descriptors, accumulators double-buffered in
// TMEM; tcgen05.commit hands the stage back to the producer; four epilogue warps read the
// accumulators with tcgen05.ld (one row per thread) and run the fused epilogue while the next
// row group is already being multiplied.
// When a CTA's range leaves a row group its partial result is folded: alone -> epilogue; shared
// -> global scratch + counter, the last contributor sums the parts in CTA order (deterministic).
//
// float32 ("ring") kernel: weights streamed by plain loads through a register ring, fp32 FMAs --
// the parity path.
#include <type_traits>

#include "gemv.cuh"
#include "pdl.cuh"

namespace lmb {

namespace {

constexpr float kInvLn2 = 1.4426950408889634f;      // Float32(1/log(2)) as the reference rounds it
constexpr float kHalfPi = 1.5707963267948966f;
constexpr size_t kMaxSmem = 224 * 1024;

int g_variant = GEMV_TCGEN05;

// gelu(a) = a*0.5*(1 + tanh(0.7978845608*a*(1 + 0.044715*a*a))), tanh(z) = sigmoid(2z)*2 - 1,
// sigmoid through exp2 -- the reference's decomposition, src/HighLevelOps.jl:153-168
__device__ __forceinline__ float gelu_ref(float a) {
  const float inner = (0.7978845608f * a) * (1.0f + (0.044715f * a) * a);
  const float z = inner * 2.0f;
  const float sg = 1.0f / (1.0f + exp2f((z * -1.0f) * kInvLn2));
  const float th = sg * 2.0f + -1.0f;
  return (a * 0.5f) * (1.0f + th);
}

// ---------------------------------------------------------------------------------------------
// Epilogue over a finished tile in shared memory: tile[r * RP + b], r < RPC rows of the CTA's row
// group starting at logical internal row row0.
// ---------------------------------------------------------------------------------------------
template <typename WT>
__device__ __forceinline__ void run_epilogue(const GemvParams& p, const float* tile, int RPC, int RP, int Bp,
                                             int row0, int tid, int nthreads) {
  if (p.epi == EPI_STORE_F32) {
    for (int i = tid; i < RPC * Bp; i += nthreads) {
      const int b = i / RPC, r = i - b * RPC;
      const int row = row0 + r;
      if (b < p.B && row < p.rows)
        p.out[(int64_t)b * p.out_pitch + row] = tile[r * RP + b] + (p.bias ? p.bias[row] : 0.f);
    }
  } else if (p.epi == EPI_GELU_ACT) {
    WT* act = reinterpret_cast<WT*>(p.act);
    for (int i = tid; i < RPC * Bp; i += nthreads) {
      const int b = i / RPC, r = i - b * RPC;
      const int row = row0 + r;
      if (b < p.B && row < p.n_act)
        act[Layout<WT>::x_offset(b, row, Bp)] = from_f32<WT>(gelu_ref(tile[r * RP + b] + (p.bias ? p.bias[row] : 0.f)));
    }
  } else if (p.epi == EPI_SILU_GATE) {
    WT* act = reinterpret_cast<WT*>(p.act);
    for (int i = tid; i < (RPC / 2) * Bp; i += nthreads) {
      const int b = i / (RPC / 2), j = i - b * (RPC / 2);
      const int m = j >> 3, r = j & 7;
      const int o = row0 / 2 + j;
      if (b < p.B && o < p.n_act) {
        const float a = tile[(16 * m + r) * RP + b], u = tile[(16 * m + r + 8) * RP + b];
        // silu(a) = a * (1 / (1 + exp2((a * -1) * (1/ln2))))     src/HighLevelOps.jl:153-160
        const float e = exp2f((a * -1.0f) * kInvLn2);
        const float sg = 1.0f / (1.0f + e);
        act[Layout<WT>::x_offset(b, o, Bp)] = from_f32<WT>((a * sg) * u);
      }
    }
  } else {  // EPI_QKV_ROPE
    WT* q_out = reinterpret_cast<WT*>(p.q_out);
    WT* kv = reinterpret_cast<WT*>(p.kv_layer);
    const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
    for (int i = tid; i < (RPC / 2) * Bp; i += nthreads) {
      const int b = i / (RPC / 2), j = i - b * (RPC / 2);
      const int m = j >> 3, r = j & 7;
      const int gt = row0 / 16 + m;                  // global 16-row tile
      if (b >= p.B || gt >= p.RB) continue;
      const int pos = p.pos[b];                      // every sequence has its own position
      const float fpos = (float)pos;
      const int hs = gt / tiles_per_head, jj = gt - hs * tiles_per_head;
      float v0 = tile[(16 * m + r) * RP + b], v1 = tile[(16 * m + r + 8) * RP + b];
      if (p.bias) { v0 += p.bias[gt * 16 + r]; v1 += p.bias[gt * 16 + r + 8]; }
      if (hs < p.Hl + p.KVl) {
        // rows r / r+8 of the tile are the RoPE pair (d0, d0 + D/2)      src/NN.jl:253-303
        const int d0 = 8 * jj + r;
        float o0, o1;
        if (p.rope) {
          const float ang = fpos * p.inv_freq[d0];
          const float sn = sinf(ang);
          const float cs = sinf(kHalfPi + ang * -1.0f);   // cos(a) = sin(pi/2 - a)
          o0 = v0 * cs + (v1 * sn) * -1.0f;
          o1 = v0 * sn + v1 * cs;
        } else {
          o0 = v0 * p.qk_scale;
          o1 = v1 * p.qk_scale;
        }
        if (hs < p.Hl) {
          WT* q = q_out + (int64_t)b * p.q_pitch + hs * D;
          q[d0] = from_f32<WT>(o0);
          q[d0 + half] = from_f32<WT>(o1);
        } else {
          WT* kc = kv + b * p.kv_batch_stride + (hs - p.Hl) * p.kv_head_stride;
          kc[kcache_offset(pos, d0, D)] = from_f32<WT>(o0);
          kc[kcache_offset(pos, d0 + half, D)] = from_f32<WT>(o1);
        }
      } else {
        WT* vc = kv + b * p.kv_batch_stride + (hs - p.Hl - p.KVl) * p.kv_head_stride;
        const int d = 16 * jj + r;
        vc[vcache_offset(pos, d, D)] = from_f32<WT>(v0);
        vc[vcache_offset(pos, d + 8, D)] = from_f32<WT>(v1);
      }
    }
  }
}

// sum `n` partial tiles (dense [RPC*Bp] each, `stride` floats apart) into tile[r*RP+b]
__device__ __forceinline__ void sum_partials(float* tile, const float* part, int n, int64_t stride, int RPC, int RP,
                                             int Bp, int tid, int nthreads) {
  const int total = RPC * Bp;
  for (int i0 = tid; i0 < total; i0 += nthreads * 4) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < n; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j * nthreads;
        if (i < total) s[j] += __ldcg(part + (int64_t)k * stride + i);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = i0 + j * nthreads;
      if (i < total) { const int r = i / Bp, b = i - r * Bp; tile[r * RP + b] = s[j]; }
    }
  }
}

// =============================================================================================
// ring kernel
// =============================================================================================
constexpr int kRingThreads = 256;

template <typename WT> struct Unit;   // 16 rows x 32 k of weights as seen by one lane
template <> struct Unit<__nv_bfloat16> { uint4 v[2]; };
template <> struct Unit<float> { uint4 v[4]; };

template <typename WT>
__device__ __forceinline__ void load_unit(Unit<WT>& u, const WT* W, int64_t rb, int KC, int kc, int lane) {
  constexpr int N = sizeof(Unit<WT>) / 16;
  const uint4* p = reinterpret_cast<const uint4*>(W + ((rb * KC + kc) * 32 + lane) * 16);
#pragma unroll
  for (int i = 0; i < N; ++i) u.v[i] = __ldcs(p + i);
}
template <typename WT>
__device__ __forceinline__ void zero_unit(Unit<WT>& u) {
  constexpr int N = sizeof(Unit<WT>) / 16;
#pragma unroll
  for (int i = 0; i < N; ++i) u.v[i] = make_uint4(0, 0, 0, 0);
}

template <typename WT, int NB, int MT, int STAGES>
__global__ void __launch_bounds__(kRingThreads, 1) gemv_ring_kernel(const GemvParams p) {
  constexpr int Bp = 8 * NB;
  constexpr int RPC = 2 * MT * 16;
  constexpr bool kBf16 = std::is_same<WT, __nv_bfloat16>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  WT* xs = reinterpret_cast<WT*>(smem_raw);           // [chunks][Bp][32], a copy of the global slice
  float* red = reinterpret_cast<float*>(smem_raw);
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rg = warp >> 2, kw = warp & 3;
  const int kc0 = blockIdx.y * p.kc_per_split;
  const int kc1 = min(p.KC, kc0 + p.kc_per_split);
  const int64_t rb_base = (int64_t)blockIdx.x * (2 * MT) + rg * MT;
  const WT* W = reinterpret_cast<const WT*>(p.W);

  pdl_launch_dependents();
  // prefetch the first weight units before touching the activations
  Unit<WT> ring[STAGES][MT];
#pragma unroll
  for (int s = 0; s < STAGES; ++s) {
    const int kc = kc0 + kw + 4 * s;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (s < STAGES - 1 && kc < kc1 && rb_base + mt < p.RB) load_unit<WT>(ring[s][mt], W, rb_base + mt, p.KC, kc, lane);
      else zero_unit<WT>(ring[s][mt]);
    }
  }
  pdl_wait();      // everything below reads or writes what earlier kernels produced
  {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const WT*>(p.x) + (int64_t)kc0 * Bp * 32);
    uint4* dst = reinterpret_cast<uint4*>(xs);
    const int nvec = (kc1 - kc0) * Bp * 32 * (int)sizeof(WT) / 16;
#pragma unroll 8
    for (int i = tid; i < nvec; i += kRingThreads) dst[i] = src[i];
  }
  __syncthreads();

  float acc[MT][kBf16 ? NB : 2 * Bp][kBf16 ? 4 : 1];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < (kBf16 ? NB : 2 * Bp); ++j)
#pragma unroll
      for (int k = 0; k < (kBf16 ? 4 : 1); ++k) acc[i][j][k] = 0.f;

  for (int base = kc0 + kw; base < kc1; base += 4 * STAGES) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const int cur = base + 4 * s;
      if (cur < kc1) {
        const int nxt = cur + 4 * (STAGES - 1);      // refill the slot freed by the previous iteration
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          if (nxt < kc1 && rb_base + mt < p.RB)
            load_unit<WT>(ring[(s + STAGES - 1) % STAGES][mt], W, rb_base + mt, p.KC, nxt, lane);
        }
        const WT* xc = xs + (cur - kc0) * (Bp * 32) + 8 * t;
        if constexpr (kBf16) {
          uint4 bx[NB];
#pragma unroll
          for (int nt = 0; nt < NB; ++nt) bx[nt] = *reinterpret_cast<const uint4*>(xc + (8 * nt + g) * 32);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint4 lo = ring[s][mt].v[0], hi = ring[s][mt].v[1];
#pragma unroll
            for (int nt = 0; nt < NB; ++nt) {
              mma_bf16(acc[mt][nt], lo.x, hi.x, lo.y, hi.y, bx[nt].x, bx[nt].y);
              mma_bf16(acc[mt][nt], lo.z, hi.z, lo.w, hi.w, bx[nt].z, bx[nt].w);
            }
          }
        } else {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const float4 l0 = *reinterpret_cast<const float4*>(&ring[s][mt].v[0]);
            const float4 l1 = *reinterpret_cast<const float4*>(&ring[s][mt].v[1]);
            const float4 h0 = *reinterpret_cast<const float4*>(&ring[s][mt].v[2]);
            const float4 h1 = *reinterpret_cast<const float4*>(&ring[s][mt].v[3]);
#pragma unroll
            for (int c = 0; c < Bp; ++c) {
              const float4 x0 = *reinterpret_cast<const float4*>(xc + c * 32);
              const float4 x1 = *reinterpret_cast<const float4*>(xc + c * 32 + 4);
              float lo = acc[mt][2 * c][0], hi = acc[mt][2 * c + 1][0];
              lo = fmaf(l0.x, x0.x, lo); lo = fmaf(l0.y, x0.y, lo); lo = fmaf(l0.z, x0.z, lo); lo = fmaf(l0.w, x0.w, lo);
              lo = fmaf(l1.x, x1.x, lo); lo = fmaf(l1.y, x1.y, lo); lo = fmaf(l1.z, x1.z, lo); lo = fmaf(l1.w, x1.w, lo);
              hi = fmaf(h0.x, x0.x, hi); hi = fmaf(h0.y, x0.y, hi); hi = fmaf(h0.z, x0.z, hi); hi = fmaf(h0.w, x0.w, hi);
              hi = fmaf(h1.x, x1.x, hi); hi = fmaf(h1.y, x1.y, hi); hi = fmaf(h1.z, x1.z, hi); hi = fmaf(h1.w, x1.w, hi);
              acc[mt][2 * c][0] = lo; acc[mt][2 * c + 1][0] = hi;
            }
          }
        }
      }
    }
  }
  __syncthreads();   // everyone is done with xs; reuse the memory for the k-warp reduction

  // red[kw][r][b] (row pitch RP = Bp+1 against bank conflicts), r = row inside the CTA tile
  constexpr int RP = Bp + 1;
  constexpr int SLAB = RPC * RP;
  {
    float* mine = red + kw * SLAB;
    if constexpr (kBf16) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r0 = (rg * MT + mt) * 16 + g;
#pragma unroll
        for (int nt = 0; nt < NB; ++nt) {
          const int c = 8 * nt + 2 * t;
          mine[r0 * RP + c] = acc[mt][nt][0];
          mine[r0 * RP + c + 1] = acc[mt][nt][1];
          mine[(r0 + 8) * RP + c] = acc[mt][nt][2];
          mine[(r0 + 8) * RP + c + 1] = acc[mt][nt][3];
        }
      }
    } else {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r0 = (rg * MT + mt) * 16 + g;
#pragma unroll
        for (int c = 0; c < Bp; ++c) {
          float lo = acc[mt][2 * c][0], hi = acc[mt][2 * c + 1][0];
          lo += __shfl_xor_sync(0xffffffffu, lo, 1);
          lo += __shfl_xor_sync(0xffffffffu, lo, 2);
          hi += __shfl_xor_sync(0xffffffffu, hi, 1);
          hi += __shfl_xor_sync(0xffffffffu, hi, 2);
          if (t == 0) {
            mine[r0 * RP + c] = lo;
            mine[(r0 + 8) * RP + c] = hi;
          }
        }
      }
    }
  }
  __syncthreads();
  // sum the 4 k-warp slabs into slab 0 (each thread owns its (r,b) positions: no hazard)
  for (int i = tid; i < RPC * Bp; i += kRingThreads) {
    const int r = i / Bp, b = i - r * Bp, o = r * RP + b;
    red[o] = (red[o] + red[SLAB + o]) + (red[2 * SLAB + o] + red[3 * SLAB + o]);
  }
  if (p.ksplit > 1) {
    float* my_part = p.partials + ((int64_t)blockIdx.x * p.ksplit + blockIdx.y) * (RPC * Bp);
    for (int i = tid; i < RPC * Bp; i += kRingThreads) {
      const int r = i / Bp, b = i - r * Bp;
      my_part[i] = red[r * RP + b];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned prev = atomicAdd(&p.counters[blockIdx.x], 1u);
      s_last = (prev == (unsigned)p.ksplit - 1u);
    }
    __syncthreads();
    if (!s_last) return;
    if (tid == 0) p.counters[blockIdx.x] = 0u;   // ready for the next launch
    __threadfence();
    sum_partials(red, p.partials + (int64_t)blockIdx.x * p.ksplit * (RPC * Bp), p.ksplit, RPC * Bp, RPC, RP, Bp, tid,
                 kRingThreads);
  }
  __syncthreads();
  run_epilogue<WT>(p, red, RPC, RP, Bp, blockIdx.x * RPC, tid, kRingThreads);
}

// =============================================================================================
// bf16 stream-K kernels
// =============================================================================================
constexpr int kStages = 5;
constexpr int kWStage = 32768;                   // 128 rows x 128 k, bf16
constexpr long long kWaitLimit = 4000000000LL;   // clock cycles (~2 s) before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  After a time-out the thread stops waiting for good (`dead`), so control flow --
// and with it every barrier -- stays the same for all threads; the launch is flagged as failed.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, bool& dead, int* err) {
  if (dead) return;
  if (mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitLimit) {
      dead = true;
      if (err) atomicExch(err, 1);
      return;
    }
  }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// The producer warp's last act: one 32 KB L2 prefetch per lane and round over this CTA's share of the
// next GEMV's weight heads (see GemvParams::pf_base).
__device__ __forceinline__ void prefetch_next_weights(const GemvParams& p, int lane) {
  if (!p.pf_base) return;
  const long long total = (long long)p.pf_parts * p.pf_chunk;
  const int n0 = (int)((long long)blockIdx.x * total / gridDim.x), n1 = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
  for (int n = n0 + lane; n < n1; n += 32) {
    const int part = n / p.pf_chunk, within = n - part * p.pf_chunk;
    const long long unit = (long long)part * p.pf_units / p.pf_parts + within;
    const char* a = reinterpret_cast<const char*>(p.pf_base) + unit * 32768;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(a), "r"(32768u) : "memory");
  }
}

struct UnitRange {
  int KS, nrbg, u0, u1;
  long long U, G;
};
__device__ __forceinline__ UnitRange unit_range(const GemvParams& p) {
  UnitRange ur;
  ur.KS = (p.K + 127) >> 7;
  ur.nrbg = (p.rows + 127) >> 7;
  ur.U = (long long)ur.nrbg * ur.KS;
  ur.G = gridDim.x;
  ur.u0 = (int)((long long)blockIdx.x * ur.U / ur.G);
  ur.u1 = (int)((long long)(blockIdx.x + 1) * ur.U / ur.G);
  return ur;
}
// CTAs that share row group r: CTA of unit u is ceil((u+1)*G/U) - 1
__device__ __forceinline__ void contributors(const UnitRange& ur, int r, int* c_first, int* n) {
  const long long ua = (long long)r * ur.KS, ub = ua + ur.KS - 1;
  *c_first = (int)(((ua + 1) * ur.G + ur.U - 1) / ur.U) - 1;
  const int c_last = (int)(((ub + 1) * ur.G + ur.U - 1) / ur.U) - 1;
  *n = c_last - *c_first + 1;
}

// producer loop shared by both kernels: one 32 KB weight copy + one activation copy per unit
template <int Bp>
__device__ __forceinline__ void produce(const GemvParams& p, const UnitRange& ur, unsigned char* smem,
                                        uint64_t* full_bar, uint64_t* empty_bar, int lane, int* err) {
  constexpr int kXStage = Bp * 256;
  constexpr int kStage = kWStage + kXStage;
  uint64_t pol_w, pol_x;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol_w));
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(pol_x));
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.W);
  const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.x);
  bool dead = false;
  // The weights never change: the first stages' weight copies go out before this kernel waits for
  // its predecessor; the activation copies (and everything else) come after the wait.
  const int n_units = ur.u1 - ur.u0;
  const int n_pre = n_units < kStages ? n_units : kStages;
  if (lane == 0) {
    for (int it = 0; it < n_pre; ++it) {
      const int u = ur.u0 + it;
      const int r = u / ur.KS, ks = u - r * ur.KS;
      mbar_expect_tx(&full_bar[it], (uint32_t)kStage);
      bulk_g2s(smem + it * kStage, W + ((int64_t)r * ur.KS + ks) * 16384, (uint32_t)kWStage, &full_bar[it], pol_w);
    }
  }
  pdl_wait();
  if (lane == 0) {
    for (int it = 0; it < n_pre; ++it) {
      const int ks = (ur.u0 + it) % ur.KS;
      bulk_g2s(smem + it * kStage + kWStage, X + (int64_t)ks * (128 * Bp), (uint32_t)kXStage, &full_bar[it], pol_x);
    }
  }
  __syncwarp();
  int it = n_pre;
  for (int u = ur.u0 + n_pre; u < ur.u1; ++u, ++it) {
    const int s = it % kStages, k = it / kStages;
    mbar_wait(&empty_bar[s], (k & 1) ^ 1, dead, err);
    const int r = u / ur.KS, ks = u - r * ur.KS;
    if (lane == 0) {
      unsigned char* st = smem + s * kStage;
      mbar_expect_tx(&full_bar[s], (uint32_t)kStage);
      bulk_g2s(st, W + ((int64_t)r * ur.KS + ks) * 16384, (uint32_t)kWStage, &full_bar[s], pol_w);
      bulk_g2s(st + kWStage, X + (int64_t)ks * (128 * Bp), (uint32_t)kXStage, &full_bar[s], pol_x);
    }
    __syncwarp();
  }
  prefetch_next_weights(p, lane);
}

// ---------------------------------------------------------------------------------------------
// tcgen05 variant
// ---------------------------------------------------------------------------------------------
constexpr int kTcThreads = 6 * 32;    // warp 0 producer, warp 1 MMA issue + TMEM, warps 2..5 epilogue

__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  // K-major, no swizzle: start address, leading (K-direction) and stride (M/N-direction) byte
  // offsets between 8x8 core matrices, all in 16-byte units; bit 46 = descriptor version 1.
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
         ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

template <int N> __device__ __forceinline__ void tmem_load_row(float (&v)[N], uint32_t taddr);
template <>
__device__ __forceinline__ void tmem_load_row<32>(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
template <>
__device__ __forceinline__ void tmem_load_row<16>(float (&v)[16], uint32_t taddr) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Epilogue of one accumulator row held by one thread (v[b], b < N).  Rows g and g+8 of a 16-row
// block -- the pairs the fused epilogues combine -- are 8 lanes apart in the same warp.
// The thread holds batch columns b0 .. b0+NV-1 of the row (the whole row when NV == BP); BP is the
// batch padding of the activation buffers.
template <int NV, int BP>
__device__ __forceinline__ void row_epilogue(const GemvParams& p, float (&v)[NV], int row, int b0, const float* s_inv) {
  typedef Layout<__nv_bfloat16> LY;
  constexpr int N = NV;
  const int rb = row >> 4, rr = row & 15, g = rr & 7, hi = rr >> 3;
  if (s_inv) {                                   // the norm scale of the input, one per sequence (InvScale)
#pragma unroll
    for (int b = 0; b < N; ++b) v[b] *= s_inv[b0 + b];
    if (p.ln_wg) {                               // LayerNorm: the mean's share, inv * mu * (W g)[row]
      const float wg = row < p.rows ? p.ln_wg[row] : 0.f;
#pragma unroll
      for (int b = 0; b < N; ++b) v[b] -= s_inv[32 + b0 + b] * wg;
    }
  }
  if (p.bias) {
    const float bias = row < p.rows ? p.bias[row] : 0.f;
#pragma unroll
    for (int b = 0; b < N; ++b) v[b] += bias;
  }
  if (p.epi == EPI_STORE_F32) {
    if (row < p.rows) {
#pragma unroll
      for (int b = 0; b < N; ++b)
        if (b0 + b < p.B) p.out[(int64_t)(b0 + b) * p.out_pitch + row] = v[b];
    }
    return;
  }
  if (p.epi == EPI_GELU_ACT) {
    if (row < p.n_act) {
      __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p.act);
#pragma unroll
      for (int b = 0; b < N; ++b)
        if (b0 + b < p.B) act[LY::x_offset(b0 + b, row, BP)] = __float2bfloat16_rn(gelu_ref(v[b]));
    }
    return;
  }
  float w[N];                                   // the partner row's values
#pragma unroll
  for (int b = 0; b < N; ++b) w[b] = __shfl_xor_sync(0xffffffffu, v[b], 8);
  if (row >= p.rows) return;
  if (p.epi == EPI_SILU_GATE) {
    const int o = rb * 8 + g;
    if (hi == 0 && o < p.n_act) {
      __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p.act);
#pragma unroll
      for (int b = 0; b < N; ++b) {
        if (b0 + b < p.B) {
          const float a = v[b], u = w[b];
          // silu(a) = a * (1 / (1 + exp2((a * -1) * (1/ln2))))     src/HighLevelOps.jl:153-160
          const float ex = exp2f((a * -1.0f) * kInvLn2);
          const float sg = 1.0f / (1.0f + ex);
          act[LY::x_offset(b0 + b, o, BP)] = __float2bfloat16_rn((a * sg) * u);
        }
      }
    }
    return;
  }
  // EPI_QKV_ROPE
  __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(p.kv_layer);
  const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
  // One position per sequence.  When the host knows they are all equal (pos_uniform) the rotation's sine and
  // cosine are computed once per row; otherwise once per batch column.
  int pos = p.pos[0];
  const int hs = rb / tiles_per_head, jj = rb - hs * tiles_per_head;
  if (hs < p.Hl + p.KVl) {
    // rows g / g+8 of the block are the RoPE pair (d0, d0 + D/2)      src/NN.jl:253-303
    const int d0 = 8 * jj + g;
    float sn = 0.f, cs = p.qk_scale;                // no rotation: q and k rows are only scaled
    const float inv_f = p.rope ? p.inv_freq[d0] : 0.f;
    if (p.rope) {
      const float ang = (float)pos * inv_f;
      sn = sinf(ang);
      cs = sinf(kHalfPi + ang * -1.0f);             // cos(a) = sin(pi/2 - a)
    }
    const int d = hi ? d0 + half : d0;
#pragma unroll
    for (int b = 0; b < N; ++b) {
      if (b0 + b < p.B) {
        if (!p.pos_uniform) {
          pos = p.pos[b0 + b];
          if (p.rope) {
            const float ang = (float)pos * inv_f;
            sn = sinf(ang);
            cs = sinf(kHalfPi + ang * -1.0f);
          }
        }
        // low row: x0*cos - x1*sin; high row: x0*sin + x1*cos (x0 = the low row's value)
        const float o = hi ? (w[b] * sn + v[b] * cs) : (v[b] * cs + (w[b] * sn) * -1.0f);
        if (hs < p.Hl) {
          reinterpret_cast<__nv_bfloat16*>(p.q_out)[(int64_t)(b0 + b) * p.q_pitch + hs * D + d] = __float2bfloat16_rn(o);
        } else {
          kv[(b0 + b) * p.kv_batch_stride + (hs - p.Hl) * p.kv_head_stride + kcache_offset(pos, d, D)] = __float2bfloat16_rn(o);
        }
      }
    }
  } else {
    const int d = 16 * jj + rr;
#pragma unroll
    for (int b = 0; b < N; ++b)
      if (b0 + b < p.B) {
        if (!p.pos_uniform) pos = p.pos[b0 + b];
        kv[(b0 + b) * p.kv_batch_stride + (hs - p.Hl - p.KVl) * p.kv_head_stride + vcache_offset(pos, d, D)] =
            __float2bfloat16_rn(v[b]);
      }
  }
}

// Optional per-CTA phase stamps (SM clock) for tuning; compiled in only with -DLMB_GEMV_TRACE.
#ifdef LMB_GEMV_TRACE
__device__ long long g_gemv_trace[160 * 16];
__device__ __forceinline__ long long gtime_ns() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
}  // namespace
int32_t gemv_trace_copy(long long* out) {
  return cudaMemcpyFromSymbol(out, g_gemv_trace, sizeof(g_gemv_trace)) == cudaSuccess ? 0 : -3;
}
namespace {
#define LMB_TRACE(slot) (g_gemv_trace[blockIdx.x * 16 + (slot)] = clock64())
#define LMB_TRACE_NS(slot) (g_gemv_trace[blockIdx.x * 16 + (slot)] = gtime_ns())
#else
#define LMB_TRACE(slot) ((void)0)
#define LMB_TRACE_NS(slot) ((void)0)
#endif

// The epilogue group (128 threads, e = 0..127) turns the producer's per-CTA sums of squares into the
// per-sequence scale 1 / sqrt(mean(x*x) + eps) (src/HighLevelOps.jl:299-304).  Four lanes share a
// sequence; each adds every fourth slot in ascending order and the four are combined pairwise, the
// same arithmetic in every CTA and on every rank.
__device__ __forceinline__ void compute_inv_scale(const InvScale& iv, float* s_inv, int e) {
  if (!iv.ssq) return;
  const int b = e >> 2, part = e & 3;
  float s = 0.f, sx = 0.f;
  for (int t = part; t < iv.tiles; t += 4) s += __ldcg(iv.ssq + t * 32 + b);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  if (iv.sum) {
    for (int t = part; t < iv.tiles; t += 4) sx += __ldcg(iv.sum + t * 32 + b);
    sx += __shfl_xor_sync(0xffffffffu, sx, 1);
    sx += __shfl_xor_sync(0xffffffffu, sx, 2);
  }
  if (part == 0) {
    const float rn = 1.0f / (float)iv.n;
    const float mu = sx * rn;                                   // 0 for RMSNorm
    const float inv = 1.0f / sqrtf(fmaxf(s * rn - mu * mu, 0.f) + iv.eps);
    s_inv[b] = inv;
    s_inv[32 + b] = mu * inv;
  }
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
}

__device__ __forceinline__ uint4 peer_load16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void peer_store16(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// bf16 -0.0 marks "not written yet" in a push buffer: a partial that rounds to it is sent as +0.0
__device__ __forceinline__ uint32_t pack_bf16x2_sendable(float a, float b) {
  uint32_t w = pack_bf16x2(a, b);
  if ((w & 0xFFFFu) == 0x8000u) w &= 0xFFFF0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000FFFFu;
  return w;
}
__device__ __forceinline__ bool has_empty_bf16(const uint4& u) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  bool any = false;
#pragma unroll
  for (int i = 0; i < 4; ++i) any = any || (w[i] & 0xFFFFu) == 0x8000u || (w[i] >> 16) == 0x8000u;
  return any;
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// EPI_RESID_NORM on the tile a cluster CTA finalises (rows_per = 128 / C rows of row group r, all Bp
// batch columns), run by the 128 epilogue threads once every partial row of the cluster sits in `recv`.
// Thread e owns rows (e >> 2) + 32 j and the 8 batch columns 8 (e & 3) .. + 7, so that a warp covers
// 8 consecutive rows x Bp columns: its peer stores and its reads of x are contiguous 512-byte runs.
template <int N>
__device__ __forceinline__ void resid_norm_tile(const GemvParams& p, const unsigned char* recv_raw, int C, int c, int r,
                                                int e, float* s_red) {
  constexpr int BG = N / 8;
  const int lane = e & 31, we = e >> 5;
  const int rows_per = 128 / C;
  const int bg = e & 3, rl0 = e >> 2;
  const int row0 = r * 128 + c * rows_per;
  const int iters = (rows_per + 31) >> 5;                      // 1, 1, 2, 4 for 16, 32, 64, 128 rows
  const float4* recv = reinterpret_cast<const float4*>(recv_raw);
  const int n = p.push.n, me = p.push.rank;
  float acc[4][8];
  bool valid[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int rl = rl0 + 32 * j;
    valid[j] = j < iters && bg < BG && rl < rows_per && row0 + rl < p.rows;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
    if (valid[j]) {
      for (int src = 0; src < C; ++src) {                      // the cluster's partials, in CTA order
        const float4 t0 = recv[((src * rows_per + rl) * N + 8 * bg) / 4], t1 = recv[((src * rows_per + rl) * N + 8 * bg) / 4 + 1];
        acc[j][0] += t0.x; acc[j][1] += t0.y; acc[j][2] += t0.z; acc[j][3] += t0.w;
        acc[j][4] += t1.x; acc[j][5] += t1.y; acc[j][6] += t1.z; acc[j][7] += t1.w;
      }
    }
  }
  if (n > 1) {
    const unsigned long long epoch = *p.push.step * kPeerEpochStride + p.push.phase;
    // this rank's partial, rounded to bf16 (never the "not written yet" pattern), into the same place of every peer's region
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!valid[j]) continue;
      uint4 u;
      u.x = pack_bf16x2_sendable(acc[j][0], acc[j][1]); u.y = pack_bf16x2_sendable(acc[j][2], acc[j][3]);
      u.z = pack_bf16x2_sendable(acc[j][4], acc[j][5]); u.w = pack_bf16x2_sendable(acc[j][6], acc[j][7]);
      unpack_bf16x8(u, acc[j]);                                // what this rank adds is what its peers receive
      const size_t at = ((size_t)me * p.rows + (row0 + rl0 + 32 * j)) * N + 8 * bg;
#pragma unroll
      for (int rk = 0; rk < 8; ++rk)
        if (rk < n && rk != me) peer_store16(p.push.part[rk] + at, u);
    }
    if (e < n && e != me) {                                    // validity channel, unordered with the data
      const bool poisoned = *reinterpret_cast<volatile int*>(p.push.broken) != 0;
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.push.flag[e] + me * kPushMaxCtas + blockIdx.x),
                   "l"(epoch | (poisoned ? kPeerPoison : 0ull))
                   : "memory");
    }
    const uint4 empty = make_uint4(kPeerEmptyPair, kPeerEmptyPair, kPeerEmptyPair, kPeerEmptyPair);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!valid[j]) continue;
      __nv_bfloat16* mine = p.push.part[me] + ((size_t)(row0 + rl0 + 32 * j)) * N + 8 * bg;      // + rk * rows * N
      const size_t src_stride = (size_t)p.rows * N;
      uint4 got[8];
      unsigned pending = 0;
#pragma unroll
      for (int rk = 0; rk < 8; ++rk)
        if (rk < n && rk != me) pending |= 1u << rk;
      const long long t0 = clock64();
      unsigned spins = 0;
      while (pending) {
#pragma unroll
        for (int rk = 0; rk < 8; ++rk)
          if (pending & (1u << rk)) got[rk] = peer_load16(mine + rk * src_stride);
#pragma unroll
        for (int rk = 0; rk < 8; ++rk)
          if ((pending & (1u << rk)) && !has_empty_bf16(got[rk])) pending &= ~(1u << rk);
        if (pending && (++spins & 63u) == 0u) {
          if (*reinterpret_cast<volatile int*>(p.push.broken) != 0) break;       // an earlier wait of this rank already failed
          if (clock64() - t0 > p.push.wait_cycles) { peer_mark_failed(p.push.dev_err, p.push.broken, 1); break; }
        }
      }
      float tot[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) tot[i] = 0.f;
#pragma unroll
      for (int rk = 0; rk < 8; ++rk) {                         // rank order, the same on every rank
        if (rk >= n) continue;
        float pv[8];
        if (rk == me) {
#pragma unroll
          for (int i = 0; i < 8; ++i) pv[i] = acc[j][i];
        } else {
          unpack_bf16x8(got[rk], pv);
          *reinterpret_cast<uint4*>(mine + rk * src_stride) = empty;   // ready for the reduction after the next
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) tot[i] += pv[i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = tot[i];
    }
    if (e < n && e != me) {                                    // the senders' validity marks (normally long there)
      const unsigned long long* flag = p.push.flag[me] + e * kPushMaxCtas + blockIdx.x;
      const long long t0 = clock64();
      unsigned spins = 0;
      for (;;) {
        unsigned long long v;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
        bool bad = false;
        if (peer_signal_ok(v, epoch, &bad)) {
          if (bad) peer_mark_failed(p.push.dev_err, p.push.broken, 2);
          break;
        }
        if ((++spins & 63u) == 0u) {
          if (*reinterpret_cast<volatile int*>(p.push.broken) != 0) break;
          if (clock64() - t0 > p.push.wait_cycles) { peer_mark_failed(p.push.dev_err, p.push.broken, 1); break; }
        }
      }
    }
  }
  // residual add, the next Linear's input x * gain, this tile's share of the sum of squares (and, for a LayerNorm, of the sum)
  float ssq[8], sxv[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { ssq[i] = 0.f; sxv[i] = 0.f; }
  __nv_bfloat16* xg = reinterpret_cast<__nv_bfloat16*>(p.rn.xg);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (!valid[j]) continue;
    const int grow = row0 + rl0 + 32 * j;
    float4* xr = reinterpret_cast<float4*>(p.rn.x + (size_t)grow * N + 8 * bg);
    float4 x0 = xr[0], x1 = xr[1];
    const float bias = p.bias ? p.bias[grow] : 0.f;             // the projection's own bias (Whisper)
    x0.x += acc[j][0] + bias; x0.y += acc[j][1] + bias; x0.z += acc[j][2] + bias; x0.w += acc[j][3] + bias;
    x1.x += acc[j][4] + bias; x1.y += acc[j][5] + bias; x1.z += acc[j][6] + bias; x1.w += acc[j][7] + bias;
    xr[0] = x0; xr[1] = x1;
    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const float g = p.rn.gain[grow];
    __nv_bfloat16* o = xg + (size_t)(grow >> 3) * (N * 8) + bg * 64 + (grow & 7);      // Layout::x_offset(8 bg + i, grow, N) = o + 8 i
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o[8 * i] = __float2bfloat16_rn(xv[i] * g);
      ssq[i] += xv[i] * xv[i];
      sxv[i] += xv[i];
    }
    if (p.rn.capture) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (8 * bg + i < p.B) p.rn.capture[(size_t)(8 * bg + i) * p.rows + grow] = xv[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {                                // over the 8 rows of the warp that share these batch columns
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 4);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 8);
    ssq[i] += __shfl_xor_sync(0xffffffffu, ssq[i], 16);
  }
  if (lane < 4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) s_red[we * 32 + 8 * lane + i] = ssq[i];
  }
  asm volatile("bar.sync 1, 128;\n" ::: "memory");
  if (e < 32) p.rn.ssq[(size_t)blockIdx.x * 32 + e] = ((s_red[e] + s_red[32 + e]) + s_red[64 + e]) + s_red[96 + e];
  if (p.rn.sum) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sxv[i] += __shfl_xor_sync(0xffffffffu, sxv[i], 4);
      sxv[i] += __shfl_xor_sync(0xffffffffu, sxv[i], 8);
      sxv[i] += __shfl_xor_sync(0xffffffffu, sxv[i], 16);
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");         // s_red has been read
    if (lane < 4) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s_red[we * 32 + 8 * lane + i] = sxv[i];
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (e < 32) p.rn.sum[(size_t)blockIdx.x * 32 + e] = ((s_red[e] + s_red[32 + e]) + s_red[64 + e]) + s_red[96 + e];
  }
}

template <int N>
__global__ void __launch_bounds__(kTcThreads, 1) gemv_tc_kernel(const GemvParams p, int* err) {
  constexpr int kXStage = N * 256;
  constexpr int kStage = kWStage + kXStage;
  constexpr uint32_t kTmemCols = 2 * N;       // two accumulator buffers (32 or 64 columns)
  // instruction descriptor, kind::f16: D = f32 (bit 4), A = B = bf16 (bits 7, 10), both K-major,
  // N >> 3 at bit 17, M >> 4 at bit 24
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ float s_inv_buf[64];        // [0, 32): inv per sequence, [32, 64): mean * inv (LayerNorm)
  const float* s_inv = p.inv.ssq ? s_inv_buf : nullptr;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const UnitRange ur = unit_range(p);
  if (tid == 0) {
    LMB_TRACE(0); LMB_TRACE_NS(10);
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full[0], 1); mbar_init(&acc_full[1], 1);
    mbar_init(&acc_empty[0], 4); mbar_init(&acc_empty[1], 4);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  bool dead = false;
  pdl_launch_dependents();
  if (tid == 0) LMB_TRACE(1);

  if (warp == 0) {
    produce<N>(p, ur, smem, full_bar, empty_bar, lane, err);
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) LMB_TRACE(2);
    // ---------------- MMA issue ----------------
    int it = 0, seg = 0;
    for (int u = ur.u0; u < ur.u1; ++u, ++it) {
      const int ks = u % ur.KS;
      const bool first = (u == ur.u0) || ks == 0;
      const bool last = (u == ur.u1 - 1) || ks == ur.KS - 1;
      const int buf = seg & 1;
      if (first) mbar_wait(&acc_empty[buf], ((seg >> 1) & 1) ^ 1, dead, err);   // epilogue has drained this buffer
      const int s = it % kStages, k = it / kStages;
      mbar_wait(&full_bar[s], k & 1, dead, err);
      tc_fence_after();
      if (lane == 0 && it == 0) LMB_TRACE(3);
      if (lane == 0) {
        const uint32_t st = smem_u32(smem + s * kStage);
        const uint64_t adesc = smem_desc(st, 2048, 128);
        const uint64_t bdesc = smem_desc(st + kWStage, N * 16, 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)     // 8 k-steps of 16: two core matrices along K each
          tc_mma_f16(tmem_base + buf * N, adesc + (uint64_t)(j * (4096 >> 4)), bdesc + (uint64_t)(j * ((2 * N * 16) >> 4)),
                     kIdesc, (first && j == 0) ? 0u : 1u);
        tc_commit(&empty_bar[s]);       // stage free once these MMAs have read it
        if (last) tc_commit(&acc_full[buf]);
      }
      __syncwarp();
      if (last) ++seg;
    }
    if (lane == 0) LMB_TRACE(4);
  } else {
    // ---------------- epilogue: warp quarter q owns TMEM lanes / rows 32q .. 32q+31 ----------------
    // A row group whose k range is shared by n > 1 CTAs is folded by all of them together: each
    // stores its partial accumulator and counts itself in; once this CTA has finished its own
    // units it waits until every contributor of the group has arrived and then sums, in contributor
    // order, the 16-row blocks that fall to it (block j goes to contributor j mod n) and runs
    // their epilogue.  The sum order is fixed, so results do not depend on timing.
    pdl_wait();
    const int q = warp & 3;
    const int e = tid - 64;                      // 0..127 inside the epilogue group
    compute_inv_scale(p.inv, s_inv_buf, e);
    int seg = 0;
    int pend_r[2], pend_first[2], pend_n[2], n_pend = 0;
    for (int u = ur.u0; u < ur.u1; ++seg) {
      const int r = u / ur.KS;
      const int u_end = min(ur.u1, (r + 1) * ur.KS);
      u = u_end;
      const int buf = seg & 1;
      mbar_wait(&acc_full[buf], (seg >> 1) & 1, dead, err);
      tc_fence_after();
      float v[N];
      tmem_load_row<N>(v, tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(buf * N));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (tid == 64) LMB_TRACE(5);
      const int row_in_group = 32 * q + lane;
      int c_first, n;
      contributors(ur, r, &c_first, &n);
      if (n == 1) {
        row_epilogue<N, N>(p, v, r * 128 + row_in_group, 0, s_inv);
        continue;
      }
      float4* part = reinterpret_cast<float4*>(p.partials) + (int64_t)r * p.ksplit * (128 * N / 4);
      float4* mine = part + (int64_t)((int)blockIdx.x - c_first) * (128 * N / 4) + row_in_group * (N / 4);
#pragma unroll
      for (int i = 0; i < N / 4; ++i) mine[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      __threadfence();
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (e == 0) atomicAdd(&p.counters[r * 8], 1u);
      if (tid == 64) LMB_TRACE(6);
      if (n_pend < 2) { pend_r[n_pend] = r; pend_first[n_pend] = c_first; pend_n[n_pend] = n; ++n_pend; }
    }
    // wait for every contributor of the shared row groups.  The last segment is shared with CTAs
    // that finished it long ago, the first one with a CTA that ends on it about now.
    if (e == 0) {
      const long long t0 = clock64();
      for (int ip = n_pend - 1; ip >= 0; --ip) {
        for (;;) {
          unsigned seen;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(p.counters + pend_r[ip] * 8) : "memory");
          if (seen >= (unsigned)pend_n[ip] || dead) break;
          if (clock64() - t0 > kWaitLimit) { dead = true; if (err) atomicExch(err, 1); break; }
        }
      }
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (tid == 64) LMB_TRACE(7);
    const int row16 = lane & 15, cg = e >> 4;               // one float4 (4 batch columns) per thread
    if (cg < N / 4 && n_pend > 0) {                          // warp-uniform: whole warps drop out for N = 16
      // Per shared row group this contributor owns the 16-row blocks ci, ci + n, ... (at most 4) and
      // sums each over the contributors in ascending order.  A round trip to L2 at the end of a
      // kernel costs microseconds, so every partial this thread needs is fetched with one wave of
      // cp.async into the (now idle) pipeline stages, slot s of thread e at byte s * 2048 + e * 16,
      // and summed from shared memory afterwards.
      constexpr int kSlots = (kStages * kStage) / 2048;
      constexpr int64_t kPartStride = 128 * N / 4;           // float4s per contributor
      const uint32_t fs = smem_u32(smem) + (uint32_t)e * 16u;
      int n_[2], ci_[2], nj_[2];
      const float4* part_[2];
#pragma unroll
      for (int ip = 0; ip < 2; ++ip) {
        const bool on = ip < n_pend;
        n_[ip] = on ? pend_n[ip] : 1;
        ci_[ip] = on ? (int)blockIdx.x - pend_first[ip] : 8;
        nj_[ip] = ci_[ip] < 8 ? (8 - ci_[ip] + n_[ip] - 1) / n_[ip] : 0;
        part_[ip] = reinterpret_cast<const float4*>(p.partials) + (int64_t)(on ? pend_r[ip] : 0) * p.ksplit * kPartStride +
                    row16 * (N / 4) + cg;
      }
      auto issue = [&](int ip, int slot, int k0, int k1) -> int {
        for (int jj = 0; jj < nj_[ip]; ++jj) {
          const float4* src = part_[ip] + 16 * (ci_[ip] + jj * n_[ip]) * (N / 4);
          for (int k = k0; k < k1; ++k, ++slot)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(fs + (uint32_t)slot * 2048u), "l"(src + k * kPartStride) : "memory");
        }
        return slot;
      };
      auto lds4 = [&](int slot) -> float4 {
        float4 t;
        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "r"(fs + (uint32_t)slot * 2048u));
        return t;
      };
      auto consume = [&](int ip, int slot) -> int {
        for (int jj = 0; jj < nj_[ip]; ++jj) {
          float v4[4] = {0.f, 0.f, 0.f, 0.f};
          for (int k = 0; k < n_[ip]; ++k, ++slot) {
            const float4 t = lds4(slot);
            v4[0] += t.x; v4[1] += t.y; v4[2] += t.z; v4[3] += t.w;
          }
          row_epilogue<4, N>(p, v4, pend_r[ip] * 128 + 16 * (ci_[ip] + jj * n_[ip]) + row16, 4 * cg, s_inv);
        }
        return slot;
      };
      const int cnt0 = nj_[0] * n_[0], cnt1 = nj_[1] * n_[1];
      if (cnt0 + cnt1 <= kSlots) {
        const int s1 = issue(0, 0, 0, n_[0]);
        issue(1, s1, 0, n_[1]);
        asm volatile("cp.async.wait_all;\n" ::: "memory");
        if (tid == 64) LMB_TRACE(12);
        consume(1, consume(0, 0));
      } else {
        // a row group shared by more CTAs than there are slots (tiny matrices): waves over k
#pragma unroll 1
        for (int ip = 0; ip < 2; ++ip) {
          if (nj_[ip] == 0) continue;
          if (nj_[ip] * n_[ip] <= kSlots) {
            issue(ip, 0, 0, n_[ip]);
            asm volatile("cp.async.wait_all;\n" ::: "memory");
            consume(ip, 0);
            continue;
          }
          float v4[4] = {0.f, 0.f, 0.f, 0.f};          // n > kSlots > 8, so there is one block
          for (int k0 = 0; k0 < n_[ip]; k0 += kSlots) {
            const int k1 = min(n_[ip], k0 + kSlots);
            issue(ip, 0, k0, k1);
            asm volatile("cp.async.wait_all;\n" ::: "memory");
            for (int sl = 0; sl < k1 - k0; ++sl) {
              const float4 t = lds4(sl);
              v4[0] += t.x; v4[1] += t.y; v4[2] += t.z; v4[3] += t.w;
            }
          }
          row_epilogue<4, N>(p, v4, pend_r[ip] * 128 + 16 * ci_[ip] + row16, 4 * cg, s_inv);
        }
      }
      if (tid == 64) LMB_TRACE(13);
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (e < n_pend) {
      const int r = pend_r[e], n = pend_n[e];
      const unsigned prev = atomicAdd(&p.counters[r * 8 + 1], 1u);
      if (prev == (unsigned)n - 1u) {                       // every contributor has read: ready for the next launch
        p.counters[r * 8] = 0u;
        p.counters[r * 8 + 1] = 0u;
      }
    }
    if (tid == 64) LMB_TRACE(8);
  }
  // all roles meet before the accumulator memory is given back
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (tid == 0) { LMB_TRACE(9); LMB_TRACE_NS(11); }
}

// =============================================================================================
// Cluster variant for small matrices.  The stream-K kernel folds a shared row group through
// global scratch: store, fence, count, wait, fetch -- about 6 us after the last MMA, more than
// the streaming itself once a matrix is a few tens of MB (tensor-parallel shards, q/k/v, o_proj).
// Here a thread-block cluster of C CTAs owns one 128-row group, CTA c streams the c-th share of
// its k range, and the partial accumulators are exchanged through distributed shared memory:
// every CTA sends each peer the rows that peer finalises (128 / C of them), one cluster barrier,
// then every CTA sums its rows over the C sources in rank order and runs their epilogue.
// =============================================================================================
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void dsmem_store4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

template <int N>
__global__ void __launch_bounds__(kTcThreads, 1) gemv_cl_kernel(const GemvParams p, int* err) {
  constexpr int kXStage = N * 256;
  constexpr int kStage = kWStage + kXStage;
  constexpr uint32_t kTmemCols = N < 32 ? 32 : N;     // an allocation is at least 32 columns
  constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
  extern __shared__ __align__(1024) unsigned char smem[];       // kStages stages, then recv[C][128 / C][N] floats
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ float s_inv_buf[64];        // [0, 32): inv per sequence, [32, 64): mean * inv (LayerNorm)
  __shared__ float s_red[128];
  const float* s_inv = p.inv.ssq ? s_inv_buf : nullptr;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = (int)cluster_nctarank(), c = (int)cluster_ctarank();
  const int r = (int)blockIdx.x / C;                              // row group of this cluster
  const int KS = (p.K + 127) >> 7;
  const int ks0 = (int)((long long)c * KS / C), ks1 = (int)((long long)(c + 1) * KS / C);
  const int n_steps = ks1 - ks0;
  if (tid == 0) {
    LMB_TRACE(0); LMB_TRACE_NS(10);
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  bool dead = false;
  pdl_launch_dependents();
  if (tid == 0) LMB_TRACE(1);

  if (warp == 0) {
    // ---------------- producer: weights before the dependency wait, activations after ----------------
    uint64_t pol_w, pol_x;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol_w));
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(pol_x));
    const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.W) + ((int64_t)r * KS + ks0) * 16384;
    const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.x) + (int64_t)ks0 * (128 * N);
    const int n_pre = n_steps < kStages ? n_steps : kStages;
    if (lane == 0) {
      for (int i = 0; i < n_pre; ++i) {
        mbar_expect_tx(&full_bar[i], (uint32_t)kStage);
        bulk_g2s(smem + i * kStage, W + (int64_t)i * 16384, (uint32_t)kWStage, &full_bar[i], pol_w);
      }
    }
    pdl_wait();
    if (lane == 0) {
      for (int i = 0; i < n_pre; ++i)
        bulk_g2s(smem + i * kStage + kWStage, X + (int64_t)i * (128 * N), (uint32_t)kXStage, &full_bar[i], pol_x);
    }
    __syncwarp();
    for (int i = n_pre; i < n_steps; ++i) {
      const int s = i % kStages, k = i / kStages;
      mbar_wait(&empty_bar[s], (k & 1) ^ 1, dead, err);
      if (lane == 0) {
        unsigned char* sp = smem + s * kStage;
        mbar_expect_tx(&full_bar[s], (uint32_t)kStage);
        bulk_g2s(sp, W + (int64_t)i * 16384, (uint32_t)kWStage, &full_bar[s], pol_w);
        bulk_g2s(sp + kWStage, X + (int64_t)i * (128 * N), (uint32_t)kXStage, &full_bar[s], pol_x);
      }
      __syncwarp();
    }
    prefetch_next_weights(p, lane);
  } else if (warp == 1) {
    // ---------------- MMA issue ----------------
    pdl_wait();
    if (lane == 0) LMB_TRACE(2);
    for (int i = 0; i < n_steps; ++i) {
      const int s = i % kStages, k = i / kStages;
      mbar_wait(&full_bar[s], k & 1, dead, err);
      tc_fence_after();
      if (lane == 0 && i == 0) LMB_TRACE(3);
      if (lane == 0) {
        const uint32_t sa = smem_u32(smem + s * kStage);
        const uint64_t adesc = smem_desc(sa, 2048, 128);
        const uint64_t bdesc = smem_desc(sa + kWStage, N * 16, 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          tc_mma_f16(tmem_base, adesc + (uint64_t)(j * (4096 >> 4)), bdesc + (uint64_t)(j * ((2 * N * 16) >> 4)), kIdesc,
                     (i == 0 && j == 0) ? 0u : 1u);
        tc_commit(&empty_bar[s]);
        if (i == n_steps - 1) tc_commit(&acc_full);
      }
      __syncwarp();
    }
    if (lane == 0) LMB_TRACE(4);
  } else {
    // ---------------- epilogue warps: send every row to the CTA that finalises it ----------------
    pdl_wait();
    const int q = warp & 3;
    compute_inv_scale(p.inv, s_inv_buf, tid - 64);
    float v[N];
    if (n_steps > 0) {
      mbar_wait(&acc_full, 0, dead, err);
      tc_fence_after();
      tmem_load_row<N>(v, tmem_base + ((uint32_t)(32 * q) << 16));
      tc_fence_before();
      if (tid == 64) LMB_TRACE(5);
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] = 0.f;
    }
    const int rows_per = 128 / C;
    const int row = 32 * q + lane;
    const int owner = row / rows_per, row_local = row - owner * rows_per;
    const uint32_t recv_local = smem_u32(smem + kStages * kStage) + (uint32_t)(((c * rows_per + row_local) * N) * 4);
    const uint32_t dst = dsmem_addr(recv_local, (uint32_t)owner);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) dsmem_store4(dst + 16u * i, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    if (tid == 64) LMB_TRACE(6);
  }
  // every partial row is in its owner's shared memory once all CTAs of the cluster are here
  cluster_sync_all();
  if (tid == 64) LMB_TRACE(7);
  if (warp >= 2 && p.epi == EPI_RESID_NORM) {
    resid_norm_tile<N>(p, smem + kStages * kStage, C, c, r, tid - 64, s_red);
  } else if (warp >= 2) {
    const int e = tid - 64;
    const int rows_per = 128 / C;
    const int row16 = lane & 15, cg = e >> 4;               // one float4 (4 batch columns) per thread
    if (cg < N / 4) {
      const float4* recv = reinterpret_cast<const float4*>(smem + kStages * kStage);
      for (int j = 0; j < rows_per / 16; ++j) {
        float v4[4] = {0.f, 0.f, 0.f, 0.f};
        for (int src = 0; src < C; ++src) {
          const float4 t = recv[((src * rows_per + 16 * j + row16) * N) / 4 + cg];
          v4[0] += t.x; v4[1] += t.y; v4[2] += t.z; v4[3] += t.w;
        }
        row_epilogue<4, N>(p, v4, r * 128 + c * rows_per + 16 * j + row16, 4 * cg, s_inv);
      }
    }
  }
  if (tid == 64) LMB_TRACE(8);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
  if (tid == 0) { LMB_TRACE(9); LMB_TRACE_NS(11); }
}

template <int Bp>
constexpr size_t cluster_smem() {
  return (size_t)kStages * (kWStage + Bp * 256) + 128 * Bp * 4 + 1024;
}

template <int Bp>
int32_t launch_cluster(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(ceil_div(p.rows, 128) * p.cluster));
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = cluster_smem<Bp>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  LMB_CUDA(cudaLaunchKernelEx(&cfg, gemv_cl_kernel<Bp>, p, ctx->dev_err));
  ctx->launches++;
  return LMB200_OK;
}

// The largest cluster size (8, 4, 2) that keeps rows/128 x C CTAs on the device in one wave and
// gives every CTA at least one k step; 0: use the stream-K kernel.
template <int Bp>
int cluster_choice(const Ctx* ctx, int rows, int K) {
  const int nrbg = (int)ceil_div(rows, 128), KS = (int)ceil_div(K, 128);
  for (int C = 8; C >= 2; C >>= 1) {
    if (C > KS || (int64_t)nrbg * C > ctx->sm_count) continue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nrbg * C));
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = cluster_smem<Bp>();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&n_clusters, gemv_cl_kernel<Bp>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    if (n_clusters >= nrbg) return C;
  }
  return 0;
}

template <typename WT, int NB, int MT, int STAGES>
int32_t launch_ring(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  constexpr int Bp = 8 * NB, RPC = 2 * MT * 16;
  const size_t xs_bytes = (size_t)p.kc_per_split * Bp * 32 * sizeof(WT);
  const size_t red_bytes = (size_t)4 * RPC * (Bp + 1) * sizeof(float);
  const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  LMB_REQUIRE(smem <= kMaxSmem, "gemv: %zu bytes of shared memory exceed the configured %zu", smem, kMaxSmem);
  dim3 grid((unsigned)ceil_div(p.RB, 2 * MT), (unsigned)p.ksplit);
  LMB_CUDA(launch_k(gemv_ring_kernel<WT, NB, MT, STAGES>, grid, dim3(kRingThreads), smem, stream, p));
  ctx->launches++;
  return LMB200_OK;
}

template <int Bp>
constexpr size_t stream_smem() {
  return (size_t)kStages * (kWStage + Bp * 256) + 1024;
}

template <int Bp>
int32_t launch_bf16(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  if (p.cluster >= 1) return launch_cluster<Bp>(ctx, p, stream);
  LMB_CUDA(launch_k(gemv_tc_kernel<Bp>, dim3(p.grid), dim3(kTcThreads), stream_smem<Bp>(), stream, p, ctx->dev_err));
  ctx->launches++;
  return LMB200_OK;
}

constexpr int kMtF32 = 1;
constexpr size_t kMaxXsBytes = 96 * 1024;

}  // namespace

void gemv_set_variant(int variant) { (void)variant; g_variant = GEMV_TCGEN05; }
int gemv_variant() { return g_variant; }

void gemv_prefetch_next(GemvParams& p, const Ctx* ctx, int dtype, const void* next_W, int next_rows, int next_K,
                        const GemvPlan& next_plan) {
  (void)ctx;
  static const int budget_mb = [] { const char* e = getenv("LMB200_L2_PREFETCH_MB"); return e ? atoi(e) : 24; }();
  if (dtype != LMB200_BF16 || g_variant != GEMV_TCGEN05 || budget_mb <= 0 || !next_W) return;
  const int KS = (int)ceil_div(next_K, 128), nrbg = (int)ceil_div(next_rows, 128);
  const int64_t U = (int64_t)nrbg * KS;
  const int parts = next_plan.cluster >= 1 ? nrbg * next_plan.cluster : next_plan.grid;
  if (parts <= 0 || U / parts < 1) return;
  int64_t chunk = ((int64_t)budget_mb * 1000000 / 32768) / parts;
  if (chunk < 1) chunk = 1;
  if (chunk > U / parts) chunk = U / parts;
  p.pf_base = next_W; p.pf_units = (int)U; p.pf_parts = parts; p.pf_chunk = (int)chunk;
}

GemvPlan gemv_plan(const Ctx* ctx, int dtype, int B, int rows, int K) {
  GemvPlan pl;
  if (dtype == LMB200_BF16) {
    const int Bp = Layout<__nv_bfloat16>::batch_pad(B);
    const int KS = (int)ceil_div(K, 128);
    const int nrbg = (int)ceil_div(rows, 128);
    const int64_t U = (int64_t)nrbg * KS;
    int G = ctx->sm_count;
    if (G > U) G = (int)U;
    pl.grid = G;
    const int64_t upc_min = U / G;                       // >= 1
    pl.ksplit = (int)ceil_div(KS, upc_min) + 1;          // contributors reserved per row group
    pl.kc_per_split = KS;
    pl.partial_floats = (int64_t)nrbg * pl.ksplit * 128 * Bp;   // [row group][contributor][128 x Bp]
    pl.n_counters = nrbg * 8;
    // small matrices: a cluster per row group, partials through distributed shared memory
    const char* ce = getenv("LMB200_GEMV_CLUSTER");             // 0: never; N (MB): size limit, default 128
    const int64_t limit_mb = ce ? atoi(ce) : 128;
    if (g_variant == GEMV_TCGEN05 && (int64_t)rows * K * 2 <= limit_mb * 1000000)
      pl.cluster = Bp == 16 ? cluster_choice<16>(ctx, rows, K) : cluster_choice<32>(ctx, rows, K);
    return pl;
  }
  const int Bp = Layout<float>::batch_pad(B);
  const int RB = (int)ceil_div(rows, 16), KC = (int)ceil_div(K, 32);
  const int MT = kMtF32;
  const int RPC = 2 * MT * 16;
  const size_t esz = 4;
  const int nrbg = (int)ceil_div(RB, 2 * MT);
  // One CTA per SM is resident (register ring).  Pick the k-split that minimises
  //   waves * (chunks per CTA + fixed cost of staging x and the epilogue, in chunk units)
  // with the activation slice fitting shared memory and at least one chunk per k-warp.
  const int per_max = (int)(kMaxXsBytes / (Bp * 32 * esz));
  const int kFixed = 6;
  int best_ks = 1, best_per = KC;
  double best_cost = 1e30;
  for (int ks_try = 1; ks_try <= KC; ++ks_try) {
    const int per_try = (int)ceil_div(KC, ks_try);
    if (per_try > per_max) continue;
    if (per_try < 4 && ks_try > 1) break;
    const int ks_eff = (int)ceil_div(KC, per_try);
    const double waves = (double)ceil_div((int64_t)nrbg * ks_eff, ctx->sm_count);
    const double cost = waves * (per_try + kFixed) + 0.02 * ks_eff;
    if (cost < best_cost) { best_cost = cost; best_ks = ks_eff; best_per = per_try; }
  }
  pl.ksplit = best_ks;
  pl.kc_per_split = best_per;
  pl.grid = nrbg * best_ks;
  pl.partial_floats = best_ks > 1 ? (int64_t)nrbg * best_ks * RPC * Bp : 0;
  pl.n_counters = nrbg;
  return pl;
}

GemvPlan gemv_plan_resid(const Ctx* ctx, int B, int rows, int K) {
  GemvPlan pl = gemv_plan(ctx, LMB200_BF16, B, rows, K);
  const int Bp = Layout<__nv_bfloat16>::batch_pad(B);
  const int nrbg = (int)ceil_div(rows, 128);
  pl.cluster = 0;
  if (g_variant != GEMV_TCGEN05) return pl;
  pl.cluster = Bp == 16 ? cluster_choice<16>(ctx, rows, K) : cluster_choice<32>(ctx, rows, K);
  if (pl.cluster == 0 && nrbg <= ctx->sm_count && nrbg <= kPushMaxCtas) pl.cluster = 1;
  if (nrbg * pl.cluster > kPushMaxCtas) pl.cluster = 0;
  return pl;
}

int gemv_plan_ctas(const GemvPlan& pl, int rows) {
  return pl.cluster >= 1 ? (int)ceil_div(rows, 128) * pl.cluster : pl.grid;
}

// Raise the dynamic shared-memory limit of every instantiation once per device, outside any
// stream capture.
int32_t gemv_configure() {
#define LMB_CFG(KERN, BYTES) \
  LMB_CUDA(cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(BYTES)))
  LMB_CFG((gemv_ring_kernel<float, 1, kMtF32, 3>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<float, 2, kMtF32, 3>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<float, 4, kMtF32, 2>), kMaxSmem);
  LMB_CFG(gemv_tc_kernel<16>, stream_smem<16>());
  LMB_CFG(gemv_tc_kernel<32>, stream_smem<32>());
  LMB_CFG(gemv_cl_kernel<16>, cluster_smem<16>());
  LMB_CFG(gemv_cl_kernel<32>, cluster_smem<32>());
#undef LMB_CFG
  return LMB200_OK;
}

int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream) {
  LMB_REQUIRE(p.B >= 1 && p.B <= 32, "gemv: batch %d outside 1..32", p.B);
  if (dtype == LMB200_BF16) {
    LMB_REQUIRE(p.grid >= 1 && p.partials && p.counters, "gemv: the bf16 kernels need a plan and scratch");
    return Layout<__nv_bfloat16>::batch_pad(p.B) == 16 ? launch_bf16<16>(ctx, p, stream) : launch_bf16<32>(ctx, p, stream);
  }
  LMB_REQUIRE(dtype == LMB200_F32, "gemv: dtype %d", dtype);
  LMB_REQUIRE(p.ksplit >= 1 && p.kc_per_split >= 1 && (int64_t)p.ksplit * p.kc_per_split >= p.KC,
              "gemv: bad k split");
  LMB_REQUIRE(p.ksplit == 1 || (p.partials && p.counters), "gemv: split-K needs scratch");
  switch (Layout<float>::batch_pad(p.B) / 8) {
    case 1: return launch_ring<float, 1, kMtF32, 3>(ctx, p, stream);
    case 2: return launch_ring<float, 2, kMtF32, 3>(ctx, p, stream);
    default: return launch_ring<float, 4, kMtF32, 2>(ctx, p, stream);
  }
}

}  // namespace lmb

#ifdef LMB_GEMV_TRACE
extern "C" int32_t lmb200_debug_gemv_trace(long long* out) {
  return lmb::gemv_trace_copy(out);
}
#endif
