// Bandwidth-bound decode GEMV with fused epilogues (store / SiLU-gate / RoPE + KV append).
//
// bf16 "stream" kernel (default): stream-K over bulk-TMA.  The weight matrix is cut into units of
// 128 rows x 128 k (32 KB, eight contiguous 4 KB runs of the tiled layout); the grid is one CTA
// per SM and CTA c takes the contiguous unit range [c*U/G, (c+1)*U/G), so every SM streams the
// same number of bytes in a single wave whatever the matrix shape.  A producer warp keeps a ring
// of STAGES shared-memory stages full with cp.async.bulk copies (weights evict-first, plus the
// matching slice of the tiled activations) signalled through mbarriers; 8 consumer warps read
// their MMA operands from the stage with conflict-free 16-byte loads
// and issue mma.sync m16n8k16; each consumer warp owns one 16-row block of the group, so nothing
// is reduced across warps and the fused epilogue runs from the accumulator registers.  When a
// CTA's range leaves a row group its warps fold their fragments: alone -> epilogue; shared ->
// global scratch + a per-row-block counter, the last contributing warp sums the fragments in CTA
// order (deterministic) and runs the epilogue.  No CTA-wide barrier after start-up.
//
// "ring" kernel: weights streamed by plain loads through a register ring; used for float32 (the
// parity path, fp32 FMAs) and selectable for bf16 (A/B comparison).
#include <type_traits>

#include "gemv.cuh"

namespace lmb {

namespace {

constexpr float kInvLn2 = 1.4426950408889634f;      // Float32(1/log(2)) as the reference rounds it
constexpr float kHalfPi = 1.5707963267948966f;
constexpr size_t kMaxSmem = 224 * 1024;

bool g_use_stream = true;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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
      if (b < p.B && row < p.rows) p.out[(int64_t)b * p.out_pitch + row] = tile[r * RP + b];
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
        act[xtile_offset(b, o, Bp)] = from_f32<WT>((a * sg) * u);
      }
    }
  } else {  // EPI_QKV_ROPE
    WT* q_out = reinterpret_cast<WT*>(p.q_out);
    WT* kv = reinterpret_cast<WT*>(p.kv_layer);
    const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
    const int pos = *p.pos;
    const float fpos = (float)pos;
    for (int i = tid; i < (RPC / 2) * Bp; i += nthreads) {
      const int b = i / (RPC / 2), j = i - b * (RPC / 2);
      const int m = j >> 3, r = j & 7;
      const int gt = row0 / 16 + m;                  // global 16-row tile
      if (b >= p.B || gt >= p.RB) continue;
      const int hs = gt / tiles_per_head, jj = gt - hs * tiles_per_head;
      const float v0 = tile[(16 * m + r) * RP + b], v1 = tile[(16 * m + r + 8) * RP + b];
      if (hs < p.Hl + p.KVl) {
        // rows r / r+8 of the tile are the RoPE pair (d0, d0 + D/2)      src/NN.jl:253-303
        const int d0 = 8 * jj + r;
        const float ang = fpos * p.inv_freq[d0];
        const float sn = sinf(ang);
        const float cs = sinf(kHalfPi + ang * -1.0f);   // cos(a) = sin(pi/2 - a)
        const float o0 = v0 * cs + (v1 * sn) * -1.0f;
        const float o1 = v0 * sn + v1 * cs;
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
// stream kernel (bf16)
// =============================================================================================
constexpr int kConsumerWarps = 8;
constexpr int kStreamThreads = (kConsumerWarps + 1) * 32;
constexpr int kCH = 4;              // k-chunks per stage (one per k-warp)
constexpr int kRPC = 128;           // rows per row group (8 row blocks)
constexpr int kStages = 5;
constexpr int kWStage = 8 * kCH * 1024;
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

// Epilogue of one 16-row block straight from the accumulator fragments of the warp that owns it:
// lane (g,t) holds, per batch tile nt, rows g (c0,c1) and g+8 (c2,c3) at columns 8nt+2t, +1 --
// and rows g / g+8 are exactly the pairs the fused epilogues combine.
template <int NB>
__device__ __forceinline__ void fragment_epilogue(const GemvParams& p, const float (&acc)[NB][4], int rb, int g, int t) {
  constexpr int Bp = 8 * NB;
  if (p.epi == EPI_STORE_F32) {
    const int row = rb * 16 + g;
#pragma unroll
    for (int nt = 0; nt < NB; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int b = 8 * nt + 2 * t + e;
        if (b < p.B) {
          if (row < p.rows) p.out[(int64_t)b * p.out_pitch + row] = acc[nt][e];
          if (row + 8 < p.rows) p.out[(int64_t)b * p.out_pitch + row + 8] = acc[nt][2 + e];
        }
      }
    }
  } else if (p.epi == EPI_SILU_GATE) {
    __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(p.act);
    const int o = rb * 8 + g;
    if (o < p.n_act) {
#pragma unroll
      for (int nt = 0; nt < NB; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int b = 8 * nt + 2 * t + e;
          if (b < p.B) {
            const float a = acc[nt][e], u = acc[nt][2 + e];
            // silu(a) = a * (1 / (1 + exp2((a * -1) * (1/ln2))))     src/HighLevelOps.jl:153-160
            const float ex = exp2f((a * -1.0f) * kInvLn2);
            const float sg = 1.0f / (1.0f + ex);
            act[xtile_offset(b, o, Bp)] = __float2bfloat16_rn((a * sg) * u);
          }
        }
      }
    }
  } else {  // EPI_QKV_ROPE
    __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(p.q_out);
    __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(p.kv_layer);
    const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
    const int pos = *p.pos;
    const int hs = rb / tiles_per_head, jj = rb - hs * tiles_per_head;
    float sn = 0.f, cs = 1.f;
    const bool rope = hs < p.Hl + p.KVl;
    const int d0 = 8 * jj + g;
    if (rope) {
      // rows g / g+8 of the block are the RoPE pair (d0, d0 + D/2)      src/NN.jl:253-303
      const float ang = (float)pos * p.inv_freq[d0];
      sn = sinf(ang);
      cs = sinf(kHalfPi + ang * -1.0f);   // cos(a) = sin(pi/2 - a)
    }
#pragma unroll
    for (int nt = 0; nt < NB; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int b = 8 * nt + 2 * t + e;
        if (b >= p.B) continue;
        const float v0 = acc[nt][e], v1 = acc[nt][2 + e];
        if (rope) {
          const float o0 = v0 * cs + (v1 * sn) * -1.0f;
          const float o1 = v0 * sn + v1 * cs;
          if (hs < p.Hl) {
            __nv_bfloat16* q = q_out + (int64_t)b * p.q_pitch + hs * D;
            q[d0] = __float2bfloat16_rn(o0);
            q[d0 + half] = __float2bfloat16_rn(o1);
          } else {
            __nv_bfloat16* kc = kv + b * p.kv_batch_stride + (hs - p.Hl) * p.kv_head_stride;
            kc[kcache_offset(pos, d0, D)] = __float2bfloat16_rn(o0);
            kc[kcache_offset(pos, d0 + half, D)] = __float2bfloat16_rn(o1);
          }
        } else {
          __nv_bfloat16* vc = kv + b * p.kv_batch_stride + (hs - p.Hl - p.KVl) * p.kv_head_stride;
          const int d = 16 * jj + g;
          vc[vcache_offset(pos, d, D)] = __float2bfloat16_rn(v0);
          vc[vcache_offset(pos, d + 8, D)] = __float2bfloat16_rn(v1);
        }
      }
    }
  }
}

template <int NB>
__global__ void __launch_bounds__(kStreamThreads, 1) gemv_stream_kernel(const GemvParams p, int* err) {
  constexpr int Bp = 8 * NB;
  constexpr int kXStage = kCH * Bp * 64;
  constexpr int kStage = kWStage + kXStage;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int KS = (p.KC + kCH - 1) / kCH;              // stage units per row group
  const int nrbg = (p.RB + 7) / 8;
  const long long U = (long long)nrbg * KS;
  const long long G = gridDim.x;
  const int u0 = (int)((long long)blockIdx.x * U / G);
  const int u1 = (int)((long long)(blockIdx.x + 1) * U / G);

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  bool dead = false;
  if (warp == kConsumerWarps) {
    // ---------------- producer ----------------
    uint64_t pol_w, pol_x;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(pol_w));
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;\n" : "=l"(pol_x));
    const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.W);
    const __nv_bfloat16* X = reinterpret_cast<const __nv_bfloat16*>(p.x);
    int it = 0;
    for (int u = u0; u < u1; ++u, ++it) {
      const int s = it % kStages, k = it / kStages;
      mbar_wait(&empty_bar[s], (k & 1) ^ 1, dead, err);
      const int r = u / KS, ks = u - r * KS;
      const int chunk0 = ks * kCH;
      const int nch = min(kCH, p.KC - chunk0);
      const int nrb = min(8, p.RB - r * 8);
      unsigned char* st = smem + s * kStage;
      if (lane == 0) mbar_expect_tx(&full_bar[s], (uint32_t)(nrb * nch * 1024 + nch * Bp * 64));
      __syncwarp();
      if (lane < nrb)
        bulk_g2s(st + lane * (kCH * 1024), W + ((int64_t)(r * 8 + lane) * p.KC + chunk0) * 512, (uint32_t)(nch * 1024),
                 &full_bar[s], pol_w);
      else if (lane == 8)
        bulk_g2s(st + kWStage, X + (int64_t)chunk0 * (Bp * 32), (uint32_t)(nch * Bp * 64), &full_bar[s], pol_x);
    }
    return;
  }

  // ---------------- consumers: warp w owns row block 8r + w of the current row group ----------------
  const int g = lane >> 2, t = lane & 3;
  float acc[NB][4];
  auto zero_acc = [&]() {
#pragma unroll
    for (int j = 0; j < NB; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  };
  // Fold the accumulators of row group r, which this CTA's unit range has just left.  Everything
  // is warp-local: alone -> epilogue; shared -> fragment to scratch, per-row-block counter, the
  // last contributor sums the fragments in CTA order and runs the epilogue.
  auto flush = [&](int r) {
    const int rb = r * 8 + warp;
    if (rb >= p.RB) return;
    const long long ua = (long long)r * KS, ub = ua + KS - 1;
    const int c_first = (int)(((ua + 1) * G + U - 1) / U) - 1;     // CTA of unit u: ceil((u+1)G/U) - 1
    const int c_last = (int)(((ub + 1) * G + U - 1) / U) - 1;
    const int n = c_last - c_first + 1;
    if (n > 1) {
      float4* part = reinterpret_cast<float4*>(p.partials) + (int64_t)rb * p.ksplit * (32 * NB);
      float4* mine = part + (int64_t)((int)blockIdx.x - c_first) * (32 * NB) + lane * NB;
#pragma unroll
      for (int nt = 0; nt < NB; ++nt) mine[nt] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
      __threadfence();
      __syncwarp();
      unsigned prev = 0;
      if (lane == 0) prev = atomicAdd(&p.counters[rb], 1u);
      prev = __shfl_sync(0xffffffffu, prev, 0);
      if (prev != (unsigned)n - 1u) return;
      if (lane == 0) p.counters[rb] = 0u;          // ready for the next launch
      __threadfence();
      zero_acc();
      for (int k0 = 0; k0 < n; k0 += 4) {
        float4 v[4][NB];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
          for (int nt = 0; nt < NB; ++nt)
            v[kk][nt] = (k0 + kk < n) ? __ldcg(part + (int64_t)(k0 + kk) * (32 * NB) + lane * NB + nt)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
          for (int nt = 0; nt < NB; ++nt) {
            acc[nt][0] += v[kk][nt].x; acc[nt][1] += v[kk][nt].y; acc[nt][2] += v[kk][nt].z; acc[nt][3] += v[kk][nt].w;
          }
      }
    }
    fragment_epilogue<NB>(p, acc, rb, g, t);
  };

  zero_acc();
  int seg_r = u0 < u1 ? u0 / KS : -1;
  int it = 0;
  for (int u = u0; u < u1; ++u, ++it) {
    const int r = u / KS, ks = u - r * KS;
    if (r != seg_r) {
      flush(seg_r);
      zero_acc();
      seg_r = r;
    }
    const int s = it % kStages, k = it / kStages;
    const int nch = min(kCH, p.KC - ks * kCH);
    mbar_wait(&full_bar[s], k & 1, dead, err);
    if (r * 8 + warp < p.RB) {
      const unsigned char* st = smem + s * kStage;
      const unsigned char* xst = st + kWStage + g * 64 + t * 16;
      const unsigned char* wst = st + warp * (kCH * 1024) + lane * 32;
#pragma unroll
      for (int c = 0; c < kCH; ++c) {
        if (c < nch) {
          const uint4 lo = *reinterpret_cast<const uint4*>(wst + c * 1024);
          const uint4 hi = *reinterpret_cast<const uint4*>(wst + c * 1024 + 16);
#pragma unroll
          for (int nt = 0; nt < NB; ++nt) {
            const uint4 bx = *reinterpret_cast<const uint4*>(xst + c * (Bp * 64) + nt * 512);
            mma_bf16(acc[nt], lo.x, hi.x, lo.y, hi.y, bx.x, bx.y);
            mma_bf16(acc[nt], lo.z, hi.z, lo.w, hi.w, bx.z, bx.w);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }
  if (seg_r >= 0) flush(seg_r);
}

template <typename WT, int NB, int MT, int STAGES>
int32_t launch_ring(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  constexpr int Bp = 8 * NB, RPC = 2 * MT * 16;
  const size_t xs_bytes = (size_t)p.kc_per_split * Bp * 32 * sizeof(WT);
  const size_t red_bytes = (size_t)4 * RPC * (Bp + 1) * sizeof(float);
  const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  LMB_REQUIRE(smem <= kMaxSmem, "gemv: %zu bytes of shared memory exceed the configured %zu", smem, kMaxSmem);
  dim3 grid((unsigned)ceil_div(p.RB, 2 * MT), (unsigned)p.ksplit);
  gemv_ring_kernel<WT, NB, MT, STAGES><<<grid, kRingThreads, smem, stream>>>(p);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

template <int NB>
constexpr size_t stream_smem() {
  return (size_t)kStages * (kWStage + kCH * 8 * NB * 64);
}

template <int NB>
int32_t launch_stream(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  gemv_stream_kernel<NB><<<p.grid, kStreamThreads, stream_smem<NB>(), stream>>>(p, ctx->dev_err);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

constexpr int kMtBf16 = 4;
constexpr int kMtF32 = 1;
constexpr size_t kMaxXsBytes = 96 * 1024;

}  // namespace

void gemv_set_stream_kernel(bool on) { g_use_stream = on; }

GemvPlan gemv_plan(const Ctx* ctx, int dtype, int B, int RB, int KC) {
  GemvPlan pl;
  const int Bp = batch_pad(B);
  if (dtype == LMB200_BF16 && g_use_stream) {
    const int KS = (int)ceil_div(KC, kCH);
    const int nrbg = (int)ceil_div(RB, 8);
    const int64_t U = (int64_t)nrbg * KS;
    int G = ctx->sm_count;
    if (G > U) G = (int)U;
    pl.grid = G;
    const int64_t upc_min = U / G;                       // >= 1
    pl.ksplit = (int)ceil_div(KS, upc_min) + 1;          // contributors reserved per row group
    pl.kc_per_split = KC;
    pl.partial_floats = (int64_t)nrbg * pl.ksplit * kRPC * Bp;    // [row block][contributor][16 x Bp fragment]
    pl.n_counters = nrbg * 8;
    return pl;
  }
  const int MT = dtype == LMB200_BF16 ? kMtBf16 : kMtF32;
  const int RPC = 2 * MT * 16;
  const size_t esz = dtype == LMB200_BF16 ? 2 : 4;
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

// Raise the dynamic shared-memory limit of every instantiation once per device, outside any
// stream capture.
int32_t gemv_configure() {
#define LMB_CFG(KERN, BYTES)                                                                           \
  LMB_CUDA(cudaFuncSetAttribute(KERN, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(BYTES)));     \
  LMB_CUDA(cudaFuncSetAttribute(KERN, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared))
  LMB_CFG((gemv_ring_kernel<__nv_bfloat16, 1, kMtBf16, 4>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<__nv_bfloat16, 2, kMtBf16, 4>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<__nv_bfloat16, 4, kMtBf16, 3>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<float, 1, kMtF32, 3>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<float, 2, kMtF32, 3>), kMaxSmem);
  LMB_CFG((gemv_ring_kernel<float, 4, kMtF32, 2>), kMaxSmem);
  LMB_CFG(gemv_stream_kernel<1>, stream_smem<1>());
  LMB_CFG(gemv_stream_kernel<2>, stream_smem<2>());
  LMB_CFG(gemv_stream_kernel<4>, stream_smem<4>());
#undef LMB_CFG
  return LMB200_OK;
}

int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream) {
  LMB_REQUIRE(p.B >= 1 && p.B <= 32, "gemv: batch %d outside 1..32", p.B);
  const int nb = batch_pad(p.B) / 8;
  if (dtype == LMB200_BF16 && g_use_stream) {
    LMB_REQUIRE(p.grid >= 1 && p.partials && p.counters, "gemv: stream kernel needs a plan and scratch");
    switch (nb) {
      case 1: return launch_stream<1>(ctx, p, stream);
      case 2: return launch_stream<2>(ctx, p, stream);
      default: return launch_stream<4>(ctx, p, stream);
    }
  }
  LMB_REQUIRE(p.ksplit >= 1 && p.kc_per_split >= 1 && (int64_t)p.ksplit * p.kc_per_split >= p.KC,
              "gemv: bad k split");
  LMB_REQUIRE(p.ksplit == 1 || (p.partials && p.counters), "gemv: split-K needs scratch");
  if (dtype == LMB200_BF16) {
    switch (nb) {
      case 1: return launch_ring<__nv_bfloat16, 1, kMtBf16, 4>(ctx, p, stream);
      case 2: return launch_ring<__nv_bfloat16, 2, kMtBf16, 4>(ctx, p, stream);
      default: return launch_ring<__nv_bfloat16, 4, kMtBf16, 3>(ctx, p, stream);
    }
  } else if (dtype == LMB200_F32) {
    switch (nb) {
      case 1: return launch_ring<float, 1, kMtF32, 3>(ctx, p, stream);
      case 2: return launch_ring<float, 2, kMtF32, 3>(ctx, p, stream);
      default: return launch_ring<float, 4, kMtF32, 2>(ctx, p, stream);
    }
  }
  return fail(LMB200_EINVAL, "gemv: dtype %d", dtype);
}

}  // namespace lmb
