// Bandwidth-bound decode GEMV with fused epilogues (store / SiLU-gate / RoPE + KV append).
//
// One CTA = 8 warps = 2 row groups x 4 k-warps and owns 2*MT 16-row blocks of the tiled weight
// matrix for one k-split.  The activation slice [B, Ks] is staged in shared memory once; the
// weights never touch shared memory: every lane streams its own 32 contiguous bytes of each
// 1 KB unit (evict-first) through a STAGES-deep register ring and feeds them straight to
// mma.sync m16n8k16 (bf16) or to fp32 FMAs (the float32 parity path).  Partial tiles of the 4
// k-warps are summed through shared memory; with ksplit > 1 the CTAs of one row group leave
// their tiles in global scratch and the last one to arrive (a counter) sums them in fixed
// order, so results do not depend on scheduling.
#include <type_traits>

#include "gemv.cuh"

namespace lmb {

namespace {

constexpr int kThreads = 256;
constexpr size_t kMaxSmem = 112 * 1024;
constexpr float kInvLn2 = 1.4426950408889634f;      // Float32(1/log(2)) as the reference rounds it
constexpr float kHalfPi = 1.5707963267948966f;

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename WT> struct Unit;   // 16 rows x 32 k of weights as seen by one lane
template <> struct Unit<__nv_bfloat16> { uint4 v[2]; };
template <> struct Unit<float> { uint4 v[4]; };

template <typename WT>
__device__ __forceinline__ void load_unit(Unit<WT>& u, const WT* W, int64_t rb, int KC, int kc, int lane) {
  constexpr int N = sizeof(Unit<WT>) / 16;
  const uint4* p = reinterpret_cast<const uint4*>(W + ((rb * KC + kc) * 32 + lane) * 16);
#pragma unroll
  for (int i = 0; i < N; ++i) u.v[i] = ld_stream(p + i);
}
template <typename WT>
__device__ __forceinline__ void zero_unit(Unit<WT>& u) {
  constexpr int N = sizeof(Unit<WT>) / 16;
#pragma unroll
  for (int i = 0; i < N; ++i) u.v[i] = make_uint4(0, 0, 0, 0);
}

template <typename WT, int NB, int MT, int STAGES>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvParams p) {
  constexpr int Bp = 8 * NB;
  constexpr int RPC = 2 * MT * 16;
  constexpr bool kBf16 = std::is_same<WT, __nv_bfloat16>::value;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  WT* xs = reinterpret_cast<WT*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw);
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rg = warp >> 2, kw = warp & 3;
  const int kc0 = blockIdx.y * p.kc_per_split;
  const int kc1 = min(p.KC, kc0 + p.kc_per_split);
  const int Ks = (kc1 - kc0) * 32;
  const int xs_pitch = kBf16 ? (Ks + ((Ks & 63) == 32 ? 0 : 32)) : Ks + 4;
  const int64_t rb_base = (int64_t)blockIdx.x * (2 * MT) + rg * MT;
  const WT* W = reinterpret_cast<const WT*>(p.W);

  // prefetch the first weight units before touching the activations
  Unit<WT> ring[STAGES][MT];
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    const int kc = kc0 + kw + 4 * s;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (kc < kc1 && rb_base + mt < p.RB) load_unit<WT>(ring[s][mt], W, rb_base + mt, p.KC, kc, lane);
      else zero_unit<WT>(ring[s][mt]);
    }
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt) zero_unit<WT>(ring[STAGES - 1][mt]);

  // stage x[:, kc0*32 .. kc1*32) into shared memory, rows >= B zero
  {
    constexpr int EPV = 16 / sizeof(WT);
    const int vec_per_row = Ks / EPV;
    const WT* x = reinterpret_cast<const WT*>(p.x);
    for (int i = tid; i < Bp * vec_per_row; i += kThreads) {
      const int b = i / vec_per_row, v = i - b * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (b < p.B) val = *reinterpret_cast<const uint4*>(x + (int64_t)b * p.x_pitch + kc0 * 32 + v * EPV);
      *reinterpret_cast<uint4*>(xs + b * xs_pitch + v * EPV) = val;
    }
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
        {  // refill the slot freed by the previous iteration
          const int nxt = cur + 4 * (STAGES - 1);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (nxt < kc1 && rb_base + mt < p.RB)
              load_unit<WT>(ring[(s + STAGES - 1) % STAGES][mt], W, rb_base + mt, p.KC, nxt, lane);
          }
        }
        const int koff = (cur - kc0) * 32 + 8 * t;
        if constexpr (kBf16) {
          uint4 bx[NB];
#pragma unroll
          for (int nt = 0; nt < NB; ++nt)
            bx[nt] = *reinterpret_cast<const uint4*>(xs + (8 * nt + g) * xs_pitch + koff);
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
              const float4 x0 = *reinterpret_cast<const float4*>(xs + c * xs_pitch + koff);
              const float4 x1 = *reinterpret_cast<const float4*>(xs + c * xs_pitch + koff + 4);
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
  for (int i = tid; i < RPC * Bp; i += kThreads) {
    const int r = i / Bp, b = i - r * Bp, o = r * RP + b;
    red[o] = (red[o] + red[SLAB + o]) + (red[2 * SLAB + o] + red[3 * SLAB + o]);
  }
  if (p.ksplit > 1) {
    float* my_part = p.partials + ((int64_t)blockIdx.x * p.ksplit + blockIdx.y) * (RPC * Bp);
    for (int i = tid; i < RPC * Bp; i += kThreads) {
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
    const float* part = p.partials + (int64_t)blockIdx.x * p.ksplit * (RPC * Bp);
    for (int i = tid; i < RPC * Bp; i += kThreads) {
      const int r = i / Bp, b = i - r * Bp;
      float s = 0.f;
      for (int k = 0; k < p.ksplit; ++k) s += __ldcg(part + (int64_t)k * (RPC * Bp) + i);
      red[r * RP + b] = s;
    }
  }
  __syncthreads();
  auto tile = [&](int r, int b) -> float { return red[r * RP + b]; };

  const int row0 = blockIdx.x * RPC;
  if (p.epi == EPI_STORE_F32) {
    for (int i = tid; i < RPC * Bp; i += kThreads) {
      const int b = i / RPC, r = i - b * RPC;
      const int row = row0 + r;
      if (b < p.B && row < p.rows) p.out[(int64_t)b * p.out_pitch + row] = tile(r, b);
    }
  } else if (p.epi == EPI_SILU_GATE) {
    WT* act = reinterpret_cast<WT*>(p.act);
    for (int i = tid; i < (RPC / 2) * Bp; i += kThreads) {
      const int b = i / (RPC / 2), j = i - b * (RPC / 2);
      const int m = j >> 3, r = j & 7;
      const int o = row0 / 2 + j;
      if (b < p.B && o < p.n_act) {
        const float a = tile(16 * m + r, b), u = tile(16 * m + r + 8, b);
        // silu(a) = a * (1 / (1 + exp2((a * -1) * (1/ln2))))     src/HighLevelOps.jl:153-160
        const float e = exp2f((a * -1.0f) * kInvLn2);
        const float sg = 1.0f / (1.0f + e);
        act[(int64_t)b * p.act_pitch + o] = from_f32<WT>((a * sg) * u);
      }
    }
  } else {  // EPI_QKV_ROPE
    WT* q_out = reinterpret_cast<WT*>(p.q_out);
    WT* kv = reinterpret_cast<WT*>(p.kv_layer);
    const int D = p.D, tiles_per_head = D >> 4, half = D >> 1;
    const int pos = *p.pos;
    const float fpos = (float)pos;
    for (int i = tid; i < (RPC / 2) * Bp; i += kThreads) {
      const int b = i / (RPC / 2), j = i - b * (RPC / 2);
      const int m = j >> 3, r = j & 7;
      const int gt = row0 / 16 + m;                  // global 16-row tile
      if (b >= p.B || gt >= p.RB) continue;
      const int hs = gt / tiles_per_head, jj = gt - hs * tiles_per_head;
      const float v0 = tile(16 * m + r, b), v1 = tile(16 * m + r + 8, b);
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

template <typename WT, int NB, int MT, int STAGES>
int32_t launch_t(Ctx* ctx, const GemvParams& p, cudaStream_t stream) {
  constexpr int Bp = 8 * NB, RPC = 2 * MT * 16;
  const int Ks = p.kc_per_split * 32;
  const size_t xs_bytes = (size_t)Bp * (Ks + 32) * sizeof(WT);
  const size_t red_bytes = (size_t)4 * RPC * (Bp + 1) * sizeof(float);
  const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  auto kern = gemv_kernel<WT, NB, MT, STAGES>;
  LMB_REQUIRE(smem <= kMaxSmem, "gemv: %zu bytes of shared memory exceed the configured %zu", smem, kMaxSmem);
  dim3 grid((unsigned)ceil_div(p.RB, 2 * MT), (unsigned)p.ksplit);
  kern<<<grid, kThreads, smem, stream>>>(p);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  return LMB200_OK;
}

constexpr int kMtBf16 = 4;
constexpr int kMtF32 = 1;
constexpr size_t kMaxXsBytes = 96 * 1024;

}  // namespace

void gemv_plan(const Ctx* ctx, int dtype, int B, int RB, int KC, int* ksplit, int* kc_per_split,
               int64_t* partial_floats, int* n_counters) {
  const int MT = dtype == LMB200_BF16 ? kMtBf16 : kMtF32;
  const int NB = B <= 8 ? 1 : (B <= 16 ? 2 : 4);
  const int Bp = 8 * NB, RPC = 2 * MT * 16;
  const size_t esz = dtype == LMB200_BF16 ? 2 : 4;
  const int nrbg = (int)ceil_div(RB, 2 * MT);
  // One CTA per SM is resident (register ring).  Pick the k-split that minimises
  //   waves * (chunks per CTA + fixed cost of staging x and the epilogue, in chunk units)
  // with the activation slice fitting shared memory and at least one chunk per k-warp.
  const int per_max = (int)(kMaxXsBytes / (Bp * esz) / 32) - 1;
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
  int ks = best_ks, per = best_per;
  *ksplit = ks;
  *kc_per_split = per;
  *partial_floats = ks > 1 ? (int64_t)nrbg * ks * RPC * Bp : 0;
  *n_counters = nrbg;
}

// Raise the dynamic shared-memory limit of every instantiation once per device, outside any
// stream capture.
int32_t gemv_configure() {
#define LMB_CFG(...)                                                                              \
  LMB_CUDA(cudaFuncSetAttribute(gemv_kernel<__VA_ARGS__>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                (int)kMaxSmem))
  LMB_CFG(__nv_bfloat16, 1, kMtBf16, 4);
  LMB_CFG(__nv_bfloat16, 2, kMtBf16, 4);
  LMB_CFG(__nv_bfloat16, 4, kMtBf16, 3);
  LMB_CFG(float, 1, kMtF32, 3);
  LMB_CFG(float, 2, kMtF32, 3);
  LMB_CFG(float, 4, kMtF32, 2);
#undef LMB_CFG
  return LMB200_OK;
}

int32_t gemv_launch(Ctx* ctx, int dtype, GemvParams p, cudaStream_t stream) {
  LMB_REQUIRE(p.B >= 1 && p.B <= 32, "gemv: batch %d outside 1..32", p.B);
  LMB_REQUIRE(p.ksplit >= 1 && p.kc_per_split >= 1 && (int64_t)p.ksplit * p.kc_per_split >= p.KC,
              "gemv: bad k split");
  LMB_REQUIRE(p.ksplit == 1 || (p.partials && p.counters), "gemv: split-K needs scratch");
  const int nb = p.B <= 8 ? 1 : (p.B <= 16 ? 2 : 4);
  if (dtype == LMB200_BF16) {
    switch (nb) {
      case 1: return launch_t<__nv_bfloat16, 1, kMtBf16, 4>(ctx, p, stream);
      case 2: return launch_t<__nv_bfloat16, 2, kMtBf16, 4>(ctx, p, stream);
      default: return launch_t<__nv_bfloat16, 4, kMtBf16, 3>(ctx, p, stream);
    }
  } else if (dtype == LMB200_F32) {
    switch (nb) {
      case 1: return launch_t<float, 1, kMtF32, 3>(ctx, p, stream);
      case 2: return launch_t<float, 2, kMtF32, 3>(ctx, p, stream);
      default: return launch_t<float, 4, kMtF32, 2>(ctx, p, stream);
    }
  }
  return fail(LMB200_EINVAL, "gemv: dtype %d", dtype);
}

}  // namespace lmb
