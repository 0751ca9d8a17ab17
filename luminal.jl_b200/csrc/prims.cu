// Primitive graph ops on float32 row-major device tensors: what the reference's execute_op!
// dispatches to, one call per node (src/Execution.jl:216-371, 580-618), plus the stand-alone
// forms of the fused layer ops.  These are the op-by-op path of execute() on the B200 device;
// the decode session does not go through them.
#include <math.h>

#include "common.cuh"

namespace lmb {
namespace {

constexpr int kMaxRank = 8;
constexpr float kInvLn2 = 1.4426950408889634f;
constexpr float kHalfPi = 1.5707963267948966f;

struct Idx {
  int rank;
  int64_t out_d[kMaxRank];
  int64_t sa[kMaxRank], sb[kMaxRank], sc[kMaxRank];   // operand strides (0 = broadcast)
};

__device__ __forceinline__ float apply_op(int op, float a, float b, float c) {
  switch (op) {
    case LMB200_OP_ADD: return a + b;
    case LMB200_OP_MUL: return a * b;
    case LMB200_OP_MOD: return fmodf(a, b);
    case LMB200_OP_LESSTHAN: return a < b ? 1.0f : 0.0f;
    case LMB200_OP_MAX: return fmaxf(a, b);
    case LMB200_OP_LOG2: return log2f(a);
    case LMB200_OP_EXP2: return exp2f(a);
    case LMB200_OP_SIN: return sinf(a);
    case LMB200_OP_COS: return cosf(a);
    case LMB200_OP_SQRT: return sqrtf(a);
    case LMB200_OP_RECIP: return 1.0f / a;
    case LMB200_OP_RELU: return fmaxf(a, 0.0f);
    case LMB200_OP_COPY: return a;
    case LMB200_OP_FUSED_MUL_ADD: return __fadd_rn(__fmul_rn(a, b), c);   // (a .* b) .+ c, two roundings
    case LMB200_OP_FUSED_ADD_RELU: return fmaxf(a + b, 0.0f);
  }
  return 0.f;
}

__global__ void ew_kernel(int op, float* out, const float* a, const float* b, const float* c, Idx ix, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = o, oa = 0, ob = 0, oc = 0;
    for (int k = ix.rank - 1; k >= 0; --k) {
      const int64_t i = rem % ix.out_d[k];
      rem /= ix.out_d[k];
      oa += i * ix.sa[k]; ob += i * ix.sb[k]; oc += i * ix.sc[k];
    }
    out[o] = apply_op(op, a ? a[oa] : 0.f, b ? b[ob] : 0.f, c ? c[oc] : 0.f);
  }
}

// One element-wise fusion group per launch: a postfix program over up to 8 broadcast inputs,
// interpreted per output element with every operation rounded to float32 on its own (no
// contraction), so the result equals running the group's nodes one by one.
// Stands in for FusedElementwiseOp (src/Compiler.jl:323-357, executor src/Execution.jl:552-563).
constexpr int kFusedMaxInputs = 8, kFusedMaxInstr = 64, kFusedMaxStack = 16;
enum FusedOp { F_PUSH_IN = 0, F_PUSH_CONST = 1, F_ADD = 2, F_MUL = 3, F_MOD = 4, F_LT = 5, F_MAX = 6, F_LOG2 = 7, F_EXP2 = 8,
               F_SIN = 9, F_COS = 10, F_SQRT = 11, F_RECIP = 12, F_RELU = 13, F_FMA = 14, F_ADD_RELU = 15 };
struct FusedProgram {
  int n_in, n_instr, rank;
  int64_t out_d[kMaxRank];
  int64_t st[kFusedMaxInputs][kMaxRank];      // input strides over the output's axes (0 = broadcast)
  const float* in[kFusedMaxInputs];
  int op[kFusedMaxInstr];
  float arg[kFusedMaxInstr];                  // PUSH_IN: input index; PUSH_CONST: the value
};
__global__ void fused_ew_kernel(float* out, const FusedProgram pg, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t off[kFusedMaxInputs];
#pragma unroll
    for (int i = 0; i < kFusedMaxInputs; ++i) off[i] = 0;
    int64_t rem = o;
    for (int k = pg.rank - 1; k >= 0; --k) {
      const int64_t idx = rem % pg.out_d[k];
      rem /= pg.out_d[k];
#pragma unroll
      for (int i = 0; i < kFusedMaxInputs; ++i)
        if (i < pg.n_in) off[i] += idx * pg.st[i][k];
    }
    float stack[kFusedMaxStack];
    int sp = 0;
    for (int pc = 0; pc < pg.n_instr; ++pc) {
      const int op = pg.op[pc];
      if (op == F_PUSH_IN) { const int i = (int)pg.arg[pc]; stack[sp++] = pg.in[i][off[i]]; continue; }
      if (op == F_PUSH_CONST) { stack[sp++] = pg.arg[pc]; continue; }
      if (op == F_FMA) {
        const float c = stack[--sp], b = stack[--sp], a = stack[sp - 1];
        stack[sp - 1] = __fadd_rn(__fmul_rn(a, b), c);
        continue;
      }
      if (op >= F_LOG2 && op <= F_RELU) {
        const float a = stack[sp - 1];
        float r = a;
        switch (op) {
          case F_LOG2: r = log2f(a); break;
          case F_EXP2: r = exp2f(a); break;
          case F_SIN: r = sinf(a); break;
          case F_COS: r = cosf(a); break;
          case F_SQRT: r = sqrtf(a); break;
          case F_RECIP: r = 1.0f / a; break;
          case F_RELU: r = fmaxf(a, 0.0f); break;
        }
        stack[sp - 1] = r;
        continue;
      }
      const float b = stack[--sp], a = stack[sp - 1];
      float r = 0.f;
      switch (op) {
        case F_ADD: r = __fadd_rn(a, b); break;
        case F_MUL: r = __fmul_rn(a, b); break;
        case F_MOD: r = fmodf(a, b); break;
        case F_LT: r = a < b ? 1.0f : 0.0f; break;
        case F_MAX: r = fmaxf(a, b); break;
        case F_ADD_RELU: r = fmaxf(__fadd_rn(a, b), 0.0f); break;
      }
      stack[sp - 1] = r;
    }
    out[o] = stack[0];
  }
}

// out[o] = in[offset + sum idx_k * stride_k] over the OUT shape: permute / expand / slice
struct Gather {
  int rank;
  int64_t out_d[kMaxRank];
  int64_t st[kMaxRank];
  int64_t offset;
};
__global__ void strided_copy_kernel(float* out, const float* in, Gather gt, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = o, src = gt.offset;
    for (int k = gt.rank - 1; k >= 0; --k) {
      const int64_t i = rem % gt.out_d[k];
      rem /= gt.out_d[k];
      src += i * gt.st[k];
    }
    out[o] = in[src];
  }
}

struct Pad {
  int rank;
  int64_t out_d[kMaxRank], in_d[kMaxRank], left[kMaxRank];
};
__global__ void pad_kernel(float* out, const float* in, Pad pd, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = o, src = 0, mul = 1;
    bool inside = true;
    for (int k = pd.rank - 1; k >= 0; --k) {
      const int64_t i = rem % pd.out_d[k] - pd.left[k];
      rem /= pd.out_d[k];
      if (i < 0 || i >= pd.in_d[k]) inside = false;
      src += i * mul;
      mul *= pd.in_d[k];
    }
    out[o] = inside ? in[src] : 0.f;
  }
}

// column-major-order-preserving reshape between two row-major tensors
struct Reshape {
  int in_rank, out_rank;
  int64_t in_d[kMaxRank], out_d[kMaxRank];
};
__global__ void reshape_cm_kernel(float* out, const float* in, Reshape rs, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    // row-major index of out -> multi-index -> column-major linear index
    int64_t rem = o, lin = 0;
    int64_t idx[kMaxRank];
    for (int k = rs.out_rank - 1; k >= 0; --k) { idx[k] = rem % rs.out_d[k]; rem /= rs.out_d[k]; }
    int64_t mul = 1;
    for (int k = 0; k < rs.out_rank; ++k) { lin += idx[k] * mul; mul *= rs.out_d[k]; }
    // column-major linear index -> multi-index of in -> row-major offset
    int64_t src = 0;
    for (int k = 0; k < rs.in_rank; ++k) { idx[k] = lin % rs.in_d[k]; lin /= rs.in_d[k]; }
    for (int k = 0; k < rs.in_rank; ++k) src = src * rs.in_d[k] + idx[k];
    out[o] = in[src];
  }
}

// reduce over one axis: in viewed as [outer, n, inner]
__global__ void reduce_kernel(int kind, float* out, const float* in, int64_t outer, int64_t n, int64_t inner) {
  const int64_t total = outer * inner;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t a = o / inner, c = o - a * inner;
    const float* p = in + a * n * inner + c;
    float acc = kind == LMB200_REDUCE_SUM ? 0.f : -INFINITY;
    for (int64_t i = 0; i < n; ++i) {
      const float v = p[i * inner];
      acc = kind == LMB200_REDUCE_SUM ? acc + v : fmaxf(acc, v);
    }
    out[o] = acc;
  }
}

// C[bt] = A[bt] (MxK) * B[bt] (KxN), 32x32 tiles, plain fp32 FMAs
__global__ void __launch_bounds__(1024) matmul_kernel(float* C, const float* A, const float* Bm, int M, int N, int K,
                                                      int64_t sA, int64_t sB, int64_t sC) {
  __shared__ float As[32][33], Bs[32][33];
  const int bt = blockIdx.z;
  const float* a = A + bt * sA;
  const float* b = Bm + bt * sB;
  float* c = C + bt * sC;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int row = blockIdx.y * 32 + ty, col = blockIdx.x * 32 + tx;
  float acc = 0.f;
  for (int k0 = 0; k0 < K; k0 += 32) {
    As[ty][tx] = (row < M && k0 + tx < K) ? a[(int64_t)row * K + k0 + tx] : 0.f;
    Bs[ty][tx] = (k0 + ty < K && col < N) ? b[(int64_t)(k0 + ty) * N + col] : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; ++k) acc = fmaf(As[ty][k], Bs[k][tx], acc);
    __syncthreads();
  }
  if (row < M && col < N) c[(int64_t)row * N + col] = acc;
}

__global__ void gather_kernel(float* out, const float* table, int64_t vocab, int64_t dim, const float* ids, int64_t n_ids) {
  const int64_t total = n_ids * dim;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = o / dim, c = o - r * dim;
    const int64_t id = (int64_t)ids[r];
    out[o] = (id >= 0 && id < vocab) ? table[id * dim + c] : 0.f;
  }
}

// im2col of the last axis: out[bc, o, k] = a[bc, o*stride + k*dilation]   (src/Execution.jl:481-504)
__global__ void unfold1d_kernel(float* out, const float* a, int64_t BC, int64_t Lin, int64_t O, int64_t K, int64_t stride,
                                int64_t dilation) {
  const int64_t total = BC * O * K;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t k = i % K, o = (i / K) % O, bc = i / (K * O);
    out[i] = a[bc * Lin + o * stride + k * dilation];
  }
}

__global__ void cumsum_kernel(float* out, const float* in, int64_t rows, int64_t n) {
  const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float acc = 0.f;
  for (int64_t i = 0; i < n; ++i) { acc += in[r * n + i]; out[r * n + i] = acc; }
}

// mode 0: RMSNorm(+scale); mode 1: LayerNorm (mean-centred, optional w and bias)
__global__ void __launch_bounds__(256) norm_kernel(float* y, const float* x, const float* w, const float* bias,
                                                   int64_t n, float eps, int mean_centre) {
  __shared__ float red[8];
  const int tid = threadIdx.x;
  const float* xr = x + blockIdx.x * n;
  float* yr = y + blockIdx.x * n;
  auto block_sum = [&](float v) -> float {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i];
    return t;
  };
  float mean = 0.f;
  if (mean_centre) {
    float s = 0.f;
    for (int64_t i = tid; i < n; i += 256) s += xr[i];
    mean = block_sum(s) * (1.0f / (float)n);
  }
  float ss = 0.f;
  for (int64_t i = tid; i < n; i += 256) { const float v = xr[i] + mean * -1.0f; ss += v * v; }
  const float var = block_sum(ss) * (1.0f / (float)n);
  const float inv = 1.0f / sqrtf(var + eps);
  for (int64_t i = tid; i < n; i += 256) {
    float v = (xr[i] + mean * -1.0f) * inv;
    if (w) v = v * w[i];
    if (bias) v = v + bias[i];
    yr[i] = v;
  }
}

__global__ void silu_gate_kernel(float* out, const float* gate, const float* up, int64_t n) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < n; o += (int64_t)gridDim.x * blockDim.x) {
    const float a = gate[o];
    const float e = exp2f((a * -1.0f) * kInvLn2);
    const float sg = 1.0f / (1.0f + e);
    out[o] = (a * sg) * up[o];
  }
}

__global__ void rope_kernel(float* out, const float* x, int64_t BH, int64_t S, int64_t D, int64_t prev_seq, float l2base) {
  const int64_t half = D / 2;
  const int64_t total = BH * S * half;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = o % half, s = (o / half) % S, bh = o / (half * S);
    // inv_freq = recip(exp2((i*2*(1/D)) * log2(base)));  angle = (s + prev) * inv_freq
    const float fr = __fmul_rn(__fmul_rn(__fmul_rn((float)i, 2.0f), 1.0f / (float)D), l2base);
    const float inv = 1.0f / exp2f(fr);
    const float ang = __fmul_rn((float)s + (float)prev_seq, inv);
    const float sn = sinf(ang), cs = sinf(kHalfPi + ang * -1.0f);
    const float* xr = x + (bh * S + s) * D;
    float* yr = out + (bh * S + s) * D;
    const float x0 = xr[i], x1 = xr[i + half];
    yr[i] = x0 * cs + (x1 * sn) * -1.0f;
    yr[i + half] = x0 * sn + x1 * cs;
  }
}

__global__ void __launch_bounds__(256) argmax_kernel(int32_t* out, const float* x, int64_t n) {
  __shared__ float sv[256];
  __shared__ int si[256];
  const int tid = threadIdx.x;
  const float* row = x + blockIdx.x * n;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int64_t i = tid; i < n; i += 256) {
    const float v = row[i];
    if (v > best || (v == best && (int)i < bi)) { best = v; bi = (int)i; }
  }
  sv[tid] = best; si[tid] = bi;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (tid < off) {
      const float v = sv[tid + off];
      const int i = si[tid + off];
      if (v > sv[tid] || (v == sv[tid] && i < si[tid])) { sv[tid] = v; si[tid] = i; }
    }
    __syncthreads();
  }
  if (tid == 0) out[blockIdx.x] = si[0];
}

int grid_for(int64_t total) {
  int64_t g = ceil_div(total, 256);
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return (int)g;
}

int32_t check_dims(int32_t rank, const int64_t* dims, int64_t* total) {
  LMB_REQUIRE(rank >= 0 && rank <= kMaxRank, "rank %d outside 0..%d", rank, kMaxRank);
  LMB_REQUIRE(rank == 0 || dims, "null dims");
  int64_t t = 1;
  for (int i = 0; i < rank; ++i) {
    LMB_REQUIRE(dims[i] >= 1, "dimension %d is %lld", i, (long long)dims[i]);
    t *= dims[i];
  }
  *total = t;
  return LMB200_OK;
}

// strides of an operand broadcast against out (1-dims prepended, src/Execution.jl:207-214)
int32_t bcast_strides(int out_rank, const int64_t* out_d, int rank, const int64_t* d, int64_t* st, const char* what) {
  LMB_REQUIRE(rank <= out_rank, "%s: operand rank %d above output rank %d", what, rank, out_rank);
  const int shift = out_rank - rank;
  int64_t mul = 1;
  for (int k = out_rank - 1; k >= 0; --k) {
    const int j = k - shift;
    if (j < 0) { st[k] = 0; continue; }
    if (d[j] == out_d[k]) { st[k] = d[j] == 1 ? 0 : mul; }
    else if (d[j] == 1) st[k] = 0;
    else return fail(LMB200_EINVAL, "%s: dimension mismatch in broadcasting: %lld vs %lld", what, (long long)d[j],
                     (long long)out_d[k]);
    mul *= d[j];
  }
  return LMB200_OK;
}

}  // namespace
}  // namespace lmb

using namespace lmb;

#define CTX_OR_FAIL()                  \
  Ctx* ctx = ctx_from(h);              \
  if (!ctx) return LMB200_EINVAL;      \
  LMB_CUDA(cudaSetDevice(ctx->device))

#define LAUNCHED()          \
  ctx->launches++;          \
  LMB_CUDA(cudaGetLastError())

extern "C" int32_t lmb200_ew(lmb200_ctx h, int32_t opcode, float* out, int32_t out_rank, const int64_t* out_dims,
                             const float* a, int32_t a_rank, const int64_t* a_dims, const float* b, int32_t b_rank,
                             const int64_t* b_dims, const float* c, int32_t c_rank, const int64_t* c_dims) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && a, "ew: null pointer");
  const bool binary = opcode <= LMB200_OP_MAX || opcode >= LMB200_OP_FUSED_MUL_ADD;
  const bool ternary = opcode == LMB200_OP_FUSED_MUL_ADD;
  LMB_REQUIRE((opcode >= 0 && opcode <= LMB200_OP_MAX) || (opcode >= LMB200_OP_LOG2 && opcode <= LMB200_OP_FUSED_ADD_RELU),
              "ew: opcode %d", opcode);
  LMB_REQUIRE(!binary || b, "ew: opcode %d needs operand b", opcode);
  LMB_REQUIRE(!ternary || c, "ew: opcode %d needs operand c", opcode);
  Idx ix{};
  int64_t total, tmp;
  LMB_TRY(check_dims(out_rank, out_dims, &total));
  ix.rank = out_rank;
  for (int i = 0; i < out_rank; ++i) ix.out_d[i] = out_dims[i];
  LMB_TRY(check_dims(a_rank, a_dims, &tmp));
  LMB_TRY(bcast_strides(out_rank, out_dims, a_rank, a_dims, ix.sa, "ew a"));
  if (binary) {
    LMB_TRY(check_dims(b_rank, b_dims, &tmp));
    LMB_TRY(bcast_strides(out_rank, out_dims, b_rank, b_dims, ix.sb, "ew b"));
  }
  if (ternary) {
    LMB_TRY(check_dims(c_rank, c_dims, &tmp));
    LMB_TRY(bcast_strides(out_rank, out_dims, c_rank, c_dims, ix.sc, "ew c"));
  }
  ew_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(opcode, out, a, binary ? b : nullptr, ternary ? c : nullptr, ix, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_fused_ew(lmb200_ctx h, float* out, int32_t out_rank, const int64_t* out_dims, int32_t n_inputs,
                                   const float* const* inputs, const int32_t* in_ranks, const int64_t* in_dims,
                                   int32_t n_instr, const int32_t* ops, const float* args) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && ops && args && in_ranks && n_inputs >= 0 && (n_inputs == 0 || (inputs && in_dims)), "fused_ew: null pointer");
  LMB_REQUIRE(n_inputs <= kFusedMaxInputs, "fused_ew: %d inputs (at most %d)", n_inputs, kFusedMaxInputs);
  LMB_REQUIRE(n_instr >= 1 && n_instr <= kFusedMaxInstr, "fused_ew: %d instructions (1..%d)", n_instr, kFusedMaxInstr);
  FusedProgram pg{};
  int64_t total, tmp;
  LMB_TRY(check_dims(out_rank, out_dims, &total));
  pg.rank = out_rank; pg.n_in = n_inputs; pg.n_instr = n_instr;
  for (int i = 0; i < out_rank; ++i) pg.out_d[i] = out_dims[i];
  const int64_t* d = in_dims;
  for (int i = 0; i < n_inputs; ++i) {
    LMB_REQUIRE(inputs[i], "fused_ew: input %d is null", i);
    LMB_TRY(check_dims(in_ranks[i], d, &tmp));
    LMB_TRY(bcast_strides(out_rank, out_dims, in_ranks[i], d, pg.st[i], "fused_ew input"));
    pg.in[i] = inputs[i];
    d += in_ranks[i];
  }
  int depth = 0;                                   // the program must be well-formed postfix: checked here, not on the device
  for (int pc = 0; pc < n_instr; ++pc) {
    const int op = ops[pc];
    LMB_REQUIRE(op >= F_PUSH_IN && op <= F_ADD_RELU, "fused_ew: opcode %d at %d", op, pc);
    int need = 0, push = 1;
    if (op == F_PUSH_IN) LMB_REQUIRE(args[pc] >= 0 && (int)args[pc] < n_inputs && (float)(int)args[pc] == args[pc], "fused_ew: input index at %d", pc);
    if (op == F_FMA) need = 3;
    else if (op >= F_LOG2 && op <= F_RELU) need = 1;
    else if (op >= F_ADD) need = 2;
    LMB_REQUIRE(depth >= need, "fused_ew: stack underflow at instruction %d", pc);
    depth += push - need;
    LMB_REQUIRE(depth <= kFusedMaxStack, "fused_ew: stack deeper than %d at instruction %d", kFusedMaxStack, pc);
    pg.op[pc] = op; pg.arg[pc] = args[pc];
  }
  LMB_REQUIRE(depth == 1, "fused_ew: the program leaves %d values", depth);
  if (total == 0) return LMB200_OK;
  fused_ew_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(out, pg, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_reduce(lmb200_ctx h, int32_t kind, float* out, const float* in, int32_t rank,
                                 const int64_t* dims, int32_t axis) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in, "reduce: null pointer");
  LMB_REQUIRE(kind == LMB200_REDUCE_SUM || kind == LMB200_REDUCE_MAX, "reduce: kind %d", kind);
  int64_t total;
  LMB_TRY(check_dims(rank, dims, &total));
  LMB_REQUIRE(axis >= 0 && axis < rank, "reduce: axis %d of rank %d", axis, rank);
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < axis; ++i) outer *= dims[i];
  for (int i = axis + 1; i < rank; ++i) inner *= dims[i];
  reduce_kernel<<<grid_for(outer * inner), 256, 0, ctx->stream>>>(kind, out, in, outer, dims[axis], inner);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_matmul(lmb200_ctx h, float* out, const float* a, int32_t a_rank, const int64_t* a_dims,
                                 const float* b, int32_t b_rank, const int64_t* b_dims) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && a && b, "matmul: null pointer");
  int64_t ta, tb;
  LMB_TRY(check_dims(a_rank, a_dims, &ta));
  LMB_TRY(check_dims(b_rank, b_dims, &tb));
  // the four cases of batch_matmul (src/Execution.jl:12-54); anything else is the reference's error
  const bool ok = (a_rank == 2 && b_rank == 2) || (a_rank == 3 && b_rank == 2) || (a_rank == 3 && b_rank == 3) ||
                  (a_rank == 4 && b_rank == 4);
  LMB_REQUIRE(ok, "Batch matmul not implemented for %dD and %dD", a_rank, b_rank);
  const int64_t M = a_dims[a_rank - 2], K = a_dims[a_rank - 1], N = b_dims[b_rank - 1];
  LMB_REQUIRE(b_dims[b_rank - 2] == K, "matmul: inner dimensions %lld vs %lld", (long long)K, (long long)b_dims[b_rank - 2]);
  int64_t batch = 1;
  for (int i = 0; i < a_rank - 2; ++i) batch *= a_dims[i];
  if (b_rank > 2)
    for (int i = 0; i < b_rank - 2; ++i)
      LMB_REQUIRE(a_dims[i] == b_dims[i], "Batch dimensions must match: %lld vs %lld", (long long)a_dims[i], (long long)b_dims[i]);
  LMB_REQUIRE(batch <= 65535, "matmul: batch %lld too large", (long long)batch);
  dim3 grid((unsigned)ceil_div(N, 32), (unsigned)ceil_div(M, 32), (unsigned)batch);
  matmul_kernel<<<grid, dim3(32, 32), 0, ctx->stream>>>(out, a, b, (int)M, (int)N, (int)K, M * K, b_rank > 2 ? K * N : 0, M * N);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_permute(lmb200_ctx h, float* out, const float* in, int32_t rank, const int64_t* in_dims,
                                  const int32_t* perm) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in && perm, "permute: null pointer");
  int64_t total;
  LMB_TRY(check_dims(rank, in_dims, &total));
  int64_t in_st[kMaxRank];
  int64_t mul = 1;
  for (int k = rank - 1; k >= 0; --k) { in_st[k] = mul; mul *= in_dims[k]; }
  Gather gt{};
  gt.rank = rank;
  bool seen[kMaxRank] = {false};
  for (int k = 0; k < rank; ++k) {
    LMB_REQUIRE(perm[k] >= 0 && perm[k] < rank && !seen[perm[k]], "permute: bad permutation");
    seen[perm[k]] = true;
    gt.out_d[k] = in_dims[perm[k]];
    gt.st[k] = in_st[perm[k]];
  }
  strided_copy_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(out, in, gt, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_reshape_colmajor(lmb200_ctx h, float* out, const float* in, int32_t in_rank,
                                           const int64_t* in_dims, int32_t out_rank, const int64_t* out_dims) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in, "reshape: null pointer");
  int64_t ti, to;
  LMB_TRY(check_dims(in_rank, in_dims, &ti));
  LMB_TRY(check_dims(out_rank, out_dims, &to));
  LMB_REQUIRE(ti == to, "Length mismatch in Reshape!: %lld vs %lld", (long long)to, (long long)ti);
  Reshape rs{};
  rs.in_rank = in_rank; rs.out_rank = out_rank;
  for (int i = 0; i < in_rank; ++i) rs.in_d[i] = in_dims[i];
  for (int i = 0; i < out_rank; ++i) rs.out_d[i] = out_dims[i];
  reshape_cm_kernel<<<grid_for(to), 256, 0, ctx->stream>>>(out, in, rs, to);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_expand(lmb200_ctx h, float* out, const float* in, int32_t in_rank, const int64_t* in_dims,
                                 int32_t axis, int64_t size) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in, "expand: null pointer");
  int64_t ti;
  LMB_TRY(check_dims(in_rank, in_dims, &ti));
  LMB_REQUIRE(in_rank < kMaxRank && axis >= 0 && axis <= in_rank && size >= 1, "expand: axis %d size %lld", axis, (long long)size);
  Gather gt{};
  gt.rank = in_rank + 1;
  int64_t mul = 1;
  int64_t in_st[kMaxRank];
  for (int k = in_rank - 1; k >= 0; --k) { in_st[k] = mul; mul *= in_dims[k]; }
  for (int k = 0, j = 0; k < gt.rank; ++k) {
    if (k == axis) { gt.out_d[k] = size; gt.st[k] = 0; }
    else { gt.out_d[k] = in_dims[j]; gt.st[k] = in_st[j]; ++j; }
  }
  const int64_t total = ti * size;
  strided_copy_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(out, in, gt, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_slice(lmb200_ctx h, float* out, const float* in, int32_t rank, const int64_t* in_dims,
                                const int64_t* starts, const int64_t* stops) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in && starts && stops, "slice: null pointer");
  int64_t ti;
  LMB_TRY(check_dims(rank, in_dims, &ti));
  Gather gt{};
  gt.rank = rank;
  int64_t mul = 1, total = 1;
  for (int k = rank - 1; k >= 0; --k) {
    const int64_t s = starts[k] < 0 ? 0 : starts[k];
    const int64_t e = stops[k] > in_dims[k] ? in_dims[k] : stops[k];
    LMB_REQUIRE(e > s, "slice: empty range on axis %d", k);
    gt.out_d[k] = e - s;
    gt.st[k] = mul;
    gt.offset += s * mul;
    mul *= in_dims[k];
    total *= e - s;
  }
  strided_copy_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(out, in, gt, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_pad(lmb200_ctx h, float* out, const float* in, int32_t rank, const int64_t* in_dims,
                              const int64_t* left, const int64_t* right) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in && left && right, "pad: null pointer");
  int64_t ti;
  LMB_TRY(check_dims(rank, in_dims, &ti));
  Pad pd{};
  pd.rank = rank;
  int64_t total = 1;
  for (int k = 0; k < rank; ++k) {
    LMB_REQUIRE(left[k] >= 0 && right[k] >= 0, "pad: negative padding");
    pd.in_d[k] = in_dims[k]; pd.left[k] = left[k];
    pd.out_d[k] = in_dims[k] + left[k] + right[k];
    total *= pd.out_d[k];
  }
  pad_kernel<<<grid_for(total), 256, 0, ctx->stream>>>(out, in, pd, total);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_gather(lmb200_ctx h, float* out, const float* table, int64_t vocab, int64_t dim,
                                 const float* ids, int64_t n_ids) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && table && ids && vocab >= 1 && dim >= 1 && n_ids >= 1, "gather: bad argument");
  gather_kernel<<<grid_for(n_ids * dim), 256, 0, ctx->stream>>>(out, table, vocab, dim, ids, n_ids);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_unfold1d(lmb200_ctx h, float* out, const float* in, int64_t rows, int64_t length, int64_t kernel,
                                   int64_t stride, int64_t dilation) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in && rows >= 1 && kernel >= 1 && stride >= 1 && dilation >= 1, "unfold: bad argument");
  const int64_t O = (length - dilation * (kernel - 1) - 1) / stride + 1;
  LMB_REQUIRE(O >= 1, "unfold: length %lld too short for kernel %lld", (long long)length, (long long)kernel);
  unfold1d_kernel<<<grid_for(rows * O * kernel), 256, 0, ctx->stream>>>(out, in, rows, length, O, kernel, stride, dilation);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_cumsum_last(lmb200_ctx h, float* out, const float* in, int64_t rows, int64_t n) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && in && rows >= 1 && n >= 1, "cumsum: bad argument");
  cumsum_kernel<<<(unsigned)ceil_div(rows, 128), 128, 0, ctx->stream>>>(out, in, rows, n);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_rmsnorm_scale(lmb200_ctx h, float* y, const float* x, const float* w, int64_t rows,
                                        int64_t n, float eps) {
  CTX_OR_FAIL();
  LMB_REQUIRE(y && x && rows >= 1 && n >= 1, "rmsnorm: bad argument");
  norm_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(y, x, w, nullptr, n, eps, 0);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_layernorm(lmb200_ctx h, float* y, const float* x, const float* w, const float* bias,
                                    int64_t rows, int64_t n, float eps) {
  CTX_OR_FAIL();
  LMB_REQUIRE(y && x && rows >= 1 && n >= 1, "layernorm: bad argument");
  norm_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(y, x, w, bias, n, eps, 1);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_silu_gate(lmb200_ctx h, float* out, const float* gate, const float* up, int64_t n) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && gate && up && n >= 1, "silu_gate: bad argument");
  silu_gate_kernel<<<grid_for(n), 256, 0, ctx->stream>>>(out, gate, up, n);
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_rope(lmb200_ctx h, float* out, const float* x, int64_t B, int64_t H, int64_t S, int64_t D,
                               int64_t prev_seq, float base) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && x && B >= 1 && H >= 1 && S >= 1 && D >= 2 && D % 2 == 0, "rope: bad argument");
  rope_kernel<<<grid_for(B * H * S * (D / 2)), 256, 0, ctx->stream>>>(out, x, B * H, S, D, prev_seq, log2f(base));
  LAUNCHED();
  return LMB200_OK;
}

extern "C" int32_t lmb200_argmax(lmb200_ctx h, int32_t* out, const float* x, int64_t rows, int64_t n) {
  CTX_OR_FAIL();
  LMB_REQUIRE(out && x && rows >= 1 && n >= 1, "argmax: bad argument");
  argmax_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(out, x, n);
  LAUNCHED();
  return LMB200_OK;
}
