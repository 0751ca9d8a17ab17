// lmb200_decode_attention_noalloc: split-KV decode attention for callers that must not allocate.
//
// Who that is: a host runtime that has already handed all device memory to its own pool (Julia's
// CUDA.jl, a serving framework's arena) sees any further cudaMalloc fail or fragment the pool;
// and a caller sitting inside a latency-critical loop cannot afford the device-wide
// synchronisation an allocation may bring.  For them the per-split partial results of the
// attention kernel -- the only global memory it needs beyond its inputs and outputs -- live in a
// fixed array that is part of the library image, and this entry point never calls cudaMalloc,
// cudaFree or any routine that allocates.
//
// The array is shared by every call on a device and keeps whatever the previous call left in it.
// Nothing in it has to start at zero: each launch rewrites every slot that its merge step reads.
// Two calls whose kernels overlap on the GPU (different streams, different contexts of the same
// process) would write the same slots and race; issue them one after the other.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "attention.cuh"
#include "common.cuh"

namespace {

// 2 Mi floats = 8 MiB per GPU that loads the library, held until the process exits.
constexpr int64_t kScratchFloats = 2 * 1024 * 1024;
static __device__ __align__(256) float g_attn_scratch[kScratchFloats];

// In host code `g_attn_scratch` is only a handle for the runtime, not a device address: the
// address a kernel can use has to be asked for, once per device, with that device current.
// The table is filled without a lock: two host threads that race on a device's first call both
// look up and store the same address.
constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

int32_t scratch_for_current_device(int device, float** out) {
  if (device < 0 || device >= kMaxDevices) return lmb::fail(LMB200_EINVAL, "noalloc: device ordinal %d", device);
  if (!g_scratch_ptr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_scratch);
    if (e != cudaSuccess || !p)
      return lmb::fail(LMB200_ECUDA, "noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_ptr[device] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[device];
  return LMB200_OK;
}

}  // namespace

extern "C" int32_t lmb200_decode_attention_noalloc(lmb200_ctx h, int32_t dtype, const void* q_dptr, void* out_dptr,
                                                   const void* kv_layer_dptr, int64_t kv_batch_stride,
                                                   int64_t kv_head_stride, int32_t batch, int32_t n_kv_heads,
                                                   int32_t group, int32_t head_dim, int32_t T) {
  using namespace lmb;
  Ctx* ctx = ctx_from(h);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(q_dptr && out_dptr && kv_layer_dptr, "decode_attention_noalloc: null pointer");
  LMB_REQUIRE(dtype == LMB200_F32 || dtype == LMB200_BF16, "decode_attention_noalloc: dtype %d", dtype);
  LMB_REQUIRE(batch >= 1 && n_kv_heads >= 1 && group >= 1 && T >= 1, "decode_attention_noalloc: bad shape");
  LMB_REQUIRE(head_dim >= 16 && head_dim % 16 == 0 && head_dim <= 256, "decode_attention_noalloc: head_dim %d", head_dim);
  LMB_REQUIRE(dtype != LMB200_BF16 || group <= 8,
              "decode_attention_noalloc: %d query heads per kv head (max 8 on the bf16 path)", group);
  // sizes are checked in 64-bit before anything is narrowed to int
  const int64_t q_pitch64 = (int64_t)n_kv_heads * group * head_dim;
  const int64_t T_padded64 = round_up((int64_t)T, 64);
  LMB_REQUIRE(q_pitch64 <= INT32_MAX && (int64_t)batch * n_kv_heads <= INT32_MAX && T_padded64 <= INT32_MAX,
              "decode_attention_noalloc: shape too large (q row of %lld elements, context %d)", (long long)q_pitch64, T);
  // The kernels read ceil(T / 16) blocks of 32 * head_dim elements per (sequence, kv head): the strides
  // must describe a tiled layer that holds at least that many, or the reads would leave the cache.
  const int64_t need_head = ceil_div((int64_t)T, 16) * kv_block_elems(head_dim);
  LMB_REQUIRE(kv_head_stride >= need_head,
              "decode_attention_noalloc: context %d needs a kv head stride of at least %lld elements, got %lld "
              "(T exceeds the layer's capacity?)", T, (long long)need_head, (long long)kv_head_stride);
  LMB_REQUIRE(kv_batch_stride >= (int64_t)n_kv_heads * kv_head_stride,
              "decode_attention_noalloc: kv batch stride %lld is smaller than %d heads x head stride %lld",
              (long long)kv_batch_stride, n_kv_heads, (long long)kv_head_stride);
  LMB_CUDA(cudaSetDevice(ctx->device));
  float* scratch = nullptr;
  LMB_TRY(scratch_for_current_device(ctx->device, &scratch));

  AttnParams a;
  int64_t po = 0, pml = 0;
  attn_plan(ctx, batch, n_kv_heads, group, head_dim, (int)T_padded64, &a.keys_per_cta, &a.nsplit, &po, &pml);
  if (po + pml > kScratchFloats)
    return fail(LMB200_EINVAL,
                "decode_attention_noalloc: batch %d x kv heads %d x group %d x head_dim %d at context %d needs %lld "
                "scratch floats, the built-in array holds %lld; use lmb200_decode_attention_splitkv",
                batch, n_kv_heads, group, head_dim, T, (long long)(po + pml), (long long)kScratchFloats);
  a.q = q_dptr; a.q_pitch = (int)q_pitch64;
  a.kv_layer = kv_layer_dptr; a.kv_batch_stride = kv_batch_stride; a.kv_head_stride = kv_head_stride;
  a.B = batch; a.KVl = n_kv_heads; a.G = group; a.D = head_dim;
  a.pos = nullptr; a.T_fixed = T;
  a.scale = 1.0f / sqrtf((float)head_dim);
  a.part_o = scratch;
  a.part_ml = scratch + po;
  a.out = out_dptr; a.out_pitch = a.q_pitch;
  return attn_decode_launch(ctx, dtype, a, ctx->stream);
}
