// Shared declarations of libluminal_b200: context, error reporting, the tiled ("fragment-major")
// weight / KV-cache layouts and the counter-based generator.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/luminal_b200.h"

namespace lmb {

// ---------------------------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t fail(int32_t code, const char* fmt, ...);

#define LMB_CUDA(expr)                                                                       \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return lmb::fail(LMB200_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                       __FILE__, __LINE__);                                                  \
  } while (0)

#define LMB_REQUIRE(cond, ...)                                \
  do {                                                        \
    if (!(cond)) return lmb::fail(LMB200_EINVAL, __VA_ARGS__); \
  } while (0)

#define LMB_TRY(expr)              \
  do {                             \
    int32_t _r = (expr);           \
    if (_r != LMB200_OK) return _r; \
  } while (0)

// ---------------------------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------------------------
struct Ctx {
  uint32_t magic = 0x4C4D4231;
  int device = 0;
  int sm_count = 148;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  int64_t launches = 0;
  int* dev_err = nullptr;        // mapped pinned word: a kernel whose bounded wait gave up sets it
  int* dev_broken = nullptr;     // device word: set with dev_err by a tensor-parallel wait that failed; while it is
                                 // set every signal this rank sends to its peers is marked invalid (see PeerReduce)
  bool comm_broken = false;      // a tensor-parallel step failed: steps are refused until lmb200_comm_resync
  // NCCL (resolved with dlopen so that the library loads on hosts without it)
  void* nccl_comm = nullptr;
  int tp_size = 1;
  int tp_rank = 0;
  // Peer exchange region of the in-kernel all-reduce, one per communicator, mapped into every rank
  // with CUDA IPC: two partial buffers of kPeerBufFloats floats, then one 64-bit flag per source
  // rank.  peer_n == 0: not set up, the NCCL all-reduce is used instead.
  int peer_n = 0;
  void* peer_base[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  unsigned long long* peer_step = nullptr;   // device counter: decode steps enqueued on this communicator
  float* peer_scratch = nullptr;             // 1 float for the teardown barrier
  long long peer_wait_cycles = 0;            // SM cycles a kernel waits for a peer's signal (LMB200_PEER_WAIT_MS, default 10 s)
  // Scratch of the stand-alone ops that need some (the float32 flash attention's bf16 halves): grows to the largest
  // request and stays until shutdown, so that a call neither allocates nor waits for the device
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  // lmb200_capture_begin .. lmb200_capture_end: the op-level launches of this context are recorded into a CUDA graph
  // instead of run; calls that copy to or from the host, allocate, free or wait are refused meanwhile
  bool capturing = false;
  int64_t capture_launches0 = 0;
  bool scratch_in_graph = false;   // a recorded graph reads `scratch`: when it must grow, the old block is retired, not freed
  std::vector<void*> retired_scratch;   // blocks recorded graphs may still read; freed with the last graph or at shutdown
  int live_graphs = 0;
};

// Region layout (bytes): two 4 MiB buffers read by the peers (the norm kernels' all-reduce), two 4 MiB
// buffers written by the peers (the projections that do their own exchange; kept at the "nothing here
// yet" bit pattern between uses), then the flags of either protocol.
constexpr int64_t kPeerBufFloats = 1 << 20;
constexpr int64_t kPeerPushOffset = 2 * kPeerBufFloats * 4;
constexpr int64_t kPeerFlagsOffset = 4 * kPeerBufFloats * 4;
constexpr int64_t kPeerPushFlagsOffset = kPeerFlagsOffset + 4096;    // [8 source ranks][256 CTAs] 64-bit flags
constexpr int64_t kPeerRegionBytes = kPeerPushFlagsOffset + 8 * 256 * 8;
constexpr uint32_t kPeerEmptyPair = 0x80008000u;                      // two bf16 -0.0: "not written yet" in a push buffer
constexpr unsigned long long kPeerEpochStride = 4096;                 // reductions per step < this
constexpr unsigned long long kPeerPoison = 1ull << 63;                // a signal sent by a rank whose earlier wait failed
constexpr long long kPeerWaitCycles = 20000000000ll;                  // about 10 s of SM clock

// What a kernel needs to sum the ranks' partial results of one row-parallel projection: every rank
// wrote its partial into its own region; the consumer signals the peers, waits (bounded) for their
// signals and adds the partials in rank order, so every rank gets the same bits.
struct PeerReduce {
  int n = 0, rank = 0;
  const float* part[8];                    // rank r's partial buffer of this reduction
  unsigned long long* remote_flag[8];      // this rank's slot in rank r's flag array
  const unsigned long long* local_flag;    // this rank's flag array, one slot per source rank
  const unsigned long long* step;          // steps completed so far
  unsigned phase = 0;                      // 1 + index of the reduction inside the step
  int* dev_err = nullptr;
  int* broken = nullptr;                   // Ctx::dev_broken
  long long wait_cycles = kPeerWaitCycles;
};

// A signal is the epoch (step * kPeerEpochStride + phase) of the reduction it announces.  A rank
// that is one reduction ahead may already have overwritten its slot with the next epoch, which is
// fine (its data of this epoch sits in the other buffer).  Two things are not fine and end the wait
// with an error instead of a sum of stale partials: a signal marked kPeerPoison (its sender had a
// wait run out earlier, so what it computed since is not the model's), and a signal a whole step or
// more ahead (the ranks' step counters have come apart).

#ifdef __CUDACC__
// All threads of the block call this once the kernel that produced this rank's partial is complete.
// CTA 0 publishes "rank `rank` has written reduction `epoch`" into every peer's flag array; every
// CTA then waits until all peers have published the same epoch.  A wait that runs out (or finds an
// earlier failure recorded) sets the error word and returns, so nothing spins forever.
__device__ __forceinline__ bool peer_signal_ok(unsigned long long v, unsigned long long epoch, bool* bad) {
  const unsigned long long e = v & ~kPeerPoison;
  if (e < epoch) return false;                                   // not there yet
  *bad = (v & kPeerPoison) != 0ull || e - epoch >= kPeerEpochStride;
  return true;
}
__device__ __forceinline__ void peer_mark_failed(int* dev_err, int* broken, int code) {
  *reinterpret_cast<volatile int*>(dev_err) = code;
  if (broken) *reinterpret_cast<volatile int*>(broken) = 1;
}

__device__ __forceinline__ void peer_exchange_wait(const PeerReduce& pr) {
  const unsigned long long epoch = *pr.step * kPeerEpochStride + pr.phase;
  const int t = threadIdx.x;
  if (t < pr.n && t != pr.rank) {
    if (blockIdx.x == 0) {
      const bool poisoned = pr.broken && *reinterpret_cast<volatile int*>(pr.broken) != 0;
      __threadfence_system();
      asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(pr.remote_flag[t]), "l"(epoch | (poisoned ? kPeerPoison : 0ull)) : "memory");
    }
    const long long t0 = clock64();
    unsigned spins = 0;
    for (;;) {
      unsigned long long v;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(pr.local_flag + t) : "memory");
      bool bad = false;
      if (peer_signal_ok(v, epoch, &bad)) {
        if (bad) peer_mark_failed(pr.dev_err, pr.broken, 2);
        break;
      }
      if ((++spins & 1023u) == 0u) {
        volatile int* err = pr.dev_err;
        if (*err != 0) break;
        if (clock64() - t0 > pr.wait_cycles) { peer_mark_failed(pr.dev_err, pr.broken, 1); break; }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ float4 peer_load4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
#endif

Ctx* ctx_from(lmb200_ctx h);
// LMB200_ETIMEOUT (and clears the flag) if a kernel reported a wait that ran out
int32_t check_device_error(Ctx* ctx);
int32_t nccl_allreduce_f32(Ctx* ctx, void* dptr, int64_t count, cudaStream_t stream);

// Strided view of the tensors of a tensor-core flash attention launch (elements, bf16)
struct FlashView {
  int H = 1, G = 1;                 // query heads per batch entry; query heads per kv head
  int64_t q_b = 0, q_h = 0, q_s = 0;    // q and out: batch, head, position strides
  int64_t k_b = 0, k_h = 0, k_s = 0;    // k and v
};

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// ---------------------------------------------------------------------------------------------
// Counter-based generator, identical on host and device (and in the NumPy oracle):
//   value = float(2*sum_of_12_uint16_lanes - 12*65535) * (sigma/131072) [+ offset]
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  uint64_t z = x;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ inline uint64_t stream_key(uint64_t seed, uint64_t tensor_id) {
  return splitmix64(seed * 0xD1342543DE82EF95ull + tensor_id);
}
__host__ __device__ inline float synth_value(uint64_t key, uint64_t idx, float scale /*sigma/131072*/,
                                             float offset) {
  int32_t total = 0;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    uint64_t h = splitmix64(key ^ (idx * 3ull + (uint64_t)r));
    total += (int32_t)(h & 0xFFFF) + (int32_t)((h >> 16) & 0xFFFF) + (int32_t)((h >> 32) & 0xFFFF) +
             (int32_t)((h >> 48) & 0xFFFF);
  }
  float v = (float)(2 * total - 12 * 65535);
#ifdef __CUDA_ARCH__
  v = __fmul_rn(v, scale);
  if (offset != 0.0f) v = __fadd_rn(v, offset);
#else
  v = v * scale;
  if (offset != 0.0f) v = v + offset;
#endif
  return v;
}

// ---------------------------------------------------------------------------------------------
// Tiled weight layout.  A matrix [rows, K] is stored as units of 16 rows x 32 k, unit (rb, kc)
// at ((rb*KC + kc) * 512) elements; inside a unit lane (g = row%8, t = (k%32)/8) owns 16
// consecutive elements: 8 of row g then 8 of row g+8, k = 8t..8t+7.  This is the operand order
// of two m16n8k16 MMAs (with the k index permuted identically in the activation operand), so a
// warp reads one unit with fully contiguous 2 x 16-byte loads per lane.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline int64_t wtile_offset(int64_t row, int64_t k, int64_t KC) {
  int64_t rb = row >> 4;
  int r = (int)(row & 15);
  int g = r & 7, hi = r >> 3;
  int64_t kc = k >> 5;
  int kk = (int)(k & 31);
  int t = kk >> 3, e = kk & 7;
  return ((rb * KC + kc) * 32 + (g * 4 + t)) * 16 + hi * 8 + e;
}

// ---------------------------------------------------------------------------------------------
// Tiled KV cache.  Per (layer, batch, kv head) the keys are grouped in blocks of 16; block kb
// holds D/16 K-units then D/16 V-units, each unit 16x16 elements in m16n8k16 A-operand order:
//   K unit dk (M = key, K = d):  lane (g,t): [key g][d 2t,2t+1] [key g+8][d 2t,2t+1]
//                                            [key g][d 2t+8,+9] [key g+8][d 2t+8,+9]
//   V unit dm (M = d,   K = key): lane (g,t): [d g][key 2t,2t+1] [d g+8][key 2t,2t+1]
//                                            [d g][key 2t+8,+9] [d g+8][key 2t+8,+9]
// with d = 16*unit + local.  One block is 2*16*D elements and fully contiguous.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline int64_t kv_block_elems(int D) { return 32 * (int64_t)D; }
__host__ __device__ inline int64_t kcache_offset(int64_t key, int d, int D) {
  int64_t kb = key >> 4;
  int kk = (int)(key & 15);
  int dk = d >> 4, dd = d & 15;
  int g = kk & 7, hik = kk >> 3;
  int t = (dd & 7) >> 1, e = dd & 1, hid = dd >> 3;
  return kb * kv_block_elems(D) + (int64_t)dk * 256 + (g * 4 + t) * 8 + (hid * 2 + hik) * 2 + e;
}
__host__ __device__ inline int64_t vcache_offset(int64_t key, int d, int D) {
  int64_t kb = key >> 4;
  int kk = (int)(key & 15);
  int dm = d >> 4, dd = d & 15;
  int g = dd & 7, hid = dd >> 3;
  int t = (kk & 7) >> 1, e = kk & 1, hik = kk >> 3;
  return kb * kv_block_elems(D) + (int64_t)(D / 16 + dm) * 256 + (g * 4 + t) * 8 + (hik * 2 + hid) * 2 + e;
}

// ---------------------------------------------------------------------------------------------
// Tiled activations.  A GEMV input x[b, k] (b < Bp = 8, 16 or 32 rows, zero beyond the batch) is
// stored chunk-major: [k/32][Bp][32].  The slice of any run of k-chunks is contiguous (one bulk
// copy), and the B-operand read of the MMA -- lane (g,t) takes x[8nt+g][8t..8t+7] -- touches
// 128 contiguous bytes per quarter-warp, so shared memory needs no padding or swizzle.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline int64_t xtile_offset(int b, int k, int Bp) {
  return (int64_t)(k >> 5) * (Bp * 32) + b * 32 + (k & 31);
}
static inline int batch_pad(int B) { return B <= 8 ? 8 : (B <= 16 ? 16 : 32); }

// ---------------------------------------------------------------------------------------------
// bf16 GEMV operands: the tensor-core ("UMMA") canonical K-major layout without swizzle, so that
// one contiguous bulk copy lands a stage in shared memory exactly as tcgen05.mma reads it through
// a shared-memory descriptor -- and as ldmatrix reads it for mma.sync.
//   core matrix = 8 rows x 8 k (bf16) = 128 contiguous bytes, rows 16 bytes apart.
//   weights: unit = 128 rows x 128 k = 32 KB at ((row/128)*KS + k/128) * 16384 elements, inside it
//            [k8 = (k%128)/8][m8 = (row%128)/8][row%8][k%8]
//            -> A descriptor: K-direction core-matrix stride (LBO) 2048 B, M-direction (SBO) 128 B.
//   activations x[b, k], b < Bp (16 or 32), zero beyond the batch and beyond K:
//            [k/8][b/8][b%8][k%8]  -> B descriptor: LBO = Bp*16 B, SBO = 128 B; the slice of one
//            128-k stage is Bp*256 contiguous bytes.
// K is padded to a multiple of 128 (KS stages), rows to a multiple of 128.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline int64_t wcanon_offset(int64_t row, int64_t k, int64_t KS) {
  const int64_t r = row >> 7, ks = k >> 7;
  const int m8 = (int)((row & 127) >> 3), rr = (int)(row & 7);
  const int k8 = (int)((k & 127) >> 3), kk = (int)(k & 7);
  return (r * KS + ks) * 16384 + k8 * 1024 + m8 * 64 + rr * 8 + kk;
}
__host__ __device__ inline int64_t xcanon_offset(int b, int k, int Bp) {
  return (int64_t)(k >> 3) * (Bp * 8) + (b >> 3) * 64 + (b & 7) * 8 + (k & 7);
}

// Per-dtype operand layouts of the decode GEMV: float32 uses the lane-ordered tiles of the
// register-ring kernel, bf16 the canonical tensor-core layout above.
template <typename WT> struct Layout;
template <> struct Layout<float> {
  __host__ __device__ static int batch_pad(int B) { return B <= 8 ? 8 : (B <= 16 ? 16 : 32); }
  __host__ __device__ static int64_t w_elems(int rows, int K) { return (int64_t)((rows + 15) / 16) * ((K + 31) / 32) * 512; }
  __host__ __device__ static int64_t w_offset(int row, int k, int K) { return wtile_offset(row, k, (K + 31) / 32); }
  __host__ __device__ static int64_t x_elems(int K, int Bp) { return (int64_t)((K + 31) / 32) * Bp * 32; }
  __host__ __device__ static int64_t x_offset(int b, int k, int Bp) { return xtile_offset(b, k, Bp); }
};
template <> struct Layout<__nv_bfloat16> {
  __host__ __device__ static int batch_pad(int B) { return B <= 16 ? 16 : 32; }
  __host__ __device__ static int64_t w_elems(int rows, int K) { return (int64_t)((rows + 127) / 128) * ((K + 127) / 128) * 16384; }
  __host__ __device__ static int64_t w_offset(int row, int k, int K) { return wcanon_offset(row, k, (K + 127) / 128); }
  __host__ __device__ static int64_t x_elems(int K, int Bp) { return (int64_t)((K + 127) / 128) * 128 * Bp; }
  __host__ __device__ static int64_t x_offset(int b, int k, int Bp) { return xcanon_offset(b, k, Bp); }
};

// element conversions
__device__ inline float to_f32(float v) { return v; }
__device__ inline float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ inline T from_f32(float v);
template <> __device__ inline float from_f32<float>(float v) { return v; }
template <> __device__ inline __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace lmb
