// Context, error reporting, buffers, host<->device layout conversion and the NCCL binding.
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "common.cuh"
#include "gemv.cuh"
#include "model.cuh"
#include "pdl.cuh"

namespace lmb {

int32_t flash_tc_configure();
int32_t flash_tc_f32_configure();

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

Ctx* ctx_from(lmb200_ctx h) {
  Ctx* c = reinterpret_cast<Ctx*>(h);
  if (!c || c->magic != 0x4C4D4231) {
    set_error("invalid context handle");
    return nullptr;
  }
  return c;
}

static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void pdl_set_enabled(bool on) { g_pdl = on; }

// A wait that ran out inside a tensor-parallel step leaves the ranks out of step with one another
// (this rank advanced its counters on sums it never received), so the communicator is marked broken:
// the device word keeps every later signal of this rank marked invalid, and the session calls refuse
// tensor-parallel work until lmb200_comm_resync.
int32_t check_device_error(Ctx* ctx) {
  const int code = ctx->dev_err ? *reinterpret_cast<volatile int*>(ctx->dev_err) : 0;
  if (code != 0) {
    *ctx->dev_err = 0;
    if (ctx->nccl_comm && ctx->tp_size > 1) ctx->comm_broken = true;
    if (code == 2)
      return fail(LMB200_ETIMEOUT, "a peer rank's signal was invalid (that rank had a wait run out, or the ranks' step counters "
                                   "differ): results of the last call are invalid; call lmb200_comm_resync on every rank");
    return fail(LMB200_ETIMEOUT, "a kernel gave up a bounded wait (mbarrier / flag): results of the last call are invalid%s",
                ctx->comm_broken ? "; the tensor-parallel ranks are out of step, call lmb200_comm_resync on every rank" : "");
  }
  return LMB200_OK;
}

// ---------------------------------------------------------------------------------------------
// NCCL, resolved at run time so the library loads (and its CPU-side entry points work) on a
// host without NCCL.  Only the calls below are used; the types are ABI-stable across NCCL 2.x.
// ---------------------------------------------------------------------------------------------
namespace {
struct Id128 { char b[128]; };   // ncclUniqueId: 128 opaque bytes, passed by value
struct NcclApi {
  void* lib = nullptr;
  int (*GetUniqueId)(void*) = nullptr;
  int (*CommInitRank)(void**, int, Id128, int) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;

int32_t nccl_load() {
  if (g_nccl.lib) return LMB200_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* lib = nullptr;
  for (const char* n : names) {
    lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (lib) break;
  }
  if (!lib) return fail(LMB200_ENCCL, "NCCL not found: %s", dlerror());
  g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(lib, "ncclGetUniqueId"));
  g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(lib, "ncclCommInitRank"));
  g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(lib, "ncclCommDestroy"));
  g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(lib, "ncclAllReduce"));
  g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(lib, "ncclAllGather"));
  g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(lib, "ncclGetErrorString"));
  if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce)
    return fail(LMB200_ENCCL, "NCCL library lacks a required symbol");
  g_nccl.lib = lib;
  return LMB200_OK;
}
const char* nccl_str(int r) { return g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?"; }

// What the ranks tell each other while the peer exchange region is set up.
struct PeerHello {
  cudaIpcMemHandle_t handle;
  int32_t ok;
  int32_t pad[15];
};

// Waits for the stream, but not forever: a rank whose peers never arrive gives up after `seconds`.
bool stream_done_within(cudaStream_t st, double seconds) {
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    const cudaError_t e = cudaStreamQuery(st);
    if (e == cudaSuccess) return true;
    if (e != cudaErrorNotReady) { cudaGetLastError(); return false; }
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > seconds) return false;
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

int32_t gather_hello(Ctx* c, const PeerHello& mine, PeerHello* all, void* dsend, void* drecv) {
  LMB_CUDA(cudaMemcpyAsync(dsend, &mine, sizeof(PeerHello), cudaMemcpyHostToDevice, c->own_stream));
  const int r = g_nccl.AllGather(dsend, drecv, sizeof(PeerHello), 0 /* ncclInt8 */, c->nccl_comm, c->own_stream);
  if (r != 0) return fail(LMB200_ENCCL, "ncclAllGather: %s", nccl_str(r));
  LMB_CUDA(cudaMemcpyAsync(all, drecv, sizeof(PeerHello) * c->tp_size, cudaMemcpyDeviceToHost, c->own_stream));
  LMB_CUDA(cudaStreamSynchronize(c->own_stream));
  return LMB200_OK;
}

__global__ void fill_u32_kernel(uint32_t* p, uint32_t v, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}
// This rank's push buffers back to "nothing written yet" everywhere (set-up, and after a failed step)
int32_t peer_clear_push_buffers(Ctx* c, void* region) {
  uint32_t* p = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(region) + kPeerPushOffset);
  fill_u32_kernel<<<1024, 256, 0, c->own_stream>>>(p, kPeerEmptyPair, 2 * kPeerBufFloats);
  LMB_CUDA(cudaGetLastError());
  LMB_CUDA(cudaStreamSynchronize(c->own_stream));
  return LMB200_OK;
}

// Maps one exchange region per rank into every rank (CUDA IPC inside one node) for the all-reduce
// that the decode step's norm kernels do themselves.  Every decision is taken on gathered data, so
// all ranks end up with the same answer; any failure leaves peer_n == 0 and NCCL does the sums.
int32_t peer_setup(Ctx* c) {
  const char* sel = getenv("LMB200_TP_ALLREDUCE");          // "nccl": keep ncclAllReduce (A/B runs)
  if ((sel && strcmp(sel, "nccl") == 0) || c->tp_size < 2 || c->tp_size > 8 || !g_nccl.AllGather) return LMB200_OK;
  const int n = c->tp_size;
  const char* wms = getenv("LMB200_PEER_WAIT_MS");          // how long a kernel waits for a peer's signal
  int khz = 0;                                              // SM clock the limit is converted with (clock64 ticks)
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device) != cudaSuccess || khz <= 0) { cudaGetLastError(); khz = 1965000; }
  c->peer_wait_cycles = wms && atoll(wms) > 0 ? atoll(wms) * (long long)khz : kPeerWaitCycles;
  void *region = nullptr, *dsend = nullptr, *drecv = nullptr;
  PeerHello mine, all[8];
  memset(&mine, 0, sizeof(mine));
  bool ok = cudaMalloc(&region, kPeerRegionBytes) == cudaSuccess && cudaMemset(region, 0, kPeerRegionBytes) == cudaSuccess &&
            cudaMalloc((void**)&c->peer_step, 8) == cudaSuccess && cudaMemset(c->peer_step, 0, 8) == cudaSuccess &&
            cudaMalloc((void**)&c->peer_scratch, 4) == cudaSuccess && cudaMemset(c->peer_scratch, 0, 4) == cudaSuccess &&
            peer_clear_push_buffers(c, region) == LMB200_OK &&
            cudaDeviceSynchronize() == cudaSuccess && cudaIpcGetMemHandle(&mine.handle, region) == cudaSuccess;
  cudaGetLastError();
  mine.ok = ok ? 1 : 0;
  int32_t rc = LMB200_OK;
  if (cudaMalloc(&dsend, sizeof(PeerHello)) != cudaSuccess || cudaMalloc(&drecv, sizeof(PeerHello) * 8) != cudaSuccess) {
    cudaGetLastError();
    rc = fail(LMB200_ENOMEM, "comm_init: staging allocation failed");
  }
  void* mapped[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  if (rc == LMB200_OK) rc = gather_hello(c, mine, all, dsend, drecv);
  if (rc == LMB200_OK) {
    for (int r = 0; r < n; ++r) ok = ok && all[r].ok;
    if (ok) {
      for (int r = 0; r < n; ++r) {
        if (r == c->tp_rank) { mapped[r] = region; continue; }
        if (cudaIpcOpenMemHandle(&mapped[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          cudaGetLastError();
          mapped[r] = nullptr;
          ok = false;
        }
      }
    }
    mine.ok = ok ? 1 : 0;
    rc = gather_hello(c, mine, all, dsend, drecv);       // second round: did every rank map every peer?
    if (rc == LMB200_OK)
      for (int r = 0; r < n; ++r) ok = ok && all[r].ok;
  }
  cudaFree(dsend);
  cudaFree(drecv);
  if (rc == LMB200_OK && ok) {
    for (int r = 0; r < n; ++r) c->peer_base[r] = mapped[r];
    c->peer_n = n;
    return LMB200_OK;
  }
  for (int r = 0; r < n; ++r)
    if (mapped[r] && r != c->tp_rank) cudaIpcCloseMemHandle(mapped[r]);
  cudaFree(region);
  cudaFree(c->peer_step); c->peer_step = nullptr;
  cudaFree(c->peer_scratch); c->peer_scratch = nullptr;
  cudaGetLastError();
  return rc;
}

// Peers may still be reading this rank's region (their last norm kernel), so all ranks meet in one
// NCCL all-reduce first.  If the others never come, the region is left allocated rather than freed
// under a reader.
void peer_teardown(Ctx* c) {
  if (c->peer_n == 0) return;
  cudaStreamSynchronize(c->stream);
  bool met = g_nccl.AllReduce(c->peer_scratch, c->peer_scratch, 1, 7, 0, c->nccl_comm, c->own_stream) == 0 &&
             stream_done_within(c->own_stream, 5.0);
  for (int r = 0; r < c->peer_n; ++r) {
    if (r != c->tp_rank && c->peer_base[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
    else if (r == c->tp_rank && met) cudaFree(c->peer_base[r]);
    c->peer_base[r] = nullptr;
  }
  if (met) { cudaFree(c->peer_step); cudaFree(c->peer_scratch); }
  c->peer_step = nullptr;
  c->peer_scratch = nullptr;
  c->peer_n = 0;
  cudaGetLastError();
}
}  // namespace

int32_t nccl_allreduce_f32(Ctx* ctx, void* dptr, int64_t count, cudaStream_t stream) {
  if (!ctx->nccl_comm) return fail(LMB200_ENCCL, "allreduce without a communicator");
  // ncclFloat32 = 7, ncclSum = 0
  const int r = g_nccl.AllReduce(dptr, dptr, (size_t)count, 7, 0, ctx->nccl_comm, stream);
  if (r != 0) return fail(LMB200_ENCCL, "ncclAllReduce: %s", nccl_str(r));
  return LMB200_OK;
}

// ---------------------------------------------------------------------------------------------
// layout conversion: host float32 (row- or column-major) <-> device row-major tensor
// ---------------------------------------------------------------------------------------------
struct Shape8 {
  int rank;
  int64_t d[8];
};

// src is the host image (float32) staged on the device; element (i0..ir) of a column-major
// array sits at sum i_k * prod_{j<k} d_j.
template <typename T, bool kToDevice>
__global__ void relayout_kernel(T* dev, float* stage, Shape8 s, int colmajor, int64_t total) {
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    int64_t src = o;
    if (colmajor) {
      int64_t rem = o, stride_total = total;
      src = 0;
      // walk the row-major index from the slowest dim, accumulate the column-major offset
      int64_t cm_stride[8];
      int64_t acc = 1;
      for (int k = 0; k < s.rank; ++k) { cm_stride[k] = acc; acc *= s.d[k]; }
      for (int k = 0; k < s.rank; ++k) {
        stride_total /= s.d[k];
        const int64_t ik = rem / stride_total;
        rem -= ik * stride_total;
        src += ik * cm_stride[k];
      }
    }
    if (kToDevice) dev[o] = from_f32<T>(stage[src]);
    else stage[src] = to_f32(dev[o]);
  }
}

}  // namespace lmb

using namespace lmb;

extern "C" int32_t lmb200_version(void) { return 100; }
extern "C" const char* lmb200_last_error(void) { return g_err; }

extern "C" int32_t lmb200_device_count(int32_t* count) {
  LMB_REQUIRE(count, "device_count: null argument");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *count = 0;
    return fail(LMB200_ECUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
  }
  *count = n;
  return LMB200_OK;
}

extern "C" int32_t lmb200_init(int32_t device, lmb200_ctx* out) {
  LMB_REQUIRE(out, "init: null argument");
  int n = 0;
  LMB_TRY(lmb200_device_count(&n));
  LMB_REQUIRE(device >= 0 && device < n, "init: device %d of %d", device, n);
  LMB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  LMB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(LMB200_EINVAL, "init: device %d is sm_%d%d; this library holds sm_100a code only", device,
                prop.major, prop.minor);
  Ctx* c = new Ctx();
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete c;
    return fail(LMB200_ECUDA, "init: stream creation failed");
  }
  c->stream = c->own_stream;
  if (cudaHostAlloc((void**)&c->dev_err, sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
    cudaStreamDestroy(c->own_stream);
    delete c;
    return fail(LMB200_ECUDA, "init: pinned allocation failed");
  }
  *c->dev_err = 0;
  if (cudaMalloc((void**)&c->dev_broken, sizeof(int)) != cudaSuccess || cudaMemset(c->dev_broken, 0, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(c->dev_err);
    cudaStreamDestroy(c->own_stream);
    delete c;
    return fail(LMB200_ENOMEM, "init: device allocation failed");
  }
  const char* pdl = getenv("LMB200_PDL");      // LMB200_PDL=0: plain stream-ordered launches
  pdl_set_enabled(!(pdl && atoi(pdl) == 0));
  gemv_set_variant(GEMV_TCGEN05);
  int32_t rc = gemv_configure();
  if (rc == LMB200_OK) rc = attn_configure();
  if (rc == LMB200_OK) rc = flash_tc_configure();
  if (rc == LMB200_OK) rc = flash_tc_f32_configure();
  if (rc == LMB200_OK) rc = step_kernels_configure();
  if (rc == LMB200_OK) rc = prefill_configure();
  if (rc != LMB200_OK) { cudaFree(c->dev_broken); cudaFreeHost(c->dev_err); cudaStreamDestroy(c->own_stream); delete c; return rc; }
  *out = reinterpret_cast<lmb200_ctx>(c);
  return LMB200_OK;
}

extern "C" int32_t lmb200_shutdown(lmb200_ctx h) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  peer_teardown(c);
  if (c->nccl_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->nccl_comm);
  cudaStreamDestroy(c->own_stream);
  cudaFreeHost(c->dev_err);
  cudaFree(c->dev_broken);
  cudaFree(c->scratch);
  for (void* p : c->retired_scratch) cudaFree(p);
  c->magic = 0;
  delete c;
  return LMB200_OK;
}

extern "C" int32_t lmb200_set_stream(lmb200_ctx h, void* stream) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  c->stream = stream ? reinterpret_cast<cudaStream_t>(stream) : c->own_stream;
  return LMB200_OK;
}

extern "C" int32_t lmb200_sync(lmb200_ctx h) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "sync: not between capture_begin and capture_end");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_CUDA(cudaStreamSynchronize(c->stream));
  return check_device_error(c);
}

// ---------------------------------------------------------------------------------------------
// Capture of a sequence of op-level calls into a CUDA graph (execute_with_capture, src/Device.jl:106-121)
// ---------------------------------------------------------------------------------------------
namespace {
struct HostGraph {
  uint32_t magic = 0x47525048;
  Ctx* ctx = nullptr;
  cudaGraphExec_t exec = nullptr;
  int64_t nodes = 0;                 // kernels one replay launches
};
HostGraph* graph_from(uint64_t h) {
  HostGraph* g = reinterpret_cast<HostGraph*>(h);
  if (!g || g->magic != 0x47525048) { set_error("invalid graph handle"); return nullptr; }
  return g;
}
}  // namespace

extern "C" int32_t lmb200_capture_begin(lmb200_ctx h) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  if (c->capturing) return fail(LMB200_ESTATE, "capture_begin: a capture is already open on this context");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  c->capturing = true;
  c->capture_launches0 = c->launches;
  return LMB200_OK;
}

extern "C" int32_t lmb200_capture_end(lmb200_ctx h, uint64_t* graph_out) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  if (!c->capturing) return fail(LMB200_ESTATE, "capture_end: no capture is open on this context");
  cudaSetDevice(c->device);
  cudaGraph_t g = nullptr;
  const cudaError_t e = cudaStreamEndCapture(c->stream, &g);
  c->capturing = false;
  const int64_t nodes = c->launches - c->capture_launches0;
  c->launches = c->capture_launches0;                      // recorded, not run
  if (e != cudaSuccess || !g) {
    cudaGetLastError();
    if (g) cudaGraphDestroy(g);
    return fail(LMB200_ECUDA, "capture_end: the recorded calls cannot be replayed (%s)", cudaGetErrorString(e));
  }
  if (!graph_out) { cudaGraphDestroy(g); return fail(LMB200_EINVAL, "capture_end: null argument"); }
  HostGraph* G = new HostGraph();
  G->ctx = c; G->nodes = nodes;
  const cudaError_t ei = cudaGraphInstantiate(&G->exec, g, 0);
  cudaGraphDestroy(g);
  if (ei != cudaSuccess) {
    cudaGetLastError();
    delete G;
    return fail(LMB200_ECUDA, "capture_end: cudaGraphInstantiate failed (%s)", cudaGetErrorString(ei));
  }
  c->live_graphs++;
  *graph_out = reinterpret_cast<uint64_t>(G);
  return LMB200_OK;
}

extern "C" int32_t lmb200_graph_launch(lmb200_ctx h, uint64_t graph) {
  Ctx* c = ctx_from(h);
  HostGraph* G = graph_from(graph);
  if (!c || !G) return LMB200_EINVAL;
  LMB_REQUIRE(G->ctx == c, "graph_launch: the graph belongs to another context");
  LMB_REQUIRE(!c->capturing, "graph_launch: not between capture_begin and capture_end");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_CUDA(cudaGraphLaunch(G->exec, c->stream));
  c->launches += G->nodes;
  return LMB200_OK;
}

extern "C" int32_t lmb200_graph_destroy(lmb200_ctx h, uint64_t graph) {
  Ctx* c = ctx_from(h);
  HostGraph* G = graph_from(graph);
  if (!c || !G) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "graph_destroy: not between capture_begin and capture_end");   // it waits for the stream
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  cudaGraphExecDestroy(G->exec);
  G->magic = 0;
  delete G;
  if (--c->live_graphs <= 0) {                 // nothing can replay a read of the retired scratch blocks any more
    c->live_graphs = 0;
    for (void* p : c->retired_scratch) cudaFree(p);
    c->retired_scratch.clear();
    c->scratch_in_graph = false;
  }
  return LMB200_OK;
}

extern "C" int32_t lmb200_launch_count(lmb200_ctx h, int64_t* count) {
  Ctx* c = ctx_from(h);
  if (!c || !count) return LMB200_EINVAL;
  *count = c->launches;
  return LMB200_OK;
}

extern "C" int32_t lmb200_comm_unique_id(uint8_t id_out[128]) {
  LMB_REQUIRE(id_out, "comm_unique_id: null argument");
  LMB_TRY(nccl_load());
  Id128 id;
  memset(&id, 0, sizeof(id));
  const int r = g_nccl.GetUniqueId(&id);
  if (r != 0) return fail(LMB200_ENCCL, "ncclGetUniqueId: %s", nccl_str(r));
  memcpy(id_out, &id, 128);
  return LMB200_OK;
}

extern "C" int32_t lmb200_comm_init(lmb200_ctx h, int32_t n_ranks, int32_t rank, const uint8_t id_in[128]) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(id_in && n_ranks >= 1 && rank >= 0 && rank < n_ranks, "comm_init: rank %d of %d", rank, n_ranks);
  LMB_REQUIRE(!c->nccl_comm, "comm_init: communicator already exists");
  LMB_TRY(nccl_load());
  LMB_CUDA(cudaSetDevice(c->device));
  Id128 id;
  memcpy(&id, id_in, 128);
  void* comm = nullptr;
  const int r = g_nccl.CommInitRank(&comm, n_ranks, id, rank);
  if (r != 0) return fail(LMB200_ENCCL, "ncclCommInitRank: %s", nccl_str(r));
  c->nccl_comm = comm;
  c->tp_size = n_ranks;
  c->tp_rank = rank;
  return peer_setup(c);
}

extern "C" int32_t lmb200_comm_destroy(lmb200_ctx h) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  if (c->nccl_comm) {
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    peer_teardown(c);
    g_nccl.CommDestroy(c->nccl_comm);
    c->nccl_comm = nullptr;
    c->tp_size = 1;
    c->tp_rank = 0;
  }
  return LMB200_OK;
}

// After a failed tensor-parallel step (LMB200_ETIMEOUT) the ranks' step counters differ.  Collective:
// every rank calls this between steps with nothing in flight; the ranks agree on a step number past
// every rank's (NCCL max-reduce, bounded wait), which makes all older signals stale, and the broken
// marks are cleared.  Session positions are the caller's to put back (lmb200_session_set_position).
extern "C" int32_t lmb200_comm_resync(lmb200_ctx h) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(c->nccl_comm && c->tp_size > 1, "comm_resync: no tensor-parallel communicator");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_CUDA(cudaStreamSynchronize(c->stream));
  if (c->peer_n > 1) {
    // ncclUint64 = 5, ncclMax = 2
    const int r = g_nccl.AllReduce(c->peer_step, c->peer_step, 1, 5, 2, c->nccl_comm, c->own_stream);
    if (r != 0) return fail(LMB200_ENCCL, "comm_resync: ncclAllReduce: %s", nccl_str(r));
    if (!stream_done_within(c->own_stream, 10.0))
      return fail(LMB200_ETIMEOUT, "comm_resync: the other ranks did not join within 10 s");
    unsigned long long step = 0;
    LMB_CUDA(cudaMemcpy(&step, c->peer_step, 8, cudaMemcpyDeviceToHost));
    step += 1;
    LMB_CUDA(cudaMemcpy(c->peer_step, &step, 8, cudaMemcpyHostToDevice));
    // every rank has stopped (it joined the reduction above): leftovers of the failed step out of this rank's
    // push buffers, and nobody goes on before all ranks have done so
    LMB_TRY(peer_clear_push_buffers(c, c->peer_base[c->tp_rank]));
    const int r2 = g_nccl.AllReduce(c->peer_scratch, c->peer_scratch, 1, 7, 0, c->nccl_comm, c->own_stream);
    if (r2 != 0) return fail(LMB200_ENCCL, "comm_resync: ncclAllReduce: %s", nccl_str(r2));
    if (!stream_done_within(c->own_stream, 10.0))
      return fail(LMB200_ETIMEOUT, "comm_resync: the other ranks did not join within 10 s");
  }
  LMB_CUDA(cudaMemset(c->dev_broken, 0, sizeof(int)));
  *c->dev_err = 0;
  c->comm_broken = false;
  return LMB200_OK;
}

extern "C" int32_t lmb200_allreduce_sum_f32(lmb200_ctx h, void* dptr, int64_t count) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(dptr && count > 0, "allreduce: bad argument");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_TRY(nccl_allreduce_f32(c, dptr, count, c->stream));
  LMB_CUDA(cudaStreamSynchronize(c->stream));
  return LMB200_OK;
}

extern "C" int32_t lmb200_alloc(lmb200_ctx h, int64_t bytes, void** out) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "alloc: not between capture_begin and capture_end");
  LMB_REQUIRE(out && bytes >= 0, "alloc: bad argument");
  LMB_CUDA(cudaSetDevice(c->device));
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)(bytes > 0 ? bytes : 16));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(LMB200_ENOMEM, "alloc of %lld bytes failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  *out = p;
  return LMB200_OK;
}

extern "C" int32_t lmb200_free(lmb200_ctx h, void* dptr) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "free: not between capture_begin and capture_end");
  LMB_CUDA(cudaSetDevice(c->device));
  LMB_CUDA(cudaStreamSynchronize(c->stream));
  LMB_CUDA(cudaFree(dptr));
  return LMB200_OK;
}

static int32_t shape_of(int32_t rank, const int64_t* dims, Shape8* s, int64_t* total) {
  LMB_REQUIRE(rank >= 0 && rank <= 8, "rank %d outside 0..8", rank);
  s->rank = rank;
  int64_t t = 1;
  for (int i = 0; i < rank; ++i) {
    LMB_REQUIRE(dims && dims[i] >= 0, "negative dimension");
    s->d[i] = dims[i];
    t *= dims[i];
  }
  *total = t;
  return LMB200_OK;
}

extern "C" int32_t lmb200_upload(lmb200_ctx h, void* dptr, int32_t dtype, const float* host, int32_t rank,
                                 const int64_t* dims, int32_t layout) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "upload: not between capture_begin and capture_end");
  LMB_REQUIRE(dptr && host, "upload: null pointer");
  LMB_REQUIRE(dtype == LMB200_F32 || dtype == LMB200_BF16, "upload: dtype %d", dtype);
  Shape8 s;
  int64_t total;
  LMB_TRY(shape_of(rank, dims, &s, &total));
  if (total == 0) return LMB200_OK;
  LMB_CUDA(cudaSetDevice(c->device));
  if (dtype == LMB200_F32 && (layout == LMB200_ROWMAJOR || rank <= 1)) {
    LMB_CUDA(cudaMemcpyAsync(dptr, host, (size_t)total * 4, cudaMemcpyHostToDevice, c->stream));
    LMB_CUDA(cudaStreamSynchronize(c->stream));
    return LMB200_OK;
  }
  float* stage = nullptr;
  LMB_CUDA(cudaMalloc(&stage, (size_t)total * 4));
  cudaError_t e = cudaMemcpyAsync(stage, host, (size_t)total * 4, cudaMemcpyHostToDevice, c->stream);
  if (e == cudaSuccess) {
    const int grid = (int)(ceil_div(total, 256) > 4096 ? 4096 : ceil_div(total, 256));
    if (dtype == LMB200_F32)
      relayout_kernel<float, true><<<grid, 256, 0, c->stream>>>((float*)dptr, stage, s, layout, total);
    else
      relayout_kernel<__nv_bfloat16, true><<<grid, 256, 0, c->stream>>>((__nv_bfloat16*)dptr, stage, s, layout, total);
    c->launches++;
    e = cudaGetLastError();
  }
  cudaStreamSynchronize(c->stream);
  cudaFree(stage);
  if (e != cudaSuccess) return fail(LMB200_ECUDA, "upload: %s", cudaGetErrorString(e));
  return LMB200_OK;
}

extern "C" int32_t lmb200_download(lmb200_ctx h, float* host, const void* dptr, int32_t dtype, int32_t rank,
                                   const int64_t* dims, int32_t layout) {
  Ctx* c = ctx_from(h);
  if (!c) return LMB200_EINVAL;
  LMB_REQUIRE(!c->capturing, "download: not between capture_begin and capture_end");
  LMB_REQUIRE(dptr && host, "download: null pointer");
  LMB_REQUIRE(dtype == LMB200_F32 || dtype == LMB200_BF16, "download: dtype %d", dtype);
  Shape8 s;
  int64_t total;
  LMB_TRY(shape_of(rank, dims, &s, &total));
  if (total == 0) return LMB200_OK;
  LMB_CUDA(cudaSetDevice(c->device));
  if (dtype == LMB200_F32 && (layout == LMB200_ROWMAJOR || rank <= 1)) {
    LMB_CUDA(cudaMemcpyAsync(host, dptr, (size_t)total * 4, cudaMemcpyDeviceToHost, c->stream));
    LMB_CUDA(cudaStreamSynchronize(c->stream));
    return LMB200_OK;
  }
  float* stage = nullptr;
  LMB_CUDA(cudaMalloc(&stage, (size_t)total * 4));
  const int grid = (int)(ceil_div(total, 256) > 4096 ? 4096 : ceil_div(total, 256));
  if (dtype == LMB200_F32)
    relayout_kernel<float, false><<<grid, 256, 0, c->stream>>>((float*)dptr, stage, s, layout, total);
  else
    relayout_kernel<__nv_bfloat16, false><<<grid, 256, 0, c->stream>>>((__nv_bfloat16*)dptr, stage, s, layout, total);
  c->launches++;
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyAsync(host, stage, (size_t)total * 4, cudaMemcpyDeviceToHost, c->stream);
  cudaStreamSynchronize(c->stream);
  cudaFree(stage);
  if (e != cudaSuccess) return fail(LMB200_ECUDA, "download: %s", cudaGetErrorString(e));
  return LMB200_OK;
}
