// Whisper AudioEncoder and the cross-K/V projection on the tensor cores (bf16).
//
// The reference builds the encoder from primitive nodes -- Conv1D as pad + unfold + permute +
// reshape + matmul (src/NN.jl:55-104), attention with a materialised [B, H, S, S] score tensor
// (src/Whisper.jl:238-276), LayerNorm, Linear, GELU (src/Whisper.jl:322-404) -- and projects the
// encoder output to every decoder layer's cross K/V (src/Whisper.jl:809-831).  Here each Conv1D is
// an implicit GEMM (the prompt GEMM whose activation tiles are, per pipeline step, 64 channels of one tap read
// from the token-major input through a 4-D tensor map; the weight columns keep the reference's merged index c + C*k,
// regrouped tap by tap) with a bias + GELU epilogue, the Linears are the same GEMM with bias / scale /
// GELU epilogues, attention is the tensor-core flash kernel (non-causal), and the cross K/V GEMMs
// write straight into the decode session's tiled cross cache.
//
// Head split: the reference's column-major reshape puts feature f = h + H*d in head h.  The rows of
// q/k/v (and of the cross k/v) projections and the columns of out_proj are permuted at upload so
// that the kernels see the head-major order h*D + d.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "model.cuh"

namespace lmb {

int32_t gemm_affine(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int T, int rows, int K, const float* bias, float scale,
                    int gelu, void* out, int ldo, int out_bf16, cudaStream_t st);
int32_t gemm_conv1d(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int batch, int rows_in, int C, int cpad, int taps,
                    int stride, int pad, int Lout, int out_rpb, int rows, const float* bias, int gelu, void* out, int ldo,
                    int out_bf16, cudaStream_t st);
int32_t gemm_cross_kv(Ctx* ctx, const void* W, const __nv_bfloat16* X, int ldx, int T, int rows, int K, const float* bias, float scale,
                      void* kv_layer, int64_t batch_stride, int64_t head_stride, int n_seq, int D, int is_v, cudaStream_t st);
int32_t flash_tc_launch_view(Ctx* ctx, void* out, const void* q, const void* k, const void* v, const FlashView& fv, int64_t B,
                             int64_t S, int64_t D, float scale, int causal, cudaStream_t stream);
bool flash_tc_supported(int64_t D);

namespace {

constexpr float kHalfPi = 1.5707963267948966f;

struct Bufs {
  std::vector<void*> p;
  ~Bufs() { release(); }
  void release() { for (void* q : p) cudaFree(q); p.clear(); }
  template <typename T>
  int32_t get(T** out, int64_t elems) {
    void* q = nullptr;
    if (cudaMalloc(&q, (size_t)(elems * (int64_t)sizeof(T))) != cudaSuccess) {
      cudaGetLastError();
      return fail(LMB200_ENOMEM, "whisper encoder: scratch allocation failed");
    }
    p.push_back(q);
    *out = reinterpret_cast<T*>(q);
    return LMB200_OK;
  }
};


struct EncLinear {
  void* W = nullptr;        // bf16, tensor-core weight layout
  float* bias = nullptr;    // [rows] or NULL
  int rows = 0, K = 0;
};
struct EncLayer {
  EncLinear q, k, v, o, fc1, fc2;
  float *ln1_w = nullptr, *ln1_b = nullptr, *ln2_w = nullptr, *ln2_b = nullptr;
};
struct WhisperEncoder {
  uint32_t magic = 0x57454E43;
  Ctx* ctx = nullptr;
  int d = 0, H = 0, L = 0, ffn = 0, n_mels = 0, dec_layers = 0;
  EncLinear conv1, conv2;
  std::vector<EncLayer> layers;
  float *post_w = nullptr, *post_b = nullptr;
  std::vector<EncLinear> cross_k, cross_v;
  float* inv_ts = nullptr;              // [d/2] sinusoid rates
  __nv_bfloat16* enc_b = nullptr;       // last output, bf16 [B * S, d]
  float* enc_f = nullptr;               // last output, float32
  int out_B = 0, out_S = 0;
  // scratch of the last run, kept while the input shape stays the same
  Bufs scratch;
  int scratch_B = 0, scratch_frames = 0;
  float *mel = nullptr, *x = nullptr, *delta = nullptr;
  __nv_bfloat16 *melt = nullptr, *h1 = nullptr, *xn = nullptr, *qb = nullptr, *kb = nullptr, *vb = nullptr, *attn = nullptr,
                *act = nullptr;
};

WhisperEncoder* enc_from(uint64_t h) {
  WhisperEncoder* e = reinterpret_cast<WhisperEncoder*>(h);
  if (!e || e->magic != 0x57454E43) { set_error("invalid whisper encoder handle"); return nullptr; }
  return e;
}

enum Perm { PERM_NONE = 0, PERM_ROWS = 1, PERM_COLS = 2, PERM_CONV = 3 };

// dst (tensor-core layout, zero padded) <- src [rows, cols] float32 (row- or column-major), with the
// head permutation f = h + H*dd -> h*D + dd applied to the rows or to the columns
__global__ void canon_fill_kernel(__nv_bfloat16* dst, const float* src, int rows, int cols, int cols_dst, int colmajor, int perm,
                                  int H, int D, int rows_pad, int KS) {
  const int64_t total = (int64_t)rows_pad * KS * 128;
  for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < total; o += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(o / (KS * 128)), k = (int)(o - (int64_t)r * (KS * 128));
    float v = 0.f;
    if (r < rows && k < cols_dst) {
      int sr = r, sk = k;
      if (perm == PERM_ROWS) sr = (r / D) + H * (r % D);
      if (perm == PERM_COLS) sk = (k / D) + H * (k % D);
      // convolution weights: destination column tap * cpad + c <- the reference's merged column c + C * tap (H = C, D = cpad)
      if (perm == PERM_CONV) sk = (k % D) < H ? (k % D) + H * (k / D) : -1;
      if (sk >= 0) v = colmajor ? src[(int64_t)sk * rows + sr] : src[(int64_t)sr * cols + sk];
    }
    dst[wcanon_offset(r, k, KS)] = __float2bfloat16_rn(v);
  }
}

// mel [B, C, L] float32 -> token-major bf16 [B, L, pitch] (channels contiguous, pitch >= C): the layout whose rows the
// implicit convolution's tensor map reads
__global__ void mel_tokens_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ mel, int B, int C, int L, int pitch) {
  const int64_t total = (int64_t)B * L * pitch;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % pitch);
    const int64_t row = i / pitch;
    const int l = (int)(row % L), b = (int)(row / L);
    out[i] = __float2bfloat16_rn(c < C ? mel[((int64_t)b * C + c) * L + l] : 0.f);
  }
}

// x[b, s, :] += sinusoids(d, S)[s, :]: sin(s * inv_ts[i]) for i < d/2, then cos = sin(pi/2 - .)  (src/Whisper.jl:208-231)
__global__ void add_sinusoids_kernel(float* __restrict__ x, const float* __restrict__ inv_ts, int S, int d, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % d), s = (int)((i / d) % S);
    const int half = d >> 1;
    const float a = (float)s * inv_ts[c < half ? c : c - half];
    x[i] += c < half ? sinf(a) : sinf(kHalfPi + a * -1.0f);
  }
}

// x[t, :] += delta[t, :] (if given); y = LayerNorm(x) * w + b with mean-centering (src/NN.jl:138-173)
__global__ void __launch_bounds__(256) layernorm_rows_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                             const float* __restrict__ w, const float* __restrict__ bias,
                                                             __nv_bfloat16* __restrict__ yb, float* __restrict__ yf, int n, float eps) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  float* xr = x + (int64_t)t * n;
  auto block_sum = [&](float v) -> float {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i];
    return s;
  };
  float s1 = 0.f;
  for (int i = tid; i < n; i += 256) {
    float v = xr[i];
    if (delta) { v += delta[(int64_t)t * n + i]; xr[i] = v; }
    row[i] = v;
    s1 += v;
  }
  const float mean = block_sum(s1) * (1.0f / (float)n);
  float s2 = 0.f;
  for (int i = tid; i < n; i += 256) { const float c = row[i] + mean * -1.0f; row[i] = c; s2 += c * c; }
  const float var = block_sum(s2) * (1.0f / (float)n);
  const float inv = 1.0f / sqrtf(var + eps);
  for (int i = tid; i < n; i += 256) {
    const float y = (row[i] * inv) * w[i] + bias[i];
    if (yb) yb[(int64_t)t * n + i] = __float2bfloat16_rn(y);
    if (yf) yf[(int64_t)t * n + i] = y;
  }
}

int grid_for(int64_t total) { return (int)std::min<int64_t>(ceil_div(total, 256), 8192); }

int32_t dev_alloc(void** p, int64_t bytes) {
  if (cudaMalloc(p, (size_t)(bytes > 0 ? bytes : 16)) != cudaSuccess) {
    cudaGetLastError();
    return fail(LMB200_ENOMEM, "whisper encoder: allocation of %lld bytes failed", (long long)bytes);
  }
  return LMB200_OK;
}

int32_t upload_matrix(WhisperEncoder* E, EncLinear& lin, const float* host, int rows, int cols, int layout, int perm) {
  Ctx* ctx = E->ctx;
  // a convolution's [out, C * 3] matrix is stored tap by tap with the channels of a tap padded to a multiple of 64: a
  // pipeline step of the implicit GEMM is then 64 channels of one tap
  const int conv_C = cols / 3, conv_cpad = (conv_C + 63) / 64 * 64;
  const int cols_dst = perm == PERM_CONV ? 3 * conv_cpad : cols;
  const int KS = (cols_dst + 127) / 128, rows_pad = (rows + 127) / 128 * 128;
  float* stage = nullptr;
  LMB_TRY(dev_alloc((void**)&stage, (int64_t)rows * cols * 4));
  int32_t rc = LMB200_OK;
  if (!lin.W) rc = dev_alloc(&lin.W, (int64_t)rows_pad * KS * 128 * 2);
  if (rc == LMB200_OK && cudaMemcpyAsync(stage, host, (size_t)rows * cols * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
    rc = fail(LMB200_ECUDA, "whisper encoder: upload failed");
  if (rc == LMB200_OK) {
    const bool cv = perm == PERM_CONV;
    canon_fill_kernel<<<grid_for((int64_t)rows_pad * KS * 128), 256, 0, ctx->stream>>>(
        reinterpret_cast<__nv_bfloat16*>(lin.W), stage, rows, cols, cols_dst, layout == LMB200_COLMAJOR, perm, cv ? conv_C : E->H,
        cv ? conv_cpad : E->d / E->H, rows_pad, KS);
    ctx->launches++;
    lin.rows = rows; lin.K = cols_dst;
  }
  cudaStreamSynchronize(ctx->stream);
  cudaFree(stage);
  return rc;
}

int32_t upload_vector(WhisperEncoder* E, float** dst, const float* host, int n, bool head_perm) {
  std::vector<float> tmp(host, host + n);
  if (head_perm) {
    const int H = E->H, D = E->d / E->H;
    for (int r = 0; r < n; ++r) tmp[r] = host[(r / D) + H * (r % D)];
  }
  if (!*dst) LMB_TRY(dev_alloc((void**)dst, (int64_t)n * 4));
  LMB_CUDA(cudaMemcpy(*dst, tmp.data(), (size_t)n * 4, cudaMemcpyHostToDevice));
  return LMB200_OK;
}

void free_linear(EncLinear& l) { cudaFree(l.W); cudaFree(l.bias); l.W = nullptr; l.bias = nullptr; }

}  // namespace
}  // namespace lmb

using namespace lmb;

extern "C" int32_t lmb200_whisper_encoder_create(lmb200_ctx hctx, int32_t d_model, int32_t heads, int32_t layers, int32_t ffn,
                                                 int32_t n_mels, int32_t dec_layers, uint64_t* out) {
  Ctx* ctx = ctx_from(hctx);
  if (!ctx) return LMB200_EINVAL;
  LMB_REQUIRE(out, "whisper_encoder_create: null argument");
  LMB_REQUIRE(d_model >= 16 && heads >= 1 && d_model % heads == 0 && flash_tc_supported(d_model / heads),
              "whisper_encoder_create: d_model %d with %d heads (head_dim 64, 96 or 128)", d_model, heads);
  LMB_REQUIRE(d_model % 8 == 0 && ffn % 8 == 0 && n_mels % 8 == 0 && layers >= 1 && dec_layers >= 0,
              "whisper_encoder_create: sizes must be multiples of 8");
  LMB_CUDA(cudaSetDevice(ctx->device));
  WhisperEncoder* E = new WhisperEncoder();
  E->ctx = ctx; E->d = d_model; E->H = heads; E->L = layers; E->ffn = ffn; E->n_mels = n_mels; E->dec_layers = dec_layers;
  E->layers.resize(layers);
  E->cross_k.resize(dec_layers);
  E->cross_v.resize(dec_layers);
  // sinusoid rates as the reference computes them: exp(-log(10000) / (d/2 - 1) * i) in float64, rounded to float32
  std::vector<float> inv(d_model / 2);
  const double inc = log(10000.0) / (d_model / 2 - 1);
  for (int i = 0; i < d_model / 2; ++i) inv[i] = (float)exp(-inc * i);
  if (dev_alloc((void**)&E->inv_ts, (int64_t)inv.size() * 4) != LMB200_OK ||
      cudaMemcpy(E->inv_ts, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
    delete E;
    return fail(LMB200_ECUDA, "whisper_encoder_create: setup failed");
  }
  *out = reinterpret_cast<uint64_t>(E);
  return LMB200_OK;
}

extern "C" int32_t lmb200_whisper_encoder_destroy(uint64_t h) {
  WhisperEncoder* E = enc_from(h);
  if (!E) return LMB200_EINVAL;
  cudaSetDevice(E->ctx->device);
  cudaStreamSynchronize(E->ctx->stream);
  free_linear(E->conv1); free_linear(E->conv2);
  for (EncLayer& l : E->layers) {
    free_linear(l.q); free_linear(l.k); free_linear(l.v); free_linear(l.o); free_linear(l.fc1); free_linear(l.fc2);
    cudaFree(l.ln1_w); cudaFree(l.ln1_b); cudaFree(l.ln2_w); cudaFree(l.ln2_b);
  }
  for (EncLinear& l : E->cross_k) free_linear(l);
  for (EncLinear& l : E->cross_v) free_linear(l);
  cudaFree(E->post_w); cudaFree(E->post_b); cudaFree(E->inv_ts); cudaFree(E->enc_b); cudaFree(E->enc_f);
  E->scratch.release();
  E->magic = 0;
  delete E;
  return LMB200_OK;
}

// Names as the reference registers them (src/Whisper.jl:354-404, 809-831): model.encoder.conv{1,2}.{weight,bias},
// model.encoder.layers.{i}.{self_attn.{q,k,v,out}_proj, self_attn_layer_norm, fc1, fc2, final_layer_norm}.{weight,bias},
// model.encoder.layer_norm.{weight,bias}, model.decoder.layers.{i}.encoder_attn.{k,v}_proj.{weight,bias}.
// The reference registers the tensors of its encoder blocks as layers.{i}.attn.{q,k,v,out}_proj.*, attn_layer_norm.*,
// mlp.fc1.* and mlp.fc2.* (src/Whisper.jl:330-336), while checkpoints -- and the reference's own decoder blocks
// (src/Whisper.jl:424-431) -- spell them self_attn.*, self_attn_layer_norm.*, fc1.* and fc2.*.  Both spellings name the
// same tensor; this gives the checkpoint's.
static std::string canonical_encoder_name(const std::string& n) {
  const std::string pre = "model.encoder.layers.";
  if (n.rfind(pre, 0) != 0) return n;
  const size_t dot = n.find('.', pre.size());
  if (dot == std::string::npos) return n;
  const std::string head = n.substr(0, dot + 1), t = n.substr(dot + 1);
  static const char* const kAlias[][2] = {{"attn.", "self_attn."}, {"attn_layer_norm.", "self_attn_layer_norm."},
                                          {"mlp.fc1.", "fc1."}, {"mlp.fc2.", "fc2."}};
  for (const auto& a : kAlias)
    if (t.rfind(a[0], 0) == 0) return head + a[1] + t.substr(strlen(a[0]));
  return n;
}

extern "C" int32_t lmb200_whisper_canonical_name(const char* name, char* out, int64_t capacity) {
  LMB_REQUIRE(name && out && capacity > 0, "whisper_canonical_name: null argument");
  const std::string c = canonical_encoder_name(name);
  LMB_REQUIRE((int64_t)c.size() < capacity, "whisper_canonical_name: %lld bytes do not hold %s", (long long)capacity, c.c_str());
  memcpy(out, c.c_str(), c.size() + 1);
  return LMB200_OK;
}

extern "C" int32_t lmb200_whisper_encoder_set_weight(uint64_t h, const char* name, const float* host, int32_t rank,
                                                     const int64_t* dims, int32_t layout) {
  WhisperEncoder* E = enc_from(h);
  if (!E) return LMB200_EINVAL;
  LMB_REQUIRE(name && host, "whisper_encoder_set_weight: null argument");
  LMB_REQUIRE(rank >= 1 && rank <= 2 && dims, "whisper_encoder_set_weight: %s: rank %d (expected 1 or 2 with the dimensions given)", name, rank);
  // the stated shape must be the one the encoder's configuration gives the tensor: nothing is read past it
  auto shape_is = [&](int64_t rows, int64_t cols) -> int32_t {
    const int64_t d0 = dims[0], d1 = rank == 2 ? dims[1] : 1;
    const bool ok = rows == 1 ? ((rank == 1 && d0 == cols) || (rank == 2 && ((d0 == 1 && d1 == cols) || (d0 == cols && d1 == 1))))
                              : (rank == 2 && d0 == rows && d1 == cols);
    if (!ok)
      return fail(LMB200_EINVAL, "whisper_encoder_set_weight: %s has shape [%lld, %lld] (rank %d), the encoder expects [%lld, %lld]",
                  name, (long long)d0, (long long)d1, rank, (long long)rows, (long long)cols);
    return LMB200_OK;
  };
  LMB_REQUIRE(layout == LMB200_ROWMAJOR || layout == LMB200_COLMAJOR, "whisper_encoder_set_weight: layout %d", layout);
  LMB_CUDA(cudaSetDevice(E->ctx->device));
  const std::string n = canonical_encoder_name(name);
  const int d = E->d;
  auto linear = [&](EncLinear& lin, const std::string& tail, int rows, int cols, int perm) -> int32_t {
    if (tail == "weight") { LMB_TRY(shape_is(rows, cols)); return upload_matrix(E, lin, host, rows, cols, layout, perm); }
    if (tail == "bias") { LMB_TRY(shape_is(1, rows)); return upload_vector(E, &lin.bias, host, rows, perm == PERM_ROWS); }
    return fail(LMB200_ENOTFOUND, "whisper_encoder_set_weight: unknown tensor %s", name);
  };
  auto vec = [&](float** dst, int len) -> int32_t { LMB_TRY(shape_is(1, len)); return upload_vector(E, dst, host, len, false); };
  const std::string enc = "model.encoder.", dec = "model.decoder.layers.";
  if (n.rfind(enc, 0) == 0) {
    const std::string r = n.substr(enc.size());
    if (r.rfind("conv1.", 0) == 0) return linear(E->conv1, r.substr(6), d, E->n_mels * 3, PERM_CONV);
    if (r.rfind("conv2.", 0) == 0) return linear(E->conv2, r.substr(6), d, d * 3, PERM_CONV);
    if (r == "layer_norm.weight") return vec(&E->post_w, d);
    if (r == "layer_norm.bias") return vec(&E->post_b, d);
    if (r.rfind("layers.", 0) == 0) {
      const size_t dot = r.find('.', 7);
      LMB_REQUIRE(dot != std::string::npos, "whisper_encoder_set_weight: unknown tensor %s", name);
      const int i = atoi(r.substr(7, dot - 7).c_str());
      LMB_REQUIRE(i >= 0 && i < E->L, "whisper_encoder_set_weight: layer %d of %d", i, E->L);
      EncLayer& l = E->layers[i];
      const std::string t = r.substr(dot + 1);
      if (t.rfind("self_attn.q_proj.", 0) == 0) return linear(l.q, t.substr(17), d, d, PERM_ROWS);
      if (t.rfind("self_attn.k_proj.", 0) == 0) return linear(l.k, t.substr(17), d, d, PERM_ROWS);
      if (t.rfind("self_attn.v_proj.", 0) == 0) return linear(l.v, t.substr(17), d, d, PERM_ROWS);
      if (t.rfind("self_attn.out_proj.", 0) == 0) return linear(l.o, t.substr(19), d, d, t.substr(19) == "weight" ? PERM_COLS : PERM_NONE);
      if (t == "self_attn_layer_norm.weight") return vec(&l.ln1_w, d);
      if (t == "self_attn_layer_norm.bias") return vec(&l.ln1_b, d);
      if (t == "final_layer_norm.weight") return vec(&l.ln2_w, d);
      if (t == "final_layer_norm.bias") return vec(&l.ln2_b, d);
      if (t.rfind("fc1.", 0) == 0) return linear(l.fc1, t.substr(4), E->ffn, d, PERM_NONE);
      if (t.rfind("fc2.", 0) == 0) return linear(l.fc2, t.substr(4), d, E->ffn, PERM_NONE);
    }
  } else if (n.rfind(dec, 0) == 0) {
    const size_t dot = n.find('.', dec.size());
    if (dot != std::string::npos) {
      const int i = atoi(n.substr(dec.size(), dot - dec.size()).c_str());
      const std::string t = n.substr(dot + 1);
      if (i >= 0 && i < E->dec_layers) {
        if (t.rfind("encoder_attn.k_proj.", 0) == 0) return linear(E->cross_k[i], t.substr(20), d, d, PERM_ROWS);
        if (t.rfind("encoder_attn.v_proj.", 0) == 0) return linear(E->cross_v[i], t.substr(20), d, d, PERM_ROWS);
      }
    }
  }
  return fail(LMB200_ENOTFOUND, "whisper_encoder_set_weight: unknown tensor %s", name);
}

// mel: [batch, n_mels, frames] float32 row-major on the host.  out (NULL or [batch, S, d_model] float32, S =
// (frames - 1) / 2 + 1) receives the encoder output; it also stays on the device for lmb200_whisper_encoder_cross_kv.
extern "C" int32_t lmb200_whisper_encoder_run(uint64_t h, const float* mel_host, int32_t batch, int32_t frames, float* out_host) {
  WhisperEncoder* E = enc_from(h);
  if (!E) return LMB200_EINVAL;
  LMB_REQUIRE(mel_host && batch >= 1 && frames >= 3, "whisper_encoder_run: batch %d, frames %d", batch, frames);
  Ctx* ctx = E->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  cudaStream_t st = ctx->stream;
  const int d = E->d, H = E->H, D = d / H, C1 = E->n_mels;
  LMB_REQUIRE(E->conv1.W && E->conv1.bias && E->conv2.W && E->conv2.bias && E->post_w && E->post_b, "whisper_encoder_run: weights missing");
  for (const EncLayer& l : E->layers)
    LMB_REQUIRE(l.q.W && l.q.bias && l.k.W && l.v.W && l.v.bias && l.o.W && l.o.bias && l.fc1.W && l.fc1.bias && l.fc2.W && l.fc2.bias &&
                    l.ln1_w && l.ln1_b && l.ln2_w && l.ln2_b,
                "whisper_encoder_run: layer weights missing");
  const int L1 = frames;                         // conv1: kernel 3, stride 1, padding 1
  const int S = (frames + 2 - 3) / 2 + 1;        // conv2: kernel 3, stride 2, padding 1
  const int L1p = (L1 + 1) / 2 * 2;              // rows per batch element of conv1's output: even, so that a tap of the
                                                 // stride-2 convolution is one parity of consecutive row pairs
  const int C1p = (C1 + 7) / 8 * 8;              // channel pitch of the token-major mel (rows start on 16 bytes)
  const int64_t T1 = (int64_t)batch * L1, T = (int64_t)batch * S;
  if (E->scratch_B != batch || E->scratch_frames != frames) {
    E->scratch.release();
    E->scratch_B = E->scratch_frames = 0;
    Bufs& sc = E->scratch;
    LMB_TRY(sc.get(&E->mel, (int64_t)batch * C1 * frames));
    LMB_TRY(sc.get(&E->melt, T1 * C1p));
    LMB_TRY(sc.get(&E->h1, (int64_t)batch * L1p * d));
    LMB_CUDA(cudaMemsetAsync(E->h1, 0, (size_t)batch * L1p * d * 2, st));      // the pad row of an odd length stays zero
    LMB_TRY(sc.get(&E->x, T * d));
    LMB_TRY(sc.get(&E->delta, T * d));
    LMB_TRY(sc.get(&E->xn, T * d));
    LMB_TRY(sc.get(&E->qb, T * d));
    LMB_TRY(sc.get(&E->kb, T * d));
    LMB_TRY(sc.get(&E->vb, T * d));
    LMB_TRY(sc.get(&E->attn, T * d));
    LMB_TRY(sc.get(&E->act, T * E->ffn));
    E->scratch_B = batch; E->scratch_frames = frames;
  }
  float *mel = E->mel, *x = E->x, *delta = E->delta;
  __nv_bfloat16 *melt = E->melt, *h1 = E->h1, *xn = E->xn, *qb = E->qb, *kb = E->kb, *vb = E->vb, *attn = E->attn,
                *act = E->act;
  if (E->out_B * E->out_S != T) {
    cudaFree(E->enc_b); cudaFree(E->enc_f);
    E->enc_b = nullptr; E->enc_f = nullptr;
    LMB_TRY(dev_alloc((void**)&E->enc_b, T * d * 2));
    LMB_TRY(dev_alloc((void**)&E->enc_f, T * d * 4));
  }
  E->out_B = batch; E->out_S = S;
  LMB_CUDA(cudaMemcpyAsync(mel, mel_host, (size_t)batch * C1 * frames * 4, cudaMemcpyHostToDevice, st));
  // stem: conv1 + GELU, conv2 + GELU (implicit GEMMs: the activation tiles of every tap come straight from the
  // token-major input, nothing is unfolded), positions
  mel_tokens_kernel<<<grid_for(T1 * C1p), 256, 0, st>>>(melt, mel, batch, C1, frames, C1p);
  ctx->launches++;
  LMB_TRY(gemm_conv1d(ctx, E->conv1.W, melt, C1p, batch, L1, C1, E->conv1.K / 3, 3, 1, 1, L1, L1p, d, E->conv1.bias, 1, h1, d, 1, st));
  LMB_TRY(gemm_conv1d(ctx, E->conv2.W, h1, d, batch, L1p, d, E->conv2.K / 3, 3, 2, 1, S, S, d, E->conv2.bias, 1, x, d, 0, st));
  add_sinusoids_kernel<<<grid_for(T * d), 256, 0, st>>>(x, E->inv_ts, S, d, T * d);
  ctx->launches++;
  const float scale = powf((float)d / (float)H, -0.25f);          // on q and k (src/Whisper.jl:257-260)
  const size_t ln_smem = (size_t)d * sizeof(float);
  FlashView fv;
  fv.H = H; fv.G = 1;
  fv.q_b = fv.k_b = (int64_t)S * d; fv.q_h = fv.k_h = D; fv.q_s = fv.k_s = d;
  for (int i = 0; i < E->L; ++i) {
    EncLayer& l = E->layers[i];
    layernorm_rows_kernel<<<(unsigned)T, 256, ln_smem, st>>>(x, i == 0 ? nullptr : delta, l.ln1_w, l.ln1_b, xn, nullptr, d, 1e-5f);
    ctx->launches++;
    LMB_TRY(gemm_affine(ctx, l.q.W, xn, d, (int)T, d, d, l.q.bias, scale, 0, qb, d, 1, st));
    LMB_TRY(gemm_affine(ctx, l.k.W, xn, d, (int)T, d, d, l.k.bias, scale, 0, kb, d, 1, st));
    LMB_TRY(gemm_affine(ctx, l.v.W, xn, d, (int)T, d, d, l.v.bias, 1.0f, 0, vb, d, 1, st));
    LMB_TRY(flash_tc_launch_view(ctx, attn, qb, kb, vb, fv, batch, S, D, 1.0f, 0, st));
    LMB_TRY(gemm_affine(ctx, l.o.W, attn, d, (int)T, d, d, l.o.bias, 1.0f, 0, delta, d, 0, st));
    layernorm_rows_kernel<<<(unsigned)T, 256, ln_smem, st>>>(x, delta, l.ln2_w, l.ln2_b, xn, nullptr, d, 1e-5f);
    ctx->launches++;
    LMB_TRY(gemm_affine(ctx, l.fc1.W, xn, d, (int)T, E->ffn, d, l.fc1.bias, 1.0f, 1, act, E->ffn, 1, st));
    LMB_TRY(gemm_affine(ctx, l.fc2.W, act, E->ffn, (int)T, d, E->ffn, l.fc2.bias, 1.0f, 0, delta, d, 0, st));
  }
  layernorm_rows_kernel<<<(unsigned)T, 256, ln_smem, st>>>(x, delta, E->post_w, E->post_b, E->enc_b, E->enc_f, d, 1e-5f);
  ctx->launches++;
  LMB_CUDA(cudaGetLastError());
  if (out_host) LMB_CUDA(cudaMemcpyAsync(out_host, E->enc_f, (size_t)T * d * 4, cudaMemcpyDeviceToHost, st));
  LMB_CUDA(cudaStreamSynchronize(st));
  return check_device_error(ctx);
}

// Projects the last encoder output to the cross K/V of every decoder layer and writes them into the session's
// cross cache (what project_cross_kv + lmb200_session_set_cross_kv do through the host).
extern "C" int32_t lmb200_whisper_encoder_cross_kv(uint64_t h, lmb200_session hs) {
  WhisperEncoder* E = enc_from(h);
  Session* S = session_from(hs);
  if (!E || !S) return LMB200_EINVAL;
  Model* M = S->m;
  const lmb200_model_config& c = M->cfg;
  LMB_REQUIRE(c.arch == LMB200_ARCH_WHISPER_DECODER && S->cross_kv && c.dtype == LMB200_BF16, "whisper_encoder_cross_kv: needs a bf16 Whisper decoder session");
  LMB_REQUIRE(E->enc_b && E->out_B == S->B && E->out_S == c.cross_len && c.hidden == E->d && c.n_heads == E->H && c.n_layers == E->dec_layers,
              "whisper_encoder_cross_kv: encoder output [%d, %d] does not match the session", E->out_B, E->out_S);
  Ctx* ctx = E->ctx;
  LMB_CUDA(cudaSetDevice(ctx->device));
  const int d = E->d, D = d / E->H;
  const float scale = powf((float)d / (float)E->H, -0.25f);
  const int T = E->out_B * E->out_S;
  for (int i = 0; i < E->dec_layers; ++i) {
    LMB_REQUIRE(E->cross_k[i].W && E->cross_v[i].W && E->cross_v[i].bias, "whisper_encoder_cross_kv: cross projection weights of layer %d missing", i);
    void* layer = reinterpret_cast<__nv_bfloat16*>(S->cross_kv) + (int64_t)i * S->cross_layer_stride;
    LMB_TRY(gemm_cross_kv(ctx, E->cross_k[i].W, E->enc_b, d, T, d, d, E->cross_k[i].bias, scale, layer, S->cross_batch_stride,
                          S->cross_head_stride, E->out_S, D, 0, ctx->stream));
    LMB_TRY(gemm_cross_kv(ctx, E->cross_v[i].W, E->enc_b, d, T, d, d, E->cross_v[i].bias, 1.0f, layer, S->cross_batch_stride,
                          S->cross_head_stride, E->out_S, D, 1, ctx->stream));
  }
  LMB_CUDA(cudaStreamSynchronize(ctx->stream));
  return check_device_error(ctx);
}
