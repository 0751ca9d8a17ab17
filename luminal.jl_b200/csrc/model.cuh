// Model (weights in the tiled layouts) and session (KV cache, activations, CUDA graph of a step).
#pragma once
#include <map>
#include <set>
#include <string>
#include <vector>

#include "attention.cuh"
#include "common.cuh"
#include "gemv.cuh"

namespace lmb {

enum MapKind { MAP_PLAIN = 0, MAP_QKV = 1, MAP_O = 2, MAP_GATEUP = 3, MAP_DOWN = 4 };

// How one internal (tiled) matrix maps onto up to three logical [out,in] tensors of the
// reference (src/NN.jl:330-341, 238-244) -- including the head split f = h + H*d that the
// reference's column-major reshape implies (src/NN.jl:347-354), the GQA mapping q = kv + KV*g
// (src/NN.jl:305-317), the RoPE pairing (d, d + D/2) (src/NN.jl:274-276) and the tensor-parallel
// shard of this rank.
struct WMap {
  int kind = MAP_PLAIN;
  int rows = 0, K = 0;       // internal valid extent
  int RB = 0, KC = 0;        // padded extent in 16-row blocks / 32-k chunks
  int H = 0, KV = 0, D = 0, G = 0, Hl = 0, KVl = 0, kv_off = 0;
  int inter_l = 0, inter_off = 0;
  int src_rows[3] = {0, 0, 0};
  int src_cols[3] = {0, 0, 0};
};

struct LayerWeights {
  void* wqkv = nullptr;
  void* wo = nullptr;
  void* wgu = nullptr;
  void* wdown = nullptr;
  float* attn_norm = nullptr;
  float* ffn_norm = nullptr;
  // Whisper decoder layers only
  void* wq_cross = nullptr;      // encoder_attn.q_proj
  void* wo_cross = nullptr;      // encoder_attn.out_proj
  float* attn_norm_b = nullptr;  // LayerNorm biases
  float* ffn_norm_b = nullptr;
  float* cross_norm = nullptr;
  float* cross_norm_b = nullptr;
  float* b_qkv = nullptr;        // biases in internal row order (k rows zero)
  float* b_o = nullptr;
  float* b_q_cross = nullptr;
  float* b_o_cross = nullptr;
  float* b_fc1 = nullptr;
  float* b_fc2 = nullptr;
  // Whisper, fused step: what folding a LayerNorm into the Linear that follows it needs (InvScale): W g and W b + bias
  // per internal row of q/k/v, of the cross-attention q projection and of fc1
  float *wg_qkv = nullptr, *bf_qkv = nullptr, *wg_qc = nullptr, *bf_qc = nullptr, *wg_fc1 = nullptr, *bf_fc1 = nullptr;
};

struct Model {
  bool tp_solo = false;        // profiling aid: shard of one rank, no all-reduce
  uint32_t magic = 0x4D4F444C;
  Ctx* ctx = nullptr;
  lmb200_model_config cfg{};
  int esz = 4;
  int Hl = 0, KVl = 0, G = 0, D = 0, kv_off = 0, inter_l = 0, inter_off = 0;
  WMap m_qkv, m_o, m_gu, m_down, m_head;
  WMap m_qc;                    // Whisper: cross-attention q projection (q rows only)
  float* final_norm_b = nullptr;
  float* pos_emb = nullptr;     // Whisper: [max_positions, hidden] float32
  void* embed_tiled = nullptr;  // Whisper: the embedding table in GEMV layout (tied head)
  float *wg_head = nullptr, *bf_head = nullptr;   // Whisper, fused step: the final LayerNorm folded into the head
  bool fold_valid = false;      // the folded vectors match the weights (set_weight / init_random clear it)
  std::vector<LayerWeights> layers;
  void* embed = nullptr;        // [vocab, hidden] row-major, model dtype
  float* final_norm = nullptr;
  void* lm_head = nullptr;
  float* inv_freq = nullptr;    // [D/2]
  int64_t weight_bytes = 0;
  std::set<std::string> weights_set;   // registry names given through lmb200_model_set_weight
  bool all_weights_set = false;        // lmb200_model_init_random filled everything
};

struct Session {
  uint32_t magic = 0x53455353;
  Model* m = nullptr;
  int B = 0, max_ctx = 0, cap = 0;
  int host_pos = 0;               // the furthest position of any sequence (bounds checks)
  std::vector<int> host_pos_v;    // the host's copy of the per-sequence positions
  bool ragged = false;            // the positions differ: kernels take the per-sequence RoPE path
  bool in_ragged_prefill = false; // steps of lmb200_prefill_ragged: the host positions are set at its end
  int* limit = nullptr;           // device [B]: a sequence at its limit does not advance
  float* ragged_logits = nullptr; // [B][logits_pitch]: each sequence's logits at its own last prompt position
  // cache: [L][B][KVl][cap/16][32*D]
  void* kv = nullptr;
  int64_t kv_head_stride = 0, kv_batch_stride = 0, kv_layer_stride = 0;
  // activations
  float* x = nullptr;
  float* delta = nullptr;
  float* logits = nullptr;
  void* xn = nullptr;
  void* qbuf = nullptr;
  void* attn_out = nullptr;
  void* act = nullptr;
  int Bp = 0;                   // batch padding of the tiled activation buffers (8, 16 or 32)
  int q_pitch = 0, logits_pitch = 0;
  int* tokens = nullptr;
  int* pos = nullptr;           // device [B]: one position per sequence
  int* step_ctr = nullptr;
  int* stop = nullptr;          // [0] end-of-text id or -1, [1] sequences that produced it, [2 + b] sequence b did
  int* tok_hist = nullptr;      // [cap][B]
  int* prompt = nullptr;        // staging for prefill
  int64_t prompt_cap = 0;
  // scratch
  float* gemv_partials = nullptr;
  unsigned* gemv_counters = nullptr;
  float* part_o = nullptr;
  float* part_ml = nullptr;
  unsigned* attn_counters = nullptr;   // [B*KVl], zero between launches
  float* sum_slots = nullptr;          // fused Whisper step: per-CTA sums of x beside ssq (LayerNorm's mean)
  void* prefill_buf = nullptr;         // scratch of the GEMM prompt phase, kept between prompts
  int64_t prefill_bytes = 0;
  int keys_per_cta = 0, nsplit = 0;
  GemvPlan p_qkv, p_o, p_gu, p_down, p_head, p_qc;
  // Whisper: cross-attention cache [L][B][H][cross_cap/16][32*D] and its split plan
  void* cross_kv = nullptr;
  int cross_cap = 0;
  int64_t cross_head_stride = 0, cross_batch_stride = 0, cross_layer_stride = 0;
  int cross_keys_per_cta = 0, cross_nsplit = 0;
  // fused step (bf16 Llama): the row-parallel projections do the all-reduce, the residual add and the
  // RMSNorm preparation in their epilogue, the other projections apply the norm's scale in theirs
  bool fused = false;
  float* xT = nullptr;          // residual stream [hidden][Bp] float32 (batch fastest)
  float* ssq = nullptr;         // [256][32] per-CTA sums of squares of the residual rows
  int embed_rows_per_cta = 32;
  float* capture = nullptr;     // [L][B][hidden] when enabled
  bool capture_on = false;
  // Tensor parallelism, fused step: every rank multiplies only its slice of the (replicated) head's rows and the ranks
  // exchange their (best logit, token id) pairs; the full logits are computed only when a caller asks for them
  bool head_sliced = false;
  int head_rg0 = 0, head_rows = 0;      // this rank's first 128-row group and its valid rows
  GemvPlan p_head_slice;
  float* logits_slice = nullptr;        // [B][head_pitch] float32
  int head_pitch = 0;
  cudaGraphExec_t graph_full = nullptr;   // head and logits
  cudaGraphExec_t graph_body = nullptr;   // no head
  cudaGraphExec_t graph_tok = nullptr;    // sliced head, tokens only (head_sliced)
  cudaStream_t graph_stream = nullptr;
  int graph_nodes_full = 0, graph_nodes_body = 0, graph_nodes_tok = 0;
  // a batch above 32: this session owns nothing on the device, it is a row of sub-sessions of at most 32 sequences
  std::vector<uint64_t> parts;
};

// the entry points of a session of more than 32 sequences (csrc/wide.cu): each runs the sub-sessions in turn
int32_t wide_create(Model* M, int batch, int max_ctx, lmb200_session* out);
int32_t wide_destroy(Session* S);
int32_t wide_reset(Session* S);
int32_t wide_position(Session* S, int32_t* pos);
int32_t wide_set_position(Session* S, int32_t pos);
int32_t wide_set_positions(Session* S, const int32_t* pos);
int32_t wide_positions(Session* S, int32_t* pos_out);
int32_t wide_fill_kv_random(Session* S, int32_t n_pos, uint64_t seed);
int32_t wide_set_capture(Session* S, int32_t enable);
int32_t wide_read_layer_output(Session* S, int32_t layer, float* host);
int32_t wide_prefill(Session* S, const int32_t* tokens, int32_t n, float* logits_out);
int32_t wide_prefill_ragged(Session* S, const int32_t* tokens, const int32_t* lengths, int32_t n_max, float* logits_out);
int32_t wide_decode_step(Session* S, const int32_t* tokens_in, int32_t* next_tokens_out, float* logits_out);
int32_t wide_decode_n(Session* S, const int32_t* first_tokens, int32_t n_steps, int32_t* tokens_out);
int32_t wide_decode_until(Session* S, const int32_t* first_tokens, int32_t max_steps, int32_t eot_token, int32_t* tokens_out,
                          int32_t* steps_done);
int32_t wide_step_bytes(Session* S, int32_t T, int64_t* bytes);

int32_t step_kernels_configure();
// prompt phase as GEMMs + flash attention (csrc/prefill.cu)
int32_t prefill_configure();
bool prefill_gemm_ok(const Session* S, int n);
// lens_dev: NULL (every sequence has n tokens) or device [B] prompt lengths <= n (the last-position rows are taken per sequence)
int32_t prefill_gemm(Session* S, const int* tokens_dev, int n, const int* lens_dev, cudaStream_t st);
int32_t prefill_linear(Ctx* ctx, const void* W, const float* x_dev, int T, int rows, int K, float* out_dev, cudaStream_t st);
Model* model_from(lmb200_model h);
Session* session_from(lmb200_session h);

}  // namespace lmb
