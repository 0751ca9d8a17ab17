/*
 * luminal_b200.h -- C ABI of libluminal_b200.so, the B200 (sm_100a) execution backend for the
 * compiled transformer decode path of Luminal.jl.
 *
 * The reference has no FFI; its extension seam is Julia multiple dispatch on the device type
 * (src/Device.jl:9-16, 82-121) and on the array type inside execute_op! (src/Execution.jl:521,
 * 566, 604).  A `B200Device <: AbstractDevice` shim binds the entry points below with `ccall`;
 * each declaration names the reference code it stands in for.
 *
 * Conventions
 *  - every function returns 0 on success, a negative LMB200_E* code otherwise, and never aborts,
 *    traps or blocks without bound; lmb200_last_error() gives the message (thread-local);
 *  - handles are opaque 64-bit integers; the caller owns host memory, the library owns device
 *    memory until the matching *_free / *_destroy;
 *  - "dptr" arguments are device addresses (from lmb200_alloc or any CUDA allocation on the
 *    context's device); every other pointer is host memory;
 *  - device tensors are row-major over the LOGICAL shape (last logical dim contiguous).  Julia
 *    arrays are column-major: pass LMB200_COLMAJOR to upload/download and the library re-lays
 *    them out, so parity is on logical indices, not on memory images;
 *  - one host thread per context, calls are synchronous with respect to their host results
 *    (like the reference: single task, src/Execution.jl:620-665);
 *  - token ids cross the ABI as int32 (the shim converts from the reference's Float32 ids,
 *    src/Execution.jl:263).
 */
#ifndef LUMINAL_B200_H
#define LUMINAL_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t lmb200_ctx;
typedef uint64_t lmb200_model;
typedef uint64_t lmb200_session;

enum { LMB200_F32 = 0, LMB200_BF16 = 1, LMB200_I32 = 2 };
enum { LMB200_ROWMAJOR = 0, LMB200_COLMAJOR = 1 };
enum {
  LMB200_OK = 0,
  LMB200_EINVAL = -1,    /* bad argument / shape mismatch (reference: error(...), @assert) */
  LMB200_ECUDA = -2,     /* a CUDA runtime call failed */
  LMB200_ENOMEM = -3,
  LMB200_ENCCL = -4,
  LMB200_ESTATE = -5,    /* call order (e.g. decode past max_ctx) */
  LMB200_ETIMEOUT = -6,  /* a bounded device-side wait gave up */
  LMB200_ENOMATCH = -8,  /* lmb200_match_decoder / lmb200_compile_node_list: the node list is not a decoder this
                            backend fuses; the message names the first node that does not fit.  Run it node by node. */
  LMB200_ENOTFOUND = -7  /* a tensor name the model does not have (the reference skips tensors that
                            are not registered, src/Weights.jl:76-91) */
};

/* element-wise opcodes of lmb200_ew: the reference's primitive and fused ops
 * (src/Ops.jl:4-22; executors src/Execution.jl:216-227, 274-285) */
enum {
  LMB200_OP_ADD = 0, LMB200_OP_MUL = 1, LMB200_OP_MOD = 2, LMB200_OP_LESSTHAN = 3,
  LMB200_OP_MAX = 4,
  LMB200_OP_LOG2 = 8, LMB200_OP_EXP2 = 9, LMB200_OP_SIN = 10, LMB200_OP_COS = 11,
  LMB200_OP_SQRT = 12, LMB200_OP_RECIP = 13, LMB200_OP_RELU = 14, LMB200_OP_COPY = 15,
  LMB200_OP_FUSED_MUL_ADD = 16,   /* a*b+c        src/Ops.jl:21, src/Execution.jl:220,278 */
  LMB200_OP_FUSED_ADD_RELU = 17   /* max(a+b,0)   src/Ops.jl:22, src/Execution.jl:221,279 */
};
enum { LMB200_REDUCE_SUM = 0, LMB200_REDUCE_MAX = 1 };

/* ---------------------------------------------------------------------------------------------
 * Library / context.  Replaces get_device()'s health check and the device structs
 * (src/Device.jl:9-74): one context per process per GPU.
 * ------------------------------------------------------------------------------------------ */
int32_t lmb200_version(void);
const char* lmb200_last_error(void);
int32_t lmb200_device_count(int32_t* count);
int32_t lmb200_init(int32_t device_ordinal, lmb200_ctx* ctx);
int32_t lmb200_shutdown(lmb200_ctx ctx);
/* run all later work of this context on an existing cudaStream_t (0 = the context's own) */
int32_t lmb200_set_stream(lmb200_ctx ctx, void* cuda_stream);
int32_t lmb200_sync(lmb200_ctx ctx);
/* number of kernels this context has launched so far (graph replays count their nodes) */
int32_t lmb200_launch_count(lmb200_ctx ctx, int64_t* count);
/* Recording a sequence of op-level calls into a CUDA graph and replaying it: what execute_with_capture is for
 * (src/Device.jl:106-121; the reference's CUDA method runs f() uncaptured, CompiledGraph keeps the `cache` it would
 * fill, src/Compiler.jl:75-100).  Between capture_begin and capture_end the primitive, fused and flash-attention entry
 * points on device tensors record their launches instead of running them (same pointers on every replay: the caller
 * keeps those buffers alive and unchanged in place); calls that copy to or from the host, allocate, free, wait, or
 * belong to a model or session are refused with an error and leave the device untouched.  capture_end returns the
 * instantiated graph, or an error if something recorded cannot be replayed; graph_launch enqueues one replay on the
 * context's stream. */
int32_t lmb200_capture_begin(lmb200_ctx ctx);
int32_t lmb200_capture_end(lmb200_ctx ctx, uint64_t* graph_out);
int32_t lmb200_graph_launch(lmb200_ctx ctx, uint64_t graph);
int32_t lmb200_graph_destroy(lmb200_ctx ctx, uint64_t graph);

/* Tensor-parallel communicator: one rank per process, NCCL over NVLink.  Not in the reference
 * (single device only, README.md:150-158); defined by the multi-GPU row of the hot-path scope.
 * Rank 0 creates the id, the launcher broadcasts the 128 bytes, every rank joins. */
int32_t lmb200_comm_unique_id(uint8_t id_out[128]);
int32_t lmb200_comm_init(lmb200_ctx ctx, int32_t n_ranks, int32_t rank, const uint8_t id[128]);
int32_t lmb200_comm_destroy(lmb200_ctx ctx);
/* Recovery after a tensor-parallel call returned LMB200_ETIMEOUT (a peer never signalled, or its
 * signal was invalid).  The ranks are then out of step, and prefill / decode calls of tensor-parallel
 * sessions return LMB200_ESTATE until every rank has called this, between steps, with nothing in
 * flight: the ranks agree on a common step number again (bounded wait for the peers) and the error
 * marks are cleared.  Session positions are not touched: put them back with
 * lmb200_session_set_position.  Not in the reference (single device). */
int32_t lmb200_comm_resync(lmb200_ctx ctx);
int32_t lmb200_allreduce_sum_f32(lmb200_ctx ctx, void* dptr, int64_t count);

/* ---------------------------------------------------------------------------------------------
 * Buffers.  Replace to_device / from_device (src/Device.jl:82-105) and the per-node buffers
 * that compile() allocates (src/Compiler.jl:217-235).
 * ------------------------------------------------------------------------------------------ */
int32_t lmb200_alloc(lmb200_ctx ctx, int64_t bytes, void** dptr_out);
int32_t lmb200_free(lmb200_ctx ctx, void* dptr);
/* host float32 array of logical shape dims[rank] in `layout` -> row-major device tensor of dtype */
int32_t lmb200_upload(lmb200_ctx ctx, void* dptr, int32_t dtype, const float* host,
                      int32_t rank, const int64_t* dims, int32_t layout);
int32_t lmb200_download(lmb200_ctx ctx, float* host, const void* dptr, int32_t dtype,
                        int32_t rank, const int64_t* dims, int32_t layout);

/* ---------------------------------------------------------------------------------------------
 * Primitive ops on float32 row-major device tensors: what execute_op! dispatches to per node.
 * ------------------------------------------------------------------------------------------ */
/* Element-wise with the reference's broadcasting (lower rank gets 1-dims PREPENDED,
 * src/Execution.jl:207-214).  Unused operands are NULL with rank 0.
 * Replaces src/Execution.jl:216-227 / 274-285. */
int32_t lmb200_ew(lmb200_ctx ctx, int32_t opcode, float* out_dptr, int32_t out_rank,
                  const int64_t* out_dims,
                  const float* a, int32_t a_rank, const int64_t* a_dims,
                  const float* b, int32_t b_rank, const int64_t* b_dims,
                  const float* c, int32_t c_rank, const int64_t* c_dims);
/* One element-wise fusion group (what compile() makes of an element-wise node and the single-consumer
 * element-wise nodes and constants feeding it): a postfix program over n_inputs float32 tensors,
 * each broadcast to the output by the rule above.  ops[i] / args[i]: 0 push input (args = its index),
 * 1 push constant (args = the value), 2 add, 3 mul, 4 mod, 5 less-than, 6 max, 7 log2, 8 exp2, 9 sin,
 * 10 cos, 11 sqrt, 12 recip, 13 relu, 14 a*b+c, 15 max(a+b, 0).  in_dims holds the inputs' dims one after
 * the other.  At most 8 inputs, 64 instructions, stack depth 16.  Every operation is rounded on its own,
 * so the result equals running the nodes one by one.
 * Replaces FusedElementwiseOp: src/Compiler.jl:196-215, 323-357, src/Execution.jl:552-563. */
int32_t lmb200_fused_ew(lmb200_ctx ctx, float* out_dptr, int32_t out_rank, const int64_t* out_dims,
                        int32_t n_inputs, const float* const* inputs, const int32_t* in_ranks,
                        const int64_t* in_dims, int32_t n_instr, const int32_t* ops, const float* args);
/* SumReduce / MaxReduce over one 0-based axis, axis dropped.  src/Execution.jl:232-233, 306-339 */
int32_t lmb200_reduce(lmb200_ctx ctx, int32_t kind, float* out_dptr, const float* in_dptr,
                      int32_t rank, const int64_t* dims, int32_t axis);
/* batch_matmul cases 2Dx2D, 3Dx2D, 3Dx3D, 4Dx4D.  src/Execution.jl:12-90 */
int32_t lmb200_matmul(lmb200_ctx ctx, float* out_dptr, const float* a, int32_t a_rank,
                      const int64_t* a_dims, const float* b, int32_t b_rank, const int64_t* b_dims);
/* Permute (0-based perm).  src/Execution.jl:229, 298-301 */
int32_t lmb200_permute(lmb200_ctx ctx, float* out_dptr, const float* in_dptr, int32_t rank,
                       const int64_t* in_dims, const int32_t* perm);
/* Reshape keeping the COLUMN-MAJOR linear order of the logical tensor.  src/Execution.jl:228 */
int32_t lmb200_reshape_colmajor(lmb200_ctx ctx, float* out_dptr, const float* in_dptr,
                                int32_t in_rank, const int64_t* in_dims,
                                int32_t out_rank, const int64_t* out_dims);
/* Expand: new axis of `size` inserted at 0-based `axis`.  src/Execution.jl:238-248, 345-371 */
int32_t lmb200_expand(lmb200_ctx ctx, float* out_dptr, const float* in_dptr, int32_t in_rank,
                      const int64_t* in_dims, int32_t axis, int64_t size);
/* Slice [start, stop) per axis (clamped).  src/Execution.jl:160-181 */
int32_t lmb200_slice(lmb200_ctx ctx, float* out_dptr, const float* in_dptr, int32_t rank,
                     const int64_t* in_dims, const int64_t* starts, const int64_t* stops);
/* Zero padding (left,right) per axis.  src/Execution.jl:183-202 */
int32_t lmb200_pad(lmb200_ctx ctx, float* out_dptr, const float* in_dptr, int32_t rank,
                   const int64_t* in_dims, const int64_t* left, const int64_t* right);
/* Gather rows of table[vocab,dim] by float ids (row Int(id), out-of-range -> 0).
 * src/Execution.jl:262-264, 580-611 */
int32_t lmb200_gather(lmb200_ctx ctx, float* out_dptr, const float* table, int64_t vocab,
                      int64_t dim, const float* ids, int64_t n_ids);
/* Unfold of the last axis (Conv1D's im2col): in [rows, length] -> out [rows, O, kernel] with
 * O = (length - dilation*(kernel-1) - 1) / stride + 1.  src/Execution.jl:481-550 */
int32_t lmb200_unfold1d(lmb200_ctx ctx, float* out_dptr, const float* in_dptr, int64_t rows,
                        int64_t length, int64_t kernel, int64_t stride, int64_t dilation);
/* CumSum along the last axis (used by arange).  src/Execution.jl:265-266, 612-613 */
int32_t lmb200_cumsum_last(lmb200_ctx ctx, float* out_dptr, const float* in_dptr,
                           int64_t rows, int64_t n);
/* FlashAttentionOp: softmax(scale*Q K^T [+causal]) V on [B,H,S,D]; dtype F32 or BF16 storage.
 * src/Ops.jl:104-107, src/Execution.jl:374-479, 565-578 */
int32_t lmb200_flash_attention(lmb200_ctx ctx, void* out_dptr, const void* q, const void* k,
                               const void* v, int32_t dtype, int64_t B, int64_t H, int64_t S,
                               int64_t D, float scale, int32_t causal);

/* ---------------------------------------------------------------------------------------------
 * Fused layer ops (what the compiled path's fusion groups become, src/Compiler.jl:196-215).
 * ------------------------------------------------------------------------------------------ */
/* y = (x * recip(sqrt(mean(x*x)+eps))) * w over the last dim.  src/NN.jl:134-173,
 * src/HighLevelOps.jl:299-304.  x,y: [rows,n] float32; w: [n] float32. */
int32_t lmb200_rmsnorm_scale(lmb200_ctx ctx, float* y, const float* x, const float* w,
                             int64_t rows, int64_t n, float eps);
/* LayerNorm with mean-centering, optional w / bias (NULL to skip).  src/NN.jl:121-173 */
int32_t lmb200_layernorm(lmb200_ctx ctx, float* y, const float* x, const float* w,
                         const float* bias, int64_t rows, int64_t n, float eps);
/* out = silu(gate) * up, silu via exp2 as in src/HighLevelOps.jl:153-160; src/NN.jl:246-249 */
int32_t lmb200_silu_gate(lmb200_ctx ctx, float* out, const float* gate, const float* up, int64_t n);
/* Half-split RoPE on [B,H,S,D] float32 at positions prev_seq..prev_seq+S-1.  src/NN.jl:253-303 */
int32_t lmb200_rope(lmb200_ctx ctx, float* out, const float* x, int64_t B, int64_t H, int64_t S,
                    int64_t D, int64_t prev_seq, float base);
/* One Linear on host data: out[b, o] = sum_i x[b, i] * W[o, i]; W [rows, K], x [batch <= 32, K],
 * out [batch, rows], all float32 row-major on the host.  dtype selects the float32 or the bf16
 * (float32-accumulate) decode GEMV; variant is reserved (pass 0: the tcgen05 / TMEM kernel).
 * The decode session runs the same kernels on resident weights; this entry uploads, runs once and
 * downloads (tests, comparisons).  Replaces NN.Linear for a single position, src/NN.jl:22-35. */
int32_t lmb200_linear_gemv(lmb200_ctx ctx, int32_t dtype, int32_t variant, int32_t rows, int32_t K,
                           int32_t batch, const float* w_host, const float* x_host, float* out_host);

/* ------------------------------------------------------------------------------------------
 * Whisper AudioEncoder + cross-K/V projection on the tensor cores (bf16 operands, float32
 * accumulation and residual stream).  Replaces running AudioEncoder (src/Whisper.jl:354-404; Conv1D
 * src/NN.jl:55-104; WhisperSelfAttention src/Whisper.jl:238-276) and project_cross_kv
 * (src/Whisper.jl:809-831) node by node.  Weights are set by the reference's registry names
 * (model.encoder.*, model.decoder.layers.{i}.encoder_attn.{k,v}_proj.*), full logical tensors.
 * ------------------------------------------------------------------------------------------ */
typedef uint64_t lmb200_whisper_encoder;
int32_t lmb200_whisper_encoder_create(lmb200_ctx ctx, int32_t d_model, int32_t heads, int32_t layers, int32_t ffn,
                                      int32_t n_mels, int32_t dec_layers, lmb200_whisper_encoder* out);
int32_t lmb200_whisper_encoder_destroy(lmb200_whisper_encoder enc);
int32_t lmb200_whisper_encoder_set_weight(lmb200_whisper_encoder enc, const char* name, const float* host, int32_t rank,
                                          const int64_t* dims, int32_t layout);
/* The reference registers its encoder blocks' tensors as model.encoder.layers.{i}.attn.*, .attn_layer_norm.*, .mlp.fc1.*,
 * .mlp.fc2.* (src/Whisper.jl:330-336); checkpoints and the reference's decoder blocks (src/Whisper.jl:424-431) spell them
 * .self_attn.*, .self_attn_layer_norm.*, .fc1.*, .fc2.*.  set_weight takes either; this writes the checkpoint's spelling
 * of `name` (any other name unchanged) into out.  No GPU is needed. */
int32_t lmb200_whisper_canonical_name(const char* name, char* out, int64_t capacity);
/* mel [batch, n_mels, frames] float32 row-major on the host; out_host NULL or [batch, (frames - 1) / 2 + 1, d_model].
 * The output also stays on the device for lmb200_whisper_encoder_cross_kv. */
int32_t lmb200_whisper_encoder_run(lmb200_whisper_encoder enc, const float* mel_host, int32_t batch, int32_t frames,
                                   float* out_host);
/* Cross K/V of every decoder layer from the last encoder output, written into the (bf16 Whisper) session's
 * cross cache: project_cross_kv + lmb200_session_set_cross_kv without the trip through the host. */
int32_t lmb200_whisper_encoder_cross_kv(lmb200_whisper_encoder enc, lmb200_session session);

/* out[t, o] = sum_i x[t, i] * w[o, i] for many rows t at once (the prompt phase) through the
 * tensor-core GEMM (bf16 operands, float32 accumulation): w [rows, K], x [n_tokens, K] and out
 * [n_tokens, rows] are float32 row-major host arrays; K must be a multiple of 8.  Replaces
 * NN.Linear -> batch_matmul on [B, S, in] (src/NN.jl:22-35, src/Execution.jl:12-54). */
int32_t lmb200_prefill_gemm(lmb200_ctx ctx, int32_t rows, int32_t K, int32_t n_tokens, const float* w_host,
                            const float* x_host, float* out_host);
/* argmax over the last dim (first maximum), 0-based ids.  src/Decoding.jl:119-124 */
int32_t lmb200_argmax(lmb200_ctx ctx, int32_t* out_ids_dptr, const float* x, int64_t rows, int64_t n);

/* ---------------------------------------------------------------------------------------------
 * Model / session API: the timed decode loop.  A model is the weights of a NN.Llama / NN.Phi3
 * shaped decoder (src/NN.jl:417-507); a session owns the preallocated GQA KV cache and the
 * CUDA graph of one decode step, and replaces the per-token graph build + execute of
 * examples/llama.jl:39-99 and src/Decoding.jl:91-130.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
  int32_t n_layers;
  int32_t hidden;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t head_dim;        /* must equal hidden / n_heads (src/NN.jl:331) */
  int32_t intermediate;
  int32_t vocab;
  float rms_eps;           /* 1e-5 in the reference (src/NN.jl:134) */
  float rope_base;         /* 500000 Llama (src/NN.jl:451), 10000 Phi-3 (src/NN.jl:503) */
  int32_t dtype;           /* LMB200_F32: everything float32; LMB200_BF16: weights, KV cache and
                              GEMV inputs bf16, accumulation and the residual stream float32 */
  int32_t tp_size;         /* tensor-parallel ranks (1 = single GPU) */
  int32_t tp_rank;
  int32_t arch;            /* LMB200_ARCH_LLAMA (NN.Llama / NN.Phi3) or LMB200_ARCH_WHISPER_DECODER
                              (TextDecoder with cached self attention and cross attention,
                              src/Whisper.jl:449-502, 584-742): LayerNorm, biases, GELU MLP, tied
                              embedding head, learned positions, no RoPE, n_kv_heads == n_heads,
                              tp_size 1 */
  int32_t max_positions;   /* Whisper: rows of embed_positions (448, src/Whisper.jl:206) */
  int32_t cross_len;       /* Whisper: encoder positions the cross attention reads (1500) */
  int32_t reserved;
} lmb200_model_config;
enum { LMB200_ARCH_LLAMA = 0, LMB200_ARCH_WHISPER_DECODER = 1 };

int32_t lmb200_model_create(lmb200_ctx ctx, const lmb200_model_config* cfg, lmb200_model* model);
/* Host-only view of the weight re-layout and tensor-parallel sharding (no GPU needed): the extent
 * of this rank's fused matrix `matrix` (0 qkv, 1 o_proj, 2 gate/up, 3 down_proj, 4 lm_head) and, for
 * one of its elements, which logical tensor (slot: q/k/v = 0/1/2, gate/up = 0/1, else 0) and which
 * [out, in] element of it sits there (-1 for padding).  Encodes src/NN.jl:305-317, 347-354
 * (q = kv + KV*g, feature f = h + H*d) and the RoPE pairing of src/NN.jl:274-276. */
int32_t lmb200_shard_extent(const lmb200_model_config* cfg, int32_t matrix, int32_t* rows, int32_t* cols);
int32_t lmb200_shard_map(const lmb200_model_config* cfg, int32_t matrix, int32_t row, int32_t col,
                         int32_t* slot, int32_t* logical_row, int32_t* logical_col);
int32_t lmb200_model_destroy(lmb200_model model);
/* Set one weight from the FULL logical float32 tensor under its registry name
 * ("model.layers.3.self_attn.q_proj.weight", "model.embed_tokens.weight", "model.norm.weight",
 * "lm_head.weight" ...: src/NN.jl:180-225, 433-445).  dims[rank] is the shape of `host` (rank 1 or
 * 2); it must equal the logical shape the configuration gives that tensor ([out, in] for a
 * Linear, [n] for gains and biases), else LMB200_EINVAL names both shapes and nothing is read.
 * A name the model does not have returns LMB200_ENOTFOUND.  The library keeps only this rank's
 * shard, in its own tiled layout.  Replaces graph.tensors / load_weights! (src/Weights.jl:60-114). */
int32_t lmb200_model_set_weight(lmb200_model model, const char* name, const float* host,
                                int32_t rank, const int64_t* dims, int32_t layout);
/* Which of the model's tensors have not been set yet: their count, and their names separated by
 * '\n' into names_out (as many as fit in `capacity` bytes, NUL-terminated; names_out may be NULL
 * with capacity 0).  Stands in for the warning load_weights! prints for missing keys
 * (src/Weights.jl:86-91). */
int32_t lmb200_model_missing_weights(lmb200_model model, char* names_out, int64_t capacity,
                                     int32_t* n_missing);
/* Fill every weight on the device from the counter-based generator (seed, tensor id, logical
 * row-major index) -> Irwin-Hall(12) approximation of N(0,sigma); norm gains get +1. */
int32_t lmb200_model_init_random(lmb200_model model, uint64_t seed, float sigma);
int32_t lmb200_model_weight_bytes(lmb200_model model, int64_t* bytes);

/* A session: `batch` sequences with a preallocated cache of max_ctx positions each (the cache the reference lacks for
 * Llama, examples/llama.jl:39-99, and keeps per graph for Whisper, src/Whisper.jl:519-541).  The model's forward takes
 * any batch (src/NN.jl:448-455): up to 32 sequences share one pass over the weights; a larger batch (Llama / Phi-3, one
 * GPU) runs as sub-sessions of at most 32 sequences, one weight pass each, behind the same handle and entry points.
 * Not offered above 32: lmb200_session_kv_layer, lmb200_decode_attention_splitkv, lmb200_decode_n_device. */
int32_t lmb200_session_create(lmb200_model model, int32_t batch, int32_t max_ctx,
                              lmb200_session* session);
int32_t lmb200_session_destroy(lmb200_session session);
int32_t lmb200_session_reset(lmb200_session session);
int32_t lmb200_session_position(lmb200_session session, int32_t* pos);
/* Rewind (or move) the position of every sequence; cache contents at and beyond it are overwritten by
 * later steps.  lmb200_session_position reports the furthest position of any sequence. */
int32_t lmb200_session_set_position(lmb200_session session, int32_t pos);
/* One position per sequence (pos[batch] / pos_out[batch]).  The reference's [batch, seq] token tensor
 * gives every sequence the same length (src/NN.jl:448-455); a batch of real prompts has one length
 * each, so the session keeps a position per sequence: RoPE angle, cache slot and attention length
 * follow it. */
int32_t lmb200_session_set_positions(lmb200_session session, const int32_t* pos);
int32_t lmb200_session_positions(lmb200_session session, int32_t* pos_out);
/* Synthetic context: fill cache positions [0,n_pos) with generator values (sigma 1 for K and V)
 * and set the position to n_pos. */
int32_t lmb200_session_fill_kv_random(lmb200_session session, int32_t n_pos, uint64_t seed);
/* Keep the residual stream after every layer of the next steps (parity tests). */
int32_t lmb200_session_set_capture(lmb200_session session, int32_t enable);
int32_t lmb200_session_read_layer_output(lmb200_session session, int32_t layer, float* host);

/* Whisper: the cross-attention keys and values of one decoder layer, as project_cross_kv computes
 * them (src/Whisper.jl:809-831; K already scaled by head_dim^-0.25): float32 [batch, heads,
 * cross_len, head_dim] in `layout`.  Stands in for the cross_kv_arrays that decode_step! feeds as
 * inputs at every step (src/Whisper.jl:770-778): here they are uploaded once. */
int32_t lmb200_session_set_cross_kv(lmb200_session session, int32_t layer, const float* k_host,
                                    const float* v_host, int32_t layout);

/* Prompt: tokens [batch, n] int32 row-major, appended at the current position.  logits_out
 * (NULL or [batch, vocab] float32) receives the LAST position's logits.
 * Replaces running the model over the prompt (src/NN.jl:448-455). */
int32_t lmb200_prefill(lmb200_session session, const int32_t* tokens, int32_t n, float* logits_out);
/* Prompts of different lengths in one batch: tokens [batch, n_max] int32 row-major, sequence b uses its
 * first lengths[b] ids (1 <= lengths[b] <= n_max), appended at that sequence's position.  logits_out
 * (NULL or [batch, vocab]) receives, per sequence, the logits of ITS last prompt position; afterwards the
 * sequences stand at different positions and lmb200_decode_step / _n / _until go on from there.
 * Replaces running the model over a batch of prompts (src/NN.jl:448-455), which the reference can only
 * do for equal lengths. */
int32_t lmb200_prefill_ragged(lmb200_session session, const int32_t* tokens, const int32_t* lengths,
                              int32_t n_max, float* logits_out);
/* One token per sequence in, greedy next token out; host buffers, copies inside the call.
 * Replaces one iteration of the generation loop (src/Decoding.jl:91-130, examples/llama.jl:73-99). */
int32_t lmb200_decode_step(lmb200_session session, const int32_t* tokens_in,
                           int32_t* next_tokens_out, float* logits_out);
/* n_steps greedy steps by CUDA-graph replay with the tokens staying on the device.
 * first_tokens [batch] host (NULL = continue from the last produced tokens);
 * tokens_out [n_steps, batch] host (NULL to skip the copy back). */
int32_t lmb200_decode_n(lmb200_session session, const int32_t* first_tokens, int32_t n_steps,
                        int32_t* tokens_out);
/* The generation loop with the reference's two exits (src/Decoding.jl:91-130): greedy steps until
 * every sequence has produced eot_token (:126-129) or max_steps, capped by the positions left in the
 * session, have run (:93-95).  A sequence that is done keeps emitting eot_token while the others go
 * on.  first_tokens [batch] host (NULL = continue); tokens_out [max_steps, batch] host receives
 * *steps_done rows, the last of which is the step in which the last sequence finished. */
int32_t lmb200_decode_until(lmb200_session session, const int32_t* first_tokens, int32_t max_steps,
                            int32_t eot_token, int32_t* tokens_out, int32_t* steps_done);
/* Same loop, asynchronous on the context's stream: tokens come from and go to device memory
 * ([batch] int32 in, [n_steps,batch] int32 out, either may be NULL), no host synchronisation. */
int32_t lmb200_decode_n_device(lmb200_session session, const int32_t* first_tokens_dptr,
                               int32_t n_steps, int32_t* tokens_out_dptr);
/* Algorithmic HBM bytes of ONE decode step on this rank at context length T (weights read once
 * + KV cache read for T keys + KV written for one key; of the replicated head only the rows this
 * rank multiplies in a token-only step under tensor parallelism). */
int32_t lmb200_session_step_bytes(lmb200_session session, int32_t T, int64_t* bytes);

/* ---------------------------------------------------------------------------------------------
 * A graph as a backend sees it: Graph.nodes (src/Graph.jl:4-26) flattened into arrays, node n (1-based, in
 * insertion = topological order) described by op[n-1], its inputs in_node[in_off[n-1] .. in_off[n]) (1-based
 * ids of earlier nodes), its output shape shape[shape_off[n-1] .. shape_off[n]) and its op fields as doubles
 * arg[arg_off[n-1] .. arg_off[n]):
 *   SumReduce / MaxReduce: dim;  Permute: dims...;  Expand: dim, size;  Reshape: shape...;
 *   Slice: (start, stop) per dim, 0-based half-open, an open end as any value >= 2^62;  Pad: (left, right) per dim;
 *   Unfold: kernel..., stride..., dilation...;  Constant: value;  FlashAttentionOp: scale, causal;  others: none.
 * Function("InputTensor" / "Gather" / "CumSum") are LMB200_NODE_INPUT / _GATHER / _CUMSUM (src/Ops.jl:4-110).
 * ------------------------------------------------------------------------------------------ */
enum {
  LMB200_NODE_LOG2 = 0, LMB200_NODE_EXP2 = 1, LMB200_NODE_SIN = 2, LMB200_NODE_SQRT = 3, LMB200_NODE_COS = 4,
  LMB200_NODE_RECIP = 5, LMB200_NODE_CONTIGUOUS = 6, LMB200_NODE_RELU = 7, LMB200_NODE_ADD = 8, LMB200_NODE_MUL = 9,
  LMB200_NODE_MOD = 10, LMB200_NODE_MAX = 11, LMB200_NODE_LESSTHAN = 12, LMB200_NODE_FUSED_MUL_ADD = 13,
  LMB200_NODE_FUSED_ADD_RELU = 14, LMB200_NODE_MATMUL = 15, LMB200_NODE_SUM_REDUCE = 16, LMB200_NODE_MAX_REDUCE = 17,
  LMB200_NODE_PERMUTE = 18, LMB200_NODE_EXPAND = 19, LMB200_NODE_RESHAPE = 20, LMB200_NODE_SLICE = 21,
  LMB200_NODE_PAD = 22, LMB200_NODE_UNFOLD = 23, LMB200_NODE_CONSTANT = 24, LMB200_NODE_INPUT = 25,
  LMB200_NODE_GATHER = 26, LMB200_NODE_CUMSUM = 27, LMB200_NODE_FLASH_ATTENTION = 28, LMB200_NODE_OTHER = 29
};
typedef struct {
  int32_t n_nodes;
  int32_t reserved;
  const int32_t* op;        /* [n_nodes] LMB200_NODE_* */
  const int32_t* in_off;    /* [n_nodes + 1] */
  const int32_t* in_node;
  const int32_t* shape_off; /* [n_nodes + 1] */
  const int64_t* shape;
  const int32_t* arg_off;   /* [n_nodes + 1] */
  const double* arg;
} lmb200_node_list;
typedef struct {
  int32_t arch;         /* LMB200_ARCH_LLAMA or LMB200_ARCH_WHISPER_DECODER: which builder's graph was recognised */
  int32_t batch;        /* the shape the graph was traced for: tokens [batch, seq] */
  int32_t seq;
  int32_t prev_seq;     /* Llama: the position offset baked into the RoPE angles (src/NN.jl:253-262); Whisper: the
                           step_pos baked into the slice positions (src/Whisper.jl:687-742) */
  int32_t tokens_node;  /* the input node the token ids enter through */
  int32_t n_weights;    /* Llama: 3 + 9 * n_layers; Whisper: 4 + 21 * n_layers */
  int32_t max_seq;      /* Whisper: positions of the past self K/V inputs */
  int32_t cross_len;    /* Whisper: positions of the encoder K/V inputs */
} lmb200_decoder_match;
/* Recognises NN.Llama / NN.Phi3 (src/NN.jl:390-507) ending in the logits node output_id:
 * lm_head(norm(block^L(embedding(tokens)))), every layer decomposed into primitives as src/NN.jl and
 * src/HighLevelOps.jl build them.  No GPU is needed.  On success cfg holds the widths, head split, epsilon and
 * RoPE base (dtype float32, tp_size 1), weight_nodes[k] (as many as fit in weight_capacity) the input node that
 * plays the role of the k-th registry name of names_out ('\n'-separated, src/NN.jl:180-225, 433-445).  A graph
 * that deviates anywhere returns LMB200_ENOMATCH and lmb200_last_error names the node and what was expected
 * there; the reference has no such step: its compile() (src/Compiler.jl:181-364) runs whatever nodes it is given. */
int32_t lmb200_match_decoder(const lmb200_node_list* list, int32_t output_id, lmb200_model_config* cfg,
                             lmb200_decoder_match* info, int32_t* weight_nodes, int32_t weight_capacity,
                             char* names_out, int64_t names_capacity);
/* The same for the Whisper TextDecoder's incremental decode step (build_decode_step!, src/Whisper.jl:687-742: cached
 * self attention with the slice-and-concat cache write of src/Whisper.jl:541-570, cross attention over encoder K/V
 * inputs, GELU MLP, LayerNorm, tied-embedding head), ending in its logits node.  cfg comes back with
 * LMB200_ARCH_WHISPER_DECODER; weight_nodes / names_out list the model.decoder.* tensors the session needs; cache_nodes
 * (as many as fit) holds, n_layers of each in this order: the encoder K inputs, encoder V inputs, past self K inputs,
 * past self V inputs, and the nodes of the updated self K and V (IncrementalDecodeGraph, src/Whisper.jl:662-672). */
int32_t lmb200_match_whisper_step(const lmb200_node_list* list, int32_t logits_id, lmb200_model_config* cfg,
                                  lmb200_decoder_match* info, int32_t* weight_nodes, int32_t weight_capacity,
                                  char* names_out, int64_t names_capacity, int32_t* cache_nodes,
                                  int32_t cache_capacity);
/* compile() for a graph one of the two matchers recognises (replaces src/Compiler.jl:181-364 + the per-token
 * re-execution of examples/llama.jl:39-99, or the per-position graph build + compile of src/Whisper.jl:679-801):
 * matches, creates the model in `dtype`, sets every weight from node_data[node - 1] (host float32 in `layout`, shape =
 * that node's; entries of other nodes may be NULL: graph.tensors filled by load_weights!, src/Weights.jl:60-114) and
 * creates a session of `batch` sequences (0 = the graph's) with room for max_ctx positions (Whisper: 0 = the graph's
 * max_seq).  The caller owns both handles.  The session starts at position 0: a Llama graph traced with prev_seq != 0
 * is refused (LMB200_ENOMATCH); a Whisper step graph of any step_pos gives the same session, and encoder K/V inputs that
 * have data are uploaded as lmb200_session_set_cross_kv does. */
int32_t lmb200_compile_node_list(lmb200_ctx ctx, const lmb200_node_list* list, int32_t output_id,
                                 const float* const* node_data, int32_t layout, int32_t dtype, int32_t batch,
                                 int32_t max_ctx, lmb200_model* model_out, lmb200_session* session_out,
                                 lmb200_decoder_match* info);

/* The Whisper AudioEncoder's graph (src/Whisper.jl:354-404: the Conv1D stem of src/NN.jl:55-104 with GELU, the
 * sinusoid table of src/Whisper.jl:208-231, pre-norm blocks of unmasked self attention and a GELU MLP, a final
 * LayerNorm), ending in its output node. */
typedef struct {
  int32_t d_model, heads, layers, ffn, n_mels;
  int32_t batch, frames;   /* the mel input the graph was traced for: [batch, n_mels, frames] */
  int32_t mel_node;        /* the input node the mel enters through */
  int32_t rates_node;      /* the input node holding the sinusoid rates exp(-log(10000) / (d_model/2 - 1) * i) */
  int32_t n_weights;       /* 6 + 15 * layers */
  float eps;               /* LayerNorm epsilon */
} lmb200_encoder_match;
/* Recognises that graph.  No GPU is needed.  weight_nodes / names_out as for lmb200_match_decoder, with the
 * model.encoder.* registry names; a graph that deviates anywhere returns LMB200_ENOMATCH naming the node. */
int32_t lmb200_match_whisper_encoder(const lmb200_node_list* list, int32_t output_id, lmb200_encoder_match* info,
                                     int32_t* weight_nodes, int32_t weight_capacity, char* names_out,
                                     int64_t names_capacity);
/* compile() for it: matches, creates the tensor-core encoder (lmb200_whisper_encoder_create with no decoder layers) and
 * sets every weight from node_data[node - 1] (host float32 in `layout`).  The sinusoid rates the graph holds must be
 * sinusoids()'s and the epsilon 1e-5, which the fused encoder has built in; lmb200_whisper_encoder_run then takes a mel
 * of any batch and length.  Replaces running the ~280 nodes of that graph one kernel each (src/Compiler.jl:181-364). */
int32_t lmb200_compile_encoder_node_list(lmb200_ctx ctx, const lmb200_node_list* list, int32_t output_id,
                                         const float* const* node_data, int32_t layout,
                                         lmb200_whisper_encoder* encoder_out, lmb200_encoder_match* info);

/* Stand-alone split-KV decode attention over a cache in the session layout (tests, profiling),
 * asynchronous on the context's stream (lmb200_sync before reading the result).
 * q: [batch, n_heads_local, head_dim] in the session dtype (device); out: same shape.
 * Local q head (kv_local*G + g) is the reference's head kv + KV*g.
 * Replaces whisper_self_attn_cached's attention over [0, step_pos] (src/Whisper.jl:606-617)
 * and the S=1 case of SelfAttention (src/NN.jl:369-386). */
int32_t lmb200_decode_attention_splitkv(lmb200_session session, int32_t layer, const void* q_dptr,
                                        void* out_dptr, int32_t T);

/* Address and strides (in elements) of one layer of the session's tiled KV cache, for callers that
 * run the attention kernels on it themselves.  The cache belongs to the session. */
int32_t lmb200_session_kv_layer(lmb200_session session, int32_t layer, void** kv_dptr,
                                int64_t* batch_stride, int64_t* head_stride);

/* Split-KV decode attention that allocates nothing.  It has no counterpart in the reference.
 * Some callers cannot call cudaMalloc: a host runtime that already owns all device memory in a
 * pool of its own (CUDA.jl, a serving arena), or a loop that cannot take the synchronisation an
 * allocation may cause.  The kernel's per-split partial results therefore go to an 8 MiB array
 * built into the library (one per GPU that loads it, kept until exit) instead of session scratch.
 *  - q, out: [batch, n_kv_heads*group, head_dim] device tensors of `dtype`, heads ordered
 *    (kv head, group member); kv_layer: a tiled cache layer as lmb200_session_kv_layer returns.
 *  - T must not exceed the capacity of the layer that the strides describe: the kernels read
 *    ceil(T / 16) blocks of 32 * head_dim elements per (sequence, kv head).  Strides too small
 *    for T (kv_head_stride < ceil(T / 16) * 32 * head_dim, or kv_batch_stride < n_kv_heads *
 *    kv_head_stride) are rejected with LMB200_EINVAL; on the bf16 path group must be <= 8.
 *  - Shapes whose partial results exceed the array (more than 2 Mi floats: roughly
 *    batch * n_kv_heads * group * splits * (head_dim + 2)) are rejected with LMB200_EINVAL.
 *  - The first call on a device looks up the array's device address; make that call outside any
 *    stream capture.  Asynchronous on the context's stream like lmb200_decode_attention_splitkv.
 *  - All calls share the array: calls whose kernels overlap on the GPU race.  Nothing in it
 *    needs clearing between calls. */
int32_t lmb200_decode_attention_noalloc(lmb200_ctx ctx, int32_t dtype, const void* q_dptr,
                                        void* out_dptr, const void* kv_layer_dptr,
                                        int64_t kv_batch_stride, int64_t kv_head_stride,
                                        int32_t batch, int32_t n_kv_heads, int32_t group,
                                        int32_t head_dim, int32_t T);

#ifdef __cplusplus
}
#endif
#endif /* LUMINAL_B200_H */
