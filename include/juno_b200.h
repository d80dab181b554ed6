/*
 * juno_b200.h — C ABI of the B200 (sm_100a) decode engine for Juno.
 *
 * This is the surface a Java host binds with java.lang.foreign
 * (Linker.nativeLinker().downcallHandle) in place of the cudart/cuBLAS symbol
 * table of node/src/main/java/cab/ml/juno/node/CudaBindings.java:139-211.
 * Conventions follow that file: every function returns an int status (0 = OK,
 * CudaBindings.java:247-250 turns non-zero into IllegalStateException), handles
 * are opaque pointers returned through out-parameters (CudaBindings.java:222-231),
 * and all host buffers are plain native memory (Panama rejects heap segments,
 * CudaMatVec.java:158-160).  No C++ types, callbacks or varargs cross the boundary.
 *
 * Threading: every entry point may be called from any thread; the library
 * selects the device itself and serialises work per context (the reference
 * holds one lock per device, GpuContext.java:99-101).
 */
#ifndef JUNO_B200_H
#define JUNO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define JUNO_OK 0
#define JUNO_ERR_INVALID_ARG (-1)
#define JUNO_ERR_OOM (-2)      /* cudaMalloc failed (the reference string-matches "cudaMalloc",
                                  LlamaTransformerHandler.java:350-352); there is no CPU fallback */
#define JUNO_ERR_CUDA (-3)
#define JUNO_ERR_NCCL (-4)     /* NCCL call failed, or the communicator was aborted after a step that timed out */
#define JUNO_ERR_TIMEOUT (-5)  /* a bounded wait ran out: a weight tile never arrived, or a tensor-parallel rank did not
                                  deliver (about a second for the peer exchange, JUNO_NCCL_TIMEOUT_S for NCCL steps);
                                  the context stays usable */
#define JUNO_ERR_CLOSED (-6)   /* handle already freed (IllegalStateException in MatVec.java:46-54) */
#define JUNO_ERR_UNSUPPORTED (-7)

/* GGML tensor type ids accepted (GgufReader.java:54-63) */
#define JUNO_TYPE_F32 0
#define JUNO_TYPE_Q8_0 8
#define JUNO_TYPE_Q4_K 12
#define JUNO_TYPE_Q6_K 14

typedef struct juno_ctx juno_ctx;
typedef struct juno_qmat juno_qmat;
typedef struct juno_model juno_model;
typedef struct juno_seq juno_seq;
typedef struct juno_kvpool juno_kvpool;
typedef struct juno_gguf juno_gguf;

/* Thread-local text of the last failure on the calling thread. */
const char *juno_last_error(void);

/* ── device discovery: replaces cudaGetDeviceCount / cudaGetDeviceProperties and
 *    the fixed-offset pokes into cudaDeviceProp (CudaBindings.java:75-79,107-118).
 *    Fails soft: with no driver or no device, count is 0 and the status is JUNO_OK. */
int juno_device_count(int32_t *count);
int juno_device_name(int32_t device, char *buf, int32_t buf_len);
int juno_device_total_mem(int32_t device, int64_t *bytes);

/* ── context: replaces GpuContext.shared/close (GpuContext.java:109-153,229-243). */
int juno_ctx_create(int32_t device, juno_ctx **out);
int juno_ctx_destroy(juno_ctx *ctx); /* idempotent on a closed handle: returns JUNO_ERR_CLOSED */
int juno_ctx_device(juno_ctx *ctx, int32_t *device);
int juno_ctx_synchronize(juno_ctx *ctx);
/* The cudaStream_t all work of this context is enqueued on (replaces the per-thread stream of
 * CudaMatVec.java:73-82); a host may record its own events on it. */
int juno_ctx_stream(juno_ctx *ctx, void **stream);

/* ── MatVec operator (boundary A) ─────────────────────────────────────────────
 * juno_qmat_upload replaces GpuMatVec.uploadHalf(float[],rows,cols)
 * (GpuMatVec.java:38-70, DeviceHalfMatrix.java:66-91): it keeps the QUANTISED
 * GGUF blocks resident (repacked into the kernels' tile order) instead of a
 * dequantised FP16 copy.  `blocks` is the row-major raw tensor as
 * GgufReader.tensorRaw returns it (GgufReader.java:329-360).  The caller keeps
 * ownership of `blocks`. */
int juno_qmat_upload(juno_ctx *ctx, const void *blocks, int32_t ggml_type, int64_t rows, int64_t cols,
                     juno_qmat **out);
int juno_qmat_free(juno_qmat *m);
int juno_qmat_shape(juno_qmat *m, int64_t *rows, int64_t *cols, int32_t *ggml_type);

/* y[b][rows] = A · x[b][cols], b < batch; host in, host out.  Semantics of
 * MatVec.sgemv(DeviceHalfMatrix, float[]) (MatVec.java:86-90, CudaMatVec.java:276-333)
 * on the quantised weights of LlamaTransformerHandler.matVec (:1200-1245):
 * inputs are not modified, JUNO_ERR_INVALID_ARG on a dimension mismatch,
 * JUNO_ERR_CLOSED on a freed matrix. */
int juno_gemv(juno_ctx *ctx, juno_qmat *m, const float *x_host, int32_t batch, float *y_host);

/* Same product with x and y already in device memory, enqueued on `stream`
 * (a cudaStream_t, NULL = the context's stream) and not synchronised. */
int juno_gemv_device(juno_ctx *ctx, juno_qmat *m, const float *x_dev, int32_t batch, float *y_dev,
                     void *stream);

/* Bit-exact dequantisation of rows [row_start, row_start+n_rows) to host FP32:
 * LlamaTransformerHandler.dequantize (:873-885).  Used for parity checks and for
 * embedding rows. */
int juno_dequantize(juno_ctx *ctx, juno_qmat *m, int64_t row_start, int64_t n_rows, float *out_host);

/* FP32 host-matrix product: MatVec.sgemv(float[] A, float[] x, rows, cols)
 * (MatVec.java:66, CudaMatVec.java:141-196). */
int juno_sgemv_f32(juno_ctx *ctx, const float *a_host, const float *x_host, int64_t rows, int64_t cols,
                   float *y_host);

/* ── paged KV cache + GQA decode attention operator ───────────────────────────
 * Replaces the per-request float[L][pos*kvDim] heap cache and the scalar gqa()
 * of LlamaTransformerHandler.java:670-733,1678-1730.  A pool holds `n_pages`
 * pages of `page_tokens` (16) positions for every layer; kv_dtype 0 = FP16,
 * 1 = FP32 (the reference's storage type). */
int juno_kvpool_create(juno_ctx *ctx, int32_t n_layers, int32_t n_kv_heads, int32_t head_dim,
                       int32_t n_pages, int32_t kv_dtype, juno_kvpool **out);
int juno_kvpool_free(juno_kvpool *p);
/* A sequence handle stands for one requestId (ForwardRequest.java:26-48);
 * freeing it is evict(requestId) (LlamaTransformerHandler.java:498-505). */
int juno_kvseq_create(juno_kvpool *p, int32_t max_tokens, juno_seq **out);
int juno_seq_free(juno_seq *s);
int juno_seq_length(juno_seq *s, int32_t *n_tokens);
/* Prefix sharing between requests (a kvcache/PrefixCache hit, PrefixCache.java, whose key belongs to another live
 * request): a new sequence that already holds the first n_tokens cached positions of src (n_tokens <= its length).
 * No data moves: the pages of the prefix are shared and counted per holder; before either sequence writes into a
 * shared page (its next position, or a rewrite of older ones) it gets a private copy of that page.  juno_seq_free of
 * one holder leaves the shared pages to the others. */
int juno_seq_fork(juno_seq *src, int32_t n_tokens, juno_seq **out);
/* Append n_tokens positions of K and V ([n_tokens][n_kv_heads*head_dim] FP32, host)
 * for one layer at positions [pos, pos+n_tokens); values are rounded to the pool dtype. */
int juno_seq_append_kv(juno_seq *s, int32_t layer, int32_t pos, int32_t n_tokens, const float *k_host,
                       const float *v_host);
/* out[i][n_heads*head_dim] = gqa(q[i], K_i, V_i, len_i) for n sequences at one layer
 * (len_i = current length of seqs[i]); host in, host out. */
int juno_attn_decode(juno_ctx *ctx, juno_kvpool *p, int32_t layer, int32_t n, juno_seq *const *seqs,
                     int32_t n_heads, const float *q_host, float *out_host);

/* The same attention for callers that must not allocate.  juno_attn_decode grows device staging buffers with
 * cudaMalloc when a call is larger than any before it; a host that has handed all of the GPU's memory to its KV pool
 * and weights (or that runs under a fixed reservation where a late cudaMalloc fails, or stalls the device with its
 * implicit synchronisation) cannot afford that.  This variant takes q and out as DEVICE pointers
 * ([n][n_heads*head_dim] FP32 each, caller-owned) and keeps its only working memory - per-split partial results and
 * 2n words of sequence metadata - in an 8 MiB array that is part of the library image (each GPU that loads the
 * library holds it until the process exits).  It calls no cudaMalloc/cudaFree and no allocating library routine.
 * Limits: n <= 256 and n * n_heads * (head_dim + 2) * 4 bytes must fit the array at least once (about 8 MiB minus
 * 2 KiB); larger calls fail with JUNO_ERR_INVALID_ARG and a message that names both numbers.  Fewer context splits
 * are used when the array is the constraint.  The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture.  All calls share the array: it keeps
 * the previous call's contents (every entry a call reads is rewritten by that call first), and two calls that
 * overlap on the GPU race - this function holds one lock per device (so two contexts of a GPU are serialised as
 * well) and returns after the stream has drained.
 * No counterpart in the reference. */
int juno_attn_decode_static(juno_ctx *ctx, juno_kvpool *p, int32_t layer, int32_t n, juno_seq *const *seqs,
                            int32_t n_heads, const float *q_dev, float *out_dev);

/* ── forward-pass operator (boundaries B and C) ───────────────────────────────
 * juno_model_* replaces the device half of LlamaTransformerHandler
 * (ForwardPassHandler.java:33-70); juno_forward with n sequences is
 * InferencePipeline.forwardBatch (InferencePipeline.java:62-69). */
typedef struct juno_model_cfg {
    int32_t struct_size;   /* sizeof(juno_model_cfg), for forward compatibility */
    int32_t hidden;        /* <arch>.embedding_length   (LlamaConfig.java:58-91) */
    int32_t n_layers;      /* <arch>.block_count */
    int32_t n_heads;       /* <arch>.attention.head_count */
    int32_t n_kv_heads;    /* <arch>.attention.head_count_kv */
    int32_t inter;         /* <arch>.feed_forward_length */
    int32_t vocab;
    float rms_eps;
    float rope_theta;
    int32_t max_batch;     /* most sequences per juno_forward call */
    int32_t max_seqs;      /* most live sequences */
    int32_t max_ctx;       /* most positions per sequence (the reference caps at 2048) */
    int32_t kv_dtype;      /* 0 = FP16 pages, 1 = FP32 pages */
    int32_t tp_rank;       /* TensorShardContext.tensorRank  (TensorShardContext.java:41-100) */
    int32_t tp_world;      /* TensorShardContext.tensorWorldSize; 1 = single GPU */
    uint8_t nccl_id[128];  /* ncclUniqueId bytes shared by all ranks when tp_world > 1 */
} juno_model_cfg;

/* tensor kinds, named after the GGUF tensors of LlamaTransformerHandler.java:238-275 */
#define JUNO_T_TOKEN_EMBD 0
#define JUNO_T_OUTPUT_NORM 1
#define JUNO_T_OUTPUT 2
#define JUNO_T_ATTN_NORM 3
#define JUNO_T_FFN_NORM 4
#define JUNO_T_ATTN_Q 5
#define JUNO_T_ATTN_K 6
#define JUNO_T_ATTN_V 7
#define JUNO_T_ATTN_OUT 8
#define JUNO_T_FFN_GATE 9
#define JUNO_T_FFN_UP 10
#define JUNO_T_FFN_DOWN 11
#define JUNO_T_ATTN_Q_BIAS 12 /* optional attn_{q,k,v}.bias (F32 vectors; LlamaTransformerHandler.java:258-262, added to */
#define JUNO_T_ATTN_K_BIAS 13 /* q, k, v before the rotation, :758-762); all three for every layer, or none */
#define JUNO_T_ATTN_V_BIAS 14

/* ── GGUF model files (host only, no GPU needed) ───────────────────────────────
 * Replaces node/GgufReader.java for the tensors and metadata the decode path reads: open (:102-180) parses header
 * (magic "GGUF", version 2 or 3), metadata (value types 0-12, :1189-1244) and the tensor table, and places the data
 * section at the next multiple of 32 after it (:169-176).  The file is mapped read-only; tensors are pointers into
 * the mapping (tensorRaw :329-340 copies them to the heap instead) and stay valid until juno_gguf_close.  A damaged
 * or foreign file gives JUNO_ERR_INVALID_ARG (the reference throws IOException), a version other than 2 or 3
 * JUNO_ERR_UNSUPPORTED.  GGUF inside a llamafile ZIP is not supported. */
int juno_gguf_open(const char *path, juno_gguf **out);
int juno_gguf_close(juno_gguf *g);
int juno_gguf_info(juno_gguf *g, int32_t *version, int64_t *n_tensors, int64_t *n_meta, int64_t *data_offset);
/* metaLong / metaFloat (:199-216): any numeric value converts, a missing key or another type gives dflt. */
int juno_gguf_meta_int(juno_gguf *g, const char *key, int64_t dflt, int64_t *out);
int juno_gguf_meta_float(juno_gguf *g, const char *key, double dflt, double *out);
/* metaString (:194-197): *len = -1 for a missing key or another type, else the length; buf (may be null) gets at
 * most buf_len-1 bytes and a terminator. */
int juno_gguf_meta_string(juno_gguf *g, const char *key, char *buf, int32_t buf_len, int32_t *len);
int juno_gguf_meta_array_len(juno_gguf *g, const char *key, int64_t *len); /* -1 if the key is not an array */
int juno_gguf_tensor_name(juno_gguf *g, int64_t index, char *buf, int32_t buf_len); /* file order */
int juno_gguf_has_tensor(juno_gguf *g, const char *name, int32_t *present);
/* tensorType / tensorDims / tensorRaw: dims4 is innermost first ([cols, rows] for a matrix, :246-248), unused entries
 * 1.  Any output pointer may be null.  Asking for data of a type without a byte-size formula gives
 * JUNO_ERR_UNSUPPORTED (UnsupportedOperationException in the reference); an unknown name JUNO_ERR_INVALID_ARG. */
int juno_gguf_tensor(juno_gguf *g, const char *name, int32_t *ggml_type, int32_t *n_dims, int64_t *dims4,
                     const void **data, int64_t *n_bytes);
int juno_gguf_raw_byte_count(int32_t ggml_type, int64_t n_elems, int64_t *bytes); /* rawByteCount :347-360 */

/* Host-only (no GPU needed): the slice of a FULL tensor of `kind` that rank tp_rank of tp_world keeps - the rule
 * juno_model_set_tensor applies itself (TensorShardContext.java:74-100: headsPerNode = numHeads / world, sliceDim =
 * hidden / world).  out6 = {rows, cols, row0, nrows, col0, ncols} of the full tensor and of the kept sub-matrix:
 * column-parallel attn_q/k/v, ffn_gate/up and output keep whole rows, row-parallel attn_output / ffn_down keep whole
 * 256-column super-blocks of every row.  A host can use it to ship only what a rank needs. */
int juno_tp_slice(int32_t hidden, int32_t n_heads, int32_t n_kv_heads, int32_t inter, int32_t vocab, int32_t kind,
                  int32_t tp_rank, int32_t tp_world, int64_t *out6);

/* Fills 128 bytes with a fresh ncclUniqueId (rank 0 calls it and ships the bytes to the other ranks). */
int juno_nccl_unique_id(uint8_t *out128);

int juno_model_create(juno_ctx *ctx, const juno_model_cfg *cfg, juno_model **out);
/* Hands one FULL (unsharded) tensor to the model; with tp_world > 1 the library keeps only
 * this rank's slice (column-parallel Q/K/V/gate/up by head and FFN rows, row-parallel
 * O/down by whole super-blocks, vocab-parallel output).  layer is ignored for the three
 * global tensors.  Omitting JUNO_T_OUTPUT ties the output projection to token_embd
 * (LlamaTransformerHandler.java:463-470). */
int juno_model_set_tensor(juno_model *m, int32_t kind, int32_t layer, const void *blocks,
                          int32_t ggml_type, int64_t rows, int64_t cols);
int juno_model_finalize(juno_model *m);
/* LlamaConfig.from (LlamaConfig.java:58-91): fills hidden, n_layers, n_heads, n_kv_heads, inter, vocab, rms_eps and
 * rope_theta of *cfg from "<general.architecture>.*" (then "llama.*", then the TinyLlama value); vocab is the larger
 * of <arch>.vocab_size and the length of tokenizer.ggml.tokens.  The other fields are left as they are. */
int juno_gguf_model_cfg(juno_gguf *g, juno_model_cfg *cfg);
/* Hands every tensor the reference constructor reads (LlamaTransformerHandler.java:238-275: token_embd, output_norm,
 * optional output, blk.N.{attn_norm, ffn_norm, attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down}) to
 * juno_model_set_tensor, straight from the mapped file; attn_{q,k,v}.bias of every layer too when blk.0.attn_q.bias exists.
 * Call juno_model_finalize afterwards. */
int juno_model_load_gguf(juno_model *m, juno_gguf *g);
int juno_model_free(juno_model *m); /* releaseGpuResources (LlamaTransformerHandler.java:424-448) */
/* How a finalized model exchanges the partial products of its row-parallel projections: 0 = one GPU (nothing to
 * exchange), 1 = NCCL all-reduce, 2 = stores into peer-mapped inboxes by the producing kernels (up to eight
 * sequences per step; larger steps still use NCCL).  Replaces the coordinator-side sum of
 * TensorParallelPipelineClient.allReduceSum (:244-272) either way. */
int juno_model_tp_mode(juno_model *m, int32_t *mode);
int juno_model_seq_create(juno_model *m, juno_seq **out);

/* One decode step for n sequences: token_ids[i] is fed at positions[i] (only the last token
 * of a request is used, LlamaTransformerHandler.java:653-655).  logits_host ([n][vocab]) and
 * argmax_out ([n], first maximum = SampleStep.java:51-58) may each be NULL. */
int juno_forward(juno_model *m, int32_t n, juno_seq *const *seqs, const int32_t *token_ids,
                 const int32_t *positions, float *logits_host, int32_t *argmax_out);
/* Prompt prefill in chunks: feeds token_ids[0..n_tokens) of ONE sequence at positions start_pos.. and fills its KV
 * pages, up to min(max_batch, 64) positions per pass through the batched dequant-GEMM kernels (causal attention
 * inside a chunk).  Replaces the token-by-token prefill loop of GenerationLoop.java:306-317 (same positions, same
 * cache contents up to the FP16 rounding of the batched path).  logits_host ([vocab]) and argmax_out (one id) are
 * optional and refer to the LAST position fed.  Tensor parallel models: logits only with an unsharded vocabulary. */
int juno_prefill(juno_model *m, juno_seq *seq, const int32_t *token_ids, int32_t n_tokens, int32_t start_pos,
                 float *logits_host, int32_t *argmax_out);

/* `steps` greedy steps kept on the device: step 0 feeds first_tokens at positions, step s>0
 * feeds the token picked at step s-1 at positions+s.  out_ids is [steps][n]. */
int juno_decode_greedy(juno_model *m, int32_t n, juno_seq *const *seqs, const int32_t *first_tokens,
                       const int32_t *positions, int32_t steps, int32_t *out_ids);
/* Residual stream after the last layer for the most recent juno_forward ([n][hidden]). */
int juno_model_last_hidden(juno_model *m, int32_t n, float *hidden_host);

/* ── counters: what a host needs to emit juno.MatVec / juno.ForwardPass events
 *    (MatVecEvent.java:41-72, ForwardPassEvent.java:50-75). */
typedef struct juno_counters {
    int64_t kernel_launches; /* kernels of this library launched (graph replays count their nodes) */
    int64_t gemv_calls;
    int64_t forward_calls;
    int64_t h2d_bytes;
    int64_t d2h_bytes;
} juno_counters;
int juno_ctx_counters(juno_ctx *ctx, juno_counters *out, int32_t reset);

/* Per-kernel timing, the device-side counterpart of juno.MatVec durations (MatVecEvent.java:46-72).
 * While enabled every launch is bracketed by CUDA events on the context stream and forward passes run
 * without CUDA graphs; juno_ctx_profile_read synchronises and returns, per category, launches, summed
 * milliseconds and the algorithmic bytes the launches had to move.  Categories: 0 Q4_K GEMV, 1 Q6_K GEMV,
 * 2 Q8_0 GEMV, 3 attention (split + merge), 4 RoPE + KV append, 5 other, 6 batched products that ran on the
 * tcgen05/TMEM kernel (also counted under their block format). */
#define JUNO_PROF_COUNT 7
typedef struct juno_profile_entry {
    int64_t launches;
    double ms;
    double algo_bytes;
} juno_profile_entry;
int juno_ctx_profile(juno_ctx *ctx, int32_t enable);
int juno_ctx_profile_read(juno_ctx *ctx, juno_profile_entry *out, int32_t n_entries, int32_t reset);

#ifdef __cplusplus
}
#endif
#endif /* JUNO_B200_H */
