// Forward-pass operator: the device half of LlamaTransformerHandler.forward
// (LlamaTransformerHandler.java:602-628,651-810) for n sequences per step, with real tensor
// parallelism (column-parallel Q/K/V/gate/up, row-parallel O/down, vocab-parallel logits) in place of
// the coordinator-side logits sum of TensorParallelPipelineClient.allReduceSum (:244-272).
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <memory>
#include <cstring>
#include <thread>
#include <string>
#include <map>
#include <vector>

#include "attn.cuh"
#include "common.cuh"
#include "dequant.cuh"
#include "gemv.cuh"
#include "qgemv.cuh"

namespace juno {

// ───────────────────────────── NCCL, resolved at run time ─────────────────────────────────
// Single-GPU hosts never load it.  In a process that already holds an NCCL (e.g. one rank per GPU under
// torch.distributed) the soname resolves to that copy.
struct NcclId {
    char internal[128];
};
typedef struct ncclComm *NcclComm;
struct NcclApi {
    void *h = nullptr;
    int (*GetUniqueId)(NcclId *) = nullptr;
    int (*CommInitRank)(NcclComm *, int, NcclId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*CommAbort)(NcclComm) = nullptr;                 // optional
    int (*CommGetAsyncError)(NcclComm, int *) = nullptr;  // optional
    int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mu;
constexpr int kNcclFloat = 7, kNcclSum = 0;

static int nccl_load() {
    std::lock_guard<std::mutex> g(g_nccl_mu);
    if (g_nccl.h) return JUNO_OK;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        set_error("tensor parallelism needs libnccl.so.2: %s", dlerror());
        return JUNO_ERR_NCCL;
    }
    g_nccl.GetUniqueId = (int (*)(NcclId *))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(NcclComm *, int, NcclId, int))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (int (*)(NcclComm))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce =
        (int (*)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t))dlsym(h, "ncclAllReduce");
    g_nccl.AllGather = (int (*)(const void *, void *, size_t, int, NcclComm, cudaStream_t))dlsym(h, "ncclAllGather");
    g_nccl.GetErrorString = (const char *(*)(int))dlsym(h, "ncclGetErrorString");
    g_nccl.CommAbort = (int (*)(NcclComm))dlsym(h, "ncclCommAbort");
    g_nccl.CommGetAsyncError = (int (*)(NcclComm, int *))dlsym(h, "ncclCommGetAsyncError");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce || !g_nccl.AllGather) {
        set_error("libnccl.so.2 lacks a required symbol");
        return JUNO_ERR_NCCL;
    }
    g_nccl.h = h;
    return JUNO_OK;
}

#define JUNO_NCCL_TRY(expr)                                                                         \
    do {                                                                                            \
        int _r = (expr);                                                                            \
        if (_r != 0) {                                                                              \
            set_error("%s failed: rc=%d (%s)", #expr, _r,                                           \
                      g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "?");                     \
            return JUNO_ERR_NCCL;                                                                   \
        }                                                                                           \
    } while (0)

// ───────────────────────────── small kernels ──────────────────────────────────────────────
// Embedding row of the dequantised token_embd (getInitialActivation :651-660): token id clamped to
// [0, vocab-1], values bit-exact with dequantizeQ4K & co.
__global__ void embed_kernel(int type, int tiled, const uint8_t *w, int64_t nb, int64_t row_bytes, int hidden, int vocab,
                             const int32_t *tokens, float *x) {
    const int seq = blockIdx.y, col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= hidden) return;
    int tok = tokens[seq];
    tok = max(0, min(tok, vocab - 1));
    float v;
    if (tiled) {
        const uint8_t *tile = w + (((int64_t)tok >> 4) * nb + (col >> 8)) * (int64_t)tile_bytes(type);
        v = tile_elem_value(type, tile, tok & 15, col & 255);
    } else {
        v = raw_elem_value(type, w + (int64_t)tok * row_bytes, col);
    }
    x[(size_t)seq * hidden + col] = v;
}

// Element (seq, v) of the logits: plain [n][V], or, after an all-gather of vocab slices, [world][n][V/world].
struct LogitsView {
    const float *base;
    int n, vocab, vloc;  // vloc == vocab: plain layout
    __device__ __forceinline__ float at(int seq, int v) const {
        if (vloc == vocab) return base[(size_t)seq * vocab + v];
        const int r = v / vloc, j = v - r * vloc;
        return base[((size_t)r * n + seq) * vloc + j];
    }
};

constexpr int kArgmaxBlocks = 32;
// First maximum (lowest index among equal values), as SampleStep.greedy (sampler/.../SampleStep.java:51-58)
// picks after a monotone softmax.
__global__ void argmax_partial_kernel(LogitsView lv, float *pval, int32_t *pidx) {
    const int seq = blockIdx.y, blk = blockIdx.x;
    const int per = (lv.vocab + kArgmaxBlocks - 1) / kArgmaxBlocks;
    const int v0 = blk * per, v1 = min(lv.vocab, v0 + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        const float x = lv.at(seq, v);
        if (x > best || (x == best && v < bi)) {
            best = x;
            bi = v;
        }
    }
    __shared__ float sv[256];
    __shared__ int si[256];
    sv[threadIdx.x] = best;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s];
            const int oi = si[threadIdx.x + s];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
                sv[threadIdx.x] = ov;
                si[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        pval[seq * kArgmaxBlocks + blk] = sv[0];
        pidx[seq * kArgmaxBlocks + blk] = si[0];
    }
}
__global__ void argmax_final_kernel(const float *pval, const int32_t *pidx, int n, int32_t *out) {
    const int seq = blockIdx.x * blockDim.x + threadIdx.x;
    if (seq >= n) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int b = 0; b < kArgmaxBlocks; b++) {
        const float v = pval[seq * kArgmaxBlocks + b];
        const int i = pidx[seq * kArgmaxBlocks + b];
        if (i != 0x7fffffff && (v > best || (v == best && i < bi))) {
            best = v;
            bi = i;
        }
    }
    out[seq] = (bi == 0x7fffffff) ? 0 : bi;  // all-NaN logits: index 0, as a loop that never finds a larger value
}

// Greedy loop kept on the device: the picked token becomes the next input, one position further.
__global__ void advance_kernel(int n, const int32_t *picked, int32_t *tokens, int32_t *positions, int32_t *seq_lens,
                               int32_t *out_ids, int32_t *step_counter) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int step = *step_counter;
    if (i < n) {
        tokens[i] = picked[i];
        positions[i] += 1;
        seq_lens[i] += 1;
        out_ids[(size_t)step * n + i] = picked[i];
    }
    __syncthreads();
    if (i == 0) *step_counter = step + 1;
}

// Vocabulary-parallel greedy pick without gathering the logits: every rank pushes the first maximum of its slice
// (value, global index) into every rank's slot, then publishes the step number; the merge waits (bounded) for all
// ranks and takes the first maximum overall - the same token a first-maximum scan of the gathered logits finds.
struct PairXchg {
    float2 *slot[8];      // slot[d]: this rank's row of n pairs inside rank d's buffer
    unsigned *flag[8];    // flag[d]: this rank's flag inside rank d's buffer
    int world;
};
__global__ void argmax_push_kernel(const float *pval, const int32_t *pidx, int n, int v0, PairXchg x, const unsigned *epoch) {
    const int seq = threadIdx.x;
    if (seq < n) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int b = 0; b < kArgmaxBlocks; b++) {
            const float v = pval[seq * kArgmaxBlocks + b];
            const int i = pidx[seq * kArgmaxBlocks + b];
            if (i != 0x7fffffff && (v > best || (v == best && i < bi))) {
                best = v;
                bi = i;
            }
        }
        const float2 pr = make_float2(best, __int_as_float(bi == 0x7fffffff ? 0x7fffffff : bi + v0));
        for (int d = 0; d < x.world; d++) x.slot[d][seq] = pr;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned e = *reinterpret_cast<const volatile unsigned *>(epoch);
        for (int d = 0; d < x.world; d++) *reinterpret_cast<volatile unsigned *>(x.flag[d]) = e;
    }
}
__global__ void argmax_merge_kernel(const float2 *slots /* [world][stride] */, int stride, const unsigned *flags, int world, int n,
                                    const unsigned *epoch, int32_t *out, unsigned *err, unsigned *failed) {
    const unsigned want = *reinterpret_cast<const volatile unsigned *>(epoch);
    if (threadIdx.x < world && *reinterpret_cast<volatile unsigned *>(failed) == 0u) {
        const volatile unsigned *f = flags + threadIdx.x;
        const long long t0 = clock64();
        while ((int)(*f - want) < 0) {
            if (clock64() - t0 > 2000000000ll) {  // about a second: the rank may have failed
                *reinterpret_cast<volatile unsigned *>(failed) = 1u;
                *reinterpret_cast<volatile unsigned *>(err) = 4u | (threadIdx.x << 8);
                break;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    const int seq = threadIdx.x;
    if (seq >= n) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < world; r++) {
        const float2 pr = __ldcg(slots + (size_t)r * stride + seq);
        const int i = __float_as_int(pr.y);
        if (i != 0x7fffffff && (pr.x > best || (pr.x == best && i < bi))) {
            best = pr.x;
            bi = i;
        }
    }
    out[seq] = (bi == 0x7fffffff) ? 0 : bi;
}

// q, k, v += bias (LlamaTransformerHandler.addInPlace :1641-1646, applied before the rotation :758-762): one row of
// biases laid out like a row of the q|k|v buffer.  Launched only for models that carry attn_{q,k,v}.bias.
__global__ void qkv_bias_kernel(float *qkv, const float *bias, int n, int width, int ld) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (i < width && b < n) qkv[(size_t)b * ld + i] = __fadd_rn(qkv[(size_t)b * ld + i], bias[i]);
}

// Start of a tensor-parallel step: the step number the ranks tag their partial products with.
__global__ void epoch_kernel(unsigned *epoch) { *epoch += 1u; }

// [world][n][vloc] -> [n][vocab]
__global__ void ungather_logits_kernel(LogitsView lv, float *out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)lv.n * lv.vocab) return;
    const int seq = (int)(idx / lv.vocab), v = (int)(idx - (size_t)seq * lv.vocab);
    out[idx] = lv.at(seq, v);
}

}  // namespace juno

// ───────────────────────────── model object ───────────────────────────────────────────────
struct JunoLayer {
    juno_qmat *w[12] = {nullptr};  // indexed by tensor kind (ATTN_Q .. FFN_DOWN); gate and up share w[FFN_GATE]
    std::vector<uint8_t> gate_host, up_host;  // row slices waiting for their partner
    int gate_type = -1, up_type = -1;
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    float *bqkv = nullptr;  // optional attn_{q,k,v}.bias of this rank, laid out like a row of the q|k|v buffer
    int bias_seen = 0;      // bit per bias kind received
};

struct JunoGraph {
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
    int seen = 0;
};

struct juno_model {
    uint32_t magic;
    juno_ctx *ctx;
    juno_model_cfg cfg;
    int hd, world, rank;
    int heads_loc, kv_loc, inter_loc, vocab_loc;  // this rank's share
    int qkv_ld;
    bool finalized = false;
    bool vocab_sharded = false;
    std::vector<JunoLayer> layers;
    juno_qmat *tok_embd = nullptr, *output = nullptr;
    bool output_is_embd = false, output_slice_of_embd = false;
    float *output_norm = nullptr;
    juno_kvpool *pool = nullptr;
    juno::NcclComm comm = nullptr;
    // activations
    float *x[2] = {nullptr, nullptr}, *qkv = nullptr, *att = nullptr, *proj = nullptr, *proj2 = nullptr;
    float *hdn = nullptr, *xsc = nullptr;  // batched path: silu(gate)*up rows; per-row factors of the three FP16 images
    uint8_t *img_h_tc = nullptr;            // batched path: the hidden-size activation again, chunk-major for the tcgen05 kernel
    unsigned *tc_err = nullptr;             // device word: a wait inside the tcgen05 kernel gave up
    bool tc_used = false;                   // the batched path ran since the word was last read
    uint8_t *img_h = nullptr, *img_att = nullptr, *img_i = nullptr;  // staged activations (K = hidden, local heads, local FFN)
    float *logits_loc = nullptr, *logits_gather = nullptr, *logits_full = nullptr;
    float *attn_scratch = nullptr;
    size_t attn_scratch_floats = 0;
    float2 *rope_cs = nullptr;
    int32_t *d_step = nullptr;  // tokens | positions | slots | seq_lens, max_batch each
    int32_t *d_argmax = nullptr, *d_pidx = nullptr, *d_out_ids = nullptr, *d_step_counter = nullptr;
    float *d_pval = nullptr;
    int out_ids_cap = 0;
    int32_t *h_step = nullptr;  // pinned mirror of d_step
    int last_n = 0, last_x = 0;
    double step_kv_bytes = 0;  // K+V bytes one layer's attention reads in the current step
    std::map<uint64_t, JunoGraph> graphs;
    bool use_graphs = true, mix_formats = true;  // JUNO_NO_GRAPH / JUNO_NO_MIXED
    // tensor parallelism without collective calls on the 1..8 sequence path: per-rank exchange buffer (flags + inbox
    // slots per row-parallel product), mapped into every peer (CUDA IPC), see enqueue_layers_q
    bool tp_push = false;
    uint8_t *tp_buf = nullptr;           // this rank's buffer
    uint8_t *tp_peer[8] = {nullptr};     // every rank's buffer as seen from here (tp_peer[rank] == tp_buf)
    size_t tp_inbox_off = 0, tp_pair_off = 0;
    int tp_bq = 0;                       // sequences an inbox slot holds
    unsigned *tp_failed = nullptr;       // device word: a wait for another rank ran out during this step
    float *tp_red = nullptr;             // [2 * n_layers][tp_bq][hidden] (value, step) pairs: the ranks' partials added by the first CTAs
    bool tp_reduce = false;              // consumers poll tp_red instead of every rank's inbox (four ranks and more)
    bool comm_failed = false;            // a collective timed out or NCCL reported an asynchronous error: no further steps
    unsigned *tp_epoch = nullptr;        // step number, incremented on the device at the start of every step
    int batched_from = 9;  // smallest batch on the FP16 one-pass kernels (JUNO_GEMM_MIN_BATCH, read when the model is created)
};

namespace juno {

static int model_check(juno_model *m) {
    if (!m) {
        set_error("model is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (m->magic != kMagicModel) {
        set_error("model handle is closed");
        return JUNO_ERR_CLOSED;
    }
    return JUNO_OK;
}

static int dev_alloc(void **p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 4);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        return JUNO_ERR_OOM;
    }
    return JUNO_OK;
}

static int upload_f32_vector(juno_ctx *c, const void *blocks, int type, int64_t rows, int64_t cols, int want, float **dst) {
    JUNO_REQUIRE(type == JUNO_TYPE_F32, "norm weights must be F32 (got GGML type %d)", type);
    JUNO_REQUIRE(rows * cols == want, "norm weight has %lld elements, expected %d", (long long)(rows * cols), want);
    if (*dst) cudaFree(*dst);
    *dst = nullptr;
    JUNO_TRY(dev_alloc((void **)dst, (size_t)want * 4));
    JUNO_CUDA_TRY(cudaMemcpyAsync(*dst, blocks, (size_t)want * 4, cudaMemcpyHostToDevice, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->h2d_bytes += want * 4;
    return JUNO_OK;
}

static void free_qmat(juno_qmat *&q) {
    if (q) {
        qmat_destroy(q);
        delete q;
        q = nullptr;
    }
}

static void model_release(juno_model *m) {
    juno_ctx *c = m->ctx;
    DeviceGuard g(c->device);
    cudaStreamSynchronize(c->stream);
    for (auto &kv : m->graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    m->graphs.clear();
    for (int r = 0; r < 8; r++)
        if (m->tp_peer[r] && m->tp_peer[r] != m->tp_buf) cudaIpcCloseMemHandle(m->tp_peer[r]);
    if (m->tp_buf) cudaFree(m->tp_buf);
    if (m->tp_failed) cudaFree(m->tp_failed);
    if (m->tp_red) cudaFree(m->tp_red);
    if (m->tp_epoch) cudaFree(m->tp_epoch);
    m->tp_buf = nullptr;
    if (m->comm) {
        // after a failure the peers may be gone: abort (returns at once) instead of the orderly teardown
        if (m->comm_failed && g_nccl.CommAbort)
            g_nccl.CommAbort(m->comm);
        else if (g_nccl.CommDestroy)
            g_nccl.CommDestroy(m->comm);
    }
    m->comm = nullptr;
    for (auto &L : m->layers) {
        for (int k = 0; k < 12; k++) free_qmat(L.w[k]);
        if (L.attn_norm) cudaFree(L.attn_norm);
        if (L.ffn_norm) cudaFree(L.ffn_norm);
        if (L.bqkv) cudaFree(L.bqkv);
    }
    m->layers.clear();
    if (m->output_is_embd) m->output = nullptr;
    free_qmat(m->output);
    free_qmat(m->tok_embd);
    if (m->pool) {
        m->pool->owned_by_model = 0;
        kvpool_destroy(m->pool);
    }
    void *bufs[] = {m->x[0], m->x[1], m->qkv, m->att, m->proj, m->proj2, m->hdn, m->xsc, m->img_h_tc, m->tc_err, m->img_h, m->img_att, m->img_i, m->logits_loc, m->logits_gather, m->logits_full,
                    m->attn_scratch, m->rope_cs, m->d_step, m->d_argmax, m->d_pidx, m->d_out_ids, m->d_step_counter,
                    m->d_pval, m->output_norm};
    for (void *b : bufs)
        if (b) cudaFree(b);
    if (m->h_step) cudaFreeHost(m->h_step);
    m->magic = kMagicDead;
}

// The slice of a full tensor one tensor-parallel rank keeps (geometry of TensorShardContext.java:74-100 turned into
// rows and columns): column-parallel attn_q/k/v (by head), ffn_gate/up (by FFN row) and the output projection (by
// vocabulary row, when the vocabulary divides); row-parallel attn_output and ffn_down (whole 256-column super-blocks).
static int tp_slice(int hidden, int n_heads, int n_kv_heads, int inter, int vocab, int kind, int rank, int world, int64_t *rows,
                    int64_t *cols, int64_t *row0, int64_t *nrows, int64_t *col0, int64_t *ncols) {
    JUNO_REQUIRE(hidden > 0 && n_heads > 0 && n_kv_heads > 0 && inter > 0 && vocab > 0 && hidden % n_heads == 0, "bad model dimensions");
    JUNO_REQUIRE(world >= 1 && rank >= 0 && rank < world, "tensorRank (%d) must be < tensorWorldSize (%d)", rank, world);
    const int64_t hd = hidden / n_heads, H = hidden, I = inter, V = vocab;
    if (world > 1) {
        JUNO_REQUIRE(n_heads % world == 0 && n_kv_heads % world == 0, "heads (%d query, %d kv) do not divide over %d ranks", n_heads,
                     n_kv_heads, world);
        JUNO_REQUIRE(inter % world == 0, "feed_forward_length %d does not divide over %d ranks", inter, world);
    }
    const int64_t hl = n_heads / world * hd, kl = n_kv_heads / world * hd, il = I / world;
    const bool vshard = world > 1 && V % world == 0;
    int64_t R = 0, C = 0, r0 = 0, nr = 0, c0 = 0, nc = 0;
    switch (kind) {
    case JUNO_T_TOKEN_EMBD: R = V; C = H; nr = V; nc = H; break;
    case JUNO_T_OUTPUT: R = V; C = H; r0 = vshard ? rank * (V / world) : 0; nr = vshard ? V / world : V; nc = H; break;
    case JUNO_T_ATTN_Q: R = H; C = H; r0 = rank * hl; nr = hl; nc = H; break;
    case JUNO_T_ATTN_K:
    case JUNO_T_ATTN_V: R = n_kv_heads * hd; C = H; r0 = rank * kl; nr = kl; nc = H; break;
    case JUNO_T_ATTN_OUT: R = H; C = H; nr = H; c0 = rank * hl; nc = hl; break;
    case JUNO_T_FFN_GATE:
    case JUNO_T_FFN_UP: R = I; C = H; r0 = rank * il; nr = il; nc = H; break;
    case JUNO_T_FFN_DOWN: R = H; C = I; nr = H; c0 = rank * il; nc = il; break;
    case JUNO_T_OUTPUT_NORM:
    case JUNO_T_ATTN_NORM:
    case JUNO_T_FFN_NORM: R = 1; C = H; nr = 1; nc = H; break;
    default: set_error("unknown tensor kind %d", kind); return JUNO_ERR_INVALID_ARG;
    }
    if (world > 1) JUNO_REQUIRE(c0 % 256 == 0 && nc % 256 == 0, "a column slice must be whole 256-column super-blocks");
    *rows = R; *cols = C; *row0 = r0; *nrows = nr; *col0 = c0; *ncols = nc;
    return JUNO_OK;
}

// Maps one exchange buffer per rank into every rank (CUDA IPC; the handles travel through an NCCL all-gather).  Any
// failure leaves the model on the NCCL collectives.
static int tp_push_setup(juno_model *m) {
    const char *e = getenv("JUNO_TP_PUSH");
    if ((e && *e == '0') || m->world > 8) return JUNO_OK;
    juno_ctx *c = m->ctx;
    const int W = m->world, H = m->cfg.hidden, n_inst = 2 * m->cfg.n_layers;
    m->tp_bq = std::min(m->cfg.max_batch, 8);
    // [greedy-pick flags: 8 words][greedy-pick pairs: 8 ranks x 8 sequences][inbox: n_inst x W slots of bq x H (value, step) pairs]
    m->tp_pair_off = 8 * 4;
    m->tp_inbox_off = (m->tp_pair_off + 8 * 8 * sizeof(float2) + 4095) & ~(size_t)4095;
    const size_t bytes = m->tp_inbox_off + (size_t)n_inst * W * m->tp_bq * H * 8;
    JUNO_TRY(dev_alloc((void **)&m->tp_buf, bytes));
    JUNO_CUDA_TRY(cudaMemset(m->tp_buf, 0, bytes));
    JUNO_TRY(dev_alloc((void **)&m->tp_failed, 4));
    JUNO_CUDA_TRY(cudaMemset(m->tp_failed, 0, 4));
    JUNO_TRY(dev_alloc((void **)&m->tp_red, (size_t)n_inst * m->tp_bq * H * 8));
    JUNO_CUDA_TRY(cudaMemset(m->tp_red, 0, (size_t)n_inst * m->tp_bq * H * 8));
    {
        // every CTA reading every rank's inbox costs L2 bandwidth in proportion to the ranks (measured 2.2 / 4.9 / 10.9 us
        // per exchange at 2 / 4 / 8 ranks); from four ranks on the first CTAs add the inboxes once for all
        const char *r = getenv("JUNO_TP_REDUCE");
        m->tp_reduce = (r && *r) ? atoi(r) != 0 : W >= 4;
    }
    JUNO_TRY(dev_alloc((void **)&m->tp_epoch, 4));
    JUNO_CUDA_TRY(cudaMemset(m->tp_epoch, 0, 4));
    cudaIpcMemHandle_t mine, all[8];
    bool ok = true;
    if (cudaIpcGetMemHandle(&mine, m->tp_buf) != cudaSuccess) {
        cudaGetLastError();
        memset(&mine, 0, sizeof(mine));
        ok = false;  // no IPC on this system: NCCL path (the ranks still meet in the two collectives below)
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    uint8_t *d_h = nullptr;
    JUNO_TRY(dev_alloc((void **)&d_h, (size_t)64 * (W + 1)));
    JUNO_CUDA_TRY(cudaMemcpyAsync(d_h, &mine, 64, cudaMemcpyHostToDevice, c->stream));
    JUNO_NCCL_TRY(g_nccl.AllGather(d_h, d_h + 64, 16, kNcclFloat, m->comm, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(all, d_h + 64, (size_t)64 * W, cudaMemcpyDeviceToHost, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    cudaFree(d_h);
    for (int r = 0; ok && r < W; r++) {
        if (r == m->rank) {
            m->tp_peer[r] = m->tp_buf;
            continue;
        }
        void *ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = false;
            break;
        }
        m->tp_peer[r] = static_cast<uint8_t *>(ptr);
    }
    // every rank must take the same path: agree on the outcome
    float *d_ok = nullptr;
    JUNO_TRY(dev_alloc((void **)&d_ok, 4));
    const float mine_ok = ok ? 0.f : 1.f;
    JUNO_CUDA_TRY(cudaMemcpyAsync(d_ok, &mine_ok, 4, cudaMemcpyHostToDevice, c->stream));
    JUNO_NCCL_TRY(g_nccl.AllReduce(d_ok, d_ok, 1, kNcclFloat, kNcclSum, m->comm, c->stream));
    float bad = 1.f;
    JUNO_CUDA_TRY(cudaMemcpyAsync(&bad, d_ok, 4, cudaMemcpyDeviceToHost, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    cudaFree(d_ok);
    m->tp_push = (bad == 0.f);
    if (!m->tp_push) {  // some rank could not map a peer: every rank drops its mappings and the group uses NCCL
        for (int r = 0; r < W; r++) {
            if (m->tp_peer[r] && m->tp_peer[r] != m->tp_buf) cudaIpcCloseMemHandle(m->tp_peer[r]);
            m->tp_peer[r] = nullptr;
        }
        cudaGetLastError();
    }
    return JUNO_OK;
}

}  // namespace juno

using namespace juno;

extern "C" {

int juno_nccl_unique_id(uint8_t *out128) {
    JUNO_REQUIRE(out128, "out is null");
    JUNO_TRY(nccl_load());
    NcclId id;
    JUNO_NCCL_TRY(g_nccl.GetUniqueId(&id));
    memcpy(out128, id.internal, 128);
    return JUNO_OK;
}

int juno_tp_slice(int32_t hidden, int32_t n_heads, int32_t n_kv_heads, int32_t inter, int32_t vocab, int32_t kind, int32_t tp_rank,
                  int32_t tp_world, int64_t *out6) {
    JUNO_REQUIRE(out6, "out is null");
    return tp_slice(hidden, n_heads, n_kv_heads, inter, vocab, kind, tp_rank, tp_world, out6, out6 + 1, out6 + 2, out6 + 3, out6 + 4, out6 + 5);
}

int juno_model_create(juno_ctx *c, const juno_model_cfg *cfg, juno_model **out) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(cfg && out, "null argument");
    JUNO_REQUIRE(cfg->struct_size == (int32_t)sizeof(juno_model_cfg), "juno_model_cfg.struct_size is %d, expected %d",
                 cfg->struct_size, (int)sizeof(juno_model_cfg));
    JUNO_REQUIRE(cfg->hidden > 0 && cfg->n_layers > 0 && cfg->n_heads > 0 && cfg->n_kv_heads > 0 && cfg->inter > 0 &&
                     cfg->vocab > 0,
                 "model dimensions must be positive");
    JUNO_REQUIRE(cfg->hidden % cfg->n_heads == 0, "hidden %d is not a multiple of n_heads %d", cfg->hidden, cfg->n_heads);
    JUNO_REQUIRE(cfg->n_heads % cfg->n_kv_heads == 0, "n_heads %d is not a multiple of n_kv_heads %d", cfg->n_heads,
                 cfg->n_kv_heads);
    JUNO_REQUIRE(cfg->max_batch >= 1 && cfg->max_batch <= 1024 && cfg->max_seqs >= 1 && cfg->max_ctx >= 1,
                 "max_batch/max_seqs/max_ctx out of range");
    JUNO_REQUIRE(cfg->tp_world >= 1 && cfg->tp_rank >= 0 && cfg->tp_rank < cfg->tp_world,
                 "tensorRank (%d) must be < tensorWorldSize (%d)", cfg->tp_rank, cfg->tp_world);
    const int hd = cfg->hidden / cfg->n_heads, w = cfg->tp_world;
    JUNO_REQUIRE(hd == 64 || hd == 128, "head_dim %d is not supported (64, 128)", hd);
    JUNO_REQUIRE(cfg->hidden % 256 == 0 && cfg->inter % 256 == 0, "hidden and feed_forward_length must be multiples of 256");
    if (w > 1) {
        // geometry of TensorShardContext (:74-100): headsPerNode = numHeads / world, sliceDim = hidden / world
        JUNO_REQUIRE(cfg->n_heads % 2 == 0, "numHeads (%d) must be divisible by 2 for tensor-parallel mode", cfg->n_heads);
        JUNO_REQUIRE(cfg->n_heads % w == 0 && cfg->n_kv_heads % w == 0,
                     "heads (%d query, %d kv) do not divide over %d ranks", cfg->n_heads, cfg->n_kv_heads, w);
        JUNO_REQUIRE((cfg->hidden / w) % 256 == 0 && (cfg->inter / w) % 256 == 0 && cfg->inter % w == 0,
                     "hidden/world and feed_forward_length/world must be multiples of 256 (whole super-blocks)");
    }
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    juno_model *m = new juno_model();
    m->magic = kMagicModel;
    m->ctx = c;
    m->cfg = *cfg;
    m->hd = hd;
    m->world = w;
    m->rank = cfg->tp_rank;
    m->heads_loc = cfg->n_heads / w;
    m->kv_loc = cfg->n_kv_heads / w;
    m->inter_loc = cfg->inter / w;
    m->vocab_sharded = (w > 1) && (cfg->vocab % w == 0);
    m->vocab_loc = m->vocab_sharded ? cfg->vocab / w : cfg->vocab;
    m->qkv_ld = (m->heads_loc + 2 * m->kv_loc) * hd;
    m->layers.resize(cfg->n_layers);
    const char *ng = getenv("JUNO_NO_GRAPH");
    m->use_graphs = !(ng && *ng == '1');
    const char *nm = getenv("JUNO_NO_MIXED");
    m->mix_formats = !(nm && *nm == '1');
    {
        const char *gm = getenv("JUNO_GEMM_MIN_BATCH");
        m->batched_from = std::max(2, (gm && *gm) ? atoi(gm) : 9);
    }
    if (w > 1) {
        int rc = nccl_load();
        if (rc == JUNO_OK) {
            NcclId id;
            memcpy(id.internal, cfg->nccl_id, 128);
            int r = g_nccl.CommInitRank(&m->comm, w, id, cfg->tp_rank);
            if (r != 0) {
                set_error("ncclCommInitRank failed: rc=%d (%s)", r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?");
                rc = JUNO_ERR_NCCL;
            }
        }
        if (rc != JUNO_OK) {
            m->magic = kMagicDead;
            delete m;
            return rc;
        }
    }
    *out = m;
    return JUNO_OK;
}

int juno_model_set_tensor(juno_model *m, int32_t kind, int32_t layer, const void *blocks, int32_t type, int64_t rows,
                          int64_t cols) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(blocks, "blocks is null");
    JUNO_REQUIRE(!m->finalized, "model is already finalized");
    JUNO_REQUIRE(kind >= 0 && kind <= JUNO_T_ATTN_V_BIAS, "unknown tensor kind %d", kind);
    juno_ctx *c = m->ctx;
    const juno_model_cfg &f = m->cfg;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    const int H = f.hidden, I = f.inter, V = f.vocab, hd = m->hd, r = m->rank;
    if (kind == JUNO_T_OUTPUT_NORM) return upload_f32_vector(c, blocks, type, rows, cols, H, &m->output_norm);
    if (kind > JUNO_T_OUTPUT) JUNO_REQUIRE(layer >= 0 && layer < f.n_layers, "layer %d out of range", layer);
    if (kind == JUNO_T_ATTN_NORM) return upload_f32_vector(c, blocks, type, rows, cols, H, &m->layers[layer].attn_norm);
    if (kind == JUNO_T_FFN_NORM) return upload_f32_vector(c, blocks, type, rows, cols, H, &m->layers[layer].ffn_norm);
    if (kind >= JUNO_T_ATTN_Q_BIAS) {
        // attn_{q,k,v}.bias: F32 vectors of hidden / kvDim elements; this rank keeps the slice of its heads
        JunoLayer &L = m->layers[layer];
        const int full = kind == JUNO_T_ATTN_Q_BIAS ? H : f.n_kv_heads * hd;
        const int loc = kind == JUNO_T_ATTN_Q_BIAS ? m->heads_loc * hd : m->kv_loc * hd;
        const int dst = kind == JUNO_T_ATTN_Q_BIAS ? 0 : kind == JUNO_T_ATTN_K_BIAS ? m->heads_loc * hd : (m->heads_loc + m->kv_loc) * hd;
        JUNO_REQUIRE(type == JUNO_TYPE_F32, "bias vectors must be F32 (got GGML type %d)", type);
        JUNO_REQUIRE(rows * cols == full, "bias kind %d has %lld elements, expected %d", kind, (long long)(rows * cols), full);
        if (!L.bqkv) {
            JUNO_TRY(dev_alloc((void **)&L.bqkv, (size_t)m->qkv_ld * 4));
            JUNO_CUDA_TRY(cudaMemset(L.bqkv, 0, (size_t)m->qkv_ld * 4));
        }
        JUNO_CUDA_TRY(cudaMemcpyAsync(L.bqkv + dst, static_cast<const float *>(blocks) + (size_t)r * loc, (size_t)loc * 4, cudaMemcpyHostToDevice, c->stream));
        JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
        c->h2d_bytes += loc * 4;
        L.bias_seen |= 1 << (kind - JUNO_T_ATTN_Q_BIAS);
        return JUNO_OK;
    }

    int64_t want_rows = 0, want_cols = 0, row0 = 0, nrows = 0, col0 = 0, ncols = 0;
    JUNO_TRY(tp_slice(f.hidden, f.n_heads, f.n_kv_heads, f.inter, f.vocab, kind, m->rank, m->world, &want_rows, &want_cols, &row0, &nrows,
                      &col0, &ncols));
    int64_t sb0 = col0 / 256, nsb = ncols / 256;
    JUNO_REQUIRE(rows == want_rows && cols == want_cols, "tensor kind %d has shape %lldx%lld, expected %lldx%lld", kind,
                 (long long)rows, (long long)cols, (long long)want_rows, (long long)want_cols);
    if (kind != JUNO_T_TOKEN_EMBD)
        JUNO_REQUIRE(type == JUNO_TYPE_Q4_K || type == JUNO_TYPE_Q6_K || type == JUNO_TYPE_Q8_0,
                     "projection weights must be Q4_K, Q6_K or Q8_0 (got GGML type %d)", type);
    if (m->world == 1) sb0 = nsb = 0;
    if (kind == JUNO_T_FFN_GATE || kind == JUNO_T_FFN_UP) {
        // gate and up rows are interleaved in groups of eight (tile rows 0-7 gate, 8-15 up) so that the GEMV
        // epilogue holds silu(gate_i) and up_i together; the first of the pair waits on the host for its partner
        JunoLayer &L = m->layers[layer];
        JUNO_REQUIRE(m->inter_loc % 8 == 0, "feed_forward_length per rank must be a multiple of 8");
        const int64_t rb = cols / raw_block_elems(type) * raw_block_bytes(type);
        const uint8_t *src = static_cast<const uint8_t *>(blocks) + row0 * rb;
        std::vector<uint8_t> &mine = kind == JUNO_T_FFN_GATE ? L.gate_host : L.up_host;
        mine.assign(src, src + nrows * rb);
        (kind == JUNO_T_FFN_GATE ? L.gate_type : L.up_type) = type;
        if (L.gate_host.empty() || L.up_host.empty()) return JUNO_OK;
        JUNO_REQUIRE(L.gate_type == L.up_type, "layer %d: ffn_gate and ffn_up must share one block format", layer);
        std::vector<uint8_t> both((size_t)2 * nrows * rb);
        for (int64_t t = 0; t < nrows / 8; t++) {
            memcpy(&both[(size_t)(2 * t) * 8 * rb], &L.gate_host[(size_t)t * 8 * rb], (size_t)8 * rb);
            memcpy(&both[(size_t)(2 * t + 1) * 8 * rb], &L.up_host[(size_t)t * 8 * rb], (size_t)8 * rb);
        }
        free_qmat(L.w[JUNO_T_FFN_GATE]);
        int rc = qmat_create(c, both.data(), type, 2 * nrows, cols, 0, 2 * nrows, 0, 0, &L.w[JUNO_T_FFN_GATE]);
        std::vector<uint8_t>().swap(L.gate_host);
        std::vector<uint8_t>().swap(L.up_host);
        return rc;
    }
    juno_qmat **slot = kind == JUNO_T_TOKEN_EMBD ? &m->tok_embd : kind == JUNO_T_OUTPUT ? &m->output : &m->layers[layer].w[kind];
    free_qmat(*slot);
    JUNO_TRY(qmat_create(c, blocks, type, rows, cols, row0, nrows, sb0, nsb, slot));
    if (kind == JUNO_T_OUTPUT) m->output_slice_of_embd = false;
    if (kind == JUNO_T_TOKEN_EMBD && m->vocab_sharded && (!m->output || m->output_slice_of_embd)) {
        // tied embeddings under vocab sharding: this rank's output projection is a row slice of token_embd
        if (type == JUNO_TYPE_Q4_K || type == JUNO_TYPE_Q6_K || type == JUNO_TYPE_Q8_0) {
            free_qmat(m->output);
            JUNO_TRY(qmat_create(c, blocks, type, rows, cols, (int64_t)r * m->vocab_loc, m->vocab_loc, 0, 0, &m->output));
            m->output_slice_of_embd = true;
        }
    }
    return JUNO_OK;
}

}  // extern "C"

// ───────────────────────────── finalize ───────────────────────────────────────────────────
extern "C" int juno_model_finalize(juno_model *m) {
    JUNO_TRY(model_check(m));
    if (m->finalized) return JUNO_OK;
    juno_ctx *c = m->ctx;
    const juno_model_cfg &f = m->cfg;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_REQUIRE(m->tok_embd && m->output_norm, "token_embd.weight and output_norm.weight are required");
    if (!m->output) {  // tied embeddings (LlamaTransformerHandler.java:463-470)
        JUNO_REQUIRE(m->tok_embd->tiled, "a tied output projection needs a Q4_K/Q6_K/Q8_0 token_embd");
        m->output = m->tok_embd;
        m->output_is_embd = true;
    }
    for (int l = 0; l < f.n_layers; l++) {
        JunoLayer &L = m->layers[l];
        JUNO_REQUIRE(L.attn_norm && L.ffn_norm, "layer %d: norm weights missing", l);
        JUNO_REQUIRE(L.bias_seen == 0 || L.bias_seen == 7, "layer %d: attn_q, attn_k and attn_v biases come together or not at all", l);
        JUNO_REQUIRE(L.bias_seen == m->layers[0].bias_seen, "layer %d: either every layer has attention biases or none (:258-262)", l);
        for (int k = JUNO_T_ATTN_Q; k <= JUNO_T_FFN_DOWN; k++)
            if (k != JUNO_T_FFN_UP) JUNO_REQUIRE(L.w[k], "layer %d: tensor kind %d missing", l, k);
    }
    const int B = f.max_batch, H = f.hidden, hd = m->hd;
    const int max_pages_per_seq = (f.max_ctx + kPageTokens - 1) / kPageTokens;
    const long long want_pages = (long long)f.max_seqs * max_pages_per_seq;
    JUNO_REQUIRE(want_pages < (1ll << 31), "KV pool too large");
    JUNO_TRY(kvpool_create(c, f.n_layers, m->kv_loc, hd, (int)want_pages, f.kv_dtype, f.max_seqs, max_pages_per_seq,
                           &m->pool));
    m->pool->owned_by_model = 1;
    JUNO_TRY(dev_alloc((void **)&m->x[0], (size_t)B * H * 4));
    JUNO_TRY(dev_alloc((void **)&m->x[1], (size_t)B * H * 4));
    JUNO_TRY(dev_alloc((void **)&m->qkv, (size_t)B * m->qkv_ld * 4));
    JUNO_TRY(dev_alloc((void **)&m->att, (size_t)B * m->heads_loc * hd * 4));
    JUNO_TRY(dev_alloc((void **)&m->proj, (size_t)B * H * 4));
    JUNO_TRY(dev_alloc((void **)&m->proj2, (size_t)B * H * 4));
    const int Bg = std::min(B, kGemmMaxBatch);
    JUNO_TRY(dev_alloc((void **)&m->img_h, gemm_image_bytes(H, Bg)));
    JUNO_TRY(dev_alloc((void **)&m->img_att, gemm_image_bytes(m->heads_loc * hd, Bg)));
    JUNO_TRY(dev_alloc((void **)&m->img_i, gemm_image_bytes(m->inter_loc, Bg)));
    JUNO_TRY(dev_alloc((void **)&m->hdn, (size_t)B * m->inter_loc * 4));
    JUNO_TRY(dev_alloc((void **)&m->xsc, (size_t)3 * B * 4));
    JUNO_TRY(dev_alloc((void **)&m->img_h_tc, gemm_tc_image_bytes(H, Bg)));
    JUNO_TRY(dev_alloc((void **)&m->tc_err, 4));
    JUNO_CUDA_TRY(cudaMemset(m->tc_err, 0, 4));
    JUNO_TRY(dev_alloc((void **)&m->logits_loc, (size_t)B * m->vocab_loc * 4));
    if (m->vocab_sharded) {
        JUNO_TRY(dev_alloc((void **)&m->logits_gather, (size_t)B * f.vocab * 4));
        JUNO_TRY(dev_alloc((void **)&m->logits_full, (size_t)B * f.vocab * 4));
    }
    m->attn_scratch_floats = (size_t)(c->sm_count * 4 + B * m->kv_loc) * (m->heads_loc / m->kv_loc) * (hd + 2) + 64;
    JUNO_TRY(dev_alloc((void **)&m->attn_scratch, m->attn_scratch_floats * 4));
    JUNO_TRY(dev_alloc((void **)&m->rope_cs, (size_t)B * (hd / 2) * sizeof(float2)));
    JUNO_TRY(dev_alloc((void **)&m->d_step, (size_t)4 * B * 4));
    JUNO_TRY(dev_alloc((void **)&m->d_argmax, (size_t)B * 4));
    JUNO_TRY(dev_alloc((void **)&m->d_pidx, (size_t)B * kArgmaxBlocks * 4));
    JUNO_TRY(dev_alloc((void **)&m->d_pval, (size_t)B * kArgmaxBlocks * 4));
    JUNO_TRY(dev_alloc((void **)&m->d_step_counter, 4));
    JUNO_CUDA_TRY(cudaMallocHost((void **)&m->h_step, (size_t)4 * B * 4));
    if (m->world > 1) JUNO_TRY(tp_push_setup(m));
    m->finalized = true;
    return JUNO_OK;
}

namespace juno {

// ───────────────────────────── one decode step, enqueued on the context stream ────────────
static int gemv_group(juno_model *m, juno_qmat *const *mats, float *const *outs, int count, const GemvArgs &proto,
                      cudaStream_t st) {
    // matrices that share the staged activation share a launch: one block format, or Q4_K mixed with Q6_K
    int i = 0;
    while (i < count) {
        int j = i + 1;
        bool mixed = false;
        while (j < count && j - i < 3) {
            const int ta = mats[i]->type, tb = mats[j]->type;
            const bool k_quant = m->mix_formats && (ta == 12 || ta == 14) && (tb == 12 || tb == 14);
            if (tb != ta && !k_quant) break;
            if (tb != mats[j - 1]->type || tb != ta) mixed = mixed || (tb != ta);
            j++;
        }
        GemvArgs a = proto;
        a.nseg = j - i;
        for (int s = 0; s < a.nseg; s++) {
            a.seg[s].w = mats[i + s]->dev;
            a.seg[s].out = outs[i + s];
            a.seg[s].rows = a.epi == EPI_SILU_PAIR ? (int)mats[i + s]->rows / 2 : (int)mats[i + s]->rows;
            a.seg[s].row_tiles = (int)mats[i + s]->row_tiles;
            a.seg[s].type = mats[i + s]->type;
        }
        a.type = mixed ? 0 : mats[i]->type;
        a.K = (int)mats[i]->cols;
        JUNO_TRY(launch_gemm(m->ctx, a, st));
        i = j;
    }
    return JUNO_OK;
}

// Layers and output projection of one step on the batched path (n >= gemm_min_batch()): every product is ONE pass
// over its weights for all n sequences (launch_gemm), with separate staging kernels in between (they need the
// whole row for its power-of-two factor).  x[0] holds the embeddings on entry; the residual stream ends in x[cur].
static int enqueue_layers_batched(juno_model *m, int n, const int32_t *d_slot, const int32_t *d_len, int n_splits, int &cur,
                                  cudaStream_t st, const int32_t *d_prefill_pos = nullptr, bool want_logits = true) {
    juno_ctx *c = m->ctx;
    const juno_model_cfg &f = m->cfg;
    const int H = f.hidden, hd = m->hd, B = f.max_batch;
    const int Hl = m->heads_loc * hd, KVl = m->kv_loc * hd, Il = m->inter_loc;
    float *sc_h = m->xsc, *sc_att = m->xsc + B, *sc_i = m->xsc + 2 * B;
    m->tc_used = true;
    auto stage = [&](int mode, const float *x, int ldx, const float *add, float *x_out, const float *normw, int K, uint8_t *img,
                     float *sc) {
        StageArgs a;
        a.mode = mode;
        a.x = x;
        a.ldx = ldx;
        a.x_add = add;
        a.x_out = x_out;
        a.normw = normw;
        a.eps = f.rms_eps;
        a.K = K;
        a.batch = n;
        a.img = img;
        return launch_stage_f16(c, a, sc, st, img == m->img_h ? m->img_h_tc : nullptr);
    };
    auto product = [&](juno_qmat *const *mats, float *const *outs, int count, int epi, int ld_out, const uint8_t *img,
                       const float *sc) {
        GemvArgs a;
        a.batch = n;
        a.ximg = img;
        a.xscale = sc;
        a.epi = epi;
        a.ld_out = ld_out;
        if (img == m->img_h) {
            a.ximg_tc = m->img_h_tc;
            a.tc_err = m->tc_err;
        }
        return gemv_group(m, mats, outs, count, a, st);
    };
    JUNO_TRY(stage(STAGE_RMSNORM, m->x[0], H, nullptr, nullptr, m->layers[0].attn_norm, H, m->img_h, sc_h));
    cur = 0;
    for (int l = 0; l < f.n_layers; l++) {
        JunoLayer &L = m->layers[l];
        juno_qmat *qkv_m[3] = {L.w[JUNO_T_ATTN_Q], L.w[JUNO_T_ATTN_K], L.w[JUNO_T_ATTN_V]};
        float *qkv_o[3] = {m->qkv, m->qkv + Hl, m->qkv + Hl + KVl};
        JUNO_TRY(product(qkv_m, qkv_o, 3, EPI_STORE, m->qkv_ld, m->img_h, sc_h));
        if (L.bqkv) {
            const int width = Hl + 2 * KVl;
            qkv_bias_kernel<<<dim3((width + 255) / 256, n), 256, 0, st>>>(m->qkv, L.bqkv, n, width, m->qkv_ld);
            JUNO_CUDA_TRY(cudaGetLastError());
            c->kernel_launches++;
        }
        AttnArgs at;
        at.pool = m->pool;
        at.layer = l;
        at.n = n;
        at.n_heads = m->heads_loc;
        at.q = m->qkv;
        at.ldq = m->qkv_ld;
        at.out = m->att;
        at.slots = d_slot;
        at.seq_lens = d_len;
        at.n_splits = n_splits;
        at.part_o = m->attn_scratch;
        at.part_ml = m->attn_scratch + (size_t)n * m->heads_loc * n_splits * hd;
        at.algo_bytes = m->step_kv_bytes;
        if (d_prefill_pos) {
            // chunked prefill: the n rows are consecutive positions of ONE sequence; their k, v are rotated and
            // appended first, so that every row finds the rows before it in the cache (causal by construction)
            JUNO_TRY(launch_rope_append(c, m->pool, l, n, m->heads_loc, m->qkv, m->qkv_ld, m->qkv + Hl, m->qkv + Hl + KVl, m->qkv_ld,
                                        d_slot, d_prefill_pos, m->rope_cs, st));
        } else {
            at.rope_cs = m->rope_cs;
            at.knew = m->qkv + Hl;
            at.vnew = m->qkv + Hl + KVl;
            at.ldkv = m->qkv_ld;
        }
        JUNO_TRY(launch_attn(c, at, st));
        JUNO_TRY(stage(STAGE_PLAIN, m->att, Hl, nullptr, nullptr, nullptr, Hl, m->img_att, sc_att));
        // x2 = x + Wo att (summed over ranks first when tensor parallel), staged rmsNorm(x2, ffn_norm)
        juno_qmat *wo[1] = {L.w[JUNO_T_ATTN_OUT]};
        float *po[1] = {m->proj};
        JUNO_TRY(product(wo, po, 1, EPI_STORE, H, m->img_att, sc_att));
        if (m->world > 1)
            JUNO_NCCL_TRY(g_nccl.AllReduce(m->proj, m->proj, (size_t)n * H, kNcclFloat, kNcclSum, m->comm, st));
        JUNO_TRY(stage(STAGE_RMSNORM, m->x[cur], H, m->proj, m->x[cur ^ 1], L.ffn_norm, H, m->img_h, sc_h));
        cur ^= 1;
        // hdn = silu(Wgate xn2) * (Wup xn2)
        juno_qmat *gu[1] = {L.w[JUNO_T_FFN_GATE]};
        float *pg[1] = {m->hdn};
        JUNO_TRY(product(gu, pg, 1, EPI_SILU_PAIR, Il, m->img_h, sc_h));
        JUNO_TRY(stage(STAGE_PLAIN, m->hdn, Il, nullptr, nullptr, nullptr, Il, m->img_i, sc_i));
        juno_qmat *wd[1] = {L.w[JUNO_T_FFN_DOWN]};
        JUNO_TRY(product(wd, po, 1, EPI_STORE, H, m->img_i, sc_i));
        if (m->world > 1)
            JUNO_NCCL_TRY(g_nccl.AllReduce(m->proj, m->proj, (size_t)n * H, kNcclFloat, kNcclSum, m->comm, st));
        const float *next_norm = (l + 1 < f.n_layers) ? m->layers[l + 1].attn_norm : m->output_norm;
        JUNO_TRY(stage(STAGE_RMSNORM, m->x[cur], H, m->proj, m->x[cur ^ 1], next_norm, H, m->img_h, sc_h));
        cur ^= 1;
    }
    if (!want_logits) return JUNO_OK;
    juno_qmat *lm[1] = {m->output};
    float *lo[1] = {m->logits_loc};
    return product(lm, lo, 1, EPI_STORE, m->vocab_loc, m->img_h, sc_h);
}

// ───────────────────────────── decode step on the integer-MMA GEMV (1..8 sequences) ───────
// Matrices that share an input share a launch: one block format, or Q4_K mixed with Q6_K.
static int q_group(juno_model *m, juno_qmat *const *mats, float *const *outs, int count, const QGemvArgs &proto, cudaStream_t st) {
    int i = 0;
    while (i < count) {
        int j = i + 1;
        while (j < count && j - i < 3) {
            const int ta = mats[i]->type, tb = mats[j]->type;
            const bool k_quant = m->mix_formats && (ta == 12 || ta == 14) && (tb == 12 || tb == 14);
            if (tb != ta && !k_quant) break;
            j++;
        }
        QGemvArgs a = proto;
        a.nseg = j - i;
        for (int s = 0; s < a.nseg; s++) {
            a.seg[s].w = mats[i + s]->dev;
            a.seg[s].out = outs[i + s];
            a.seg[s].rows = a.epi == QEPI_SILU_PAIR ? (int)mats[i + s]->rows / 2 : (int)mats[i + s]->rows;
            a.seg[s].row_tiles = (int)mats[i + s]->row_tiles;
            a.seg[s].type = mats[i + s]->type;
        }
        a.K = (int)mats[i]->cols;
        JUNO_TRY(launch_qgemv(m->ctx, a, st));
        i = j;
    }
    return JUNO_OK;
}

// Layers and output projection for n <= 8 sequences.  x[0] holds the embeddings on entry.  Activations travel between
// the kernels as plain FP32 rows; the residual additions (x + Wo att, x + Wdown hdn) and the RMSNorms are done by the
// CONSUMING product while it builds its operand, which also writes the new residual row once (x_store).  Under tensor
// parallelism the row-parallel products are all-reduced before their consumer reads them.
static int enqueue_layers_q(juno_model *m, int n, const int32_t *d_slot, const int32_t *d_len, int n_splits, int &cur, cudaStream_t st) {
    juno_ctx *c = m->ctx;
    const juno_model_cfg &f = m->cfg;
    const int H = f.hidden, hd = m->hd, W = m->world;
    const int Hl = m->heads_loc * hd, KVl = m->kv_loc * hd, Il = m->inter_loc;
    cur = 0;
    // Tensor parallel, up to tp_bq sequences that fit one launch of both row-parallel products: the partial products
    // are PUSHED into every rank's inbox by the producing kernel itself (8-byte (value, step number) stores over
    // NVLink into peer-mapped memory), and the consuming kernel polls the pairs it needs and adds the partials in
    // rank order.  No collective call, no extra launch, no fence or flag.  Otherwise: NCCL all-reduce between producer and consumer.
    const bool push = m->tp_push && n <= m->tp_bq && qgemv_batch_chunk(c, Hl, m->layers[0].w[JUNO_T_ATTN_OUT]->type, n) >= n &&
                      qgemv_batch_chunk(c, Il, m->layers[0].w[JUNO_T_FFN_DOWN]->type, n) >= n;
    int pend_inst = -1;           // exchange instance of the pending row-parallel product (push mode)
    const float *pend = nullptr;  // row-parallel product not yet added to the residual stream (NCCL mode / one GPU)
    auto inbox = [&](int rank_of_buf, int inst, int src) {
        return reinterpret_cast<float *>(m->tp_peer[rank_of_buf] + m->tp_inbox_off) + ((size_t)inst * W + src) * m->tp_bq * H * 2;
    };
    auto from_residual = [&](QGemvArgs &a, const float *normw) {
        a.batch = n;
        a.x = m->x[cur];
        a.ldx = H;
        a.normw = normw;
        a.eps = f.rms_eps;
        if (pend_inst >= 0 && m->tp_reduce) {
            a.red_dst = m->tp_red + (size_t)pend_inst * m->tp_bq * H * 2;
            for (int k = 0; k < W; k++) a.red_src[k] = inbox(m->rank, pend_inst, k);
            a.n_red = W;
            a.add[0] = a.red_dst;
            a.n_add = 1;
            a.tagged_adds = true;
            a.epoch = m->tp_epoch;
            a.peer_failed = m->tp_failed;
            a.x_store = m->x[cur ^ 1];
        } else if (pend_inst >= 0) {
            for (int k = 0; k < W; k++) a.add[k] = inbox(m->rank, pend_inst, k);
            a.n_add = W;
            a.tagged_adds = true;
            a.epoch = m->tp_epoch;
            a.peer_failed = m->tp_failed;
            a.x_store = m->x[cur ^ 1];
        } else if (pend) {
            a.add[0] = pend;
            a.n_add = 1;
            a.x_store = m->x[cur ^ 1];
        }
    };
    auto row_parallel = [&](juno_qmat *w, const float *x, int K, float *out, int inst) -> int {
        QGemvArgs a;
        a.batch = n;
        a.x = x;
        a.ldx = K;
        a.ld_out = H;
        if (push) {
            a.n_peers = W;
            for (int d = 0; d < W; d++) a.peer_out[d] = inbox(d, inst, m->rank);
            a.epoch = m->tp_epoch;
        }
        juno_qmat *ws[1] = {w};
        float *os[1] = {out};
        JUNO_TRY(q_group(m, ws, os, 1, a, st));
        if (push) {
            pend_inst = inst;
            pend = nullptr;
        } else {
            if (W > 1) JUNO_NCCL_TRY(g_nccl.AllReduce(out, out, (size_t)n * H, kNcclFloat, kNcclSum, m->comm, st));
            pend = out;
        }
        return JUNO_OK;
    };
    for (int l = 0; l < f.n_layers; l++) {
        JunoLayer &L = m->layers[l];
        {   // q, k, v = W rmsNorm(x)
            QGemvArgs a;
            from_residual(a, L.attn_norm);
            a.ld_out = m->qkv_ld;
            juno_qmat *qkv_m[3] = {L.w[JUNO_T_ATTN_Q], L.w[JUNO_T_ATTN_K], L.w[JUNO_T_ATTN_V]};
            float *qkv_o[3] = {m->qkv, m->qkv + Hl, m->qkv + Hl + KVl};
            JUNO_TRY(q_group(m, qkv_m, qkv_o, 3, a, st));
            if (L.bqkv) {
                const int width = Hl + 2 * KVl;
                qkv_bias_kernel<<<dim3((width + 255) / 256, n), 256, 0, st>>>(m->qkv, L.bqkv, n, width, m->qkv_ld);
                JUNO_CUDA_TRY(cudaGetLastError());
                c->kernel_launches++;
            }
            if (pend || pend_inst >= 0) cur ^= 1;
            pend = nullptr;
            pend_inst = -1;
        }
        AttnArgs at;
        at.pool = m->pool;
        at.layer = l;
        at.n = n;
        at.n_heads = m->heads_loc;
        at.q = m->qkv;
        at.ldq = m->qkv_ld;
        at.out = m->att;
        at.slots = d_slot;
        at.seq_lens = d_len;
        at.n_splits = n_splits;
        at.part_o = m->attn_scratch;
        at.part_ml = m->attn_scratch + (size_t)n * m->heads_loc * n_splits * hd;
        at.algo_bytes = m->step_kv_bytes;
        at.rope_cs = m->rope_cs;  // q, k are rotated and k, v appended inside the attention kernel
        at.knew = m->qkv + Hl;
        at.vnew = m->qkv + Hl + KVl;
        at.ldkv = m->qkv_ld;
        JUNO_TRY(launch_attn(c, at, st));
        // proj = Wo att (this rank's heads)
        JUNO_TRY(row_parallel(L.w[JUNO_T_ATTN_OUT], m->att, Hl, m->proj, 2 * l));
        {   // hdn = silu(Wgate xn2) * (Wup xn2), xn2 = rmsNorm(x + proj)
            QGemvArgs a;
            from_residual(a, L.ffn_norm);
            a.epi = QEPI_SILU_PAIR;
            a.ld_out = Il;
            juno_qmat *gu[1] = {L.w[JUNO_T_FFN_GATE]};
            float *go[1] = {m->hdn};
            JUNO_TRY(q_group(m, gu, go, 1, a, st));
            cur ^= 1;
            pend = nullptr;
            pend_inst = -1;
        }
        // proj2 = Wdown hdn (this rank's FFN rows)
        JUNO_TRY(row_parallel(L.w[JUNO_T_FFN_DOWN], m->hdn, Il, m->proj2, 2 * l + 1));
    }
    // logits = Wout rmsNorm(x + proj2)
    QGemvArgs a;
    from_residual(a, m->output_norm);
    a.ld_out = m->vocab_loc;
    juno_qmat *lm[1] = {m->output};
    float *lo[1] = {m->logits_loc};
    JUNO_TRY(q_group(m, lm, lo, 1, a, st));
    if (pend || pend_inst >= 0) cur ^= 1;
    return JUNO_OK;
}

static int enqueue_step(juno_model *m, int n, int n_splits, bool greedy_advance, bool want_logits, cudaStream_t st) {
    juno_ctx *c = m->ctx;
    const juno_model_cfg &f = m->cfg;
    const int H = f.hidden, hd = m->hd, B = f.max_batch;
    const int32_t *d_tok = m->d_step, *d_pos = m->d_step + B, *d_slot = m->d_step + 2 * B, *d_len = m->d_step + 3 * B;
    if (m->tp_push) {
        epoch_kernel<<<1, 1, 0, st>>>(m->tp_epoch);
        JUNO_CUDA_TRY(cudaGetLastError());
        c->kernel_launches++;
    }
    // embedding lookup -> x[0]
    {
        juno_qmat *e = m->tok_embd;
        dim3 grid((H + 255) / 256, n);
        int64_t rb = e->tiled ? 0 : e->cols / raw_block_elems(e->type) * raw_block_bytes(e->type);
        embed_kernel<<<grid, 256, 0, st>>>(e->type, e->tiled, e->dev, e->nb, rb, H, f.vocab, d_tok, m->x[0]);
        JUNO_CUDA_TRY(cudaGetLastError());
        c->kernel_launches++;
    }
    JUNO_TRY(launch_rope_table(c, d_pos, n, hd, f.rope_theta, m->rope_cs, st));
    int cur = 0;          // x[cur] holds the residual stream
    // 9..64 sequences: one pass over the weights per product on the FP16 tensor-core kernels; otherwise the exact
    // integer-MMA GEMV (batches above 64 in chunks of up to eight sequences per pass)
    const bool batched = n >= m->batched_from && n <= kGemmMaxBatch;
    if (batched)
        JUNO_TRY(enqueue_layers_batched(m, n, d_slot, d_len, n_splits, cur, st));
    else
        JUNO_TRY(enqueue_layers_q(m, n, d_slot, d_len, n_splits, cur, st));
    m->last_x = cur;
    LogitsView lv;
    lv.n = n;
    lv.vocab = f.vocab;
    // Sharded vocabulary: when the caller wants the logits they are gathered (NCCL); when only the greedy pick is
    // wanted and the ranks exchange through peer memory, (value, index) pairs travel instead and the step holds no
    // collective call at all.
    const bool pair_pick = m->vocab_sharded && m->tp_push && !want_logits && n <= 8;
    if (pair_pick) {
        lv.base = m->logits_loc;
        lv.vocab = m->vocab_loc;
        lv.vloc = m->vocab_loc;
        argmax_partial_kernel<<<dim3(kArgmaxBlocks, n), 256, 0, st>>>(lv, m->d_pval, m->d_pidx);
        PairXchg x;
        x.world = m->world;
        for (int d = 0; d < m->world; d++) {
            x.slot[d] = reinterpret_cast<float2 *>(m->tp_peer[d] + m->tp_pair_off) + m->rank * 8;
            x.flag[d] = reinterpret_cast<unsigned *>(m->tp_peer[d]) + m->rank;
        }
        argmax_push_kernel<<<1, 32, 0, st>>>(m->d_pval, m->d_pidx, n, m->rank * m->vocab_loc, x, m->tp_epoch);
        argmax_merge_kernel<<<1, 32, 0, st>>>(reinterpret_cast<const float2 *>(m->tp_buf + m->tp_pair_off), 8,
                                             reinterpret_cast<const unsigned *>(m->tp_buf), m->world, n, m->tp_epoch,
                                             m->d_argmax, c->gemv_scratch.qerr, m->tp_failed);
        JUNO_CUDA_TRY(cudaGetLastError());
        c->kernel_launches += 3;
    } else {
        if (m->vocab_sharded) {
            JUNO_NCCL_TRY(g_nccl.AllGather(m->logits_loc, m->logits_gather, (size_t)n * m->vocab_loc, kNcclFloat, m->comm, st));
            lv.base = m->logits_gather;
            lv.vloc = m->vocab_loc;
        } else {
            lv.base = m->logits_loc;
            lv.vloc = f.vocab;
        }
        argmax_partial_kernel<<<dim3(kArgmaxBlocks, n), 256, 0, st>>>(lv, m->d_pval, m->d_pidx);
        argmax_final_kernel<<<(n + 63) / 64, 64, 0, st>>>(m->d_pval, m->d_pidx, n, m->d_argmax);
        JUNO_CUDA_TRY(cudaGetLastError());
        c->kernel_launches += 2;
    }
    if (greedy_advance) {
        advance_kernel<<<1, std::max(32, (n + 31) / 32 * 32), 0, st>>>(n, m->d_argmax, m->d_step, m->d_step + B,
                                                                      m->d_step + 3 * B, m->d_out_ids, m->d_step_counter);
        JUNO_CUDA_TRY(cudaGetLastError());
        c->kernel_launches++;
    }
    return JUNO_OK;
}

// Runs one step: the first call for a (n, splits, mode) key runs eagerly (it also sizes every scratch
// buffer); the second captures the same launches into a CUDA graph, later ones replay it.
static int run_step(juno_model *m, int n, int n_splits, bool greedy_advance, bool want_logits) {
    juno_ctx *c = m->ctx;
    cudaStream_t st = c->stream;
    if (m->comm_failed) {
        set_error("the tensor-parallel communicator was aborted after a failed step: free the model and build a new group");
        return JUNO_ERR_NCCL;
    }
    if (!m->use_graphs || c->profiling) return enqueue_step(m, n, n_splits, greedy_advance, want_logits, st);
    const uint64_t key = ((uint64_t)n << 32) | ((uint64_t)n_splits << 2) | (want_logits ? 2u : 0u) | (greedy_advance ? 1u : 0u);
    JunoGraph &g = m->graphs[key];
    if (g.exec) {
        JUNO_CUDA_TRY(cudaGraphLaunch(g.exec, st));
        c->kernel_launches += g.launches;
        return JUNO_OK;
    }
    if (!g.seen) {
        g.seen = 1;
        return enqueue_step(m, n, n_splits, greedy_advance, want_logits, st);
    }
    const int64_t before = c->kernel_launches.load();
    JUNO_CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_step(m, n, n_splits, greedy_advance, want_logits, st);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(st, &graph);
    const int launches = (int)(c->kernel_launches.load() - before);
    c->kernel_launches = before;
    if (rc != JUNO_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (e != cudaSuccess || !graph) {
        set_error("graph capture failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return JUNO_ERR_CUDA;
    }
    e = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        g.exec = nullptr;
        set_error("cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
        return JUNO_ERR_CUDA;
    }
    g.launches = launches;
    JUNO_CUDA_TRY(cudaGraphLaunch(g.exec, st));
    c->kernel_launches += launches;
    return JUNO_OK;
}

// Waits for the step to drain.  A tensor-parallel step can hold NCCL collectives (more than eight sequences, gathered
// logits, the NCCL exchange mode): if a rank has died they never complete and a plain stream synchronise would block
// for ever.  So with a communicator the wait polls the stream together with the communicator's asynchronous error
// state and a deadline (JUNO_NCCL_TIMEOUT_S seconds, default 60); on either it aborts the communicator, which ends
// the collective kernels in flight, and the model refuses further steps.
static int step_sync(juno_model *m) {
    juno_ctx *c = m->ctx;
    if (m->world <= 1 || !m->comm) {
        JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
        return JUNO_OK;
    }
    static const double limit_s = [] {
        const char *e = getenv("JUNO_NCCL_TIMEOUT_S");
        const double v = (e && *e) ? atof(e) : 60.0;
        return v > 0 ? v : 60.0;
    }();
    const auto t0 = std::chrono::steady_clock::now();
    const char *why = nullptr;
    int async = 0;
    for (unsigned spin = 0;; spin++) {
        const cudaError_t e = cudaStreamQuery(c->stream);
        if (e == cudaSuccess) return JUNO_OK;
        if (e != cudaErrorNotReady) JUNO_CUDA_TRY(e);
        if ((spin & 63) == 63) {
            if (g_nccl.CommGetAsyncError && g_nccl.CommGetAsyncError(m->comm, &async) == 0 && async != 0 && async != 7 /* in progress */) {
                why = "NCCL reported an asynchronous error";
                break;
            }
            if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit_s) {
                why = "a collective did not complete before the deadline (a rank may have failed)";
                break;
            }
        }
        if (spin > 20000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    m->comm_failed = true;
    // The captured step graphs hold references on the communicator's plans, and the abort waits for them: mark the
    // graphs for destruction first (it happens when their run ends).  The abort itself sets the flag that ends the
    // collective kernels in flight; it runs on a helper thread, so that this call returns even if the teardown
    // inside the library waits for something that never comes.
    for (auto &kv : m->graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    m->graphs.clear();
    if (g_nccl.CommAbort) {
        NcclComm comm = m->comm;
        m->comm = nullptr;
        auto aborted = std::make_shared<std::atomic<bool>>(false);
        std::thread([comm, aborted] {
            g_nccl.CommAbort(comm);
            aborted->store(true);
        }).detach();
        const auto t1 = std::chrono::steady_clock::now();
        while (std::chrono::duration<double>(std::chrono::steady_clock::now() - t1).count() < 10.0) {
            if (aborted->load() && cudaStreamQuery(c->stream) != cudaErrorNotReady) break;
            std::this_thread::sleep_for(std::chrono::milliseconds(1));
        }
    }
    set_error("tensor-parallel step abandoned: %s (async state %d, limit %.0f s); the communicator was aborted", why, async, limit_s);
    return async != 0 && async != 7 ? JUNO_ERR_NCCL : JUNO_ERR_TIMEOUT;
}

// After the step has drained: did one of its kernels give up on a wait?
static int step_check(juno_model *m) {
    if (m->tc_err && m->tc_used) {
        m->tc_used = false;
        unsigned code = 0;
        if (cudaMemcpy(&code, m->tc_err, 4, cudaMemcpyDeviceToHost) == cudaSuccess && code) {
            cudaMemset(m->tc_err, 0, 4);
            set_error("batched tensor-core product gave up waiting (code %u, block %u)", code & 0xffu, code >> 8);
            return JUNO_ERR_CUDA;
        }
    }
    juno_ctx *c = m->ctx;
    const unsigned code = c->gemv_scratch.qerr_host ? *reinterpret_cast<volatile unsigned *>(c->gemv_scratch.qerr_host) : 0u;
    if (code) {
        *reinterpret_cast<volatile unsigned *>(c->gemv_scratch.qerr_host) = 0u;
        if (m->tp_failed) cudaMemset(m->tp_failed, 0, 4);
        if ((code & 0xffu) >= 3u)
            set_error("tensor-parallel rank %u did not deliver its %s within a second (this rank gave up waiting)", (code >> 8) & 0xffu,
                      (code & 0xffu) == 3u ? "partial products" : "greedy pick");
        else
            set_error("a GEMV warp gave up waiting for a weight tile (warp %u of block %u)", (code >> 8) & 0xffu, code >> 16);
        return JUNO_ERR_TIMEOUT;
    }
    return JUNO_OK;
}

static int bucket_len(int len) {
    int b = 64;
    while (b < len) b <<= 1;
    return b;
}

// Validates the step, reserves pages and ships (tokens, positions, slots, lengths) to the device.
static int prepare_step(juno_model *m, int n, juno_seq *const *seqs, const int32_t *tokens, const int32_t *positions,
                        int extra_positions, int *n_splits) {
    juno_ctx *c = m->ctx;
    const int B = m->cfg.max_batch;
    JUNO_REQUIRE(m->finalized, "model is not finalized");
    JUNO_REQUIRE(n >= 1 && n <= B, "n=%d outside [1, max_batch=%d]", n, B);
    JUNO_REQUIRE(seqs && tokens && positions, "null argument");
    int max_len = 0;
    for (int i = 0; i < n; i++) {
        juno_seq *s = seqs[i];
        JUNO_REQUIRE(s && s->magic == kMagicSeq && s->pool == m->pool, "sequence %d is closed or belongs to another model", i);
        for (int j = 0; j < i; j++) JUNO_REQUIRE(seqs[j] != s, "sequence listed twice in one step");
        JUNO_REQUIRE(positions[i] >= 0 && positions[i] + extra_positions < m->cfg.max_ctx,
                     "position %d is beyond max_ctx %d", positions[i] + extra_positions, m->cfg.max_ctx);
        // a position beyond the sequence's length would make attention read cache rows that were never written
        // (pages come back from the free list as they were left)
        JUNO_REQUIRE(positions[i] <= s->len, "sequence %d: position %d leaves a gap after its %d cached positions", i, positions[i], s->len);
        JUNO_TRY(seq_reserve(s, positions[i], positions[i] + 1 + extra_positions, c->stream));
        m->h_step[i] = tokens[i];
        m->h_step[B + i] = positions[i];
        m->h_step[2 * B + i] = s->slot;
        m->h_step[3 * B + i] = positions[i] + 1;
        max_len = std::max(max_len, positions[i] + 1 + extra_positions);
    }
    m->step_kv_bytes = 0;
    for (int i = 0; i < n; i++)
        m->step_kv_bytes += (double)(positions[i] + 1) * m->kv_loc * m->hd * 2 * m->pool->elem_bytes;
    *n_splits = attn_pick_splits(c, n, m->kv_loc, bucket_len(max_len));
    JUNO_CUDA_TRY(cudaMemcpyAsync(m->d_step, m->h_step, (size_t)4 * B * 4, cudaMemcpyHostToDevice, c->stream));
    c->h2d_bytes += 4 * n * 4;
    return JUNO_OK;
}

}  // namespace juno

extern "C" {

int juno_model_seq_create(juno_model *m, juno_seq **out) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(out, "out is null");
    JUNO_REQUIRE(m->finalized, "model is not finalized");
    std::lock_guard<std::recursive_mutex> lk(m->ctx->mu);
    return seq_create(m->pool, m->cfg.max_ctx, out);
}

int juno_forward(juno_model *m, int32_t n, juno_seq *const *seqs, const int32_t *token_ids, const int32_t *positions,
                 float *logits_host, int32_t *argmax_out) {
    JUNO_TRY(model_check(m));
    juno_ctx *c = m->ctx;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    // the pinned step buffer is reused: the previous step must have consumed it
    JUNO_TRY(step_sync(m));
    int n_splits = 1;
    JUNO_TRY(prepare_step(m, n, seqs, token_ids, positions, 0, &n_splits));
    JUNO_TRY(run_step(m, n, n_splits, false, logits_host != nullptr));
    // With collectives in the step the guarded wait comes first: a device-to-host copy into pageable memory blocks
    // the caller until the stream reaches it, and would sit behind a collective that never completes.
    if (m->world > 1) JUNO_TRY(step_sync(m));
    c->forward_calls++;
    const int V = m->cfg.vocab;
    if (logits_host) {
        const float *src = m->logits_loc;
        if (m->vocab_sharded) {
            LogitsView lv{m->logits_gather, n, V, m->vocab_loc};
            size_t tot = (size_t)n * V;
            ungather_logits_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, c->stream>>>(lv, m->logits_full);
            JUNO_CUDA_TRY(cudaGetLastError());
            c->kernel_launches++;
            src = m->logits_full;
        }
        JUNO_CUDA_TRY(cudaMemcpyAsync(logits_host, src, (size_t)n * V * 4, cudaMemcpyDeviceToHost, c->stream));
        c->d2h_bytes += (int64_t)n * V * 4;
    }
    if (argmax_out) {
        JUNO_CUDA_TRY(cudaMemcpyAsync(argmax_out, m->d_argmax, (size_t)n * 4, cudaMemcpyDeviceToHost, c->stream));
        c->d2h_bytes += n * 4;
    }
    JUNO_TRY(step_sync(m));
    JUNO_TRY(step_check(m));
    for (int i = 0; i < n; i++) seqs[i]->len = std::max(seqs[i]->len, positions[i] + 1);
    m->last_n = n;
    return JUNO_OK;
}

int juno_prefill(juno_model *m, juno_seq *seq, const int32_t *token_ids, int32_t n_tokens, int32_t start_pos,
                 float *logits_host, int32_t *argmax_out) {
    JUNO_TRY(model_check(m));
    juno_ctx *c = m->ctx;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_REQUIRE(m->finalized, "model is not finalized");
    JUNO_REQUIRE(seq && seq->magic == kMagicSeq && seq->pool == m->pool, "sequence is closed or belongs to another model");
    JUNO_REQUIRE(token_ids && n_tokens >= 1 && start_pos >= 0, "bad prefill arguments (n_tokens=%d, start_pos=%d)", n_tokens, start_pos);
    JUNO_REQUIRE(start_pos + n_tokens <= m->cfg.max_ctx, "position %d is beyond max_ctx %d", start_pos + n_tokens - 1, m->cfg.max_ctx);
    JUNO_REQUIRE(start_pos <= seq->len, "start position %d leaves a gap after the %d cached positions", start_pos, seq->len);
    JUNO_REQUIRE(m->pool->dtype == 0 || m->pool->dtype == 1, "unsupported KV type");
    const juno_model_cfg &f = m->cfg;
    const int B = f.max_batch, chunk_max = std::min(B, kGemmMaxBatch), V = f.vocab;
    cudaStream_t st = c->stream;
    for (int done = 0; done < n_tokens;) {
        const int n = std::min(chunk_max, n_tokens - done), pos0 = start_pos + done;
        const bool last = done + n == n_tokens;
        JUNO_TRY(step_sync(m));  // the pinned step buffer is reused
        JUNO_TRY(seq_reserve(seq, pos0, pos0 + n, st));
        for (int i = 0; i < n; i++) {
            m->h_step[i] = token_ids[done + i];
            m->h_step[B + i] = pos0 + i;
            m->h_step[2 * B + i] = seq->slot;
            m->h_step[3 * B + i] = pos0 + i + 1;
        }
        JUNO_CUDA_TRY(cudaMemcpyAsync(m->d_step, m->h_step, (size_t)4 * B * 4, cudaMemcpyHostToDevice, st));
        c->h2d_bytes += 4 * n * 4;
        m->step_kv_bytes = 0;
        for (int i = 0; i < n; i++) m->step_kv_bytes += (double)(pos0 + i + 1) * m->kv_loc * m->hd * 2 * m->pool->elem_bytes;
        const int n_splits = attn_pick_splits(c, n, m->kv_loc, bucket_len(pos0 + n));
        const int32_t *d_tok = m->d_step, *d_pos = m->d_step + B, *d_slot = m->d_step + 2 * B, *d_len = m->d_step + 3 * B;
        {
            juno_qmat *e = m->tok_embd;
            dim3 grid((f.hidden + 255) / 256, n);
            int64_t rb = e->tiled ? 0 : e->cols / raw_block_elems(e->type) * raw_block_bytes(e->type);
            embed_kernel<<<grid, 256, 0, st>>>(e->type, e->tiled, e->dev, e->nb, rb, f.hidden, V, d_tok, m->x[0]);
            JUNO_CUDA_TRY(cudaGetLastError());
            c->kernel_launches++;
        }
        JUNO_TRY(launch_rope_table(c, d_pos, n, m->hd, f.rope_theta, m->rope_cs, st));
        int cur = 0;
        JUNO_TRY(enqueue_layers_batched(m, n, d_slot, d_len, n_splits, cur, st, d_pos, last && (logits_host || argmax_out)));
        m->last_x = cur;
        m->last_n = n;
        c->forward_calls++;
        if (last && (logits_host || argmax_out)) {
            // row n-1 is the last prompt position
            const float *row = m->logits_loc + (size_t)(n - 1) * m->vocab_loc;
            JUNO_REQUIRE(!m->vocab_sharded, "prefill logits are not implemented for a sharded vocabulary");
            if (argmax_out) {
                LogitsView lv;
                lv.n = 1;
                lv.vocab = V;
                lv.base = row;
                lv.vloc = V;
                argmax_partial_kernel<<<dim3(kArgmaxBlocks, 1), 256, 0, st>>>(lv, m->d_pval, m->d_pidx);
                argmax_final_kernel<<<1, 64, 0, st>>>(m->d_pval, m->d_pidx, 1, m->d_argmax);
                JUNO_CUDA_TRY(cudaGetLastError());
                c->kernel_launches += 2;
                JUNO_CUDA_TRY(cudaMemcpyAsync(argmax_out, m->d_argmax, 4, cudaMemcpyDeviceToHost, st));
                c->d2h_bytes += 4;
            }
            if (logits_host) {
                JUNO_CUDA_TRY(cudaMemcpyAsync(logits_host, row, (size_t)V * 4, cudaMemcpyDeviceToHost, st));
                c->d2h_bytes += (int64_t)V * 4;
            }
        }
        done += n;
    }
    JUNO_TRY(step_sync(m));
    JUNO_TRY(step_check(m));
    seq->len = std::max(seq->len, start_pos + n_tokens);
    return JUNO_OK;
}

int juno_decode_greedy(juno_model *m, int32_t n, juno_seq *const *seqs, const int32_t *first_tokens,
                       const int32_t *positions, int32_t steps, int32_t *out_ids) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(steps >= 1 && steps <= 65536 && out_ids, "bad steps/out_ids");
    juno_ctx *c = m->ctx;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    int n_splits = 1;
    JUNO_TRY(prepare_step(m, n, seqs, first_tokens, positions, steps - 1, &n_splits));
    const int need = steps * m->cfg.max_batch;
    if (need > m->out_ids_cap) {
        if (m->d_out_ids) cudaFree(m->d_out_ids);
        m->d_out_ids = nullptr;
        m->out_ids_cap = 0;
        JUNO_TRY(dev_alloc((void **)&m->d_out_ids, (size_t)need * 4));
        m->out_ids_cap = need;
        // the buffer address is baked into captured graphs of the greedy mode
        for (auto it = m->graphs.begin(); it != m->graphs.end();) {
            if (it->first & 1u) {
                if (it->second.exec) cudaGraphExecDestroy(it->second.exec);
                it = m->graphs.erase(it);
            } else
                ++it;
        }
    }
    JUNO_CUDA_TRY(cudaMemsetAsync(m->d_step_counter, 0, 4, c->stream));
    for (int s = 0; s < steps; s++) JUNO_TRY(run_step(m, n, n_splits, true, false));
    if (m->world > 1) JUNO_TRY(step_sync(m));  // before the copy of the ids, see juno_forward
    c->forward_calls += steps;
    JUNO_CUDA_TRY(cudaMemcpyAsync(out_ids, m->d_out_ids, (size_t)steps * n * 4, cudaMemcpyDeviceToHost, c->stream));
    JUNO_TRY(step_sync(m));
    JUNO_TRY(step_check(m));
    c->d2h_bytes += (int64_t)steps * n * 4;
    for (int i = 0; i < n; i++) seqs[i]->len = std::max(seqs[i]->len, positions[i] + steps);
    m->last_n = n;
    return JUNO_OK;
}

int juno_model_last_hidden(juno_model *m, int32_t n, float *hidden_host) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(hidden_host && n >= 1 && n <= m->last_n, "no forward result for %d sequences", n);
    juno_ctx *c = m->ctx;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_CUDA_TRY(cudaMemcpyAsync(hidden_host, m->x[m->last_x], (size_t)n * m->cfg.hidden * 4, cudaMemcpyDeviceToHost,
                                  c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return JUNO_OK;
}

// Every tensor the reference constructor reads (LlamaTransformerHandler.java:238-275), by its GGUF name, straight from
// the mapped file.  GGUF dims are [cols (in), rows (out)] (GgufReader.java:246-248).
int juno_model_load_gguf(juno_model *m, juno_gguf *g) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(!m->finalized, "model is already finalized");
    const juno_model_cfg &f = m->cfg;
    auto put = [&](const std::string &name, int kind, int layer, bool optional) -> int {
        int32_t present = 0;
        JUNO_TRY(juno_gguf_has_tensor(g, name.c_str(), &present));
        if (!present && optional) return JUNO_OK;
        int32_t type = 0, nd = 0;
        int64_t dims[4] = {1, 1, 1, 1}, nbytes = 0;
        const void *data = nullptr;
        JUNO_TRY(juno_gguf_tensor(g, name.c_str(), &type, &nd, dims, &data, &nbytes));
        JUNO_REQUIRE(nd >= 1 && nd <= 2, "tensor %s has %d dimensions, expected 1 or 2", name.c_str(), nd);
        const int64_t cols = dims[0], rows = nd == 2 ? dims[1] : 1;
        return juno_model_set_tensor(m, kind, layer, data, type, rows, cols);
    };
    int32_t has_bias = 0;  // the reference decides by the first layer's attn_q.bias (:258-262)
    JUNO_TRY(juno_gguf_has_tensor(g, "blk.0.attn_q.bias", &has_bias));
    JUNO_TRY(put("token_embd.weight", JUNO_T_TOKEN_EMBD, 0, false));
    JUNO_TRY(put("output_norm.weight", JUNO_T_OUTPUT_NORM, 0, false));
    JUNO_TRY(put("output.weight", JUNO_T_OUTPUT, 0, true));  // absent: tied to token_embd (:463-470)
    static const struct { const char *suffix; int kind; } per_layer[] = {
        {"attn_norm", JUNO_T_ATTN_NORM}, {"ffn_norm", JUNO_T_FFN_NORM}, {"attn_q", JUNO_T_ATTN_Q},   {"attn_k", JUNO_T_ATTN_K},
        {"attn_v", JUNO_T_ATTN_V},       {"attn_output", JUNO_T_ATTN_OUT}, {"ffn_gate", JUNO_T_FFN_GATE}, {"ffn_up", JUNO_T_FFN_UP},
        {"ffn_down", JUNO_T_FFN_DOWN}};
    for (int l = 0; l < f.n_layers; l++) {
        for (const auto &t : per_layer) JUNO_TRY(put("blk." + std::to_string(l) + "." + t.suffix + ".weight", t.kind, l, false));
        if (has_bias) {
            JUNO_TRY(put("blk." + std::to_string(l) + ".attn_q.bias", JUNO_T_ATTN_Q_BIAS, l, false));
            JUNO_TRY(put("blk." + std::to_string(l) + ".attn_k.bias", JUNO_T_ATTN_K_BIAS, l, false));
            JUNO_TRY(put("blk." + std::to_string(l) + ".attn_v.bias", JUNO_T_ATTN_V_BIAS, l, false));
        }
    }
    return JUNO_OK;
}

int juno_model_tp_mode(juno_model *m, int32_t *mode) {
    JUNO_TRY(model_check(m));
    JUNO_REQUIRE(mode, "mode is null");
    *mode = m->world <= 1 ? 0 : (m->tp_push ? 2 : 1);
    return JUNO_OK;
}

int juno_model_free(juno_model *m) {
    JUNO_TRY(model_check(m));
    std::lock_guard<std::recursive_mutex> lk(m->ctx->mu);
    model_release(m);
    return JUNO_OK;
}

}  // extern "C"
