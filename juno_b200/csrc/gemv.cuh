// Resident quantised matrices and the device-level interface of the batched (9..64 sequences) dequant-GEMM:
// used by the MatVec entry points and by the forward pass.  The 1..8 sequence GEMV is declared in qgemv.cuh.
#pragma once
#include "common.cuh"

struct juno_qmat {
    uint32_t magic;
    juno_ctx *ctx;
    int type;          // GGML type id
    int tiled;         // 1: 16x256 tile layout (layout.cuh); 0: raw row-major blocks
    int64_t rows, cols;
    int64_t row_tiles; // ceil(rows/16) when tiled
    int64_t nb;        // cols/256 when tiled
    uint8_t *dev;
    size_t bytes;
};

namespace juno {

enum StageMode {
    STAGE_PLAIN = 0,    // v = x[i]
    STAGE_RMSNORM = 1,  // r = x[i] (+ x_add[i]); optional store of r to x_out; v = (normw[i]*r)*scale  (rmsNorm :818-828)
};

// Input of a staging kernel of the batched path (launch_stage_f16).
struct StageArgs {
    int mode = STAGE_PLAIN;
    const float *x = nullptr;  // [batch][ldx]
    int ldx = 0;
    const float *x_add = nullptr, *normw = nullptr;
    float *x_out = nullptr;
    float eps = 0.f;
    int K = 0, batch = 1;
    uint8_t *img = nullptr;    // at least gemm_image_bytes(K, batch)
};

enum GemvEpilogue {
    EPI_STORE = 0,       // out[b][row] = y
    EPI_SILU_PAIR = 1,   // tile rows 0-7 are gate rows, 8-15 the matching up rows: out[b][8*tile+row] = silu(gate)*up
    EPI_RESID_NORM = 2,  // x_out = resid + y
};

struct GemvSeg {
    const uint8_t *w; // tiled weights
    float *out;       // [batch][ld_out]
    int rows;         // valid rows
    int row_tiles;
    int type = 0;     // block format of this segment; 0 = GemvArgs.type
};

struct GemvArgs {
    GemvSeg seg[3];
    int nseg = 1;
    int type = 0;     // 12 / 14 / 8
    int K = 0;
    int batch = 1;
    int ld_out = 0;   // stride between batch rows of every seg.out
    int epi = EPI_STORE;
    const uint8_t *ximg = nullptr;  // FP16 staged activation (launch_stage_f16) for this K and batch
    // EPI_RESID_NORM
    const float *resid = nullptr;
    float *x_out = nullptr;
    int ldx = 0;
    // batched path (launch_gemm): ximg is an FP16 image (launch_stage_f16) and xscale its per-row factors
    const float *xscale = nullptr;
    // optional: the same activation in the chunk-major layout of the tcgen05 kernel, and the device word that kernel
    // reports a given-up wait in; segments with enough row tiles then run on it (gemm_tc_shape_ok)
    const uint8_t *ximg_tc = nullptr;
    unsigned *tc_err = nullptr;
};
// Batched path: one pass over the weights for up to kGemmMaxBatch sequences (FP16 operands on mma.sync, gemm.cu).
// The activation is staged as ONE FP16 column per sequence, pre-scaled per row by a power of two (xscale holds the
// factors to multiply the products with).  Epilogues: EPI_STORE, EPI_SILU_PAIR, and EPI_RESID_NORM meaning only
// x_out = resid + y.
constexpr int kGemmMaxBatch = 64;
int gemm_min_batch();               // smallest batch routed to the batched path (JUNO_GEMM_MIN_BATCH, default 9)
int gemm_padded_batch(int batch);   // image columns: batch rounded up to a multiple of 8
size_t gemm_image_bytes(int K, int batch);
int launch_stage_f16(juno_ctx *ctx, const StageArgs &a, float *xscale, cudaStream_t stream, uint8_t *img_tc = nullptr);
int launch_gemm(juno_ctx *ctx, const GemvArgs &a, cudaStream_t stream);

// tcgen05/TMEM version of the batched path (gemm_tc.cu): batches of at least JUNO_GEMM_TC_MIN_BATCH (48) sequences on
// matrices with at least sm_count/2 blocks of 128 rows; JUNO_GEMM_TCGEN05=0 switches it off.  It takes its own
// (chunk-major) FP16 image.
bool gemm_tc_enabled();
bool gemm_tc_shape_ok(const juno_ctx *ctx, int row_tiles, int batch);
int gemm_tc_padded_batch(int batch);
size_t gemm_tc_image_bytes(int K, int batch);
int launch_stage_tc(juno_ctx *ctx, const float *x, int ldx, int K, int batch, uint8_t *img, float *xscale, cudaStream_t stream);
int launch_gemm_tc(juno_ctx *ctx, const uint8_t *w, int type, int rows, int row_tiles, int K, int batch, const uint8_t *ximg,
                   const float *xscale, float *out, int ld_out, int epi, unsigned *err, cudaStream_t stream);

// Raw-layout / FP32 fallback (one warp per output), used for shapes the tile layout does not cover.
int launch_gemv_raw(juno_ctx *ctx, const juno_qmat *m, const float *x, int batch, float *y, cudaStream_t stream);
int launch_dequant(juno_ctx *ctx, const juno_qmat *m, int64_t row_start, int64_t n_rows, float *out,
                   cudaStream_t stream);
// Allocates and fills a resident matrix from raw host blocks (row range [row0,row0+nrows), super-block
// column range [sb0, sb0+nsb) of the host tensor — the slicing used by tensor parallelism).
int qmat_create(juno_ctx *ctx, const void *blocks, int type, int64_t rows_total, int64_t cols_total, int64_t row0,
                int64_t nrows, int64_t sb0, int64_t nsb, juno_qmat **out);
int qmat_destroy(juno_qmat *m);

}  // namespace juno
