// Resident quantised matrices: repack of raw GGUF blocks into the 16x256 tile layout (layout.cuh), bit-exact
// dequantisation (LlamaTransformerHandler.dequantize :873-1135) and the plain kernels for shapes the tile layout
// does not cover.  The fused dequant-GEMV itself lives in qgemv.cu (1..8 sequences) and gemm.cu / gemm_tc.cu
// (9..64 sequences).
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "gemv.cuh"
#include "layout.cuh"
#include "dequant.cuh"
#include "repack.cuh"

namespace juno {

// ───────────────────────────── repack (raw GGUF blocks -> tiles) ───────────────────────────
// raw: device copy of rows [0,nrows) of the source tensor, row stride raw_row_bytes; the tile matrix covers
// super-blocks [sb0, sb0+nsb) of each row.  One thread per 32-bit output word.

__global__ void repack_q4k_kernel(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb0, int nsb, uint8_t *out) {
    const size_t words_per_tile = kQ4KTileBytes / 4;
    size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t ntiles = (size_t)((nrows + 15) / 16) * nsb;
    if (gidx >= ntiles * words_per_tile) return;
    size_t tile = gidx / words_per_tile;
    int w = (int)(gidx - tile * words_per_tile);
    int R = (int)(tile / nsb), b = (int)(tile - (size_t)R * nsb);
    reinterpret_cast<uint32_t *>(out)[gidx] = q4k_out_word(raw, raw_row_bytes, nrows, sb0 + b, R, w);
}



__global__ void repack_q6k_kernel(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb0, int nsb, uint8_t *out) {
    const size_t words_per_tile = kQ6KTileBytes / 4;
    size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t ntiles = (size_t)((nrows + 15) / 16) * nsb;
    if (gidx >= ntiles * words_per_tile) return;
    size_t tile = gidx / words_per_tile;
    int w = (int)(gidx - tile * words_per_tile);
    int R = (int)(tile / nsb), b = (int)(tile - (size_t)R * nsb);
    reinterpret_cast<uint32_t *>(out)[gidx] = q6k_out_word(raw, raw_row_bytes, nrows, sb0 + b, R, w);
}


__global__ void repack_q80_kernel(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb0, int nsb, uint8_t *out) {
    const size_t words_per_tile = kQ80TileBytes / 4;
    size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t ntiles = (size_t)((nrows + 15) / 16) * nsb;
    if (gidx >= ntiles * words_per_tile) return;
    size_t tile = gidx / words_per_tile;
    int w = (int)(gidx - tile * words_per_tile);
    int R = (int)(tile / nsb), b = (int)(tile - (size_t)R * nsb);
    reinterpret_cast<uint32_t *>(out)[gidx] = q80_out_word(raw, raw_row_bytes, nrows, sb0 + b, R, w);
}

// ───────────────────────────── bit-exact dequantisation from tiles ─────────────────────────
// Formulas and rounding order of LlamaTransformerHandler.dequantizeQ4K/Q6K/Q8_0 (:1017-1050,
// :1095-1135, :895-913): every product and difference is rounded separately.
__global__ void dequant_tiled_kernel(int type, const uint8_t *tiles, int64_t nb, int64_t cols, int64_t row_start,
                                     int64_t n_rows, float *out) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * cols) return;
    int64_t r = idx / cols, col = idx - r * cols;
    int64_t row = row_start + r;
    const uint8_t *tile = tiles + ((row >> 4) * nb + (col >> 8)) * (int64_t)tile_bytes(type);
    out[idx] = tile_elem_value(type, tile, (int)(row & 15), (int)(col & 255));
}

// ───────────────────────────── raw-layout kernels (odd shapes, FP32) ───────────────────────
__global__ void gemv_raw_kernel(int type, const uint8_t *raw, int64_t row_bytes, int64_t rows, int64_t cols,
                                const float *x, int batch, float *y) {
    int64_t gw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (gw >= rows * batch) return;
    int64_t r = gw % rows;
    int b = (int)(gw / rows);
    const uint8_t *rowp = raw + r * row_bytes;
    const float *xv = x + (int64_t)b * cols;
    float acc = 0.f;
    for (int64_t c = lane; c < cols; c += 32) acc = fmaf(raw_elem_value(type, rowp, c), xv[c], acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[(int64_t)b * rows + r] = acc;
}

__global__ void dequant_raw_kernel(int type, const uint8_t *raw, int64_t row_bytes, int64_t cols, int64_t row_start,
                                   int64_t n_rows, float *out) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * cols) return;
    int64_t r = idx / cols, c = idx - r * cols;
    out[idx] = raw_elem_value(type, raw + (row_start + r) * row_bytes, c);
}

static int64_t raw_row_bytes(int type, int64_t cols) {
    return cols / raw_block_elems(type) * raw_block_bytes(type);
}

int launch_gemv_raw(juno_ctx *ctx, const juno_qmat *m, const float *x, int batch, float *y, cudaStream_t st) {
    int64_t warps = m->rows * batch;
    int threads = 256;
    int64_t blocks = (warps * 32 + threads - 1) / threads;
    gemv_raw_kernel<<<(unsigned)blocks, threads, 0, st>>>(m->type, m->dev, raw_row_bytes(m->type, m->cols), m->rows,
                                                         m->cols, x, batch, y);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

int launch_dequant(juno_ctx *ctx, const juno_qmat *m, int64_t row_start, int64_t n_rows, float *out, cudaStream_t st) {
    int64_t n = n_rows * m->cols;
    int threads = 256;
    int64_t blocks = (n + threads - 1) / threads;
    if (blocks == 0) return JUNO_OK;
    if (m->tiled)
        dequant_tiled_kernel<<<(unsigned)blocks, threads, 0, st>>>(m->type, m->dev, m->nb, m->cols, row_start, n_rows, out);
    else
        dequant_raw_kernel<<<(unsigned)blocks, threads, 0, st>>>(m->type, m->dev, raw_row_bytes(m->type, m->cols),
                                                                m->cols, row_start, n_rows, out);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

// ───────────────────────────── resident matrix ─────────────────────────────────────────────
int qmat_create(juno_ctx *ctx, const void *blocks, int type, int64_t rows_total, int64_t cols_total, int64_t row0,
                int64_t nrows, int64_t sb0, int64_t nsb, juno_qmat **out) {
    JUNO_REQUIRE(type == 0 || type == 8 || type == 12 || type == 14, "unsupported GGML type %d", type);
    JUNO_REQUIRE(rows_total > 0 && cols_total > 0 && nrows > 0 && row0 >= 0 && row0 + nrows <= rows_total,
                 "bad matrix shape rows=%lld cols=%lld", (long long)rows_total, (long long)cols_total);
    JUNO_REQUIRE(cols_total % raw_block_elems(type) == 0, "cols=%lld is not a multiple of the block size %d",
                 (long long)cols_total, raw_block_elems(type));
    const bool tiled = (type != 0) && (cols_total % 256 == 0);
    const int64_t rrb = raw_row_bytes(type, cols_total);
    int64_t cols = cols_total;
    if (tiled) {
        if (nsb <= 0) {
            sb0 = 0;
            nsb = cols_total / 256;
        }
        JUNO_REQUIRE(sb0 >= 0 && (sb0 + nsb) * 256 <= cols_total, "bad super-block slice");
        cols = nsb * 256;
    } else {
        JUNO_REQUIRE(nsb <= 0, "column slicing needs a 256-multiple column count");
    }
    JUNO_REQUIRE(nrows < (1ll << 31) && cols < (1ll << 31), "matrix too large");

    juno_qmat *m = new juno_qmat();
    m->magic = kMagicQmat;
    m->ctx = ctx;
    m->type = type;
    m->tiled = tiled ? 1 : 0;
    m->rows = nrows;
    m->cols = cols;
    m->row_tiles = (nrows + 15) / 16;
    m->nb = cols / 256;
    m->dev = nullptr;
    const uint8_t *src = static_cast<const uint8_t *>(blocks) + row0 * rrb;
    const size_t raw_bytes = (size_t)nrows * rrb;
    int rc = JUNO_OK;
    cudaStream_t st = ctx->stream;
    auto fail = [&](int code) {
        if (m->dev) cudaFree(m->dev);
        m->magic = kMagicDead;
        delete m;
        return code;
    };
    if (!tiled) {
        m->bytes = raw_bytes;
        if (cudaMalloc((void **)&m->dev, m->bytes) != cudaSuccess) {
            cudaGetLastError();
            set_error("cudaMalloc of %zu bytes failed", m->bytes);
            return fail(JUNO_ERR_OOM);
        }
        if (cudaMemcpyAsync(m->dev, src, raw_bytes, cudaMemcpyHostToDevice, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) {
            set_error("upload failed: %s", cudaGetErrorString(cudaGetLastError()));
            return fail(JUNO_ERR_CUDA);
        }
    } else {
        m->bytes = (size_t)m->row_tiles * m->nb * tile_bytes(type);
        uint8_t *tmp = nullptr;
        if (cudaMalloc((void **)&m->dev, m->bytes) != cudaSuccess || cudaMalloc((void **)&tmp, raw_bytes) != cudaSuccess) {
            cudaGetLastError();
            set_error("cudaMalloc of %zu + %zu bytes failed", m->bytes, raw_bytes);
            return fail(JUNO_ERR_OOM);
        }
        cudaError_t e = cudaMemcpyAsync(tmp, src, raw_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) {
            size_t words = m->bytes / 4;
            int threads = 256;
            unsigned blocks_n = (unsigned)((words + threads - 1) / threads);
            if (type == 12)
                repack_q4k_kernel<<<blocks_n, threads, 0, st>>>(tmp, (size_t)rrb, (int)nrows, (int)sb0, (int)nsb, m->dev);
            else if (type == 14)
                repack_q6k_kernel<<<blocks_n, threads, 0, st>>>(tmp, (size_t)rrb, (int)nrows, (int)sb0, (int)nsb, m->dev);
            else
                repack_q80_kernel<<<blocks_n, threads, 0, st>>>(tmp, (size_t)rrb, (int)nrows, (int)sb0, (int)nsb, m->dev);
            e = cudaGetLastError();
            ctx->kernel_launches++;
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        cudaFree(tmp);
        if (e != cudaSuccess) {
            set_error("repack failed: %s", cudaGetErrorString(e));
            rc = JUNO_ERR_CUDA;
            return fail(rc);
        }
    }
    ctx->h2d_bytes += (int64_t)raw_bytes;
    *out = m;
    return JUNO_OK;
}

int qmat_destroy(juno_qmat *m) {
    if (!m) return JUNO_ERR_INVALID_ARG;
    if (m->magic != kMagicQmat) {
        set_error("matrix handle is closed");
        return JUNO_ERR_CLOSED;
    }
    {
        DeviceGuard g(m->ctx->device);
        if (m->dev) cudaFree(m->dev);
    }
    m->dev = nullptr;
    m->magic = kMagicDead;  // the small host record is kept so a second free reports CLOSED instead of crashing
    return JUNO_OK;
}

}  // namespace juno
