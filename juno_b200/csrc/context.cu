// Context, device discovery, error text and the MatVec-operator entry points of the C ABI.
#include <cstring>
#include <string>

#include "common.cuh"
#include <algorithm>

#include "gemv.cuh"
#include "qgemv.cuh"

namespace juno {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char *get_error() { return g_err; }

int ctx_check(juno_ctx *c) {
    if (!c) {
        set_error("context is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (c->magic != kMagicCtx) {
        set_error("context is closed");
        return JUNO_ERR_CLOSED;
    }
    return JUNO_OK;
}

int ensure_device(void **ptr, size_t *cur, size_t want) {
    if (*cur >= want && *ptr) return JUNO_OK;
    void *np = nullptr;
    cudaError_t e = cudaMalloc(&np, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc of %zu bytes failed: %s", want, cudaGetErrorString(e));
        return JUNO_ERR_OOM;
    }
    if (*ptr) {
        cudaDeviceSynchronize();
        cudaFree(*ptr);
    }
    *ptr = np;
    *cur = want;
    return JUNO_OK;
}

int ensure_pinned(juno_ctx *c, size_t want) {
    if (c->pinned_bytes >= want && c->pinned) return JUNO_OK;
    if (c->pinned) cudaFreeHost(c->pinned);
    c->pinned = nullptr;
    c->pinned_bytes = 0;
    cudaError_t e = cudaMallocHost(&c->pinned, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMallocHost of %zu bytes failed: %s", want, cudaGetErrorString(e));
        return JUNO_ERR_OOM;
    }
    c->pinned_bytes = want;
    return JUNO_OK;
}

}  // namespace juno

using namespace juno;

extern "C" {

const char *juno_last_error(void) { return get_error(); }

int juno_device_count(int32_t *count) {
    if (!count) return JUNO_ERR_INVALID_ARG;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {  // no driver / no device: fail soft like CudaAvailability
        cudaGetLastError();
        n = 0;
    }
    *count = n;
    return JUNO_OK;
}

int juno_device_name(int32_t device, char *buf, int32_t buf_len) {
    JUNO_REQUIRE(buf && buf_len > 0, "name buffer missing");
    cudaDeviceProp prop;
    JUNO_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    snprintf(buf, (size_t)buf_len, "%s", prop.name);
    return JUNO_OK;
}

int juno_device_total_mem(int32_t device, int64_t *bytes) {
    JUNO_REQUIRE(bytes, "bytes is null");
    cudaDeviceProp prop;
    JUNO_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    *bytes = (int64_t)prop.totalGlobalMem;
    return JUNO_OK;
}

int juno_ctx_create(int32_t device, juno_ctx **out) {
    JUNO_REQUIRE(out, "out is null");
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error("no CUDA device available (this backend has no CPU fallback)");
        return JUNO_ERR_CUDA;
    }
    JUNO_REQUIRE(device >= 0 && device < n, "device %d out of range [0,%d)", device, n);
    cudaDeviceProp prop;
    JUNO_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
        return JUNO_ERR_UNSUPPORTED;
    }
    DeviceGuard g(device);
    juno_ctx *c = new juno_ctx();
    c->magic = kMagicCtx;
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = prop.sharedMemPerBlockOptin;
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        set_error("cudaStreamCreateWithFlags failed: rc=%d (%s)", (int)e, cudaGetErrorString(e));
        delete c;
        return JUNO_ERR_CUDA;
    }
    // one word in mapped host memory: a kernel that gave up a wait leaves its code there, the host reads it for free
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&c->gemv_scratch.qerr_host, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) {
        memset(c->gemv_scratch.qerr_host, 0, 64);
        e = cudaHostGetDevicePointer((void **)&c->gemv_scratch.qerr, c->gemv_scratch.qerr_host, 0);
    }
    if (e != cudaSuccess) {
        set_error("context set-up failed: rc=%d (%s)", (int)e, cudaGetErrorString(e));
        delete c;
        return e == cudaErrorMemoryAllocation ? JUNO_ERR_OOM : JUNO_ERR_CUDA;
    }
    *out = c;
    return JUNO_OK;
}

int juno_ctx_destroy(juno_ctx *c) {
    JUNO_TRY(ctx_check(c));
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    cudaStreamSynchronize(c->stream);
    if (c->gemv_scratch.ximg) cudaFree(c->gemv_scratch.ximg);
    if (c->gemv_scratch.xscale) cudaFree(c->gemv_scratch.xscale);
    if (c->gemv_scratch.qerr_host) cudaFreeHost(c->gemv_scratch.qerr_host);
    if (c->stage_x) cudaFree(c->stage_x);
    if (c->stage_y) cudaFree(c->stage_y);
    if (c->pinned) cudaFreeHost(c->pinned);
    cudaStreamDestroy(c->stream);
    c->magic = kMagicDead;  // record kept: a second destroy reports CLOSED
    return JUNO_OK;
}

int juno_ctx_device(juno_ctx *c, int32_t *device) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(device, "device is null");
    *device = c->device;
    return JUNO_OK;
}

int juno_ctx_synchronize(juno_ctx *c) {
    JUNO_TRY(ctx_check(c));
    DeviceGuard g(c->device);
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    return JUNO_OK;
}

int juno_ctx_stream(juno_ctx *c, void **stream) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(stream, "stream is null");
    *stream = (void *)c->stream;
    return JUNO_OK;
}

int juno_ctx_profile(juno_ctx *c, int32_t enable) {
    JUNO_TRY(ctx_check(c));
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    c->profiling = enable != 0;
    return JUNO_OK;
}

int juno_ctx_profile_read(juno_ctx *c, juno_profile_entry *out, int32_t n_entries, int32_t reset) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(out && n_entries >= 1, "bad output array");
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    for (auto &sp : c->prof_spans) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, sp.e0, sp.e1) == cudaSuccess) {
            c->prof_ms[sp.cat] += ms;
            c->prof_bytes[sp.cat] += sp.bytes;
            c->prof_launches[sp.cat]++;
        }
        cudaEventDestroy(sp.e0);
        cudaEventDestroy(sp.e1);
    }
    cudaGetLastError();
    c->prof_spans.clear();
    for (int i = 0; i < n_entries && i < PROF_COUNT; i++) {
        out[i].launches = c->prof_launches[i];
        out[i].ms = c->prof_ms[i];
        out[i].algo_bytes = c->prof_bytes[i];
    }
    if (reset)
        for (int i = 0; i < PROF_COUNT; i++) {
            c->prof_launches[i] = 0;
            c->prof_ms[i] = c->prof_bytes[i] = 0;
        }
    return JUNO_OK;
}

int juno_ctx_counters(juno_ctx *c, juno_counters *out, int32_t reset) {
    JUNO_TRY(ctx_check(c));
    if (out) {
        out->kernel_launches = c->kernel_launches.load();
        out->gemv_calls = c->gemv_calls.load();
        out->forward_calls = c->forward_calls.load();
        out->h2d_bytes = c->h2d_bytes.load();
        out->d2h_bytes = c->d2h_bytes.load();
    }
    if (reset) {
        c->kernel_launches = 0;
        c->gemv_calls = 0;
        c->forward_calls = 0;
        c->h2d_bytes = 0;
        c->d2h_bytes = 0;
    }
    return JUNO_OK;
}

// ── MatVec operator ────────────────────────────────────────────────────────────
int juno_qmat_upload(juno_ctx *c, const void *blocks, int32_t type, int64_t rows, int64_t cols, juno_qmat **out) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(blocks && out, "null argument");
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    return qmat_create(c, blocks, type, rows, cols, 0, rows, 0, 0, out);
}

int juno_qmat_free(juno_qmat *m) {
    if (!m) {
        set_error("matrix is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (m->magic != kMagicQmat) {
        set_error("matrix handle is closed");
        return JUNO_ERR_CLOSED;
    }
    std::lock_guard<std::recursive_mutex> lk(m->ctx->mu);
    return qmat_destroy(m);
}

static int qmat_check(juno_qmat *m) {
    if (!m) {
        set_error("matrix is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (m->magic != kMagicQmat) {
        set_error("matrix handle is closed");
        return JUNO_ERR_CLOSED;
    }
    return JUNO_OK;
}

int juno_qmat_shape(juno_qmat *m, int64_t *rows, int64_t *cols, int32_t *type) {
    JUNO_TRY(qmat_check(m));
    if (rows) *rows = m->rows;
    if (cols) *cols = m->cols;
    if (type) *type = m->type;
    return JUNO_OK;
}

static int gemv_on_stream(juno_ctx *c, juno_qmat *m, const float *x, int batch, float *y, cudaStream_t st) {
    if (!m->tiled) return launch_gemv_raw(c, m, x, batch, y, st);
    const bool batched = batch >= gemm_min_batch();
    if (!batched) {
        QGemvArgs q;
        q.nseg = 1;
        q.seg[0].w = m->dev;
        q.seg[0].out = y;
        q.seg[0].rows = (int)m->rows;
        q.seg[0].row_tiles = (int)m->row_tiles;
        q.seg[0].type = m->type;
        q.K = (int)m->cols;
        q.batch = batch;
        q.ld_out = (int)m->rows;
        q.x = x;
        q.ldx = (int)m->cols;
        return launch_qgemv(c, q, st);
    }
    const size_t need = gemm_image_bytes((int)m->cols, std::min(batch, kGemmMaxBatch));
    void *pi = c->gemv_scratch.ximg;
    JUNO_TRY(ensure_device(&pi, &c->gemv_scratch.ximg_bytes, need));
    c->gemv_scratch.ximg = (uint8_t *)pi;
    GemvArgs a;
    a.nseg = 1;
    a.seg[0].w = m->dev;
    a.seg[0].rows = (int)m->rows;
    a.seg[0].row_tiles = (int)m->row_tiles;
    a.type = m->type;
    a.K = (int)m->cols;
    a.ld_out = (int)m->rows;
    a.ximg = c->gemv_scratch.ximg;
    StageArgs sa;
    sa.mode = STAGE_PLAIN;
    sa.ldx = (int)m->cols;
    sa.K = (int)m->cols;
    sa.img = c->gemv_scratch.ximg;
    // one pass over the weights per group of up to kGemmMaxBatch rows
    if (!c->gemv_scratch.xscale) {
        cudaError_t e = cudaMalloc((void **)&c->gemv_scratch.xscale, (kGemmMaxBatch + 4) * sizeof(float));  // + an error word for the tcgen05 kernel
        if (e != cudaSuccess) {
            cudaGetLastError();
            set_error("cudaMalloc of %zu bytes failed: %s", kGemmMaxBatch * sizeof(float), cudaGetErrorString(e));
            return JUNO_ERR_OOM;
        }
        JUNO_CUDA_TRY(cudaMemset(c->gemv_scratch.xscale, 0, (kGemmMaxBatch + 4) * sizeof(float)));
    }
    for (int b0 = 0; b0 < batch; b0 += kGemmMaxBatch) {
        const int bc = std::min(kGemmMaxBatch, batch - b0);
        if (gemm_tc_enabled() && gemm_tc_shape_ok(c, (int)m->row_tiles, bc)) {  // tcgen05/TMEM kernel (opt-in)
            void *pt = c->gemv_scratch.ximg;
            JUNO_TRY(ensure_device(&pt, &c->gemv_scratch.ximg_bytes, gemm_tc_image_bytes((int)m->cols, bc) + 16));
            c->gemv_scratch.ximg = (uint8_t *)pt;
            unsigned *err = reinterpret_cast<unsigned *>(c->gemv_scratch.xscale + kGemmMaxBatch);
            JUNO_TRY(launch_stage_tc(c, x + (size_t)b0 * m->cols, (int)m->cols, (int)m->cols, bc, c->gemv_scratch.ximg,
                                     c->gemv_scratch.xscale, st));
            JUNO_TRY(launch_gemm_tc(c, m->dev, m->type, (int)m->rows, (int)m->row_tiles, (int)m->cols, bc, c->gemv_scratch.ximg,
                                    c->gemv_scratch.xscale, y + (size_t)b0 * m->rows, (int)m->rows, EPI_STORE, err, st));
            continue;
        }
        sa.x = x + (size_t)b0 * m->cols;
        sa.batch = bc;
        JUNO_TRY(launch_stage_f16(c, sa, c->gemv_scratch.xscale, st));
        a.seg[0].out = y + (size_t)b0 * m->rows;
        a.batch = bc;
        a.xscale = c->gemv_scratch.xscale;
        JUNO_TRY(launch_gemm(c, a, st));
    }
    return JUNO_OK;
}

int juno_gemv_device(juno_ctx *c, juno_qmat *m, const float *x_dev, int32_t batch, float *y_dev, void *stream) {
    JUNO_TRY(ctx_check(c));
    JUNO_TRY(qmat_check(m));
    JUNO_REQUIRE(m->ctx == c, "matrix belongs to another context");
    JUNO_REQUIRE(x_dev && y_dev && batch >= 1, "bad gemv arguments (batch=%d)", batch);
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    c->gemv_calls++;
    return gemv_on_stream(c, m, x_dev, batch, y_dev, stream ? (cudaStream_t)stream : c->stream);
}

int juno_gemv(juno_ctx *c, juno_qmat *m, const float *x_host, int32_t batch, float *y_host) {
    JUNO_TRY(ctx_check(c));
    JUNO_TRY(qmat_check(m));
    JUNO_REQUIRE(m->ctx == c, "matrix belongs to another context");
    JUNO_REQUIRE(x_host && y_host, "null vector");
    JUNO_REQUIRE(batch >= 1 && batch <= 4096, "batch %d out of range", batch);
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    const size_t xb = (size_t)batch * m->cols * sizeof(float), yb = (size_t)batch * m->rows * sizeof(float);
    void *px = c->stage_x, *py = c->stage_y;
    JUNO_TRY(ensure_device(&px, &c->stage_x_bytes, xb));
    c->stage_x = (float *)px;
    JUNO_TRY(ensure_device(&py, &c->stage_y_bytes, yb));
    c->stage_y = (float *)py;
    JUNO_CUDA_TRY(cudaMemcpyAsync(c->stage_x, x_host, xb, cudaMemcpyHostToDevice, c->stream));
    c->gemv_calls++;
    JUNO_TRY(gemv_on_stream(c, m, c->stage_x, batch, c->stage_y, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(y_host, c->stage_y, yb, cudaMemcpyDeviceToHost, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    if (c->gemv_scratch.xscale && batch >= gemm_min_batch()) {  // did a wait inside the tcgen05 kernel give up?
        unsigned code = 0;
        JUNO_CUDA_TRY(cudaMemcpy(&code, c->gemv_scratch.xscale + kGemmMaxBatch, 4, cudaMemcpyDeviceToHost));
        if (code) {
            set_error("batched tensor-core product gave up waiting (code %u, block %u)", code & 0xffu, code >> 8);
            return JUNO_ERR_CUDA;
        }
    }
    c->h2d_bytes += (int64_t)xb;
    c->d2h_bytes += (int64_t)yb;
    return JUNO_OK;
}

int juno_dequantize(juno_ctx *c, juno_qmat *m, int64_t row_start, int64_t n_rows, float *out_host) {
    JUNO_TRY(ctx_check(c));
    JUNO_TRY(qmat_check(m));
    JUNO_REQUIRE(out_host, "out is null");
    JUNO_REQUIRE(row_start >= 0 && n_rows >= 0 && row_start + n_rows <= m->rows, "row range [%lld,+%lld) outside %lld rows",
                 (long long)row_start, (long long)n_rows, (long long)m->rows);
    if (n_rows == 0) return JUNO_OK;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    const size_t bytes = (size_t)n_rows * m->cols * sizeof(float);
    void *py = c->stage_y;
    JUNO_TRY(ensure_device(&py, &c->stage_y_bytes, bytes));
    c->stage_y = (float *)py;
    JUNO_TRY(launch_dequant(c, m, row_start, n_rows, c->stage_y, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(out_host, c->stage_y, bytes, cudaMemcpyDeviceToHost, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->d2h_bytes += (int64_t)bytes;
    return JUNO_OK;
}

int juno_sgemv_f32(juno_ctx *c, const float *a_host, const float *x_host, int64_t rows, int64_t cols, float *y_host) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(a_host && x_host && y_host, "null argument");
    JUNO_REQUIRE(rows >= 1 && cols >= 1, "rows*cols must be positive (rows=%lld cols=%lld)", (long long)rows,
                 (long long)cols);
    juno_qmat *m = nullptr;
    JUNO_TRY(juno_qmat_upload(c, a_host, JUNO_TYPE_F32, rows, cols, &m));
    int rc = juno_gemv(c, m, x_host, 1, y_host);
    juno_qmat_free(m);
    delete m;
    return rc;
}

}  // extern "C"
