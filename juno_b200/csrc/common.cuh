// Shared host-side plumbing of the engine: status codes, thread-local error text,
// the context object and launch bookkeeping.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/juno_b200.h"

namespace juno {

void set_error(const char *fmt, ...);
const char *get_error();

#define JUNO_CUDA_TRY(expr)                                                                   \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            ::juno::set_error("%s failed: rc=%d (%s) at %s:%d", #expr, (int)_e,               \
                              cudaGetErrorString(_e), __FILE__, __LINE__);                    \
            return (_e == cudaErrorMemoryAllocation) ? JUNO_ERR_OOM : JUNO_ERR_CUDA;          \
        }                                                                                     \
    } while (0)

#define JUNO_TRY(expr)          \
    do {                        \
        int _rc = (expr);       \
        if (_rc != JUNO_OK)     \
            return _rc;         \
    } while (0)

#define JUNO_REQUIRE(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            ::juno::set_error(__VA_ARGS__); \
            return JUNO_ERR_INVALID_ARG;   \
        }                                  \
    } while (0)

constexpr uint32_t kMagicCtx = 0x4A435458;    // "JCTX"
constexpr uint32_t kMagicQmat = 0x4A514D54;   // "JQMT"
constexpr uint32_t kMagicModel = 0x4A4D444C;  // "JMDL"
constexpr uint32_t kMagicSeq = 0x4A534551;    // "JSEQ"
constexpr uint32_t kMagicPool = 0x4A4B5650;   // "JKVP"
constexpr uint32_t kMagicDead = 0xDEADDEAD;

// Scratch of the host-level MatVec entry points and the word kernels report a given-up wait in.
struct GemvScratch {
    unsigned *qerr = nullptr;       // device address of qerr_host
    unsigned *qerr_host = nullptr;  // mapped host memory: code | warp << 8 | block << 16, 0 = no failure
    uint8_t *ximg = nullptr;        // FP16 staged activation (batched path)
    size_t ximg_bytes = 0;
    float *xscale = nullptr;        // per-row factors of an FP16 staged activation, 64 floats
};

}  // namespace juno

namespace juno {
enum ProfCat { PROF_GEMV_Q4K = 0, PROF_GEMV_Q6K, PROF_GEMV_Q80, PROF_ATTN, PROF_ROPE_APPEND, PROF_OTHER, PROF_GEMM_TC, PROF_COUNT };
struct ProfSpan {
    int cat;
    double bytes;
    cudaEvent_t e0, e1;
};
}  // namespace juno

struct juno_ctx {
    uint32_t magic;
    int device;
    int sm_count;
    size_t smem_optin;
    cudaStream_t stream;
    std::recursive_mutex mu;
    juno::GemvScratch gemv_scratch;
    // staging buffers for the host-in/host-out entry points
    float *stage_x = nullptr, *stage_y = nullptr;
    size_t stage_x_bytes = 0, stage_y_bytes = 0;
    void *pinned = nullptr;
    size_t pinned_bytes = 0;
    // per-kernel timing (off by default): event pairs around launches, summed at read time
    bool profiling = false;
    std::vector<juno::ProfSpan> prof_spans;
    double prof_ms[juno::PROF_COUNT] = {0}, prof_bytes[juno::PROF_COUNT] = {0};
    int64_t prof_launches[juno::PROF_COUNT] = {0};
    std::atomic<int64_t> kernel_launches{0}, gemv_calls{0}, forward_calls{0}, h2d_bytes{0}, d2h_bytes{0};
};

namespace juno {

inline bool ctx_ok(juno_ctx *c) { return c && c->magic == kMagicCtx; }
int ctx_check(juno_ctx *c);
// Grows a device buffer (never shrinks). Returns JUNO_OK / JUNO_ERR_OOM.
int ensure_device(void **ptr, size_t *cur, size_t want);
int ensure_pinned(juno_ctx *c, size_t want);

// Brackets one launch (or a short group) with events when the context is profiling.
struct ProfScope {
    juno_ctx *c;
    cudaStream_t st;
    bool on;
    ProfSpan sp;
    ProfScope(juno_ctx *ctx, cudaStream_t stream, int cat, double bytes) : c(ctx), st(stream), on(ctx->profiling) {
        if (!on) return;
        sp.cat = cat;
        sp.bytes = bytes;
        cudaEventCreate(&sp.e0);
        cudaEventCreate(&sp.e1);
        cudaEventRecord(sp.e0, st);
    }
    ~ProfScope() {
        if (!on) return;
        cudaEventRecord(sp.e1, st);
        c->prof_spans.push_back(sp);
    }
};

// Programmatic dependent launch: a kernel launched with the attribute may be scheduled while the previous kernel of
// the stream is still running; it must execute pdl_wait() before it touches anything that kernel (or an earlier one)
// produces.  Here only weight prefetches and a launch-private work counter happen before the wait.
inline bool pdl_enabled() {
    static const bool on = [] {
        const char *v = getenv("JUNO_NO_PDL");
        return !(v && *v == '1');
    }();
    return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev)
            cudaSetDevice(dev);
        else
            prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0)
            cudaSetDevice(prev);
    }
};

}  // namespace juno
