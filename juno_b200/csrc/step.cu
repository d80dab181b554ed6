// The persistent decode-step kernel (see step.cuh).
//
// One CTA of 16 warps per SM.  Shared memory per CTA:
//   [ staged activation of the current product (bf16 limbs) + its 32-column sums | attention scratch ]
//   [ weight ring: per warp a few tile slots, each filled by one cp.async.bulk and guarded by an mbarrier ]
//   [ partial-sum buffers, phase descriptors, barriers ]
// Every warp streams its own tiles and refills a slot the moment it has pulled the tile into registers, following
// its tile sequence across phase boundaries: the weight stream is limited only by free slots, never by the grid
// barriers between phases — while a CTA waits for the other SMs, the first tiles of the next product are landing.
// Every wait in here (mbarrier, grid barrier) is bounded: when one runs out the kernel records a code, stops
// waiting everywhere and returns; the host reports the code.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <vector>

#include "step.cuh"
#include "tile_math.cuh"

namespace juno {

struct StepParams {
    const StepPhase *phases;
    int n_phases;
    unsigned *sync;      // {barrier arrivals, error code, one task counter per phase}, zeroed before the launch
    int slot_bytes;      // stride of the ring slots (largest tile of the model, multiple of 16)
    unsigned img_cap;    // bytes reserved at the start of shared memory for the activation / attention scratch
    unsigned long long *timeline;  // optional [n_phases][8] time stamps of CTA 0 (tuning aid), else null
    int dbg;  // JUNO_STEP_DEBUG bits (timing experiments, results are wrong): 1 skip the tile arithmetic, 2 skip the epilogues
};

enum StepError {
    STEP_ERR_GRID = 1,   // a grid barrier ran out
    STEP_ERR_FULL = 2,   // a computing warp never saw its tile arrive
    STEP_ERR_EMPTY = 3,  // the copy warp never got a slot back
    STEP_ERR_IMAGE = 4,  // the staged activation never arrived
    STEP_ERR_PART_FREE = 5,   // a partial-sum buffer was never released
    STEP_ERR_PART_READY = 6,  // a group's partial sums never arrived
    STEP_ERR_CLAIM = 7,       // the next CTA task was never published
    STEP_ERR_CLAIM_FREE = 8,  // a claimed-task entry was never read by every warp
    STEP_ERR_CURSOR = 9,      // a warp's copy cursor could not reach the tile in hand
};

// ───────────────────────────── primitives ─────────────────────────────────────────────────
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Non-blocking test of an mbarrier phase.  (mbarrier.try_wait may suspend the thread for a system-dependent time
// slice when the phase is not complete yet; in this kernel most waits are short, and a poll loop measured faster.)
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define STEP_STAMP(tl, ph, k)                                                       \
    do {                                                                          \
        if ((tl) && blockIdx.x == 0 && threadIdx.x == 0) (tl)[(ph) * 8 + (k)] = global_ns(); \
    } while (0)
// Every wait gives up after this many SM clock cycles (about a fifth of a second).  Measured with the SM's own cycle
// counter: reading the global nanosecond timer inside a wait loop costs more than the waits themselves.
constexpr long long kWaitLimitClk = 400000000ll;

// Records the first wait that gave up: code | warp << 8 | block << 16.
__device__ __forceinline__ void step_fail(unsigned *sync, volatile unsigned *err_s, unsigned code) {
    if (*err_s == 0) {
        *err_s = code;
        atomicCAS(sync + 1, 0u, code | ((threadIdx.x >> 5) << 8) | (blockIdx.x << 16));
    }
}
// Bounded wait on an mbarrier phase.  Returns false when the kernel is in the failed state.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity, unsigned *sync, volatile unsigned *err_s, unsigned code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*err_s) return false;
        if (clock64() - t0 > kWaitLimitClk) break;
    }
    step_fail(sync, err_s, code);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, unsigned bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Barrier of the computing warps only (the copy warp never joins).
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(kStepConsumers) : "memory"); }

// Grid-wide barrier, called by ONE thread of every CTA after csync(): arrivals are counted in sync[0], which starts
// at zero for the launch, so barrier number k is complete when the count reaches k * gridDim.x.
__device__ __forceinline__ void grid_sync(unsigned *sync, unsigned k, volatile unsigned *err_s) {
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(sync) : "memory");
    const unsigned target = k * gridDim.x;
    if (ld_acquire_gpu(sync) >= target) return;
    const long long t0 = clock64();
    unsigned i = 0;
    while (ld_acquire_gpu(sync) < target) {
        if (*err_s) return;
        if ((++i & 63u) == 0u && (ld_relaxed_gpu(sync + 1) != 0u || clock64() - t0 > kWaitLimitClk)) {
            step_fail(sync, err_s, STEP_ERR_GRID);
            return;
        }
    }
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

// A tile from its ring slot into registers (same byte layout as in global memory, layout.cuh).
__device__ __forceinline__ void ring_load(TileRegs<12> &r, uint32_t t, int lane) {
    const int r8 = lane >> 2, c = lane & 3;
    r.dm0 = lds32(t + 4 * r8);
    r.dm1 = lds32(t + 4 * (r8 + 8));
    r.sm0 = lds32(t + 4 * (16 + r8 * 4 + c));
    r.sm1 = lds32(t + 4 * (16 + (r8 + 8) * 4 + c));
#pragma unroll
    for (int g = 0; g < 4; g++) r.q[g] = lds128(t + kQ4KQsOff + 16 * (g * 32 + lane));
}
__device__ __forceinline__ void ring_load(TileRegs<14> &r, uint32_t t, int lane) {
    const int r8 = lane >> 2, c = lane & 3;
#pragma unroll
    for (int m = 0; m < 4; m++) r.ql[m] = lds128(t + 16 * (m * 32 + lane));
#pragma unroll
    for (int p = 0; p < 2; p++) r.qh[p] = lds128(t + 16 * (128 + p * 32 + lane));
    r.sc0 = lds32(t + 3072 + 4 * (r8 * 4 + c));
    r.sc1 = lds32(t + 3072 + 4 * ((r8 + 8) * 4 + c));
    r.d01 = lds16(t + 3328 + 2 * r8) | (lds16(t + 3328 + 2 * (r8 + 8)) << 16);
}
__device__ __forceinline__ void ring_load(TileRegs<8> &r, uint32_t t, int lane) {
    const int r8 = lane >> 2;
#pragma unroll
    for (int j = 0; j < 8; j++) r.q[j] = lds128(t + 16 * (j * 32 + lane));
    r.d0 = lds128(t + 16 * (256 + r8));
    r.d1 = lds128(t + 16 * (256 + r8 + 8));
}

// Shared-memory carve-up (byte offsets from the start of dynamic shared memory).
template <int NB>
struct StepSmem {
    static constexpr int NC = 3 * NB;
    static constexpr int LDC = 2 * ((NC + 1) / 2);  // columns of a warp's partial-sum block that are kept
    unsigned img_cap, ring, cs, scale_s, mg_f, mg_L, desc, stream, bars, flags, total;
    __host__ __device__ StepSmem(unsigned cap, int slot_bytes) {
        img_cap = cap;
        ring = img_cap;
        cs = ring + (unsigned)kStepRingSlots * (unsigned)slot_bytes;
        cs = (cs + 127u) & ~127u;
        scale_s = cs + (unsigned)kStepFragBufs * kStepWarps * 16u * LDC * 4u;
        mg_f = scale_s + 8u * 4u;
        mg_L = mg_f + 4u * 64u * 4u;
        desc = (mg_L + 4u * 4u + 15u) & ~15u;
        stream = (desc + 2u * (unsigned)sizeof(StepPhase) + 15u) & ~15u;
        bars = (stream + 8u * 80u + 15u) & ~15u;
        flags = bars + ((unsigned)kStepRingSlots + 2u * kStepFragBufs * kStepWarps + 1u + 2u * kStepClaimRing) * 8u;
        total = flags + 16u + 4u * kStepClaimRing;
    }
};

template <typename T>
__device__ __forceinline__ float kv_to_f32(T v);
template <>
__device__ __forceinline__ float kv_to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float kv_to_f32<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T kv_from_f32(float v);
template <>
__device__ __forceinline__ float kv_from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half kv_from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__device__ __forceinline__ void kv_load8(const T *p, float (&o)[8]);
template <>
__device__ __forceinline__ void kv_load8<__half>(const __half *p, float (&o)[8]) {
    const uint4 u = __ldcg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void kv_load8<float>(const float *p, float (&o)[8]) {
    const float4 a = __ldcg(reinterpret_cast<const float4 *>(p)), b = __ldcg(reinterpret_cast<const float4 *>(p + 4));
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

// ───────────────────────────── attention phase ────────────────────────────────────────────
// The 16 computing warps of a CTA take one (sequence, kv head, head group, context chunk) at a time: HD/8 lanes
// share a cached position, every lane keeps an online-softmax state for the GE query heads, the token slots are
// merged through shared memory, and the chunk's partial goes to global memory.  The CTA that completes the last
// chunk of a (sequence, kv head, head group) merges the chunks and emits the staged activation of Wo.
template <typename T, int HD, int GE>
__device__ __forceinline__ void attn_phase(const StepAttn &a, uint8_t *scratch, float *mg_f, float *mg_L, volatile int *flag,
                                           int tid) {
    constexpr int LPT = HD / 8, TPW = 32 / LPT, SLOTS = kStepWarps * TPW, U = 2;
    float *sm_q = reinterpret_cast<float *>(scratch);  // [GE][HD], rotated and scaled
    float *sm_m = sm_q + GE * HD;                      // [SLOTS][GE]
    float *sm_l = sm_m + SLOTS * GE;                   // [SLOTS][GE]
    float *sm_o = sm_l + SLOTS * GE;                   // [SLOTS][GE][HD]
    const int warp = tid >> 5, lane = tid & 31;
    const int G = a.n_heads / a.n_kv_heads;
    const int per_kv = a.head_groups * a.chunks, per_seq = a.n_kv_heads * per_kv, n_items = a.n * per_seq;
    const float scale = (float)(1.0 / sqrt((double)HD)) * 1.4426950408889634f;  // scores in the log2 domain
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int seq = item / per_seq;
        int r = item - seq * per_seq;
        const int kvh = r / per_kv;
        r -= kvh * per_kv;
        const int hg = r / a.chunks, c = r - hg * a.chunks;
        const int len = a.seq_lens[seq];
        const int chunk = (((len + a.chunks - 1) / a.chunks) + 15) & ~15;
        const int t0 = c * chunk, t1 = min(len, t0 + chunk);
        const int h0 = kvh * G + hg * GE;
        float *po = a.part_o + ((size_t)(seq * a.n_heads + h0) * a.chunks + c) * HD;   // head stride chunks*HD
        float *pml = a.part_ml + ((size_t)(seq * a.n_heads + h0) * a.chunks + c) * 2;  // head stride chunks*2
        // q of the head group: adjacent-pair rotation, each product rounded (rope :1657-1671), then the score scale
        for (int idx = tid; idx < GE * HD / 2; idx += kStepConsumers) {
            const int g = idx / (HD / 2), i = idx - g * (HD / 2);
            const float2 x = __ldcg(reinterpret_cast<const float2 *>(a.q + (size_t)seq * a.ldq + (size_t)(h0 + g) * HD + 2 * i));
            const float2 cs = a.rope_cs[seq * (HD / 2) + i];
            const float y0 = __fsub_rn(__fmul_rn(x.x, cs.x), __fmul_rn(x.y, cs.y));
            const float y1 = __fadd_rn(__fmul_rn(x.x, cs.y), __fmul_rn(x.y, cs.x));
            sm_q[g * HD + 2 * i] = y0 * scale;
            sm_q[g * HD + 2 * i + 1] = y1 * scale;
        }
        csync();
        if (t0 >= t1) {  // empty chunk: weight 0, and finite zeros so that 0 * partial stays 0 in the merge
            if (tid < GE) {
                pml[(size_t)tid * a.chunks * 2 + 0] = -INFINITY;
                pml[(size_t)tid * a.chunks * 2 + 1] = 0.f;
            }
            for (int idx = tid; idx < GE * HD; idx += kStepConsumers) po[(size_t)(idx / HD) * a.chunks * HD + (idx % HD)] = 0.f;
        } else {
            const int sub = lane % LPT, slot = warp * TPW + lane / LPT;
            const unsigned gmask = (LPT == 32) ? 0xffffffffu : (((1u << LPT) - 1u) << (lane - sub));
            float o[GE][8], m[GE], l[GE];
#pragma unroll
            for (int g = 0; g < GE; g++) {
#pragma unroll
                for (int e = 0; e < 8; e++) o[g][e] = 0.f;
                m[g] = -INFINITY;
                l[g] = 0.f;
            }
            const int32_t *table = a.table + (size_t)a.slots[seq] * a.max_pages_per_seq;
            const T *kbase = static_cast<const T *>(a.k), *vbase = static_cast<const T *>(a.v);
            const size_t head_off = (size_t)kvh * kPageTokens * HD + sub * 8;
            const size_t page_stride = (size_t)a.n_kv_heads * kPageTokens * HD;
            const size_t layer_off = (size_t)a.layer * a.n_pages * page_stride;
            const float *qs = sm_q + sub * 8;
            for (int tb = t0 + slot; tb < t1; tb += SLOTS * U) {
                float kv[U][8], vv[U][8];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int t = tb + u * SLOTS;
                    if (t < t1) {
                        const size_t off = layer_off + (size_t)table[t >> 4] * page_stride + head_off + (size_t)(t & 15) * HD;
                        if (t == len - 1) {  // the position being decoded: rotate, round, use and append
                            const float *kx = a.knew + (size_t)seq * a.ldkv + kvh * HD + sub * 8;
                            const float *vx = a.vnew + (size_t)seq * a.ldkv + kvh * HD + sub * 8;
                            T *kd = static_cast<T *>(a.kw) + off, *vd = static_cast<T *>(a.vw) + off;
#pragma unroll
                            for (int e = 0; e < 8; e += 2) {
                                const float2 cs = a.rope_cs[seq * (HD / 2) + sub * 4 + (e >> 1)];
                                const float2 kk = __ldcg(reinterpret_cast<const float2 *>(kx + e));
                                const float2 vq = __ldcg(reinterpret_cast<const float2 *>(vx + e));
                                const T k0 = kv_from_f32<T>(__fsub_rn(__fmul_rn(kk.x, cs.x), __fmul_rn(kk.y, cs.y)));
                                const T k1 = kv_from_f32<T>(__fadd_rn(__fmul_rn(kk.x, cs.y), __fmul_rn(kk.y, cs.x)));
                                const T v0 = kv_from_f32<T>(vq.x), v1 = kv_from_f32<T>(vq.y);
                                kd[e] = k0; kd[e + 1] = k1;
                                vd[e] = v0; vd[e + 1] = v1;
                                kv[u][e] = kv_to_f32<T>(k0); kv[u][e + 1] = kv_to_f32<T>(k1);
                                vv[u][e] = kv_to_f32<T>(v0); vv[u][e + 1] = kv_to_f32<T>(v1);
                            }
                        } else {
                            kv_load8<T>(kbase + off, kv[u]);
                            kv_load8<T>(vbase + off, vv[u]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int t = tb + u * SLOTS;
                    if (t < t1) {  // uniform over the LPT lanes of this position
                        float s[GE];
#pragma unroll
                        for (int g = 0; g < GE; g++) {
                            const float4 qa = *reinterpret_cast<const float4 *>(qs + g * HD);
                            const float4 qb = *reinterpret_cast<const float4 *>(qs + g * HD + 4);
                            float d = qa.x * kv[u][0];
                            d = fmaf(qa.y, kv[u][1], d);
                            d = fmaf(qa.z, kv[u][2], d);
                            d = fmaf(qa.w, kv[u][3], d);
                            d = fmaf(qb.x, kv[u][4], d);
                            d = fmaf(qb.y, kv[u][5], d);
                            d = fmaf(qb.z, kv[u][6], d);
                            d = fmaf(qb.w, kv[u][7], d);
                            s[g] = d;
                        }
#pragma unroll
                        for (int ofs = LPT / 2; ofs > 0; ofs >>= 1)
#pragma unroll
                            for (int g = 0; g < GE; g++) s[g] += __shfl_xor_sync(gmask, s[g], ofs);
#pragma unroll
                        for (int g = 0; g < GE; g++) {
                            const float mn = fmaxf(m[g], s[g]);
                            const float corr = exp2f(m[g] - mn), pe = exp2f(s[g] - mn);
                            l[g] = fmaf(l[g], corr, pe);
#pragma unroll
                            for (int e = 0; e < 8; e++) o[g][e] = fmaf(o[g][e], corr, pe * vv[u][e]);
                            m[g] = mn;
                        }
                    }
                }
            }
            // merge the token slots of this CTA
#pragma unroll
            for (int g = 0; g < GE; g++) {
                if (sub == 0) {
                    sm_m[slot * GE + g] = m[g];
                    sm_l[slot * GE + g] = l[g];
                }
                float *dst = sm_o + ((size_t)slot * GE + g) * HD + sub * 8;
                *reinterpret_cast<float4 *>(dst) = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
                *reinterpret_cast<float4 *>(dst + 4) = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
            }
            csync();
            for (int idx = tid; idx < GE * HD; idx += kStepConsumers) {
                const int g = idx / HD, d = idx - g * HD;
                float M = -INFINITY;
                for (int w = 0; w < SLOTS; w++) M = fmaxf(M, sm_m[w * GE + g]);
                float L = 0.f, acc = 0.f;
                for (int w = 0; w < SLOTS; w++) {
                    const float lw = sm_l[w * GE + g];
                    if (lw > 0.f) {
                        const float f = exp2f(sm_m[w * GE + g] - M);
                        L = fmaf(lw, f, L);
                        acc = fmaf(sm_o[((size_t)w * GE + g) * HD + d], f, acc);
                    }
                }
                po[(size_t)g * a.chunks * HD + d] = acc;
                if (d == 0) {
                    pml[(size_t)g * a.chunks * 2 + 0] = M;  // log2 domain
                    pml[(size_t)g * a.chunks * 2 + 1] = L;
                }
            }
        }
        // whoever completes the item group merges its chunks (nobody waits for anybody)
        __threadfence();
        csync();
        if (tid == 0) {
            unsigned *ctr = a.counters + (seq * a.n_kv_heads + kvh) * a.head_groups + hg;
            const unsigned old = atomicAdd(ctr, 1u);
            const int last = (old == (unsigned)a.chunks - 1u);
            if (last) *ctr = 0u;  // ready for the next use
            *flag = last;
        }
        csync();
        if (*flag) {
            __threadfence();
            for (int g = warp; g < GE; g += kStepWarps) {
                const float *pm = a.part_ml + (size_t)(seq * a.n_heads + h0 + g) * a.chunks * 2;
                float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
                if (lane < a.chunks) {
                    m0 = __ldcg(pm + 2 * lane);
                    l0 = __ldcg(pm + 2 * lane + 1);
                }
                if (lane + 32 < a.chunks) {  // chunks <= 64
                    m1 = __ldcg(pm + 2 * (lane + 32));
                    l1 = __ldcg(pm + 2 * (lane + 32) + 1);
                }
                float M = fmaxf(m0, m1);
#pragma unroll
                for (int ofs = 16; ofs > 0; ofs >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, ofs));
                const float f0 = (l0 > 0.f) ? exp2f(m0 - M) : 0.f, f1 = (l1 > 0.f) ? exp2f(m1 - M) : 0.f;
                mg_f[g * 64 + lane] = f0;
                mg_f[g * 64 + lane + 32] = f1;
                float L = fmaf(l0, f0, l1 * f1);
#pragma unroll
                for (int ofs = 16; ofs > 0; ofs >>= 1) L += __shfl_xor_sync(0xffffffffu, L, ofs);
                if (lane == 0) mg_L[g] = L;
            }
            csync();
            for (int idx = tid; idx < GE * HD; idx += kStepConsumers) {
                const int g = idx / HD, d = idx - g * HD, h = h0 + g;
                const float *pall = a.part_o + (size_t)(seq * a.n_heads + h) * a.chunks * HD;
                float acc = 0.f;
#pragma unroll 8
                for (int s = 0; s < a.chunks; s++) acc = fmaf(__ldcg(pall + (size_t)s * HD + d), mg_f[g * 64 + s], acc);
                const float L = mg_L[g];
                const float outv = (L > 0.f) ? acc / L : 0.f;
                if (a.out) a.out[(size_t)(seq * a.n_heads + h) * HD + d] = outv;
                if (a.stage.img) {
                    unsigned short *xb;
                    int NC, col0;
                    a.stage.locate(seq, xb, NC, col0);
                    stage_store1(xb, NC, col0, h * HD + d, outv);
                }
            }
        }
        csync();  // the scratch is reused by the next item
    }
}

// ───────────────────────────── weight stream ──────────────────────────────────────────────
// Every computing warp streams its own tiles: it owns kStepRingDepth ring slots, and right after it has pulled a
// tile into registers it issues the bulk copy of the tile kStepRingDepth rounds ahead into the slot it just freed.
// The "cursor" enumerates the warp's tiles in consumption order across phases (descriptors of the next phases are
// kept in a small shared-memory window), so the copies run ahead of the grid barriers.
struct StreamDesc {
    const uint8_t *w[3];
    int seg_type[3];
    int rt_begin[4];
    int kind, nb, kin_log2, tpt, total_rt, rot;
    int n_ctasks;
};
static_assert(sizeof(StreamDesc) == 80, "shared-memory carve-up assumes 80-byte stream descriptors");
constexpr int kStreamWindow = 8;  // descriptors resident at a time (power of two)

struct WarpStream {
    int dbg;
    volatile unsigned *err_s;  // the CTA's failed-state flag: nothing is copied any more once it is set
    int ph, j;           // cursor: phase, tile inside the task
    int task;            // cursor: CTA task (-1: the phase's first, not computed yet)
    unsigned cl;         // claimed-task entries the cursor has read so far
    uint32_t claim0;     // shared addresses: claim barriers, the claimed task ids
    const int *claimed;
    unsigned fetched, consumed;
    uint32_t full0;      // shared address of this warp's first "tile landed" barrier
    uint32_t slot0;      // shared address of this warp's first ring slot
    int slot_bytes;
};

__device__ __forceinline__ void stream_desc_load(StreamDesc *dst, const StepPhase *src) {
    dst->kind = src->kind;
    if (src->kind != STEP_GEMV) return;
    const GemvParams &g = src->g;
#pragma unroll
    for (int s = 0; s < 3; s++) {
        dst->w[s] = g.w[s];
        dst->seg_type[s] = g.seg_type[s];
    }
#pragma unroll
    for (int s = 0; s < 4; s++) dst->rt_begin[s] = g.rt_begin[s];
    dst->nb = g.nb;
    dst->kin_log2 = 31 - __clz(g.kin);
    dst->tpt = g.tpt;
    dst->total_rt = g.total_rt;
    dst->rot = src->rot;
    dst->n_ctasks = g.n_ctasks;
}

__device__ __forceinline__ int step_first_task(int rot) { return (int)((blockIdx.x + gridDim.x - (unsigned)rot) % gridDim.x); }

// CTA tasks of a phase: the first is fixed ((blockIdx + grid - rot) % grid), the following ones are claimed from a
// per-phase device counter by warp 0 and handed to the other warps through a small ring in shared memory
// (claim barrier j % kStepClaimRing completes when entry j is published; an id >= n_ctasks ends the phase).
// Every warp reads every entry twice, in the same order: once with its cursor, once when it gets to the task.
__device__ __forceinline__ bool claim_ready(uint32_t claim0, unsigned j) {
    return mbar_try_wait(claim0 + 8u * (j % kStepClaimRing), (j / kStepClaimRing) & 1u);
}

// Issues the copy of the warp's next tile, if the descriptor window and the claimed tasks reach that far.
// Warp-uniform.
__device__ __forceinline__ bool fetch_next(WarpStream &ws, const StreamDesc *stream, int hi, int warp, int lane, uint32_t token = 0) {
    if (*ws.err_s) return false;
    while (ws.ph <= hi) {
        const StreamDesc &sd = stream[ws.ph & (kStreamWindow - 1)];
        if (sd.kind == STEP_GEMV) {
            if (ws.task < 0) ws.task = step_first_task(sd.rot);
            if (ws.task < sd.n_ctasks) {
                const int kl = sd.kin_log2, kin = 1 << kl, G = kStepWarps >> kl;
                const int grp = warp >> kl, kj = warp & (kin - 1);
                const int R = ws.task * G + grp, sb = kj * sd.tpt + ws.j;
                if (R < sd.total_rt && ws.j < sd.tpt && sb < sd.nb) {
                    int s = 0;
                    if (R >= sd.rt_begin[1]) s = 1;
                    if (R >= sd.rt_begin[2]) s = 2;
                    const unsigned bytes = (unsigned)tile_bytes(sd.seg_type[s]);
                    const uint8_t *src = sd.w[s] + ((size_t)(R - sd.rt_begin[s]) * sd.nb + sb) * (size_t)bytes;
                    const unsigned slot = ws.fetched % kStepRingDepth;
                    if (lane == 0) {
                        // `token` is the last word the warp read from the slot being refilled: folding it (as zero)
                        // into the copy size keeps the copy behind the completion of those reads
                        uint32_t zero;
                        asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(token));
                        mbar_expect_tx(ws.full0 + 8u * slot, bytes);
                        bulk_g2s(ws.slot0 + slot * (unsigned)ws.slot_bytes, src, bytes + zero, ws.full0 + 8u * slot);
                    }
                    ws.fetched++;
                    ws.j++;
                    return true;
                }
                // this warp is done with the task: the next one has to be claimed already
                if (!claim_ready(ws.claim0, ws.cl)) return false;
                ws.task = ws.claimed[ws.cl % kStepClaimRing];
                ws.cl++;
                ws.j = 0;
                if (ws.task < sd.n_ctasks) continue;
            }
        }
        ws.ph++;
        ws.j = 0;
        ws.task = -1;
    }
    return false;
}

// One tile: wait for it, pull it into registers, refill the slot, compute.
template <int NC>
__device__ __forceinline__ void consume_tile(WarpStream &ws, const StreamDesc *stream, int hi, int type, int sb, const XView<NC> &xv,
                                             int warp, int lane, float (&acc)[(NC + 7) / 8][4], float (&macc)[(NC + 7) / 8][4],
                                             unsigned *sync, volatile unsigned *err_s) {
    if (*err_s) return;  // failed state: no waits, no copies, the counters stay as they are
    if (ws.fetched <= ws.consumed) {  // the cursor was held back (descriptor window, unclaimed task): catch up now
        const long long t0 = clock64();
        while (ws.fetched <= ws.consumed && !fetch_next(ws, stream, hi, warp, lane)) {
            if (*err_s) return;
            if (clock64() - t0 > kWaitLimitClk) {
                step_fail(sync, err_s, STEP_ERR_CURSOR);
                return;
            }
        }
    }
    const unsigned slot = ws.consumed % kStepRingDepth, par = (ws.consumed / kStepRingDepth) & 1u;
    const bool ok = mbar_wait(ws.full0 + 8u * slot, par, sync, err_s, STEP_ERR_FULL);
    const uint32_t t = ws.slot0 + slot * (unsigned)ws.slot_bytes;
    if (!ok) return;  // the tile stays "in flight": the exit path waits for it once more
    ws.consumed++;
    if (type == 12) {
        TileRegs<12> r;
        ring_load(r, t, lane);
        __syncwarp();
        while (ws.fetched < ws.consumed + kStepRingDepth && fetch_next(ws, stream, hi, warp, lane, r.q[3].w)) {
        }
        if (!(ws.dbg & 1)) compute_tile<NC>(r, sb, xv, lane, acc, macc);
    } else if (type == 14) {
        TileRegs<14> r;
        ring_load(r, t, lane);
        __syncwarp();
        while (ws.fetched < ws.consumed + kStepRingDepth && fetch_next(ws, stream, hi, warp, lane, r.d01)) {
        }
        if (!(ws.dbg & 1)) compute_tile<NC>(r, sb, xv, lane, acc, macc);
    } else {
        TileRegs<8> r;
        ring_load(r, t, lane);
        __syncwarp();
        while (ws.fetched < ws.consumed + kStepRingDepth && fetch_next(ws, stream, hi, warp, lane, r.d1.w)) {
        }
        if (!(ws.dbg & 1)) compute_tile<NC>(r, sb, xv, lane, acc, macc);
    }
}

// ───────────────────────────── GEMV phase ─────────────────────────────────────────────────
// A task is one row tile, worked on by a group of `kin` warps that split K; the groups of a CTA run independently.
// After its tiles a warp leaves its partial sums in shared memory and signals; one warp of the group (rotating)
// waits for the group's signals and finishes the rows: fixed-order sum over the K chunks and limbs, input scale,
// epilogue.  No CTA-wide barrier inside the loop.
template <int NB>
__device__ __forceinline__ void gemv_phase(const GemvParams &p, int rot, int need_xs, uint8_t *smem, const StepSmem<NB> &L,
                                           WarpStream &ws, const StreamDesc *stream, int hi, unsigned &it_total, uint32_t img_bar,
                                           unsigned &img_uses, uint32_t fbar0, unsigned &cl, int *claimed, unsigned *sync,
                                           volatile unsigned *err_s, int tid, unsigned long long *tl, int ph) {
    constexpr int NC = 3 * NB, NT = (NC + 7) / 8, LDC = StepSmem<NB>::LDC;
    const int warp = tid >> 5, lane = tid & 31;
    const int K = p.K;
    unsigned short *xb = reinterpret_cast<unsigned short *>(smem);
    unsigned short *xs = xb + (size_t)K * NC;
    float *frag = reinterpret_cast<float *>(smem + L.cs);  // [kStepFragBufs][kStepWarps][16][LDC]
    float *scale_s = reinterpret_cast<float *>(smem + L.scale_s);

    // RMSNorm scale of the input from the producer's per-task sums of squares (fixed summation order)
    if (warp < NB) {
        float sc = 1.f;
        if (p.ss_parts) {
            float s = 0.f;
            for (int i = lane; i < p.n_parts; i += 32) s += __ldcg(p.ss_parts + (size_t)warp * p.ss_ld + i);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            sc = __fdiv_rn(1.f, (float)sqrt((double)__fadd_rn(__fdiv_rn(s, (float)p.scale_n), p.eps)));
        }
        if (lane == 0) scale_s[warp] = sc;
    }
    // the staged activation (bulk copy issued right after the previous grid barrier)
    mbar_wait(img_bar, img_uses & 1u, sync, err_s, STEP_ERR_IMAGE);
    img_uses++;
    STEP_STAMP(tl, ph, 1);
    if (need_xs) {
        // sums of x over 32 columns, from the limbs (hi + mid + lo is x exactly): eight threads per sum
        const int total = (K / 4) * NB;
        for (int item = tid; item < total; item += kStepConsumers) {
            const int b = item / (K / 4), r = item - b * (K / 4), sub32 = r >> 3, q = r & 7;
            const int s16 = sub32 * 2 + (q >> 2), c = q & 3;
            float x4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int k = 2; k >= 0; k--) {  // lo + mid first, then hi
                const uint2 u = *reinterpret_cast<const uint2 *>(xb + ((size_t)(s16 * NC + 3 * b + k) * 4 + c) * 4);
                x4[0] += __uint_as_float(u.x << 16);
                x4[1] += __uint_as_float(u.x & 0xFFFF0000u);
                x4[2] += __uint_as_float(u.y << 16);
                x4[3] += __uint_as_float(u.y & 0xFFFF0000u);
            }
            float s = (x4[0] + x4[1]) + (x4[2] + x4[3]);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            unsigned short s3[3];
            split3(s, s3[0], s3[1], s3[2]);
            if (q == 0) {
#pragma unroll
                for (int k = 0; k < 3; k++) xs[xs_index(sub32, NC, 3 * b + k)] = s3[k];
            }
        }
    }
    csync();
    STEP_STAMP(tl, ph, 2);

    XView<NC> xv;
    {
        const int r8 = lane >> 2, c = lane & 3;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int colc = min(nt * 8 + r8, NC - 1);
            xv.xb_lane[nt] = xb + (colc * 4 + c) * 4;
            xv.xs_lane[nt] = reinterpret_cast<const uint32_t *>(xs) + colc * 4 + c;
        }
    }
    float acc[NT][4], macc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nt][i] = macc[nt][i] = 0.f;

    const int kin = p.kin, G = p.groups;
    const int grp = warp / kin, kj = warp - grp * kin, sb0 = kj * p.tpt;
    const int rows_out = (p.epi == EPI_SILU_PAIR) ? 8 : 16;
    unsigned *task_counter = sync + 2 + ph;
    const uint32_t claim0 = ws.claim0, cfree0 = claim0 + 8u * kStepClaimRing;
    int hist[kStepFinishLag];  // CTA tasks of the last iterations, for the late finish
#pragma unroll
    for (int h = 0; h < kStepFinishLag; h++) hist[h] = -1;
    // Finishes a task of this warp's group (CTA task T, global iteration itn): waits for the group's partial sums
    // (normally long there: it runs kStepFinishLag iterations late), adds them in fixed order, applies the epilogue,
    // frees the buffer.
    auto finish = [&](int T, unsigned itn) {
        const int R = T * G + grp;
        const bool row_ok = R < p.total_rt;
        const int seg = seg_of(p, min(R, p.total_rt - 1));
        const unsigned buf = itn % kStepFragBufs, par = (itn / kStepFragBufs) & 1u;
        if (lane < kin) mbar_wait(fbar0 + 8u * (kStepFragBufs * (grp * kin + lane) + buf), par, sync, err_s, STEP_ERR_PART_READY);
        __syncwarp();
        const float *gfrag = frag + ((size_t)buf * kStepWarps + grp * kin) * 16 * LDC;
        const int total = rows_out * NB;
        for (int base = 0; base < total; base += 32) {
            const int idx = base + lane;
            float sq = 0.f;
            int b = 0;
            if (idx < total && row_ok) {
                b = idx / rows_out;
                const int row = idx - b * rows_out;
                const int tile_in_seg = R - p.rt_begin[seg];
                float v = 0.f, v2 = 0.f;
                for (int k2 = 0; k2 < kin; k2++) {
                    const float *cr = gfrag + ((size_t)k2 * 16 + row) * LDC + 3 * b;
                    v += (cr[2] + cr[1]) + cr[0];
                    if (p.epi == EPI_SILU_PAIR) {
                        const float *cu = cr + 8 * LDC;
                        v2 += (cu[2] + cu[1]) + cu[0];
                    }
                }
                const float sc = scale_s[b];
                v = __fmul_rn(v, sc);
                const int orow = tile_in_seg * rows_out + row;
                if (orow < p.rows[seg]) {
                    float o = v;
                    if (p.epi == EPI_SILU_PAIR) {
                        o = __fmul_rn(silu_ref(v), __fmul_rn(v2, sc));
                    } else if (p.epi == EPI_RESID_NORM) {
                        o = __fadd_rn(__ldcg(p.resid + (size_t)b * p.ldx + orow), v);
                        p.x_out[(size_t)b * p.ldx + orow] = o;
                        sq = __fmul_rn(o, o);
                        o = __fmul_rn(p.normw_next[orow], o);
                    }
                    if (p.epi != EPI_RESID_NORM && p.out[seg]) p.out[seg][(size_t)b * p.ld_out + orow] = o;
                    if (p.img_next.img) {
                        unsigned short *nxb;
                        int nNC, ncol0;
                        p.img_next.locate(b, nxb, nNC, ncol0);
                        stage_store1(nxb, nNC, ncol0, orow, o);
                    }
                }
            }
            if (p.epi == EPI_RESID_NORM) {  // sum of squares of the row tile (16 rows = 16 lanes), fixed tree
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (idx < total && row_ok && (lane & 15) == 0) p.ss_out[(size_t)b * p.ss_out_ld + R] = sq;
            }
        }
        __syncwarp();
        if (lane < kin) mbar_arrive(fbar0 + 8u * (kStepFragBufs * (kStepWarps + grp * kin + lane) + buf));
    };

    int T = step_first_task(rot);
    for (int i = 0; T < p.n_ctasks; i++, it_total++) {
        // warp 0 claims the CTA's next task now; the id is published after this task's first tile, so the round
        // trip to the counter is hidden
        unsigned claimed_raw = 0;
        const bool publisher = (warp == 0);
        if (publisher) {
            mbar_wait(cfree0 + 8u * (cl % kStepClaimRing), ((cl / kStepClaimRing) & 1u) ^ 1u, sync, err_s, STEP_ERR_CLAIM_FREE);
            if (lane == 0) claimed_raw = atomicAdd(task_counter, 1u);
        }
        const int R = T * G + grp;
        bool published = false;
        if (R < p.total_rt) {
            const int type = p.seg_type[seg_of(p, R)];
            for (int j = 0; j < p.tpt; j++) {
                const int sb = sb0 + j;
                if (sb < p.nb) consume_tile<NC>(ws, stream, hi, type, sb, xv, warp, lane, acc, macc, sync, err_s);
                if (publisher && !published) {
                    if (lane == 0) {
                        claimed[cl % kStepClaimRing] = (int)(gridDim.x + claimed_raw);
                        mbar_arrive(claim0 + 8u * (cl % kStepClaimRing));
                    }
                    published = true;
                }
            }
        }
        if (publisher && !published && lane == 0) {
            claimed[cl % kStepClaimRing] = (int)(gridDim.x + claimed_raw);
            mbar_arrive(claim0 + 8u * (cl % kStepClaimRing));
        }
        if (!(ws.dbg & 2)) {
            // partial sums -> shared memory, once the finisher of kStepFragBufs tasks ago has let go of the buffer
            const unsigned buf = it_total % kStepFragBufs, par = (it_total / kStepFragBufs) & 1u;
            mbar_wait(fbar0 + 8u * (kStepFragBufs * (kStepWarps + warp) + buf), par ^ 1u, sync, err_s, STEP_ERR_PART_FREE);
            {
                float *mine = frag + ((size_t)buf * kStepWarps + warp) * 16 * LDC;
                const int r8 = lane >> 2, c = lane & 3;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    if (nt * 8 + 2 * c < LDC) {
                        *reinterpret_cast<float2 *>(mine + r8 * LDC + nt * 8 + 2 * c) =
                            make_float2(acc[nt][0] - macc[nt][0], acc[nt][1] - macc[nt][1]);
                        *reinterpret_cast<float2 *>(mine + (r8 + 8) * LDC + nt * 8 + 2 * c) =
                            make_float2(acc[nt][2] - macc[nt][2], acc[nt][3] - macc[nt][3]);
                    }
                    acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                    macc[nt][0] = macc[nt][1] = macc[nt][2] = macc[nt][3] = 0.f;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(fbar0 + 8u * (kStepFragBufs * warp + buf));
            // the rows of an earlier task are finished by one warp of the group (rotating), late enough that it
            // normally finds every partial sum in place and waits for nobody
            const int Te = hist[kStepFinishLag - 1];
            if (Te >= 0 && kj == ((i - kStepFinishLag) & (kin - 1))) finish(Te, it_total - (unsigned)kStepFinishLag);
#pragma unroll
            for (int h = kStepFinishLag - 1; h > 0; h--) hist[h] = hist[h - 1];
            hist[0] = T;
        }
        // the CTA's next task
        mbar_wait(claim0 + 8u * (cl % kStepClaimRing), (cl / kStepClaimRing) & 1u, sync, err_s, STEP_ERR_CLAIM);
        T = *err_s ? p.n_ctasks : claimed[cl % kStepClaimRing];
        if (ws.cl <= cl) {
            // The cursor has not read this entry yet: it has issued every tile this warp has in the task just
            // finished (possibly none, in which case it may still stand in an earlier phase).  Hand the entry over
            // now, because once this warp has signalled it as read, warp 0 may reuse the ring slot.
            ws.cl = cl + 1u;
            ws.j = 0;
            if (T < p.n_ctasks) {
                ws.ph = ph;
                ws.task = T;
            } else {
                ws.ph = ph + 1;
                ws.task = -1;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(cfree0 + 8u * (cl % kStepClaimRing));
        cl++;
        // keep the ring full across the task (and phase) boundary
        while (ws.fetched < ws.consumed + kStepRingDepth && fetch_next(ws, stream, hi, warp, lane)) {
        }
        if (T >= p.n_ctasks) {
            it_total++;
            // flush the tasks whose finish was still pending
            if (!(ws.dbg & 2)) {
#pragma unroll
                for (int h = kStepFinishLag - 1; h >= 0; h--) {
                    const int e = i - h;  // iteration index of hist[h]
                    if (hist[h] >= 0 && kj == (e & (kin - 1))) finish(hist[h], it_total - 1u - (unsigned)h);
                }
            }
            break;
        }
    }
}

// ───────────────────────────── the kernel ─────────────────────────────────────────────────
template <typename T, int HD, int GE, int NB>
__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const StepParams sp) {
    extern __shared__ __align__(128) uint8_t smem[];
    const StepSmem<NB> L(sp.img_cap, sp.slot_bytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    StepPhase *desc = reinterpret_cast<StepPhase *>(smem + L.desc);
    StreamDesc *stream = reinterpret_cast<StreamDesc *>(smem + L.stream);
    const uint32_t bars = smem_u32(smem + L.bars);
    // barriers: [ring: kStepWarps x depth][partials ready: kStepWarps x bufs][partials free: kStepWarps x bufs][image]
    //           [task claimed: ring][task entry read by all warps: ring]
    const uint32_t full0 = bars, fbar0 = bars + 8u * kStepRingSlots, img_bar = fbar0 + 8u * 2u * kStepFragBufs * kStepWarps;
    const uint32_t claim0 = img_bar + 8u;
    int *claimed = reinterpret_cast<int *>(smem + L.flags + 16);
    volatile unsigned *err_s = reinterpret_cast<volatile unsigned *>(smem + L.flags);
    volatile int *flag = reinterpret_cast<volatile int *>(smem + L.flags + 4);
    if (tid == 0) {
        for (int i = 0; i < kStepRingSlots + 2 * (int)kStepFragBufs * kStepWarps + 1 + (int)kStepClaimRing; i++) mbar_init(bars + 8u * i, 1);
        for (unsigned i = 0; i < kStepClaimRing; i++) mbar_init(claim0 + 8u * (kStepClaimRing + i), kStepWarps);
        *err_s = 0;
        *flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    // descriptor of the first phase, and the first window of stream descriptors
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(sp.phases);
        uint4 *dst = reinterpret_cast<uint4 *>(desc);
        for (int i = tid; i < (int)(sizeof(StepPhase) / 16); i += kStepThreads) dst[i] = src[i];
    }
    int hi = min(kStreamWindow - 2, sp.n_phases - 1);  // newest phase whose stream descriptor is resident
    if (tid >= 64 && tid - 64 <= hi) stream_desc_load(&stream[(tid - 64) & (kStreamWindow - 1)], sp.phases + (tid - 64));
    __syncthreads();

    WarpStream ws;
    ws.ph = 0;
    ws.task = -1;
    ws.cl = 0;
    ws.claim0 = claim0;
    ws.claimed = claimed;
    ws.j = 0;
    ws.fetched = 0;
    ws.consumed = 0;
    ws.full0 = full0 + 8u * (unsigned)(warp * kStepRingDepth);
    ws.slot0 = smem_u32(smem + L.ring) + (unsigned)(warp * kStepRingDepth) * (unsigned)sp.slot_bytes;
    ws.slot_bytes = sp.slot_bytes;
    ws.dbg = sp.dbg;
    ws.err_s = err_s;
    while (ws.fetched < (unsigned)kStepRingDepth && fetch_next(ws, stream, hi, warp, lane)) {
    }
    unsigned img_uses = 0, barriers = 0, it_total = 0, cl = 0;
    if (tid == 0 && desc[0].kind == STEP_GEMV) {
        mbar_expect_tx(img_bar, desc[0].g.img_bytes);
        bulk_g2s(smem_u32(smem), desc[0].g.ximg, desc[0].g.img_bytes, img_bar);
    }
    for (int ph = 0; ph < sp.n_phases; ph++) {
        const StepPhase &d = desc[ph & 1];
        STEP_STAMP(sp.timeline, ph, 0);
        if (ph + 1 < sp.n_phases) {  // next descriptor (immutable for the launch): fetched a phase ahead
            const uint4 *src = reinterpret_cast<const uint4 *>(sp.phases + ph + 1);
            uint4 *dst = reinterpret_cast<uint4 *>(&desc[(ph + 1) & 1]);
            if (tid < (int)(sizeof(StepPhase) / 16)) dst[tid] = src[tid];
        }
        {  // slide the stream-descriptor window (the entry it overwrites belongs to a finished phase)
            const int want = min(ph + kStreamWindow - 2, sp.n_phases - 1);
            const int q = hi + 1 + (tid - 64);
            if (tid >= 64 && q <= want) stream_desc_load(&stream[q & (kStreamWindow - 1)], sp.phases + q);
            // visible to the cursors after the next CTA barrier; until then they stop at the old limit
        }
        if (d.kind == STEP_GEMV) {
            gemv_phase<NB>(d.g, d.rot, d.need_xs, smem, L, ws, stream, hi, it_total, img_bar, img_uses, fbar0, cl, claimed, sp.sync,
                           err_s, tid, sp.timeline, ph);
        } else {
            attn_phase<T, HD, GE>(d.a, smem, reinterpret_cast<float *>(smem + L.mg_f), reinterpret_cast<float *>(smem + L.mg_L),
                                  flag, tid);
        }
        STEP_STAMP(sp.timeline, ph, 3);
        if (ph + 1 == sp.n_phases) break;
        csync();  // this CTA's outputs are written and its shared memory is free
        hi = min(ph + kStreamWindow - 2, sp.n_phases - 1);
        STEP_STAMP(sp.timeline, ph, 4);
        if (tid == 0) {
            grid_sync(sp.sync, ++barriers, err_s);
            STEP_STAMP(sp.timeline, ph, 5);
            const StepPhase &nx = desc[(ph + 1) & 1];
            if (nx.kind == STEP_GEMV) {
                fence_proxy_async();  // the image was written through the generic proxy (by other CTAs)
                mbar_expect_tx(img_bar, nx.g.img_bytes);
                bulk_g2s(smem_u32(smem), nx.g.ximg, nx.g.img_bytes, img_bar);
            }
        } else {
            ++barriers;
        }
        csync();
    }
    // Never leave with a copy in flight (only possible after a wait has given up: otherwise every tile that was
    // fetched has been consumed).
    while (ws.consumed < ws.fetched) {
        const unsigned slot = ws.consumed % kStepRingDepth, par = (ws.consumed / kStepRingDepth) & 1u;
        const long long t0 = clock64();
        while (!mbar_try_wait(ws.full0 + 8u * slot, par) && clock64() - t0 < kWaitLimitClk) {
        }
        ws.consumed++;
    }
}

// ───────────────────────────── host ───────────────────────────────────────────────────────
void step_task_geometry(int grid, int K, int total_rt, int *kin_out, int *tpt_out, int *n_ctasks_out) {
    const int nb = K / 256;
    long best_cost = -1;
    int best = 1;
    for (int d = 1; d <= kStepWarps && d <= std::max(1, nb); d *= 2) {
        const int groups = kStepWarps / d, tpt = (nb + d - 1) / d, nct = (total_rt + groups - 1) / groups;
        // time on the busiest CTA in units of one tile: its tiles plus a fixed cost per task (hand-over of the
        // partial sums, epilogue), which measured about two tiles
        static const int task_cost = getenv("JUNO_STEP_TASK_COST") ? atoi(getenv("JUNO_STEP_TASK_COST")) : 2;
        const long cost = (long)((nct + grid - 1) / grid) * (tpt + task_cost);
        if (best_cost < 0 || cost <= best_cost) {                 // ties: the wider split (smaller tasks)
            best_cost = cost;
            best = d;
        }
    }
    if (const char *e = getenv("JUNO_STEP_KIN")) {  // tuning: cap the K split
        const int cap = atoi(e);
        while (best > 1 && best > cap) best >>= 1;
    }
    const int groups = kStepWarps / best;
    *kin_out = best;
    *tpt_out = (nb + best - 1) / best;
    *n_ctasks_out = (total_rt + groups - 1) / groups;
}

static size_t step_attn_scratch_bytes(int hd, int ge) {
    const int slots = kStepWarps * (32 / (hd / 8));
    return ((size_t)ge * hd + 2 * (size_t)slots * ge + (size_t)slots * ge * hd) * 4;
}

static int step_group(int n_heads, int n_kv_heads) {
    if (n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
    const int G = n_heads / n_kv_heads;
    if (G % 4 == 0) return 4;
    if (G == 2) return 2;
    return 0;
}

bool step_supported(const juno_ctx *ctx, int n, int hd, int n_heads, int n_kv_heads, int max_K, int max_tile_bytes) {
    if (n != 1) return false;  // one sequence per step for now
    if (hd != 64 && hd != 128) return false;
    const int ge = step_group(n_heads, n_kv_heads);
    if (!ge) return false;
    const size_t img = (size_t)max_K * 6 * n + (((size_t)(max_K / 32) * 3 * n * 2 + 15) & ~(size_t)15);
    const size_t cap = (std::max(img, step_attn_scratch_bytes(hd, ge)) + 127) & ~(size_t)127;
    const StepSmem<1> L((unsigned)cap, (max_tile_bytes + 15) & ~15);
    return (size_t)L.total <= ctx->smem_optin;
}

int step_record_gemv(juno_ctx *ctx, const GemvArgs &a) {
    StepRecorder *rec = ctx->step_rec;
    JUNO_REQUIRE(a.batch == rec->n, "step recorder: batch %d != %d", a.batch, rec->n);
    JUNO_REQUIRE(gemv_batch_chunk(ctx, a.K, a.batch) == a.batch, "step recorder: activation of K=%d does not fit one chunk", a.K);
    StepPhase ph;
    memset(&ph, 0, sizeof(ph));
    ph.kind = STEP_GEMV;
    int total_rt = 0;
    for (int s = 0; s < a.nseg; s++) total_rt += a.seg[s].row_tiles;
    int kin, tpt, nct;
    step_task_geometry(rec->grid, a.K, total_rt, &kin, &tpt, &nct);
    JUNO_TRY(gemv_fill_params(ctx, a, 0, a.batch, 0, kin, tpt, kStepWarps / kin, nct, &ph.g));
    ph.g.counters = nullptr;
    for (int s = 0; s < a.nseg; s++) ph.need_xs |= (ph.g.seg_type[s] == 12);
    ph.rot = rec->next_rot;
    rec->next_rot = (rec->next_rot + nct) % rec->grid;
    rec->phases.push_back(ph);
    return JUNO_OK;
}

int step_record_attn(juno_ctx *ctx, const AttnArgs &a) {
    StepRecorder *rec = ctx->step_rec;
    const juno_kvpool *pool = a.pool;
    const int ge = step_group(a.n_heads, pool->n_kv_heads);
    JUNO_REQUIRE(ge > 0 && a.rope_cs && a.knew && a.vnew && a.n == rec->n, "step recorder: unsupported attention call");
    StepPhase ph;
    memset(&ph, 0, sizeof(ph));
    ph.kind = STEP_ATTN;
    StepAttn &s = ph.a;
    s.k = pool->k;
    s.v = pool->v;
    s.kw = pool->k;
    s.vw = pool->v;
    s.table = pool->d_table;
    s.max_pages_per_seq = pool->max_pages_per_seq;
    s.n_pages = pool->n_pages;
    s.n_kv_heads = pool->n_kv_heads;
    s.n_heads = a.n_heads;
    s.layer = a.layer;
    s.n = a.n;
    s.head_groups = (a.n_heads / pool->n_kv_heads) / ge;
    s.chunks = std::max(1, std::min(64, rec->grid / std::max(1, a.n * pool->n_kv_heads * s.head_groups)));
    s.q = a.q;
    s.ldq = a.ldq ? a.ldq : a.n_heads * pool->head_dim;
    s.knew = a.knew;
    s.vnew = a.vnew;
    s.ldkv = a.ldkv;
    s.slots = a.slots;
    s.seq_lens = a.seq_lens;
    s.rope_cs = a.rope_cs;
    s.part_o = a.part_o;  // the caller's scratch holds n * n_heads * chunks * (head_dim + 2) floats (chunks <= 64 per head group)
    s.part_ml = a.part_o + (size_t)a.n * a.n_heads * s.chunks * pool->head_dim;
    s.counters = a.merge_counters;
    s.out = a.out;
    if (a.stage_img) {
        s.stage.img = a.stage_img;
        s.stage.K = a.n_heads * pool->head_dim;
        s.stage.batch = a.n;
        s.stage.bc = a.stage_bc;
        s.stage.b0 = 0;
        s.stage.chunk_stride = a.stage_chunk_stride;
    }
    JUNO_REQUIRE(s.counters, "step recorder: attention needs its merge counters");
    rec->phases.push_back(ph);
    return JUNO_OK;
}

template <typename T, int HD, int GE>
static int step_launch_inst(juno_ctx *ctx, const StepPlan &plan, const StepParams &sp, cudaStream_t st) {
    auto kernel = decode_step_kernel<T, HD, GE, 1>;
    static std::mutex mu;
    static bool configured[16] = {false};
    {
        std::lock_guard<std::mutex> g(mu);
        const int dev = ctx->device & 15;
        if (!configured[dev]) {
            JUNO_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin));
            configured[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JUNO_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, sp));
    return JUNO_OK;
}

template <typename T>
static int step_launch_t(juno_ctx *ctx, const StepPlan &plan, const StepParams &sp, cudaStream_t st) {
    if (plan.hd == 64 && plan.ge == 2) return step_launch_inst<T, 64, 2>(ctx, plan, sp, st);
    if (plan.hd == 64 && plan.ge == 4) return step_launch_inst<T, 64, 4>(ctx, plan, sp, st);
    if (plan.hd == 128 && plan.ge == 2) return step_launch_inst<T, 128, 2>(ctx, plan, sp, st);
    if (plan.hd == 128 && plan.ge == 4) return step_launch_inst<T, 128, 4>(ctx, plan, sp, st);
    set_error("decode step kernel: head_dim %d with %d heads per group is not built", plan.hd, plan.ge);
    return JUNO_ERR_UNSUPPORTED;
}

static void step_print_timeline(const StepPlan &plan, cudaStream_t st);

int launch_step(juno_ctx *ctx, const StepPlan &plan, cudaStream_t st) {
    StepParams sp;
    sp.phases = plan.d_phases;
    sp.n_phases = plan.n_phases;
    sp.sync = plan.d_sync;
    sp.slot_bytes = plan.slot_bytes;
    sp.img_cap = plan.img_cap;
    sp.timeline = plan.d_timeline;
    {
        const char *e = getenv("JUNO_STEP_DEBUG");
        sp.dbg = e ? atoi(e) : 0;
    }
    JUNO_CUDA_TRY(cudaMemsetAsync(plan.d_sync, 0, (size_t)(2 + plan.n_phases) * 4, st));
    {
        ProfScope prof(ctx, st, PROF_STEP, plan.algo_bytes);
        JUNO_TRY(plan.kv_f32 ? step_launch_t<float>(ctx, plan, sp, st) : step_launch_t<__half>(ctx, plan, sp, st));
    }
    JUNO_CUDA_TRY(cudaMemcpyAsync(plan.h_err, plan.d_sync + 1, 4, cudaMemcpyDeviceToHost, st));
    ctx->kernel_launches++;
    if (plan.d_timeline) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(st, &cap);
        if (cap == cudaStreamCaptureStatusNone) step_print_timeline(plan, st);
    }
    return JUNO_OK;
}

// Tuning aid (JUNO_STEP_TIMELINE=1, eager launches only): where CTA 0 spent each phase, averaged over the layers.
static void step_print_timeline(const StepPlan &plan, cudaStream_t st) {
    std::vector<unsigned long long> t((size_t)plan.n_phases * 8);
    if (cudaStreamSynchronize(st) != cudaSuccess) return;
    if (cudaMemcpy(t.data(), plan.d_timeline, t.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
    const int per = plan.timeline_period > 0 ? plan.timeline_period : plan.n_phases;
    const int reps = (plan.n_phases - 1) / per;
    fprintf(stderr, "step timeline (CTA 0, us): phase | wait image | sums | compute | cta sync | grid barrier | total\n");
    double all = 0;
    for (int j = 0; j < per; j++) {
        double d[5] = {0, 0, 0, 0, 0};
        int cnt = 0;
        for (int r = 0; r < reps; r++) {
            const unsigned long long *e = &t[(size_t)(r * per + j) * 8];
            const unsigned long long k1 = e[1] ? e[1] : e[0], k2 = e[2] ? e[2] : k1;
            d[0] += (double)(k1 - e[0]);
            d[1] += (double)(k2 - k1);
            d[2] += (double)(e[3] - k2);
            d[3] += (double)(e[4] - e[3]);
            d[4] += (double)(e[5] - e[4]);
            cnt++;
        }
        double tot = 0;
        for (double &x : d) {
            x /= 1e3 * std::max(1, cnt);
            tot += x;
        }
        all += tot;
        fprintf(stderr, "  %d | %.2f | %.2f | %.2f | %.2f | %.2f | %.2f\n", j, d[0], d[1], d[2], d[3], d[4], tot);
    }
    const unsigned long long *e = &t[(size_t)(plan.n_phases - 1) * 8];
    fprintf(stderr, "  per layer %.2f us; last phase %.2f us; whole kernel %.1f us\n", all, (double)(e[3] - e[0]) / 1e3,
            (double)(e[3] - t[0]) / 1e3);
}

unsigned step_plan_error(const StepPlan &plan) { return plan.h_err ? *plan.h_err : 0u; }

int step_plan_build(juno_ctx *ctx, const StepRecorder &rec, int kv_f32, int hd, int group, StepPlan *plan) {
    JUNO_REQUIRE(!rec.phases.empty(), "step plan: nothing recorded");
    size_t img = 0;
    int slot = 0;
    double bytes = 0;
    for (const StepPhase &ph : rec.phases) {
        if (ph.kind != STEP_GEMV) continue;
        const GemvParams &g = ph.g;
        const size_t xs = (((size_t)(g.K / 32) * 3 * rec.n * 2) + 15) & ~(size_t)15;
        img = std::max(img, (size_t)g.img_bytes + xs);
        for (int s = 0; s < g.nseg; s++) {
            slot = std::max(slot, tile_bytes(g.seg_type[s]));
            bytes += (double)(g.rt_begin[s + 1] - g.rt_begin[s]) * g.nb * tile_bytes(g.seg_type[s]);
        }
    }
    const int ge = step_group(group, 1);
    JUNO_REQUIRE(ge > 0, "step plan: %d query heads per kv head is not supported", group);
    img = std::max(img, step_attn_scratch_bytes(hd, ge));
    plan->img_cap = (unsigned)((img + 127) & ~(size_t)127);
    plan->slot_bytes = (slot + 15) & ~15;
    const StepSmem<1> L(plan->img_cap, plan->slot_bytes);
    plan->smem = L.total;
    JUNO_REQUIRE(plan->smem <= ctx->smem_optin, "step plan: %zu bytes of shared memory needed, %zu available", plan->smem,
                 ctx->smem_optin);
    plan->grid = rec.grid;
    plan->n_phases = (int)rec.phases.size();
    plan->kv_f32 = kv_f32;
    plan->hd = hd;
    plan->ge = ge;
    plan->nb = rec.n;
    plan->algo_bytes = bytes;
    JUNO_CUDA_TRY(cudaMalloc((void **)&plan->d_phases, rec.phases.size() * sizeof(StepPhase)));
    JUNO_CUDA_TRY(cudaMemcpy(plan->d_phases, rec.phases.data(), rec.phases.size() * sizeof(StepPhase), cudaMemcpyHostToDevice));
    JUNO_CUDA_TRY(cudaMalloc((void **)&plan->d_sync, (size_t)(2 + plan->n_phases) * 4));
    JUNO_CUDA_TRY(cudaMemset(plan->d_sync, 0, (size_t)(2 + plan->n_phases) * 4));
    JUNO_CUDA_TRY(cudaHostAlloc((void **)&plan->h_err, 4, cudaHostAllocDefault));
    *plan->h_err = 0;
    if (const char *e = getenv("JUNO_STEP_TIMELINE")) {
        if (*e == '1') {
            JUNO_CUDA_TRY(cudaMalloc((void **)&plan->d_timeline, (size_t)plan->n_phases * 64));
            JUNO_CUDA_TRY(cudaMemset(plan->d_timeline, 0, (size_t)plan->n_phases * 64));
        }
    }
    return JUNO_OK;
}

void step_plan_free(StepPlan *plan) {
    if (plan->d_phases) cudaFree(plan->d_phases);
    if (plan->d_sync) cudaFree(plan->d_sync);
    if (plan->h_err) cudaFreeHost(plan->h_err);
    if (plan->d_timeline) cudaFree(plan->d_timeline);
    *plan = StepPlan();
}

}  // namespace juno
