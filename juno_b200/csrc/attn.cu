// Paged KV cache, RoPE + KV append, and GQA flash-decode attention with split-K over context.
//
// Replaces the per-request FP32 heap arrays and the scalar gqa()/softmax()/rope() loops of
// LlamaTransformerHandler.java:670-733,1657-1730.  One CTA handles one (sequence, kv head, context
// split): K and V pages are streamed once and shared by the G query heads of the group; each split
// keeps an online-softmax state (m, l, o) and a second small kernel merges the splits.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <type_traits>

#include "attn.cuh"

namespace juno {

// ───────────────────────────── kernels ────────────────────────────────────────────────────
struct AttnParams {
    const void *k, *v;
    const int32_t *table;
    int max_pages_per_seq, n_pages, n_kv_heads, n_heads, layer, n_splits;
    const float *q;
    int ldq;
    const int32_t *slots, *seq_lens;
    float *part_o, *part_ml, *out;
    // fused RoPE + KV append (rope_cs != nullptr): q is rotated on load, and the CTA whose split holds the newest
    // position rotates k, rounds k and v to the cache type, uses them and writes them to their page
    const float2 *rope_cs;
    const float *knew, *vnew;
    int ldkv;
    void *kw, *vw;
    // the context splits of a (sequence, kv head) form one thread-block cluster (cluster dimension y = n_splits): the
    // splits are merged through distributed shared memory inside attn_mma_kernel and no merge kernel is launched
    int cluster_merge;
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Eight consecutive head dimensions of one cached position, widened to FP32.
template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, float (&o)[8]) {
    const uint4 u = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

constexpr int kAttnWarps = 4;
constexpr int kAttnUnroll = 4;  // positions in flight per token slot

// One CTA = (kv head, context split, sequence).  HD/8 lanes share one cached position (eight head dimensions
// each, one 128-bit load for K and one for V), so a warp works on 32/(HD/8) positions at a time and every lane
// keeps an online-softmax state for the G query heads of the group; the states are merged through shared memory.
template <typename T, int HD, int G>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_split_kernel(const AttnParams p) {
    constexpr int LPT = HD / 8, TPW = 32 / LPT, SLOTS = kAttnWarps * TPW;
    pdl_launch_dependents();
    pdl_wait();
    const int kvh = blockIdx.x, split = blockIdx.y, seq = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int len = p.seq_lens[seq];
    const int chunk = (((len + p.n_splits - 1) / p.n_splits) + 15) & ~15;
    const int t0 = split * chunk, t1 = min(len, t0 + chunk);
    const int h0 = kvh * G;
    float *po = p.part_o + ((size_t)(seq * p.n_heads + h0) * p.n_splits + split) * HD;   // head stride n_splits*HD
    float *pml = p.part_ml + ((size_t)(seq * p.n_heads + h0) * p.n_splits + split) * 2;  // head stride n_splits*2
    __shared__ float sm_m[SLOTS][G], sm_l[SLOTS][G];
    __shared__ float sm_o[SLOTS][G][HD];
    if (t0 >= t1) {  // empty split: weight 0, and finite zeros so that 0 * partial stays 0 in the merge
        if (tid < G) {
            pml[(size_t)tid * p.n_splits * 2 + 0] = -INFINITY;
            pml[(size_t)tid * p.n_splits * 2 + 1] = 0.f;
        }
        for (int idx = tid; idx < G * HD; idx += kAttnWarps * 32) po[(size_t)(idx / HD) * p.n_splits * HD + (idx % HD)] = 0.f;
    } else {
    const int sub = lane % LPT, slot = warp * TPW + lane / LPT;
    const unsigned gmask = (LPT == 32) ? 0xffffffffu : (((1u << LPT) - 1u) << (lane - sub));
    // scores in the log2 domain: exp(x) = exp2(x * log2(e))
    const float scale = (float)(1.0 / sqrt((double)HD)) * 1.4426950408889634f;
    float qr[G][8], o[G][8], m[G], l[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        const float *qp = p.q + (size_t)seq * p.ldq + (size_t)(h0 + g) * HD + sub * 8;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            float x0 = qp[e], x1 = qp[e + 1];
            if (p.rope_cs) {  // adjacent-pair rotation, each product rounded (rope :1657-1671)
                const float2 cs = p.rope_cs[seq * (HD / 2) + sub * 4 + (e >> 1)];
                const float y0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
                const float y1 = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
                x0 = y0;
                x1 = y1;
            }
            qr[g][e] = x0 * scale;
            qr[g][e + 1] = x1 * scale;
            o[g][e] = o[g][e + 1] = 0.f;
        }
        m[g] = -INFINITY;
        l[g] = 0.f;
    }
    const int32_t *table = p.table + (size_t)p.slots[seq] * p.max_pages_per_seq;
    const T *kbase = static_cast<const T *>(p.k), *vbase = static_cast<const T *>(p.v);
    const size_t head_off = (size_t)kvh * kPageTokens * HD + sub * 8;
    const size_t page_stride = (size_t)p.n_kv_heads * kPageTokens * HD;
    const size_t layer_off = (size_t)p.layer * p.n_pages * page_stride;
    for (int tb = t0 + slot; tb < t1; tb += SLOTS * kAttnUnroll) {
        float kv[kAttnUnroll][8], vv[kAttnUnroll][8];
#pragma unroll
        for (int u = 0; u < kAttnUnroll; u++) {
            const int t = tb + u * SLOTS;
            if (t < t1) {
                const size_t off = layer_off + (size_t)table[t >> 4] * page_stride + head_off + (size_t)(t & 15) * HD;
                if (p.rope_cs && t == len - 1) {  // the position being decoded: rotate, round, use and append
                    const float *kx = p.knew + (size_t)seq * p.ldkv + kvh * HD + sub * 8;
                    const float *vx = p.vnew + (size_t)seq * p.ldkv + kvh * HD + sub * 8;
                    T *kd = static_cast<T *>(p.kw) + off, *vd = static_cast<T *>(p.vw) + off;
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float2 cs = p.rope_cs[seq * (HD / 2) + sub * 4 + (e >> 1)];
                        const float x0 = kx[e], x1 = kx[e + 1];
                        const T k0 = from_f32<T>(__fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y)));
                        const T k1 = from_f32<T>(__fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x)));
                        const T v0 = from_f32<T>(vx[e]), v1 = from_f32<T>(vx[e + 1]);
                        kd[e] = k0; kd[e + 1] = k1;
                        vd[e] = v0; vd[e + 1] = v1;
                        kv[u][e] = to_f32<T>(k0); kv[u][e + 1] = to_f32<T>(k1);
                        vv[u][e] = to_f32<T>(v0); vv[u][e + 1] = to_f32<T>(v1);
                    }
                } else {
                    load8<T>(kbase + off, kv[u]);
                    load8<T>(vbase + off, vv[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kAttnUnroll; u++) {
            const int t = tb + u * SLOTS;
            if (t < t1) {  // uniform over the LPT lanes of this position
                float s[G];
#pragma unroll
                for (int g = 0; g < G; g++) {
                    float d = 0.f;
#pragma unroll
                    for (int e = 0; e < 8; e++) d = fmaf(qr[g][e], kv[u][e], d);
                    s[g] = d;
                }
#pragma unroll
                for (int ofs = LPT / 2; ofs > 0; ofs >>= 1)
#pragma unroll
                    for (int g = 0; g < G; g++) s[g] += __shfl_xor_sync(gmask, s[g], ofs);
#pragma unroll
                for (int g = 0; g < G; g++) {
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
    for (int g = 0; g < G; g++) {
        if (sub == 0) {
            sm_m[slot][g] = m[g];
            sm_l[slot][g] = l[g];
        }
#pragma unroll
        for (int e = 0; e < 8; e++) sm_o[slot][g][sub * 8 + e] = o[g][e];
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += kAttnWarps * 32) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < SLOTS; w++) M = fmaxf(M, sm_m[w][g]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < SLOTS; w++) {
            if (sm_l[w][g] > 0.f) {
                const float f = exp2f(sm_m[w][g] - M);
                L = fmaf(sm_l[w][g], f, L);
                acc = fmaf(sm_o[w][g][d], f, acc);
            }
        }
        po[(size_t)g * p.n_splits * HD + d] = acc;
        if (d == 0) {
            pml[(size_t)g * p.n_splits * 2 + 0] = M;  // log2 domain
            pml[(size_t)g * p.n_splits * 2 + 1] = L;
        }
    }
    }  // non-empty split
}

// ───────────────────────────── tensor-core variant (FP16 pages) ───────────────────────────
// Same work split as attn_split_kernel (one CTA per kv head, context split and sequence; partials in the same
// layout), but the scores and the weighted sums run on mma.sync.m16n8k16: a warp takes whole 16-position pages,
// copies the page's K and V rows (16 x HD halfs each, contiguous in the pool) into its own shared-memory tiles with
// cp.async (next page in flight while the current one is computed), and per page does
//   S = Q K^T   : A = q as two FP16 limbs (hi + lo, so the scores keep FP32-level accuracy), B = K via ldmatrix
//   online softmax on the FP32 fragment (row max / sum across the four lanes that share a row)
//   O += P V    : A = P (the score fragment re-used as an A fragment, FP16), B = V via ldmatrix.trans
// Rows of the 16-row MMA tile are the G query heads of the group (G <= 8; rows 8..15 stay zero).
constexpr int kMmaWarps = 4;

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// K/V pages are read once per step: evict-first, so that they do not push the activations, the norm weights and the
// kernels' instructions out of the L2.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, uint64_t pol) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "l"(pol) : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <int HD, int G>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) attn_mma_kernel(const AttnParams p) {
    constexpr int LDT = HD + 8;             // tile row stride in halfs (the pad keeps ldmatrix rows on distinct banks)
    constexpr int TILE = 16 * LDT;          // halfs per K or V tile
    constexpr int KS = HD / 16, DN = HD / 8;
    static_assert(G <= 8, "the query heads of a group occupy rows 0..7 of the MMA tile");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *sm_q = reinterpret_cast<__half *>(smem_raw);                 // [2 limbs][8 rows][LDT]
    __half *sm_kv = sm_q + 2 * 8 * LDT;                                   // [warp][stage 2][K | V][TILE]
    pdl_launch_dependents();
    // Sequence lengths, page table and the cached positions were written by earlier steps (or, inside a prefill pass, by
    // kernels that are not launched programmatically): only q and the k, v of the position being decoded come from
    // the kernel before this one.  So the first K/V page of every warp is requested before the wait.
    const int kvh = blockIdx.x, split = blockIdx.y, seq = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, r8 = lane >> 2, c = lane & 3;
    const int len = p.seq_lens[seq];
    const int chunk = (((len + p.n_splits - 1) / p.n_splits) + 15) & ~15;
    const int t0 = split * chunk, t1 = min(len, t0 + chunk);
    const int h0 = kvh * G;
    float *po = p.part_o + ((size_t)(seq * p.n_heads + h0) * p.n_splits + split) * HD;   // head stride n_splits*HD
    float *pml = p.part_ml + ((size_t)(seq * p.n_heads + h0) * p.n_splits + split) * 2;  // head stride n_splits*2
    const int32_t *table = p.table + (size_t)p.slots[seq] * p.max_pages_per_seq;
    const __half *kbase = static_cast<const __half *>(p.k), *vbase = static_cast<const __half *>(p.v);
    const size_t page_stride = (size_t)p.n_kv_heads * kPageTokens * HD;
    const size_t layer_off = (size_t)p.layer * p.n_pages * page_stride + (size_t)kvh * kPageTokens * HD;
    __half *my_kv = sm_kv + (size_t)warp * 4 * TILE;
    const uint32_t my_kv_s = (uint32_t)__cvta_generic_to_shared(my_kv);
    const int pg0 = t0 >> 4, pg1 = (t1 + 15) >> 4;
    uint64_t l2_pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(l2_pol));
    auto issue = [&](int pg, int stage) {  // this warp's copy of page pg into its stage
        const size_t off = layer_off + (size_t)table[pg] * page_stride;
        const uint32_t kd = my_kv_s + (uint32_t)(stage * 2 * TILE) * 2u, vd = kd + TILE * 2u;
#pragma unroll
        for (int i = 0; i < HD / 16; i++) {  // 16 rows x HD/8 chunks of 16 bytes = 32 lanes x HD/16
            const int ch = i * 32 + lane, row = ch / (HD / 8), col8 = ch - row * (HD / 8);
            cp_async_16(kd + (uint32_t)(row * LDT + col8 * 8) * 2u, kbase + off + (size_t)row * HD + col8 * 8, l2_pol);
            cp_async_16(vd + (uint32_t)(row * LDT + col8 * 8) * 2u, vbase + off + (size_t)row * HD + col8 * 8, l2_pol);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int pg = pg0 + warp, stage = 0;
    if (pg < pg1) issue(pg, 0);
    pdl_wait();
    // An empty split leaves at once, except as a member of a cluster: there it takes part in the merge with sum 0.
    if (t0 >= t1 && !p.cluster_merge) {  // empty split: weight 0, and finite zeros so that 0 * partial stays 0 in the merge
        if (tid < G) {
            pml[(size_t)tid * p.n_splits * 2 + 0] = -INFINITY;
            pml[(size_t)tid * p.n_splits * 2 + 1] = 0.f;
        }
        for (int idx = tid; idx < G * HD; idx += kMmaWarps * 32) po[(size_t)(idx / HD) * p.n_splits * HD + (idx % HD)] = 0.f;
        return;
    }
    // q of the group: rotate (rope :1657-1671), scale into the log2 domain, split into two FP16 limbs
    const float scale = (float)(1.0 / sqrt((double)HD)) * 1.4426950408889634f;
    for (int idx = tid; idx < 8 * (HD / 2); idx += kMmaWarps * 32) {
        const int g = idx / (HD / 2), i = idx - g * (HD / 2);
        float y0 = 0.f, y1 = 0.f;
        if (g < G) {
            const float *qp = p.q + (size_t)seq * p.ldq + (size_t)(h0 + g) * HD + 2 * i;
            float x0 = qp[0], x1 = qp[1];
            if (p.rope_cs) {
                const float2 cs = p.rope_cs[seq * (HD / 2) + i];
                const float a = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
                const float b = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
                x0 = a;
                x1 = b;
            }
            y0 = x0 * scale;
            y1 = x1 * scale;
        }
        const __half h0h = __float2half_rn(y0), h1h = __float2half_rn(y1);
        sm_q[g * LDT + 2 * i] = h0h;
        sm_q[g * LDT + 2 * i + 1] = h1h;
        sm_q[8 * LDT + g * LDT + 2 * i] = __float2half_rn(y0 - __half2float(h0h));
        sm_q[8 * LDT + g * LDT + 2 * i + 1] = __float2half_rn(y1 - __half2float(h1h));
    }
    __syncthreads();
    // A fragments of q (rows 0..7 only): a0 = (row r8, k 2c..2c+1), a2 = (row r8, k 2c+8..2c+9) of every 16-column step
    uint32_t qh[KS][2], ql[KS][2];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        qh[ks][0] = *reinterpret_cast<const uint32_t *>(sm_q + r8 * LDT + ks * 16 + 2 * c);
        qh[ks][1] = *reinterpret_cast<const uint32_t *>(sm_q + r8 * LDT + ks * 16 + 2 * c + 8);
        ql[ks][0] = *reinterpret_cast<const uint32_t *>(sm_q + 8 * LDT + r8 * LDT + ks * 16 + 2 * c);
        ql[ks][1] = *reinterpret_cast<const uint32_t *>(sm_q + 8 * LDT + r8 * LDT + ks * 16 + 2 * c + 8);
    }
    float o[DN][2], m_run = -INFINITY, l_run = 0.f;  // row r8: output columns dn*8 + 2c, +1; running max; this lane's share of the sum
#pragma unroll
    for (int dn = 0; dn < DN; dn++) o[dn][0] = o[dn][1] = 0.f;
    for (; pg < pg1; pg += kMmaWarps, stage ^= 1) {
        const bool more = pg + kMmaWarps < pg1;
        if (more) issue(pg + kMmaWarps, stage ^ 1);
        if (more)
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        else
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        __half *kt = my_kv + (size_t)stage * 2 * TILE, *vt = kt + TILE;
        const int pos0 = pg << 4;
        if (p.rope_cs && len - 1 >= pos0 && len - 1 < pos0 + 16) {
            // the position being decoded lives in this page: rotate k, round k and v to FP16, use them and append them
            const int row = (len - 1) & 15;
            const size_t off = layer_off + (size_t)table[pg] * page_stride + (size_t)row * HD;
            __half *kd = static_cast<__half *>(p.kw) + off, *vd = static_cast<__half *>(p.vw) + off;
            const float *kx = p.knew + (size_t)seq * p.ldkv + kvh * HD, *vx = p.vnew + (size_t)seq * p.ldkv + kvh * HD;
            for (int i = lane; i < HD / 2; i += 32) {
                const float2 cs = p.rope_cs[seq * (HD / 2) + i];
                const float x0 = kx[2 * i], x1 = kx[2 * i + 1];
                const __half k0 = __float2half_rn(__fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y)));
                const __half k1 = __float2half_rn(__fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x)));
                const __half v0 = __float2half_rn(vx[2 * i]), v1 = __float2half_rn(vx[2 * i + 1]);
                kt[row * LDT + 2 * i] = k0;
                kt[row * LDT + 2 * i + 1] = k1;
                vt[row * LDT + 2 * i] = v0;
                vt[row * LDT + 2 * i + 1] = v1;
                kd[2 * i] = k0;
                kd[2 * i + 1] = k1;
                vd[2 * i] = v0;
                vd[2 * i + 1] = v1;
            }
            __syncwarp();
        }
        // rows of V beyond the attended range must not inject NaN/inf through 0 * x: zero them
        if (pos0 + 16 > t1) {
            const int first_bad = t1 - pos0;  // 1..15
            for (int i = lane; i < (16 - first_bad) * (HD / 2); i += 32) {
                const int row = first_bad + i / (HD / 2), cc = i - (i / (HD / 2)) * (HD / 2);
                *reinterpret_cast<uint32_t *>(vt + row * LDT + 2 * cc) = 0u;
            }
            __syncwarp();
        }
        const uint32_t kts = (uint32_t)__cvta_generic_to_shared(kt), vts = (uint32_t)__cvta_generic_to_shared(vt);
        // scores of the 16 positions: two n-tiles of 8
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const int mi = lane >> 3, rr = (lane & 7) + 8 * (mi >> 1), cc = 8 * (mi & 1);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                uint32_t b[4];  // (pos 0-7, k lo), (pos 0-7, k hi), (pos 8-15, k lo), (pos 8-15, k hi)
                ldmatrix_x4(b, kts + (uint32_t)(rr * LDT + ks * 16 + cc) * 2u);
                mma_f16(s0, qh[ks][0], 0u, qh[ks][1], 0u, b[0], b[1]);
                mma_f16(s1, qh[ks][0], 0u, qh[ks][1], 0u, b[2], b[3]);
                mma_f16(s0, ql[ks][0], 0u, ql[ks][1], 0u, b[0], b[1]);
                mma_f16(s1, ql[ks][0], 0u, ql[ks][1], 0u, b[2], b[3]);
            }
        }
        // this lane holds row r8, positions pos0 + 2c, +1 (s0) and pos0 + 8 + 2c, +1 (s1)
        float sc[4] = {s0[0], s0[1], s1[0], s1[1]};
        if (pos0 + 16 > t1) {
            if (pos0 + 2 * c >= t1) sc[0] = -INFINITY;
            if (pos0 + 2 * c + 1 >= t1) sc[1] = -INFINITY;
            if (pos0 + 8 + 2 * c >= t1) sc[2] = -INFINITY;
            if (pos0 + 8 + 2 * c + 1 >= t1) sc[3] = -INFINITY;
        }
        float mloc = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 1));
        mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 2));
        const float mn = fmaxf(m_run, mloc);  // finite: position pos0 is inside the range
        const float corr = exp2f(m_run - mn);
        float pe[4];
#pragma unroll
        for (int i = 0; i < 4; i++) pe[i] = exp2f(sc[i] - mn);
        l_run = fmaf(l_run, corr, (pe[0] + pe[1]) + (pe[2] + pe[3]));
        m_run = mn;
#pragma unroll
        for (int dn = 0; dn < DN; dn++) {
            o[dn][0] *= corr;
            o[dn][1] *= corr;
        }
        // the weights as two FP16 limbs (hi + lo), like q: the weighted sum keeps FP32-level accuracy
        const uint32_t pa0 = pack_h2(pe[0], pe[1]), pa2 = pack_h2(pe[2], pe[3]);
        float pl[4];
        {
            const __half2 h01 = *reinterpret_cast<const __half2 *>(&pa0), h23 = *reinterpret_cast<const __half2 *>(&pa2);
            pl[0] = pe[0] - __low2float(h01);
            pl[1] = pe[1] - __high2float(h01);
            pl[2] = pe[2] - __low2float(h23);
            pl[3] = pe[3] - __high2float(h23);
        }
        const uint32_t pb0 = pack_h2(pl[0], pl[1]), pb2 = pack_h2(pl[2], pl[3]);
        {
            const int mi = lane >> 3, rr = (lane & 7) + 8 * (mi & 1), cc = 8 * (mi >> 1);
#pragma unroll
            for (int dn = 0; dn < DN; dn += 2) {
                uint32_t b[4];  // (pos 0-7, dims dn), (pos 8-15, dims dn), (pos 0-7, dims dn+1), (pos 8-15, dims dn+1), transposed
                ldmatrix_x4_trans(b, vts + (uint32_t)(rr * LDT + dn * 8 + cc) * 2u);
                float acc0[4] = {o[dn][0], o[dn][1], 0.f, 0.f}, acc1[4] = {o[dn + 1][0], o[dn + 1][1], 0.f, 0.f};
                mma_f16(acc0, pa0, 0u, pa2, 0u, b[0], b[1]);
                mma_f16(acc1, pa0, 0u, pa2, 0u, b[2], b[3]);
                mma_f16(acc0, pb0, 0u, pb2, 0u, b[0], b[1]);
                mma_f16(acc1, pb0, 0u, pb2, 0u, b[2], b[3]);
                o[dn][0] = acc0[0];
                o[dn][1] = acc0[1];
                o[dn + 1][0] = acc1[0];
                o[dn + 1][1] = acc1[1];
            }
        }
        __syncwarp();  // everybody is done with this stage before it is refilled two pages later
    }
    // this lane's share of the row sum -> row sum
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    // merge the four warps through shared memory (the K/V tiles are dead)
    __syncthreads();
    float *mg_o = reinterpret_cast<float *>(sm_kv);       // [warp][G][HD]
    float *mg_m = mg_o + kMmaWarps * G * HD;               // [warp][G]
    float *mg_l = mg_m + kMmaWarps * G;                    // [warp][G]
    float *cl_o = mg_l + kMmaWarps * G;                    // [G][HD]   this CTA's merged split, read by the cluster
    float *cl_m = cl_o + G * HD, *cl_l = cl_m + G;
    if (r8 < G) {
#pragma unroll
        for (int dn = 0; dn < DN; dn++)
            *reinterpret_cast<float2 *>(mg_o + ((size_t)warp * G + r8) * HD + dn * 8 + 2 * c) = make_float2(o[dn][0], o[dn][1]);
        if (c == 0) {
            mg_m[warp * G + r8] = m_run;
            mg_l[warp * G + r8] = l_run;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += kMmaWarps * 32) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) M = fmaxf(M, mg_m[w * G + g]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) {
            const float lw = mg_l[w * G + g];
            if (lw > 0.f) {
                const float f = exp2f(mg_m[w * G + g] - M);
                L = fmaf(lw, f, L);
                acc = fmaf(mg_o[((size_t)w * G + g) * HD + d], f, acc);
            }
        }
        if (p.cluster_merge) {
            cl_o[g * HD + d] = acc;
            if (d == 0) {
                cl_m[g] = M;
                cl_l[g] = L;
            }
        } else {
            po[(size_t)g * p.n_splits * HD + d] = acc;
            if (d == 0) {
                pml[(size_t)g * p.n_splits * 2 + 0] = M;  // log2 domain
                pml[(size_t)g * p.n_splits * 2 + 1] = L;
            }
        }
    }
    if (!p.cluster_merge) return;
    // Merge of the splits inside the cluster: every CTA keeps its (max, sum, output) in its own shared memory; CTA r
    // then finishes the slice [r, r+1) * G*HD/S of the outputs, reading the S partial results over distributed shared
    // memory in split order (fixed order: bitwise repeatable).  An empty split carries sum 0 and is skipped.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    {
        const int S = (int)cluster.num_blocks(), r = (int)cluster.block_rank();
        const int per = (G * HD) / S;
        for (int idx = r * per + tid; idx < (r + 1) * per; idx += kMmaWarps * 32) {
            const int g = idx / HD, d = idx - g * HD;
            float M = -INFINITY;
            for (int sp = 0; sp < S; sp++) M = fmaxf(M, *cluster.map_shared_rank(cl_m + g, sp));
            float L = 0.f, acc = 0.f;
            for (int sp = 0; sp < S; sp++) {
                const float lw = *cluster.map_shared_rank(cl_l + g, sp);
                if (lw > 0.f) {
                    const float f = exp2f(*cluster.map_shared_rank(cl_m + g, sp) - M);
                    L = fmaf(lw, f, L);
                    acc = fmaf(*cluster.map_shared_rank(cl_o + g * HD + d, sp), f, acc);
                }
            }
            p.out[(size_t)(seq * p.n_heads + h0 + g) * HD + d] = (L > 0.f) ? acc / L : 0.f;
        }
    }
    cluster.sync();  // nobody leaves while its shared memory may still be read
}

// Merges the context splits of one (sequence, head): blockDim = kCombineParts * HD threads.  The split weights are
// computed once in parallel (one split per thread of the first HD threads); then thread (part, d) adds the splits
// s = part, part + kCombineParts, ... of output dimension d with all its loads in flight at once, and the parts are
// added in fixed order.
constexpr int kCombineParts = 4;
template <int HD>
__global__ void __launch_bounds__(kCombineParts * HD) attn_combine_kernel(const AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x, d = tid % HD, part = tid / HD, lane = tid & 31, warp = tid >> 5;
    const float *po = p.part_o + (size_t)(seq * p.n_heads + h) * p.n_splits * HD;
    const float *pml = p.part_ml + (size_t)(seq * p.n_heads + h) * p.n_splits * 2;
    __shared__ float f[64], red[HD / 32], red2[HD / 32], acc_s[kCombineParts][HD];
    float ms = -INFINITY, ls = 0.f;
    if (tid < p.n_splits) {  // n_splits <= 64 <= HD
        ms = pml[2 * tid];
        ls = pml[2 * tid + 1];
    }
    float M = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0 && warp < HD / 32) red[warp] = M;
    __syncthreads();
    M = red[0];
#pragma unroll
    for (int w = 1; w < HD / 32; w++) M = fmaxf(M, red[w]);
    const float fs = (ls > 0.f) ? exp2f(ms - M) : 0.f;  // maxima are kept in the log2 domain
    if (tid < 64) f[tid] = fs;
    float L = ls * fs;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0 && warp < HD / 32) red2[warp] = L;
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 64 / kCombineParts; i++) {
        const int s = part + i * kCombineParts;
        if (s < p.n_splits) acc = fmaf(po[(size_t)s * HD + d], f[s], acc);
    }
    acc_s[part][d] = acc;
    __syncthreads();
    if (part != 0) return;
    L = 0.f;
#pragma unroll
    for (int w = 0; w < HD / 32; w++) L += red2[w];
    acc = acc_s[0][d];
#pragma unroll
    for (int q = 1; q < kCombineParts; q++) acc += acc_s[q][d];
    const float outv = (L > 0.f) ? acc / L : 0.f;
    p.out[(size_t)(seq * p.n_heads + h) * HD + d] = outv;
}

// cos/sin of pos * theta^(-2i/hd) in binary64, cast to float, as LlamaTransformerHandler.rope (:1662-1666).
__global__ void rope_table_kernel(const int32_t *positions, int n, int hd, float theta, float2 *table) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    int half = hd / 2;
    if (idx >= n * half) return;
    int seq = idx / half, i = idx - seq * half;
    double freq = 1.0 / pow((double)theta, (2.0 * i) / hd);
    double angle = positions[seq] * freq;
    table[idx] = make_float2((float)cos(angle), (float)sin(angle));
}

struct RopeParams {
    void *k, *v;
    const int32_t *table;
    int max_pages_per_seq, n_pages, n_kv_heads, n_heads, layer, hd;
    float *q;
    int ldq;
    const float *kin, *vin;
    int ldkv;
    const int32_t *slots, *positions;
    const float2 *cs;
};

template <typename T>
__global__ void rope_append_kernel(const RopeParams p) {
    const int seq = blockIdx.x, head = blockIdx.y, i = threadIdx.x;  // i: pair index
    const float2 cs = p.cs[seq * (p.hd / 2) + i];
    if (head < p.n_heads) {
        float *x = p.q + (size_t)seq * p.ldq + head * p.hd + 2 * i;
        const float x0 = x[0], x1 = x[1];
        x[0] = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
        x[1] = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
    } else {
        const int kvh = head - p.n_heads;
        const int pos = p.positions[seq];
        const int page = p.table[(size_t)p.slots[seq] * p.max_pages_per_seq + (pos >> 4)];
        const size_t off =
            ((((size_t)p.layer * p.n_pages + page) * p.n_kv_heads + kvh) * kPageTokens + (pos & 15)) * p.hd + 2 * i;
        const float *kx = p.kin + (size_t)seq * p.ldkv + kvh * p.hd + 2 * i;
        const float *vx = p.vin + (size_t)seq * p.ldkv + kvh * p.hd + 2 * i;
        const float x0 = kx[0], x1 = kx[1];
        T *kd = static_cast<T *>(p.k) + off, *vd = static_cast<T *>(p.v) + off;
        kd[0] = from_f32<T>(__fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y)));
        kd[1] = from_f32<T>(__fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x)));
        vd[0] = from_f32<T>(vx[0]);
        vd[1] = from_f32<T>(vx[1]);
    }
}

// Scatter of host-provided K/V rows (already on the device as FP32) into pages, for the operator API.
template <typename T>
__global__ void kv_scatter_kernel(void *kpool, void *vpool, const int32_t *table_row, int n_pages, int n_kv_heads, int hd,
                                  int layer, int pos0, int n_tokens, const float *kin, const float *vin) {
    const int kvdim = n_kv_heads * hd;
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tokens * kvdim) return;
    const int j = (int)(idx / kvdim), e = (int)(idx - (size_t)j * kvdim), kvh = e / hd, d = e - kvh * hd;
    const int pos = pos0 + j, page = table_row[pos >> 4];
    const size_t off = ((((size_t)layer * n_pages + page) * n_kv_heads + kvh) * kPageTokens + (pos & 15)) * hd + d;
    static_cast<T *>(kpool)[off] = from_f32<T>(kin[idx]);
    static_cast<T *>(vpool)[off] = from_f32<T>(vin[idx]);
}

// ───────────────────────────── host: launches ─────────────────────────────────────────────
size_t attn_scratch_floats(int n, int n_heads, int hd, int n_splits) {
    return (size_t)n * n_heads * n_splits * (hd + 2);
}

// Largest split count the cluster-merged kernel takes (a power of two, at most 16); 0 = the splits are always merged by
// attn_combine_kernel.  Off by default: on the batch-1 decode step at context 2048 the cluster merge measured 7 %
// slower than eighteen independent splits plus the merge kernel (clusters are placed later and wait for their slowest
// member twice).  JUNO_ATTN_CLUSTER=8 or 16 switches it on; read at every call so that tests can cover both paths.
static int attn_cluster_max() {
    const char *e = getenv("JUNO_ATTN_CLUSTER");
    const int m = e ? atoi(e) : 0;
    return std::max(0, std::min(m, 16));
}

int attn_pick_splits(const juno_ctx *ctx, int n, int n_kv_heads, int max_len) {
    const int target = ctx->sm_count * 4;  // CTAs of 128 threads wanted in flight
    int by_occupancy = (target + n * n_kv_heads - 1) / std::max(1, n * n_kv_heads);
    // at least 128 positions per split (two pages per warp): in the batch-1 step at context 2048, 16-32 splits
    // measured 2.27 ms/step against 2.36 ms with 64 (fewer partials to merge, same occupancy where it matters)
    int by_length = std::max(1, (max_len + 127) / 128);
    int s = std::max(1, std::min(by_occupancy, by_length));
    if (const char *e = getenv("JUNO_ATTN_SPLITS")) s = std::max(1, std::min(s, atoi(e)));
    s = std::min(s, 64);
    // Up to twice the cluster limit the count is rounded down to a power of two within it, so that the splits of a
    // (sequence, kv head) can be one thread-block cluster and merge on chip; longer contexts keep their many splits
    // and the separate merge kernel.
    const int cmax = attn_cluster_max();
    if (cmax > 0 && s <= 2 * cmax) {
        int p2 = 1;
        while (2 * p2 <= std::min(s, cmax)) p2 *= 2;
        s = p2;
    }
    return s;
}

static bool attn_use_mma() {
    static const bool on = [] {
        const char *e = getenv("JUNO_ATTN_SCALAR");  // JUNO_ATTN_SCALAR=1: the FMA/shuffle kernel also for FP16 pages
        return !(e && *e == '1');
    }();
    return on;
}

template <int HD, int G>
static size_t attn_mma_smem() {
    return ((size_t)2 * 8 * (HD + 8) + (size_t)kMmaWarps * 4 * 16 * (HD + 8)) * sizeof(__half);
}

// Whether a cluster of `splits` CTAs of the tensor-core kernel can be co-scheduled on this device (asked once per size).
template <int HD, int G>
static bool attn_cluster_fits(int splits) {
    static int fits[64][5] = {{0}};  // per device, per log2(splits): 0 unknown, 1 yes, 2 no
    int dev = 0, lg = 0;
    cudaGetDevice(&dev);
    while ((1 << lg) < splits) lg++;
    int &f = fits[dev & 63][lg];
    if (f == 0) {
        const size_t smem = attn_mma_smem<HD, G>();
        cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, splits, 1);
        cfg.blockDim = dim3(kMmaWarps * 32);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = (unsigned)splits;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, attn_mma_kernel<HD, G>, &cfg);
        if (e != cudaSuccess) cudaGetLastError();
        f = (e == cudaSuccess && n > 0) ? 1 : 2;
    }
    return f == 1;
}
static bool attn_cluster_fits_any(int hd, int G, int splits) {
    if (hd == 128) return G == 1 ? attn_cluster_fits<128, 1>(splits) : G == 2 ? attn_cluster_fits<128, 2>(splits) : G == 4 ? attn_cluster_fits<128, 4>(splits) : G == 8 ? attn_cluster_fits<128, 8>(splits) : false;
    return G == 1 ? attn_cluster_fits<64, 1>(splits) : G == 2 ? attn_cluster_fits<64, 2>(splits) : G == 4 ? attn_cluster_fits<64, 4>(splits) : G == 8 ? attn_cluster_fits<64, 8>(splits) : false;
}

template <typename T, int HD, int G>
static void attn_launch_inst(const AttnParams &p, int n, cudaStream_t st) {
    dim3 grid(p.n_kv_heads, p.n_splits, n);
    if constexpr (std::is_same<T, __half>::value) {
        if (attn_use_mma()) {
            const size_t smem = attn_mma_smem<HD, G>();
            static bool configured[64] = {false};  // per device
            int dev = 0;
            cudaGetDevice(&dev);
            if (!configured[dev & 63]) {
                cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                configured[dev & 63] = true;
            }
            if (p.cluster_merge) {
                static bool np_set[64] = {false};
                if (!np_set[dev & 63]) {
                    cudaFuncSetAttribute(attn_mma_kernel<HD, G>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                    np_set[dev & 63] = true;
                }
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = grid;
                cfg.blockDim = dim3(kMmaWarps * 32);
                cfg.dynamicSmemBytes = smem;
                cfg.stream = st;
                cudaLaunchAttribute attr[2];
                attr[0].id = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 1;
                attr[0].val.clusterDim.y = (unsigned)p.n_splits;
                attr[0].val.clusterDim.z = 1;
                attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[1].val.programmaticStreamSerializationAllowed = 1;
                cfg.attrs = attr;
                cfg.numAttrs = pdl_enabled() ? 2 : 1;
                cudaLaunchKernelEx(&cfg, attn_mma_kernel<HD, G>, p);
                return;
            }
            launch_pdl(attn_mma_kernel<HD, G>, grid, dim3(kMmaWarps * 32), smem, st, p);
            return;
        }
    }
    launch_pdl(attn_split_kernel<T, HD, G>, grid, dim3(kAttnWarps * 32), 0, st, p);
}

template <typename T, int HD>
static int attn_launch_g(const AttnParams &p, int n, int G, cudaStream_t st) {
    switch (G) {
    case 1: attn_launch_inst<T, HD, 1>(p, n, st); return JUNO_OK;
    case 2: attn_launch_inst<T, HD, 2>(p, n, st); return JUNO_OK;
    case 4: attn_launch_inst<T, HD, 4>(p, n, st); return JUNO_OK;
    case 8: attn_launch_inst<T, HD, 8>(p, n, st); return JUNO_OK;
    default: break;
    }
    set_error("attention: query/kv head ratio %d is not supported (1, 2, 4, 8)", G);
    return JUNO_ERR_UNSUPPORTED;
}

int launch_attn(juno_ctx *ctx, const AttnArgs &a, cudaStream_t st) {
    const juno_kvpool *pool = a.pool;
    JUNO_REQUIRE(a.n_heads % pool->n_kv_heads == 0, "n_heads %d is not a multiple of n_kv_heads %d", a.n_heads,
                 pool->n_kv_heads);
    const int G = a.n_heads / pool->n_kv_heads, hd = pool->head_dim;
    JUNO_REQUIRE(hd == 64 || hd == 128, "attention: head_dim %d is not supported (64, 128)", hd);
    AttnParams p;
    p.k = pool->k;
    p.v = pool->v;
    p.table = pool->d_table;
    p.max_pages_per_seq = pool->max_pages_per_seq;
    p.n_pages = pool->n_pages;
    p.n_kv_heads = pool->n_kv_heads;
    p.n_heads = a.n_heads;
    p.layer = a.layer;
    p.n_splits = a.n_splits;
    p.q = a.q;
    p.ldq = a.ldq > 0 ? a.ldq : a.n_heads * hd;
    p.slots = a.slots;
    p.seq_lens = a.seq_lens;
    p.part_o = a.part_o;
    p.part_ml = a.part_ml;
    p.out = a.out;
    p.rope_cs = a.rope_cs;
    p.knew = a.knew;
    p.vnew = a.vnew;
    p.ldkv = a.ldkv;
    p.kw = pool->k;
    p.vw = pool->v;
    // FP16 pages, a power-of-two split count that fits one cluster and divides the group's outputs: merge in-cluster
    p.cluster_merge = 0;
    if (pool->dtype == 0 && attn_use_mma() && a.n_splits <= attn_cluster_max() &&
        (a.n_splits & (a.n_splits - 1)) == 0 && (G * hd) % a.n_splits == 0 && attn_cluster_fits_any(hd, G, a.n_splits))
        p.cluster_merge = 1;
    ProfScope prof(ctx, st, PROF_ATTN, a.algo_bytes);
    int rc;
    if (pool->dtype == 0)
        rc = hd == 128 ? attn_launch_g<__half, 128>(p, a.n, G, st) : attn_launch_g<__half, 64>(p, a.n, G, st);
    else
        rc = hd == 128 ? attn_launch_g<float, 128>(p, a.n, G, st) : attn_launch_g<float, 64>(p, a.n, G, st);
    JUNO_TRY(rc);
    JUNO_CUDA_TRY(cudaGetLastError());
    if (p.cluster_merge) {
        ctx->kernel_launches += 1;
        return JUNO_OK;
    }
    dim3 cgrid(a.n_heads, a.n);
    if (hd == 128)
        launch_pdl(attn_combine_kernel<128>, cgrid, dim3(kCombineParts * 128), 0, st, p);
    else
        launch_pdl(attn_combine_kernel<64>, cgrid, dim3(kCombineParts * 64), 0, st, p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches += 2;
    return JUNO_OK;
}

int launch_rope_table(juno_ctx *ctx, const int32_t *positions, int n, int hd, float theta, float2 *table,
                      cudaStream_t st) {
    int total = n * hd / 2;
    rope_table_kernel<<<(total + 127) / 128, 128, 0, st>>>(positions, n, hd, theta, table);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

int launch_rope_append(juno_ctx *ctx, const juno_kvpool *pool, int layer, int n, int n_heads, float *q, int ldq,
                       const float *k, const float *v, int ldkv, const int32_t *slots, const int32_t *positions,
                       const float2 *cs_table, cudaStream_t st) {
    RopeParams p;
    p.k = pool->k;
    p.v = pool->v;
    p.table = pool->d_table;
    p.max_pages_per_seq = pool->max_pages_per_seq;
    p.n_pages = pool->n_pages;
    p.n_kv_heads = pool->n_kv_heads;
    p.n_heads = n_heads;
    p.layer = layer;
    p.hd = pool->head_dim;
    p.q = q;
    p.ldq = ldq;
    p.kin = k;
    p.vin = v;
    p.ldkv = ldkv;
    p.slots = slots;
    p.positions = positions;
    p.cs = cs_table;
    ProfScope prof(ctx, st, PROF_ROPE_APPEND, 0);
    dim3 grid(n, n_heads + pool->n_kv_heads);
    if (pool->dtype == 0)
        rope_append_kernel<__half><<<grid, pool->head_dim / 2, 0, st>>>(p);
    else
        rope_append_kernel<float><<<grid, pool->head_dim / 2, 0, st>>>(p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

// ───────────────────────────── pool and sequences ─────────────────────────────────────────
int kvpool_create(juno_ctx *ctx, int n_layers, int n_kv_heads, int head_dim, int n_pages, int dtype, int max_slots,
                  int max_pages_per_seq, juno_kvpool **out) {
    JUNO_REQUIRE(n_layers > 0 && n_kv_heads > 0 && n_pages > 0 && max_slots > 0 && max_pages_per_seq > 0,
                 "bad KV pool geometry");
    JUNO_REQUIRE(head_dim == 64 || head_dim == 128, "head_dim %d is not supported (64, 128)", head_dim);
    JUNO_REQUIRE(dtype == 0 || dtype == 1, "kv_dtype %d (0 = f16, 1 = f32)", dtype);
    juno_kvpool *p = new juno_kvpool();
    p->magic = kMagicPool;
    p->ctx = ctx;
    p->n_layers = n_layers;
    p->n_kv_heads = n_kv_heads;
    p->head_dim = head_dim;
    p->n_pages = n_pages;
    p->dtype = dtype;
    p->page_tokens = kPageTokens;
    p->elem_bytes = dtype == 0 ? 2 : 4;
    p->max_slots = max_slots;
    p->max_pages_per_seq = max_pages_per_seq;
    p->k = p->v = nullptr;
    p->d_table = p->h_table = nullptr;
    p->owned_by_model = 0;
    const size_t bytes = (size_t)n_layers * n_pages * n_kv_heads * kPageTokens * head_dim * p->elem_bytes;
    const size_t tbytes = (size_t)max_slots * max_pages_per_seq * sizeof(int32_t);
    cudaError_t e = cudaMalloc(&p->k, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->v, bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&p->d_table, tbytes);
    if (e == cudaSuccess) e = cudaMallocHost((void **)&p->h_table, tbytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->d_table, 0, tbytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->k, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(p->v, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaMalloc of the KV pool (2 x %zu bytes) failed: %s", bytes, cudaGetErrorString(e));
        if (p->k) cudaFree(p->k);
        if (p->v) cudaFree(p->v);
        if (p->d_table) cudaFree(p->d_table);
        if (p->h_table) cudaFreeHost(p->h_table);
        delete p;
        return e == cudaErrorMemoryAllocation ? JUNO_ERR_OOM : JUNO_ERR_CUDA;
    }
    memset(p->h_table, 0, tbytes);
    p->free_pages.reserve(n_pages);
    for (int i = n_pages - 1; i >= 0; i--) p->free_pages.push_back(i);
    p->page_refs.assign((size_t)n_pages, 0);
    for (int i = max_slots - 1; i >= 0; i--) p->free_slots.push_back(i);
    *out = p;
    return JUNO_OK;
}

int kvpool_destroy(juno_kvpool *p) {
    if (!p) return JUNO_ERR_INVALID_ARG;
    if (p->magic != kMagicPool) {
        set_error("KV pool is closed");
        return JUNO_ERR_CLOSED;
    }
    DeviceGuard g(p->ctx->device);
    cudaStreamSynchronize(p->ctx->stream);
    cudaFree(p->k);
    cudaFree(p->v);
    cudaFree(p->d_table);
    cudaFreeHost(p->h_table);
    p->k = p->v = nullptr;
    p->magic = kMagicDead;
    return JUNO_OK;
}

int seq_create(juno_kvpool *p, int max_tokens, juno_seq **out) {
    JUNO_REQUIRE(max_tokens > 0, "max_tokens %d", max_tokens);
    const int need_pages = (max_tokens + kPageTokens - 1) / kPageTokens;
    JUNO_REQUIRE(need_pages <= p->max_pages_per_seq, "max_tokens %d exceeds the pool's per-sequence limit %d", max_tokens,
                 p->max_pages_per_seq * kPageTokens);
    if (p->free_slots.empty()) {
        set_error("no free sequence slot (max %d live sequences)", p->max_slots);
        return JUNO_ERR_OOM;
    }
    juno_seq *s = new juno_seq();
    s->magic = kMagicSeq;
    s->pool = p;
    s->max_tokens = max_tokens;
    s->len = 0;
    s->slot = p->free_slots.back();
    p->free_slots.pop_back();
    *out = s;
    return JUNO_OK;
}

// Copies one page (all layers, K and V) to another on the device, ordered on `st`.
static int page_copy(juno_kvpool *p, int dst, int src, cudaStream_t st) {
    const size_t page_bytes = (size_t)p->n_kv_heads * kPageTokens * p->head_dim * p->elem_bytes;
    for (int layer = 0; layer < p->n_layers; layer++) {
        const size_t d = ((size_t)layer * p->n_pages + dst) * page_bytes, s = ((size_t)layer * p->n_pages + src) * page_bytes;
        JUNO_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t *>(p->k) + d, static_cast<const uint8_t *>(p->k) + s, page_bytes, cudaMemcpyDeviceToDevice, st));
        JUNO_CUDA_TRY(cudaMemcpyAsync(static_cast<uint8_t *>(p->v) + d, static_cast<const uint8_t *>(p->v) + s, page_bytes, cudaMemcpyDeviceToDevice, st));
    }
    return JUNO_OK;
}

int seq_reserve(juno_seq *s, int from, int upto, cudaStream_t st) {
    juno_kvpool *p = s->pool;
    JUNO_REQUIRE(upto <= s->max_tokens, "position %d is beyond this sequence's limit of %d", upto - 1, s->max_tokens);
    const int need = (upto + kPageTokens - 1) / kPageTokens;
    const int have = (int)s->pages.size();
    // pages of [from, upto) that another sequence holds too (a shared prefix): this sequence writes into its own copy
    const int first = std::max(0, from) / kPageTokens, last = std::min(need, have) - 1;
    int shared = 0;
    for (int i = first; i <= last; i++) shared += p->page_refs[(size_t)s->pages[(size_t)i]] > 1 ? 1 : 0;
    const int fresh = std::max(0, need - have) + shared;
    if (fresh == 0) return JUNO_OK;
    if ((int)p->free_pages.size() < fresh) {
        set_error("KV pool exhausted: %d pages free, %d needed", (int)p->free_pages.size(), fresh);
        return JUNO_ERR_OOM;
    }
    int32_t *row = p->h_table + (size_t)s->slot * p->max_pages_per_seq;
    int lo = need, hi = -1;  // table entries that change
    for (int i = first; i <= last; i++) {
        const int old = s->pages[(size_t)i];
        if (p->page_refs[(size_t)old] <= 1) continue;
        const int pg = p->free_pages.back();
        p->free_pages.pop_back();
        JUNO_TRY(page_copy(p, pg, old, st));
        p->page_refs[(size_t)old]--;
        p->page_refs[(size_t)pg] = 1;
        s->pages[(size_t)i] = pg;
        row[i] = pg;
        lo = std::min(lo, i);
        hi = std::max(hi, i);
    }
    for (int i = have; i < need; i++) {
        int pg = p->free_pages.back();
        p->free_pages.pop_back();
        p->page_refs[(size_t)pg] = 1;
        s->pages.push_back(pg);
        row[i] = pg;
        lo = std::min(lo, i);
        hi = std::max(hi, i);
    }
    JUNO_CUDA_TRY(cudaMemcpyAsync(p->d_table + (size_t)s->slot * p->max_pages_per_seq + lo, row + lo,
                                  (size_t)(hi - lo + 1) * sizeof(int32_t), cudaMemcpyHostToDevice, st));
    return JUNO_OK;
}

static int seq_check(juno_seq *s) {
    if (!s) {
        set_error("sequence is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (s->magic != kMagicSeq || !s->pool || s->pool->magic != kMagicPool) {
        set_error("sequence handle is closed");
        return JUNO_ERR_CLOSED;
    }
    return JUNO_OK;
}

}  // namespace juno

using namespace juno;

extern "C" {

int juno_kvpool_create(juno_ctx *c, int32_t n_layers, int32_t n_kv_heads, int32_t head_dim, int32_t n_pages,
                       int32_t kv_dtype, juno_kvpool **out) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(out, "out is null");
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    return kvpool_create(c, n_layers, n_kv_heads, head_dim, n_pages, kv_dtype, 256, std::min(n_pages, 8192), out);
}

int juno_kvpool_free(juno_kvpool *p) {
    if (!p) {
        set_error("pool is null");
        return JUNO_ERR_INVALID_ARG;
    }
    if (p->magic != kMagicPool) {
        set_error("KV pool is closed");
        return JUNO_ERR_CLOSED;
    }
    JUNO_REQUIRE(!p->owned_by_model, "this pool belongs to a model; free the model instead");
    std::lock_guard<std::recursive_mutex> lk(p->ctx->mu);
    return kvpool_destroy(p);
}

int juno_kvseq_create(juno_kvpool *p, int32_t max_tokens, juno_seq **out) {
    JUNO_REQUIRE(p && out, "null argument");
    if (p->magic != kMagicPool) {
        set_error("KV pool is closed");
        return JUNO_ERR_CLOSED;
    }
    std::lock_guard<std::recursive_mutex> lk(p->ctx->mu);
    return seq_create(p, max_tokens, out);
}

int juno_seq_free(juno_seq *s) {
    JUNO_TRY(seq_check(s));
    juno_kvpool *p = s->pool;
    std::lock_guard<std::recursive_mutex> lk(p->ctx->mu);
    {
        DeviceGuard g(p->ctx->device);
        cudaStreamSynchronize(p->ctx->stream);  // no kernel may still read these pages
    }
    for (int pg : s->pages)
        if (--p->page_refs[(size_t)pg] == 0) p->free_pages.push_back(pg);  // a shared page stays with its other holders
    p->free_slots.push_back(s->slot);
    s->pages.clear();
    s->magic = kMagicDead;
    return JUNO_OK;
}

int juno_seq_fork(juno_seq *src, int32_t n_tokens, juno_seq **out) {
    JUNO_TRY(seq_check(src));
    JUNO_REQUIRE(out, "out is null");
    JUNO_REQUIRE(n_tokens >= 0 && n_tokens <= src->len, "cannot share %d positions of a sequence that holds %d", n_tokens, src->len);
    juno_kvpool *p = src->pool;
    std::lock_guard<std::recursive_mutex> lk(p->ctx->mu);
    DeviceGuard g(p->ctx->device);
    juno_seq *s = nullptr;
    JUNO_TRY(seq_create(p, src->max_tokens, &s));
    const int n_pg = (n_tokens + kPageTokens - 1) / kPageTokens;
    int32_t *row = p->h_table + (size_t)s->slot * p->max_pages_per_seq;
    for (int i = 0; i < n_pg; i++) {
        const int pg = src->pages[(size_t)i];
        p->page_refs[(size_t)pg]++;
        s->pages.push_back(pg);
        row[i] = pg;
    }
    s->len = n_tokens;
    if (n_pg) {
        cudaError_t e = cudaMemcpyAsync(p->d_table + (size_t)s->slot * p->max_pages_per_seq, row, (size_t)n_pg * sizeof(int32_t),
                                        cudaMemcpyHostToDevice, p->ctx->stream);
        if (e != cudaSuccess) {
            for (int pg : s->pages) p->page_refs[(size_t)pg]--;
            p->free_slots.push_back(s->slot);
            s->magic = kMagicDead;
            delete s;
            JUNO_CUDA_TRY(e);
        }
    }
    *out = s;
    return JUNO_OK;
}

int juno_seq_length(juno_seq *s, int32_t *n_tokens) {
    JUNO_TRY(seq_check(s));
    JUNO_REQUIRE(n_tokens, "n_tokens is null");
    *n_tokens = s->len;
    return JUNO_OK;
}

int juno_seq_append_kv(juno_seq *s, int32_t layer, int32_t pos, int32_t n_tokens, const float *k_host,
                       const float *v_host) {
    JUNO_TRY(seq_check(s));
    juno_kvpool *p = s->pool;
    juno_ctx *c = p->ctx;
    JUNO_REQUIRE(k_host && v_host, "null K/V");
    JUNO_REQUIRE(layer >= 0 && layer < p->n_layers, "layer %d out of range", layer);
    JUNO_REQUIRE(pos >= 0 && n_tokens >= 0, "bad position range");
    if (n_tokens == 0) return JUNO_OK;
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    JUNO_TRY(seq_reserve(s, pos, pos + n_tokens, c->stream));
    const int kvdim = p->n_kv_heads * p->head_dim;
    const size_t bytes = (size_t)n_tokens * kvdim * sizeof(float);
    void *px = c->stage_x, *py = c->stage_y;
    JUNO_TRY(ensure_device(&px, &c->stage_x_bytes, bytes));
    c->stage_x = (float *)px;
    JUNO_TRY(ensure_device(&py, &c->stage_y_bytes, bytes));
    c->stage_y = (float *)py;
    JUNO_CUDA_TRY(cudaMemcpyAsync(c->stage_x, k_host, bytes, cudaMemcpyHostToDevice, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(c->stage_y, v_host, bytes, cudaMemcpyHostToDevice, c->stream));
    const size_t total = (size_t)n_tokens * kvdim;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    const int32_t *row = p->d_table + (size_t)s->slot * p->max_pages_per_seq;
    if (p->dtype == 0)
        kv_scatter_kernel<__half><<<blocks, 256, 0, c->stream>>>(p->k, p->v, row, p->n_pages, p->n_kv_heads, p->head_dim,
                                                                  layer, pos, n_tokens, c->stage_x, c->stage_y);
    else
        kv_scatter_kernel<float><<<blocks, 256, 0, c->stream>>>(p->k, p->v, row, p->n_pages, p->n_kv_heads, p->head_dim,
                                                                 layer, pos, n_tokens, c->stage_x, c->stage_y);
    JUNO_CUDA_TRY(cudaGetLastError());
    c->kernel_launches++;
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->h2d_bytes += (int64_t)(2 * bytes);
    s->len = std::max(s->len, pos + n_tokens);
    return JUNO_OK;
}

int juno_attn_decode(juno_ctx *c, juno_kvpool *p, int32_t layer, int32_t n, juno_seq *const *seqs, int32_t n_heads,
                     const float *q_host, float *out_host) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(p && seqs && q_host && out_host, "null argument");
    if (p->magic != kMagicPool) {
        set_error("KV pool is closed");
        return JUNO_ERR_CLOSED;
    }
    JUNO_REQUIRE(p->ctx == c, "pool belongs to another context");
    JUNO_REQUIRE(n >= 1 && n <= 4096, "n=%d out of range", n);
    JUNO_REQUIRE(layer >= 0 && layer < p->n_layers, "layer %d out of range", layer);
    JUNO_REQUIRE(n_heads > 0 && n_heads % p->n_kv_heads == 0, "n_heads %d is not a multiple of n_kv_heads %d", n_heads,
                 p->n_kv_heads);
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    int max_len = 0;
    std::vector<int32_t> meta(2 * (size_t)n);
    for (int i = 0; i < n; i++) {
        JUNO_TRY(seq_check(seqs[i]));
        JUNO_REQUIRE(seqs[i]->pool == p, "sequence %d belongs to another pool", i);
        JUNO_REQUIRE(seqs[i]->len > 0, "sequence %d is empty", i);
        meta[i] = seqs[i]->slot;
        meta[n + i] = seqs[i]->len;
        max_len = std::max(max_len, seqs[i]->len);
    }
    const int hd = p->head_dim, qdim = n_heads * hd;
    const int n_splits = attn_pick_splits(c, n, p->n_kv_heads, max_len);
    const size_t qbytes = (size_t)n * qdim * sizeof(float);
    const size_t scratch = attn_scratch_floats(n, n_heads, hd, n_splits) * sizeof(float);
    const size_t meta_bytes = meta.size() * sizeof(int32_t);
    // stage_x: q | meta ; stage_y: out | scratch
    const size_t qoff = (qbytes + 255) & ~(size_t)255;
    void *px = c->stage_x, *py = c->stage_y;
    JUNO_TRY(ensure_device(&px, &c->stage_x_bytes, qoff + meta_bytes));
    c->stage_x = (float *)px;
    JUNO_TRY(ensure_device(&py, &c->stage_y_bytes, qoff + scratch));
    c->stage_y = (float *)py;
    int32_t *d_meta = reinterpret_cast<int32_t *>(reinterpret_cast<uint8_t *>(c->stage_x) + qoff);
    JUNO_CUDA_TRY(cudaMemcpyAsync(c->stage_x, q_host, qbytes, cudaMemcpyHostToDevice, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(d_meta, meta.data(), meta_bytes, cudaMemcpyHostToDevice, c->stream));
    AttnArgs a;
    a.pool = p;
    a.layer = layer;
    a.n = n;
    a.n_heads = n_heads;
    a.q = c->stage_x;
    a.out = c->stage_y;
    a.slots = d_meta;
    a.seq_lens = d_meta + n;
    a.n_splits = n_splits;
    for (int i = 0; i < n; i++) a.algo_bytes += (double)seqs[i]->len * p->n_kv_heads * hd * 2 * p->elem_bytes;
    float *sc = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(c->stage_y) + qoff);
    a.part_o = sc;
    a.part_ml = sc + (size_t)n * n_heads * n_splits * hd;
    JUNO_TRY(launch_attn(c, a, c->stream));
    JUNO_CUDA_TRY(cudaMemcpyAsync(out_host, c->stage_y, qbytes, cudaMemcpyDeviceToHost, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));  // meta (pageable host memory) is consumed by now
    c->h2d_bytes += (int64_t)(qbytes + meta_bytes);
    c->d2h_bytes += (int64_t)qbytes;
    return JUNO_OK;
}


// ── attention without any allocation ─────────────────────────────────────────────────────────
// Scratch for juno_attn_decode_static: the per-split partial outputs, the (max, sum) pairs and the per-sequence
// page-table row / length words.  It lives in the library image, so every GPU that loads the library holds these
// 8 MiB until the process exits.
constexpr size_t kStaticAttnScratchBytes = 8u << 20;
constexpr int kStaticAttnMaxSeqs = 256;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticAttnScratchBytes];
static std::mutex g_static_attn_mu[64];                // one per device ordinal: held for a whole call, because the array is per device
static void *g_static_attn_ptr[64] = {nullptr};  // device address of the array, per device ordinal

int juno_attn_decode_static(juno_ctx *c, juno_kvpool *p, int32_t layer, int32_t n, juno_seq *const *seqs, int32_t n_heads,
                            const float *q_dev, float *out_dev) {
    JUNO_TRY(ctx_check(c));
    JUNO_REQUIRE(p && seqs && q_dev && out_dev, "null argument");
    if (p->magic != kMagicPool) {
        set_error("KV pool is closed");
        return JUNO_ERR_CLOSED;
    }
    JUNO_REQUIRE(p->ctx == c, "pool belongs to another context");
    JUNO_REQUIRE(n >= 1 && n <= kStaticAttnMaxSeqs, "n=%d outside [1,%d] (limit of the allocation-free entry point)", n,
                 kStaticAttnMaxSeqs);
    JUNO_REQUIRE(layer >= 0 && layer < p->n_layers, "layer %d out of range", layer);
    JUNO_REQUIRE(n_heads > 0 && n_heads % p->n_kv_heads == 0, "n_heads %d is not a multiple of n_kv_heads %d", n_heads,
                 p->n_kv_heads);
    JUNO_REQUIRE(c->device >= 0 && c->device < 64, "device ordinal %d not supported here", c->device);
    // Two contexts of one device share the array: the per-device lock is held until this call's kernels have drained.
    std::lock_guard<std::mutex> dev_lock(g_static_attn_mu[c->device]);
    std::lock_guard<std::recursive_mutex> lk(c->mu);
    DeviceGuard g(c->device);
    // One-time set-up per device, with that device current: in host code the array's name is only a handle, the
    // address a kernel can use comes from cudaGetSymbolAddress.
    void *base = nullptr;
    {
        if (!g_static_attn_ptr[c->device]) {
            void *ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_attn_scratch);
            if (e != cudaSuccess || !ptr) {
                set_error("cudaGetSymbolAddress(static attention scratch) failed: rc=%d (%s)", (int)e, cudaGetErrorString(e));
                return JUNO_ERR_CUDA;
            }
            g_static_attn_ptr[c->device] = ptr;
        }
        base = g_static_attn_ptr[c->device];
    }
    int32_t meta[2 * kStaticAttnMaxSeqs];
    int max_len = 0;
    for (int i = 0; i < n; i++) {
        JUNO_TRY(seq_check(seqs[i]));
        JUNO_REQUIRE(seqs[i]->pool == p, "sequence %d belongs to another pool", i);
        JUNO_REQUIRE(seqs[i]->len > 0, "sequence %d is empty", i);
        meta[i] = seqs[i]->slot;
        meta[n + i] = seqs[i]->len;
        max_len = std::max(max_len, seqs[i]->len);
    }
    const int hd = p->head_dim;
    const size_t meta_bytes = 2 * (size_t)kStaticAttnMaxSeqs * sizeof(int32_t);
    const size_t per_split = (size_t)n * n_heads * (hd + 2) * sizeof(float);
    const size_t room = kStaticAttnScratchBytes - meta_bytes;
    if (per_split > room) {
        set_error("n=%d sequences x %d heads x head_dim %d need %zu bytes of scratch per context split; the allocation-free "
                  "entry point has %zu", n, n_heads, hd, per_split, room);
        return JUNO_ERR_INVALID_ARG;
    }
    int n_splits = attn_pick_splits(c, n, p->n_kv_heads, max_len);
    n_splits = (int)std::min<size_t>((size_t)n_splits, room / per_split);
    int32_t *d_meta = static_cast<int32_t *>(base);
    float *sc = reinterpret_cast<float *>(static_cast<unsigned char *>(base) + meta_bytes);
    JUNO_CUDA_TRY(cudaMemcpyAsync(d_meta, meta, 2 * (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, c->stream));
    AttnArgs a;
    a.pool = p;
    a.layer = layer;
    a.n = n;
    a.n_heads = n_heads;
    a.q = q_dev;
    a.out = out_dev;
    a.slots = d_meta;
    a.seq_lens = d_meta + n;
    a.n_splits = n_splits;
    a.part_o = sc;  // every (sequence, head, split) entry is rewritten by this call: nothing has to start at zero
    a.part_ml = sc + (size_t)n * n_heads * n_splits * hd;
    for (int i = 0; i < n; i++) a.algo_bytes += (double)seqs[i]->len * p->n_kv_heads * hd * 2 * p->elem_bytes;
    JUNO_TRY(launch_attn(c, a, c->stream));
    JUNO_CUDA_TRY(cudaStreamSynchronize(c->stream));  // `meta` lives on this stack frame
    return JUNO_OK;
}

}  // extern "C"
