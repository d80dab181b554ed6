// Fused dequant-GEMV for GGUF Q4_K / Q6_K / Q8_0 weights, batched over decode sequences.
//
// y[b][r] = sum_c w(r,c) * x[b][c] with w dequantised on the fly exactly as
// LlamaTransformerHandler.matVecQ4Kraw/Q6Kraw/Q8_0raw do (LlamaTransformerHandler.java:1428-1508,
// 1587-1638), but accumulated in a different order (FP32 throughout).
//
// Data flow per warp: 128-bit coalesced loads of one 16x256 tile straight from HBM into registers
// (layout.cuh), 4/6/8-bit fields unpacked in registers into exact small-integer bf16 pairs, one
// mma.sync.m16n8k16 per 16 columns against the activation held in shared memory as three bf16
// limbs (x = hi+mid+lo exactly, so the products are exact FP32 terms), the per-sub-block scale
// applied to the FP32 accumulator fragment, and the Q4_K "min" term handled the same way with an
// m16n8k8 MMA of the 6-bit mins against per-sub-block sums of x.  Tensor cores are used here as an
// exact integer-times-float dot-product unit; the kernel is bound by HBM, not by the tensor pipe.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "gemv.cuh"
#include "layout.cuh"
#include "dequant.cuh"
#include "stage.cuh"
#include "tile_math.cuh"
#include "gemv_params.cuh"
#include "step.cuh"

namespace juno {

// ───────────────────────────── activation staging ─────────────────────────────────────────
// One CTA per batch row writes that row's three limb columns of the staged image.
struct StageParams {
    int mode;
    const float *x;
    int ldx;
    const float *x_add, *normw;
    float *x_out;
    float eps;
    StageImage im;
};

size_t stage_chunk_bytes(int K, int rows_in_chunk) { return (size_t)K * 3 * rows_in_chunk * 2; }

constexpr int kStageThreads = 256;

__global__ void __launch_bounds__(kStageThreads) stage_kernel(const StageParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.im.K;
    unsigned short *xb;
    int NC, col0;
    p.im.locate(b, xb, NC, col0);
    const float *xrow = p.x + (size_t)b * p.ldx;
    const float *arow = p.x_add ? p.x_add + (size_t)b * p.ldx : nullptr;
    float scale = 1.f;
    __shared__ float red[kStageThreads / 32];
    if (p.mode == STAGE_RMSNORM) {
        float part = 0.f;
        for (int i = tid; i < K; i += kStageThreads) {
            float r = xrow[i];
            if (arow) r = __fadd_rn(r, arow[i]);
            part = fmaf(r, r, part);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        float ss = 0.f;
#pragma unroll
        for (int w8 = 0; w8 < kStageThreads / 32; w8++) ss += red[w8];
        // rmsNorm (:818-828): 1f / (float) Math.sqrt(ss / n + eps)
        scale = __fdiv_rn(1.f, (float)sqrt((double)__fadd_rn(__fdiv_rn(ss, (float)K), p.eps)));
    }
    // each thread handles 4 consecutive columns = one (s16, c) group of the feed order
    for (int i4 = tid * 4; i4 < K; i4 += kStageThreads * 4) {
        float v[4];
        const float4 xv = *reinterpret_cast<const float4 *>(xrow + i4);
        v[0] = xv.x; v[1] = xv.y; v[2] = xv.z; v[3] = xv.w;
        if (p.mode == STAGE_RMSNORM) {
            if (arow) {
                const float4 av = *reinterpret_cast<const float4 *>(arow + i4);
                v[0] = __fadd_rn(v[0], av.x); v[1] = __fadd_rn(v[1], av.y);
                v[2] = __fadd_rn(v[2], av.z); v[3] = __fadd_rn(v[3], av.w);
            }
            if (p.x_out) *reinterpret_cast<float4 *>(p.x_out + (size_t)b * p.ldx + i4) = make_float4(v[0], v[1], v[2], v[3]);
            const float4 wv = *reinterpret_cast<const float4 *>(p.normw + i4);
            v[0] = __fmul_rn(__fmul_rn(wv.x, v[0]), scale);
            v[1] = __fmul_rn(__fmul_rn(wv.y, v[1]), scale);
            v[2] = __fmul_rn(__fmul_rn(wv.z, v[2]), scale);
            v[3] = __fmul_rn(__fmul_rn(wv.w, v[3]), scale);
        }
        unsigned short l[3][4];
#pragma unroll
        for (int t = 0; t < 4; t++) split3(v[t], l[0][t], l[1][t], l[2][t]);
        const int s16 = i4 >> 4, c = (i4 >> 2) & 3;
        unsigned short *dst = xb + ((size_t)(s16 * NC + col0) * 4 + c) * 4;
#pragma unroll
        for (int k = 0; k < 3; k++) {  // feed order: columns (4c, 4c+2, 4c+1, 4c+3)
            uint2 w;
            w.x = (uint32_t)l[k][0] | ((uint32_t)l[k][2] << 16);
            w.y = (uint32_t)l[k][1] | ((uint32_t)l[k][3] << 16);
            *reinterpret_cast<uint2 *>(dst + k * 16) = w;
        }
    }
}

// ───────────────────────────── the GEMV kernel ────────────────────────────────────────────
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;


// Address of tile (R, sb) and, for mixed launches, the block format of R's segment.
template <int TYPE>
__device__ __forceinline__ const uint8_t *tile_addr(const GemvParams &p, int R, int sb, int &type) {
    const int s = seg_of(p, R);
    type = (TYPE == 0) ? p.seg_type[s] : TYPE;
    return p.w[s] + ((size_t)(R - p.rt_begin[s]) * p.nb + sb) * (size_t)tile_bytes(type);
}

// Hint: bring [a, a+bytes) into the L2 (16-byte aligned, bytes a multiple of 16).  No completion, no dependency.
__device__ __forceinline__ void l2_prefetch_range(const uint8_t *a, unsigned bytes) {
    for (unsigned o = 0; o < bytes; o += 32768u) {
        const unsigned n = min(32768u, bytes - o);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a + o), "r"(n) : "memory");
    }
}

template <int TYPE>
__device__ __forceinline__ void gemv_prefetch_own(const GemvParams &p, int tid) {
    // own weights: the row tiles of CTA tasks blockIdx.x, blockIdx.x + grid, ... below pf_rt, one row tile per thread
    for (int i = tid;; i += kThreads) {
        const int r = i / p.groups, g = i - r * p.groups;
        const int ct = blockIdx.x + r * gridDim.x;
        if (ct >= p.n_ctasks || ct * p.groups >= p.pf_rt) break;
        const int R = ct * p.groups + g;
        if (R < p.pf_rt) {
            int ty;
            const uint8_t *a = tile_addr<TYPE>(p, R, 0, ty);
            l2_prefetch_range(a, (unsigned)(p.nb * tile_bytes(ty)));
        }
    }
}

// The products that follow: each CTA one slice per range, issued by the first lane of warps 1..3.
__device__ __forceinline__ void gemv_prefetch_next(const GemvParams &p, int tid) {
    if ((tid & 31) == 0 && tid >= 32 && tid < 128) {
        const int r = (tid >> 5) - 1;
        const unsigned bytes = p.pfx_bytes[r];
        if (bytes) {
            const unsigned per = (((bytes + gridDim.x - 1) / gridDim.x) + 15u) & ~15u;
            const unsigned long long off = (unsigned long long)blockIdx.x * per;
            if (off < bytes) l2_prefetch_range(p.pfx[r] + off, min(per, (unsigned)(bytes - off)));
        }
    }
}

template <int TYPE, int NB>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvParams p) {
    constexpr int NC = 3 * NB, NT = (NC + 7) / 8, LD = 8 * NT;
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = p.K;
    unsigned short *xb = reinterpret_cast<unsigned short *>(smem);  // K*NC bf16 limbs
    unsigned short *xs = xb + (size_t)K * NC;                       // (K/32)*NC bf16: 32-column sums (Q4_K only)
    const size_t xs_bytes = (TYPE == 12 || TYPE == 0) ? ((((size_t)(K / 32) * NC * 2) + 15) & ~(size_t)15) : 0;
    float *cs = reinterpret_cast<float *>(smem + p.img_bytes + xs_bytes);  // [2][kWarps][16][LD]
    float *sqbuf = cs + 2 * kWarps * 16 * LD;                               // [groups*16*NB] (EPI_RESID_NORM)
    float *scale_s = sqbuf + kWarps * 16 * NB;                              // [NB]
    int *next_task = reinterpret_cast<int *>(scale_s + 8);

    // A CTA task is `groups` row tiles; the kin warps of a group split K.  Task ids beyond the first come
    // from a device counter, so CTAs that finish early take more.
    const int grp = warp / p.kin, kj = warp - grp * p.kin;
    const int sb0 = kj * p.tpt;
    int ct = blockIdx.x;
    if (tid == 0) next_task[0] = gridDim.x + (int)atomicAdd(p.counters, 1u);

    if (p.pf_rt > 0) gemv_prefetch_own<TYPE>(p, tid);
    if (p.pfx_bytes[0] && !p.pf_late) gemv_prefetch_next(p, tid);
    // Issue the first tile's loads before touching x: the weights do not depend on the producer of x.
    TileRegs<TYPE> bufA, bufB;
    int R = ct * p.groups + grp;
    bool have = (ct < p.n_ctasks) && (R < p.total_rt);
    int cur_type = TYPE, next_type = TYPE;
    const uint8_t *cur_ptr = have ? tile_addr<TYPE>(p, R, sb0, cur_type) : nullptr;
    if (have) load_tile_t<TYPE>(bufA, cur_ptr, lane, cur_type);
    pdl_wait();  // everything below reads what earlier kernels of the stream wrote

    // staged activation -> shared memory
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.ximg);
        uint4 *dst = reinterpret_cast<uint4 *>(smem);
        const int n16 = (int)(p.img_bytes >> 4);
        for (int i = tid; i < n16; i += kThreads) dst[i] = src[i];
    }
    // RMSNorm scale of the input from the producer's per-task sums of squares (fixed summation order)
    if (warp < NB) {
        float sc = 1.f;
        if (p.ss_parts) {
            float s = 0.f;
            for (int i = lane; i < p.n_parts; i += 32) s += p.ss_parts[(size_t)warp * p.ss_ld + i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            sc = __fdiv_rn(1.f, (float)sqrt((double)__fadd_rn(__fdiv_rn(s, (float)p.scale_n), p.eps)));
        }
        if (lane == 0) scale_s[warp] = sc;
    }
    __syncthreads();
    if (TYPE == 12 || TYPE == 0) {
        // sums of x over 32 columns, from the limbs (hi + mid + lo is x exactly): eight threads per sum
        const int total = (K / 4) * NB;
        for (int item = tid; item < total; item += kThreads) {
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
        __syncthreads();
    }

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

    int phase = 0, it = 0;
    while (ct < p.n_ctasks) {
        const int nct = next_task[it & 1];
        if (tid == 0) next_task[(it + 1) & 1] = gridDim.x + (int)atomicAdd(p.counters, 1u);
        const int nR = nct * p.groups + grp;
        const bool nhave = (nct < p.n_ctasks) && (nR < p.total_rt);
        // first tile of this warp in the next task (prefetched while the last tile of this one is computed)
        const uint8_t *next_base = nhave ? tile_addr<TYPE>(p, nR, sb0, next_type) : nullptr;
        if (have) {
            for (int j = 0; j < p.tpt; j++) {
                const bool more = j + 1 < p.tpt;
                const uint8_t *np = more ? cur_ptr + tile_bytes(cur_type) : next_base;
                const int np_type = more ? cur_type : next_type;
                if (phase == 0) {
                    if (np) load_tile_t<TYPE>(bufB, np, lane, np_type);
                    if constexpr (TYPE == 0)
                        compute_tile_mixed<NC>(bufA, cur_type, sb0 + j, xv, lane, acc, macc);
                    else
                        compute_tile_t<TYPE, NC>(bufA, cur_type, sb0 + j, xv, lane, acc, macc);
                } else {
                    if (np) load_tile_t<TYPE>(bufA, np, lane, np_type);
                    if constexpr (TYPE == 0)
                        compute_tile_mixed<NC>(bufB, cur_type, sb0 + j, xv, lane, acc, macc);
                    else
                        compute_tile_t<TYPE, NC>(bufB, cur_type, sb0 + j, xv, lane, acc, macc);
                }
                cur_ptr = np;
                phase ^= 1;
            }
            cur_type = next_type;
        } else if (nhave) {  // idle in this task, but the next one has work: fetch its first tile
            if (phase == 0)
                load_tile_t<TYPE>(bufA, next_base, lane, next_type);
            else
                load_tile_t<TYPE>(bufB, next_base, lane, next_type);
            cur_ptr = next_base;
            cur_type = next_type;
        }
        // fragments -> shared memory (double-buffered: one barrier per task)
        float *mycs = cs + ((it & 1) * kWarps + warp) * 16 * LD;
        {
            const int r8 = lane >> 2, c = lane & 3;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float *row0 = mycs + r8 * LD + nt * 8 + 2 * c;
                float *row1 = mycs + (r8 + 8) * LD + nt * 8 + 2 * c;
                *reinterpret_cast<float2 *>(row0) = make_float2(acc[nt][0] - macc[nt][0], acc[nt][1] - macc[nt][1]);
                *reinterpret_cast<float2 *>(row1) = make_float2(acc[nt][2] - macc[nt][2], acc[nt][3] - macc[nt][3]);
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
                macc[nt][0] = macc[nt][1] = macc[nt][2] = macc[nt][3] = 0.f;
            }
        }
        __syncthreads();
        // cooperative epilogue: add the K chunks of each row in warp order, then the three limbs
        {
            const float *csb = cs + (it & 1) * kWarps * 16 * LD;
            const int rows_out = (p.epi == EPI_SILU_PAIR) ? 8 : 16;
            const int per_b = p.groups * rows_out, total = per_b * NB;
            // successive tasks start their epilogue on successive warps, so no single warp carries it every time
            const int etid = (tid + 32 * (it & 7)) & (kThreads - 1);
            for (int idx = etid; idx < total; idx += kThreads) {
                const int b = idx / per_b, rg = idx - b * per_b, g = rg / rows_out, row = rg - g * rows_out;
                const int Rg = ct * p.groups + g;
                float sq = 0.f;
                if (Rg < p.total_rt) {
                    int s = 0;
                    if (p.nseg > 1 && Rg >= p.rt_begin[1]) s = 1;
                    if (p.nseg > 2 && Rg >= p.rt_begin[2]) s = 2;
                    const int tile_in_seg = Rg - p.rt_begin[s];
                    float v = 0.f, v2 = 0.f;
                    for (int k2 = 0; k2 < p.kin; k2++) {
                        const float *cr = csb + ((g * p.kin + k2) * 16 + row) * LD + 3 * b;
                        v += (cr[2] + cr[1]) + cr[0];
                        if (p.epi == EPI_SILU_PAIR) {
                            const float *cu = cr + 8 * LD;
                            v2 += (cu[2] + cu[1]) + cu[0];
                        }
                    }
                    const float sc = scale_s[b];
                    v = __fmul_rn(v, sc);
                    const int orow = tile_in_seg * rows_out + row;
                    if (orow < p.rows[s]) {
                        float o = v;
                        if (p.epi == EPI_SILU_PAIR) {
                            o = __fmul_rn(silu_ref(v), __fmul_rn(v2, sc));
                        } else if (p.epi == EPI_RESID_NORM) {
                            o = __fadd_rn(p.resid[(size_t)b * p.ldx + orow], v);
                            p.x_out[(size_t)b * p.ldx + orow] = o;
                            sq = __fmul_rn(o, o);
                            o = __fmul_rn(p.normw_next[orow], o);
                        }
                        if (p.epi != EPI_RESID_NORM && p.out[s]) p.out[s][(size_t)b * p.ld_out + orow] = o;
                        if (p.img_next.img) {
                            unsigned short *nxb;
                            int nNC, ncol0;
                            p.img_next.locate(b, nxb, nNC, ncol0);
                            stage_store1(nxb, nNC, ncol0, orow, o);
                        }
                    }
                }
                if (p.epi == EPI_RESID_NORM) sqbuf[idx] = sq;
            }
            if (p.epi == EPI_RESID_NORM) {  // per-task sum of squares, rows in order
                __syncthreads();
                if (etid < NB) {
                    float s = 0.f;
                    for (int i = 0; i < per_b; i++) s += sqbuf[etid * per_b + i];
                    p.ss_out[(size_t)etid * p.ss_out_ld + ct] = s;
                }
            }
        }
        ct = nct;
        R = nR;
        have = nhave;
        it++;
    }
    if (p.pfx_bytes[0] && p.pf_late) gemv_prefetch_next(p, tid);  // HBM goes idle as the CTAs run out of tasks
    // the last CTA to leave zeroes the counters for the next launch that uses this pair
    if (tid == 0) {
        const unsigned done = atomicAdd(p.counters + 1, 1u);
        if (done == gridDim.x - 1) {
            p.counters[0] = 0u;
            p.counters[1] = 0u;
        }
    }
}

// ───────────────────────────── host: launch ───────────────────────────────────────────────
static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

static size_t gemv_smem_bytes(int K, int nb_batch) {
    const int NT = (3 * nb_batch + 7) / 8;
    const size_t xs = ((((size_t)(K / 32) * 3 * nb_batch * 2) + 15) & ~(size_t)15);
    return stage_chunk_bytes(K, nb_batch) + xs + (size_t)2 * kWarps * 16 * 8 * NT * 4 + (size_t)kWarps * 16 * nb_batch * 4 +
           32 + 16;
}

int gemv_batch_chunk(const juno_ctx *ctx, int K, int batch) {
    int bc = std::min(batch, 8);
    while (bc > 1 && gemv_smem_bytes(K, bc) > ctx->smem_optin) bc--;
    return bc;
}

size_t stage_image_bytes(const juno_ctx *ctx, int K, int batch) {
    const int bc = gemv_batch_chunk(ctx, K, batch);
    const int chunks = (batch + bc - 1) / bc;
    return (size_t)chunks * stage_chunk_bytes(K, bc);
}

StageImage stage_image_desc(const juno_ctx *ctx, uint8_t *img, int K, int batch) {
    StageImage im;
    im.img = img;
    im.K = K;
    im.batch = batch;
    im.bc = gemv_batch_chunk(ctx, K, batch);
    im.b0 = 0;
    im.chunk_stride = stage_chunk_bytes(K, im.bc);
    return im;
}

int launch_stage(juno_ctx *ctx, const StageArgs &a, cudaStream_t st) {
    JUNO_REQUIRE(a.K > 0 && a.K % 256 == 0 && a.batch >= 1 && a.x && a.img, "stage: bad arguments (K=%d)", a.K);
    JUNO_REQUIRE(a.ldx % 4 == 0, "stage: row stride %d must be a multiple of 4", a.ldx);
    StageParams p;
    p.mode = a.mode;
    p.x = a.x;
    p.ldx = a.ldx;
    p.x_add = a.x_add;
    p.normw = a.normw;
    p.x_out = a.x_out;
    p.eps = a.eps;
    p.im = stage_image_desc(ctx, a.img, a.K, a.batch);
    ProfScope prof(ctx, st, PROF_OTHER, 0);
    JUNO_CUDA_TRY(launch_pdl(stage_kernel, dim3(a.batch), dim3(kStageThreads), 0, st, p));
    ctx->kernel_launches++;
    return JUNO_OK;
}

template <int TYPE, int NB>
static int launch_inst(juno_ctx *ctx, const GemvParams &p, int grid, size_t smem, cudaStream_t st) {
    static std::mutex mu;
    static size_t configured[16] = {0};  // per device
    {
        std::lock_guard<std::mutex> g(mu);
        int dev = ctx->device & 15;
        if (smem > 48 * 1024 && smem > configured[dev]) {
            JUNO_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<TYPE, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)ctx->smem_optin));
            configured[dev] = ctx->smem_optin;
        }
    }
    JUNO_CUDA_TRY(launch_pdl(gemv_kernel<TYPE, NB>, dim3(grid), dim3(kThreads), smem, st, p));
    ctx->kernel_launches++;
    return JUNO_OK;
}

template <int TYPE>
static int launch_type(juno_ctx *ctx, const GemvParams &p, int NB, int grid, size_t smem, cudaStream_t st) {
    switch (NB) {
    case 1: return launch_inst<TYPE, 1>(ctx, p, grid, smem, st);
    case 2: return launch_inst<TYPE, 2>(ctx, p, grid, smem, st);
    case 3: return launch_inst<TYPE, 3>(ctx, p, grid, smem, st);
    case 4: return launch_inst<TYPE, 4>(ctx, p, grid, smem, st);
    case 5: return launch_inst<TYPE, 5>(ctx, p, grid, smem, st);
    case 6: return launch_inst<TYPE, 6>(ctx, p, grid, smem, st);
    case 7: return launch_inst<TYPE, 7>(ctx, p, grid, smem, st);
    case 8: return launch_inst<TYPE, 8>(ctx, p, grid, smem, st);
    default: break;
    }
    set_error("gemv: unsupported batch chunk %d", NB);
    return JUNO_ERR_UNSUPPORTED;
}

// CTA-task geometry of a product; producers and consumers of per-task sums of squares must agree on it.
void gemv_task_geometry(const juno_ctx *ctx, int K, int batch_chunk, int total_rt, int *kin_out, int *n_ctasks_out) {
    const int nb = K / 256;
    const size_t smem = gemv_smem_bytes(K, batch_chunk);
    const int ctas_per_sm = (smem * 2 + 2048 <= ctx->smem_optin) ? 2 : 1;
    const int max_grid = ctx->sm_count * ctas_per_sm;
    // warps per row tile (K split inside the CTA): the smallest split that still yields several CTA tasks per
    // resident CTA (for balance), else the largest one (for parallelism); at least two tiles per warp per task
    int kin = 1;
    for (int d = 1; d <= kWarps; d *= 2) {
        if (nb % d || (d > 1 && nb / d < 2)) break;
        kin = d;
        const int groups = kWarps / d;
        if ((total_rt + groups - 1) / groups >= 4 * max_grid) break;
    }
    kin = env_int("JUNO_GEMV_KIN", kin);
    if (kin < 1 || kin > kWarps || (kin & (kin - 1)) || nb % kin) kin = 1;
    const int groups = kWarps / kin;
    *kin_out = kin;
    *n_ctasks_out = (total_rt + groups - 1) / groups;
}

int gemv_n_ctasks(const juno_ctx *ctx, int K, int batch, int total_rt) {
    if (ctx->step_rec) return total_rt;  // the step kernel writes one sum of squares per row tile
    int kin, n;
    gemv_task_geometry(ctx, K, gemv_batch_chunk(ctx, K, batch), total_rt, &kin, &n);
    return n;
}

static int gemv_check_args(const GemvArgs &a) {
    JUNO_REQUIRE(a.nseg >= 1 && a.nseg <= 3, "gemv: nseg %d", a.nseg);
    JUNO_REQUIRE(a.type == 0 || a.type == 12 || a.type == 14 || a.type == 8, "gemv: type %d has no tiled kernel", a.type);
    if (a.type == 0)
        for (int s = 0; s < a.nseg; s++)
            JUNO_REQUIRE(a.seg[s].type == 12 || a.seg[s].type == 14, "gemv: mixed launches take Q4_K and Q6_K segments only");
    JUNO_REQUIRE(a.K > 0 && a.K % 256 == 0, "gemv: K=%d must be a multiple of 256", a.K);
    JUNO_REQUIRE(a.batch >= 1 && a.ximg, "gemv: batch %d / missing staged activation", a.batch);
    if (a.epi == EPI_RESID_NORM)
        JUNO_REQUIRE(a.nseg == 1 && a.resid && a.x_out && a.normw_next && a.ss_out && a.img_next, "gemv: residual epilogue needs its buffers");
    return JUNO_OK;
}

size_t gemv_l2_prefetch_bytes() {
    static const size_t v = [] {
        const char *e = getenv("JUNO_L2_PREFETCH_MB");
        const long mb = e ? atol(e) : 0;  // measured: no gain at 8-16 MB, 2-6 % slower at 48-96 MB (the step is not latency bound on HBM)
        return (size_t)std::max(0L, std::min(mb, 96L)) << 20;
    }();
    return v;
}

int gemv_fill_params(juno_ctx *ctx, const GemvArgs &a, int b0, int bc, int chunk, int kin, int tpt, int groups, int n_ctasks,
                     GemvParams *out) {
    JUNO_TRY(gemv_check_args(a));
    GemvParams &p = *out;
    memset(&p, 0, sizeof(p));
    const size_t chunk_stride = stage_chunk_bytes(a.K, gemv_batch_chunk(ctx, a.K, a.batch));
    int rt = 0;
    for (int s = 0; s < a.nseg; s++) {
        p.w[s] = a.seg[s].w;
        p.out[s] = a.seg[s].out ? a.seg[s].out + (size_t)b0 * a.ld_out : nullptr;
        p.rows[s] = a.seg[s].rows;
        p.seg_type[s] = a.seg[s].type ? a.seg[s].type : a.type;
        p.rt_begin[s] = rt;
        rt += a.seg[s].row_tiles;
    }
    for (int s = a.nseg; s < 4; s++) p.rt_begin[s] = rt;
    p.nseg = a.nseg;
    p.total_rt = rt;
    p.K = a.K;
    p.nb = a.K / 256;
    p.kin = kin;
    p.tpt = tpt;
    p.groups = groups;
    p.n_ctasks = n_ctasks;
    p.ld_out = a.ld_out;
    p.epi = a.epi;
    p.ximg = a.ximg + (size_t)chunk * chunk_stride;
    p.img_bytes = (unsigned)stage_chunk_bytes(a.K, bc);
    p.ss_parts = a.ss_parts ? a.ss_parts + (size_t)b0 * a.ss_ld : nullptr;
    p.n_parts = a.n_parts;
    p.ss_ld = a.ss_ld;
    p.scale_n = a.scale_n;
    p.eps = a.eps;
    p.resid = a.resid ? a.resid + (size_t)b0 * a.ldx : nullptr;
    p.x_out = a.x_out ? a.x_out + (size_t)b0 * a.ldx : nullptr;
    p.ldx = a.ldx;
    p.normw_next = a.normw_next;
    p.ss_out = a.ss_out ? a.ss_out + (size_t)b0 * a.ss_out_ld : nullptr;
    p.ss_out_ld = a.ss_out_ld;
    if (b0 == 0) {
        const size_t budget = gemv_l2_prefetch_bytes();
        int max_tb = 0;
        for (int s = 0; s < a.nseg; s++) max_tb = std::max(max_tb, tile_bytes(p.seg_type[s]));
        static const int mode = [] {
            const char *e = getenv("JUNO_L2_PREFETCH_MODE");  // 1 own weights, 2 next at entry, 4 next at exit
            return e ? atoi(e) : 7;
        }();
        if (budget && max_tb && (mode & 1)) p.pf_rt = (int)std::min<size_t>((size_t)p.total_rt, budget / ((size_t)p.nb * max_tb));
        for (int r = 0, k = 0; r < 3 && budget; r++) {
            if (!a.pf_next[r] || !a.pf_next_bytes[r] || !(mode & (a.pf_next_late ? 4 : 2))) continue;
            p.pfx[k] = a.pf_next[r];
            p.pfx_bytes[k] = (unsigned)std::min<size_t>(a.pf_next_bytes[r] & ~(size_t)15, budget);
            k++;
        }
        p.pf_late = a.pf_next_late;
    }
    if (a.img_next) {
        // the next product chunks the batch by ITS K; rows b0.. of this launch map to rows b0.. of that image
        p.img_next = stage_image_desc(ctx, a.img_next, a.img_next_K, a.batch);
        p.img_next.b0 = b0;
    }
    return JUNO_OK;
}

int launch_gemv(juno_ctx *ctx, const GemvArgs &a, cudaStream_t st) {
    JUNO_TRY(gemv_check_args(a));
    if (ctx->step_rec) return step_record_gemv(ctx, a);
    int total_rt = 0;
    for (int s = 0; s < a.nseg; s++) total_rt += a.seg[s].row_tiles;
    JUNO_REQUIRE(gemv_smem_bytes(a.K, 1) <= ctx->smem_optin, "gemv: K=%d does not fit shared memory", a.K);

    double algo_bytes = (double)a.batch * a.K * 4;
    {
        for (int s = 0; s < a.nseg; s++) {
            const int t = a.seg[s].type ? a.seg[s].type : a.type;
            const double bpw = t == 12 ? 144.0 / 256 : t == 14 ? 210.0 / 256 : 34.0 / 32;
            algo_bytes += (double)a.seg[s].rows * a.K * bpw + (double)a.batch * a.seg[s].rows * 4;
        }
    }
    ProfScope prof(ctx, st, (a.type == 12 || a.type == 0) ? PROF_GEMV_Q4K : a.type == 14 ? PROF_GEMV_Q6K : PROF_GEMV_Q80, algo_bytes);

    const int bc_full = gemv_batch_chunk(ctx, a.K, a.batch);
    int kin = 1, n_ctasks = 1;
    gemv_task_geometry(ctx, a.K, bc_full, total_rt, &kin, &n_ctasks);
    for (int b0 = 0, chunk = 0; b0 < a.batch; b0 += bc_full, chunk++) {
        const int bc = std::min(bc_full, a.batch - b0);
        const size_t smem = gemv_smem_bytes(a.K, bc);
        const int ctas_per_sm = (gemv_smem_bytes(a.K, bc_full) * 2 + 2048 <= ctx->smem_optin) ? 2 : 1;
        const int max_grid = ctx->sm_count * ctas_per_sm;
        GemvParams p;
        JUNO_TRY(gemv_fill_params(ctx, a, b0, bc, chunk, kin, (a.K / 256) / kin, kWarps / kin, n_ctasks, &p));
        p.counters = ctx->gemv_scratch.counters + 2 * (ctx->gemv_scratch.next_slot++ % kGemvCounterSlots);
        int grid = std::min(max_grid, p.n_ctasks);
        grid = std::max(1, std::min(env_int("JUNO_GEMV_GRID", grid), p.n_ctasks));
        int rc;
        if (a.type == 0)
            rc = launch_type<0>(ctx, p, bc, grid, smem, st);
        else if (a.type == 12)
            rc = launch_type<12>(ctx, p, bc, grid, smem, st);
        else if (a.type == 14)
            rc = launch_type<14>(ctx, p, bc, grid, smem, st);
        else
            rc = launch_type<8>(ctx, p, bc, grid, smem, st);
        JUNO_TRY(rc);
    }
    return JUNO_OK;
}

// ───────────────────────────── repack (raw GGUF blocks -> tiles) ───────────────────────────
// raw: device copy of rows [0,nrows) of the source tensor, row stride raw_row_bytes; the tile matrix covers
// super-blocks [sb0, sb0+nsb) of each row.  One thread per 32-bit output word.
__host__ __device__ inline uint32_t q4k_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
                                                 int w) {
    // w: 32-bit word index inside the 2368-byte tile (0..591)
    if (w < 16) {  // d | dmin
        int row = R * 16 + w;
        if (row >= nrows) return 0;
        const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 144;
        return (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
    } else if (w < 80) {  // scales and mins of sub-blocks 2c, 2c+1 as bytes
        int v = w - 16, row16 = v >> 2, c = v & 3;
        int row = R * 16 + row16;
        if (row >= nrows) return 0;
        const uint8_t *sc = raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 144 + 4;
        return (uint32_t)q4k_scale6(sc, 2 * c) | ((uint32_t)q4k_scale6(sc, 2 * c + 1) << 8) |
               ((uint32_t)q4k_min6(sc, 2 * c) << 16) | ((uint32_t)q4k_min6(sc, 2 * c + 1) << 24);
    } else {
        int row16, off;
        q4k_qs_word_src(w - 80, row16, off);
        int row = R * 16 + row16;
        if (row >= nrows) return 0;
        const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 144 + off;
        return (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
    }
}

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

__host__ __device__ inline uint32_t q6k_tile_word(const uint8_t *blk_row /* raw block of (row, sb) or null */, int w,
                                                  int lane_c, bool ql_section, int mp, int k4) {
    // Builds one ql word W[j] or qh word H[i] for lane column group c from a raw block.
    (void)w;
    uint32_t v = 0;
    if (!blk_row) return 0;
    if (ql_section) {
        int j = 2 * mp + (k4 & 1);
        for (int odd = 0; odd < 2; odd++)
            for (int t = 0; t < 4; t++) {
                int e = 16 * (2 * j + odd) + 4 * lane_c + t;
                int nu = 2 * feed_pos(t) + odd;
                v |= (uint32_t)(q6k_raw_u6(blk_row, e) & 15) << (4 * nu);
            }
    } else {
        int i = 2 * mp + (k4 & 1);
        for (int isB = 0; isB < 2; isB++) {
            int j = 2 * i + isB;
            for (int odd = 0; odd < 2; odd++)
                for (int t = 0; t < 4; t++) {
                    int e = 16 * (2 * j + odd) + 4 * lane_c + t;
                    int nu = 2 * feed_pos(t) + odd;
                    v |= (uint32_t)(q6k_raw_u6(blk_row, e) >> 4) << q6k_field_bit(isB, nu);
                }
        }
    }
    return v;
}

__host__ __device__ inline uint32_t q6k_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
                                                 int w) {
    // w: 32-bit word index inside the 3360-byte tile (0..839)
    if (w < 768) {  // ql (512 words) then qh (256 words)
        bool ql = w < 512;
        int v = ql ? w : w - 512;
        int mp = v >> 7, lane = (v >> 2) & 31, k4 = v & 3;
        int row = R * 16 + (lane >> 2) + 8 * (k4 >> 1);
        const uint8_t *blk = (row < nrows) ? raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 210 : nullptr;
        return q6k_tile_word(blk, w, lane & 3, ql, mp, k4);
    } else if (w < 832) {  // sc: 16 rows x 16 bytes
        int v = w - 768, row16 = v >> 2, q = v & 3;
        int row = R * 16 + row16;
        if (row >= nrows) return 0;
        const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 210 + 192 + q * 4;
        return (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
    } else {  // d: 16 rows x f16, two per word
        int v = w - 832;
        uint32_t outv = 0;
        for (int h = 0; h < 2; h++) {
            int row = R * 16 + 2 * v + h;
            if (row < nrows) {
                const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)sb_abs * 210 + 208;
                outv |= ((uint32_t)s[0] | ((uint32_t)s[1] << 8)) << (16 * h);
            }
        }
        return outv;
    }
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

__host__ __device__ inline uint32_t q80_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
                                                 int w) {
    if (w < 1024) {
        int j = w >> 7, lane = (w >> 2) & 31, k4 = w & 3;
        int row = R * 16 + (lane >> 2) + 8 * (k4 >> 1);
        if (row >= nrows) return 0;
        const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)(sb_abs * 8 + j) * 34 + 2 + 16 * (k4 & 1) + 4 * (lane & 3);
        return (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
    } else {  // d[row16][8] f16: 4 words per row
        int v = w - 1024, row16 = v >> 2, q = v & 3;
        int row = R * 16 + row16;
        if (row >= nrows) return 0;
        uint32_t outv = 0;
        for (int h = 0; h < 2; h++) {
            const uint8_t *s = raw + (size_t)row * raw_row_bytes + (size_t)(sb_abs * 8 + 2 * q + h) * 34;
            outv |= ((uint32_t)s[0] | ((uint32_t)s[1] << 8)) << (16 * h);
        }
        return outv;
    }
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

// Host mirror of the repack, for layout tests that run without a GPU.
extern "C" int juno_dbg_repack_host(int type, const uint8_t *raw, int64_t rows, int64_t cols, uint8_t *out) {
    if (cols % 256 || rows < 1) return JUNO_ERR_INVALID_ARG;
    int nsb = (int)(cols / 256), RT = (int)((rows + 15) / 16);
    size_t rrb = (size_t)nsb * (type == 12 ? 144 : type == 14 ? 210 : 8 * 34);
    int wpt = tile_bytes(type) / 4;
    if (!wpt) return JUNO_ERR_UNSUPPORTED;
    uint32_t *o = reinterpret_cast<uint32_t *>(out);
    for (int R = 0; R < RT; R++)
        for (int b = 0; b < nsb; b++)
            for (int w = 0; w < wpt; w++) {
                uint32_t v = 0;
                if (type == 12) {
                    v = q4k_out_word(raw, rrb, (int)rows, b, R, w);
                } else if (type == 14) {
                    v = q6k_out_word(raw, rrb, (int)rows, b, R, w);
                } else {
                    v = q80_out_word(raw, rrb, (int)rows, b, R, w);
                }
                o[((size_t)R * nsb + b) * wpt + w] = v;
            }
    return JUNO_OK;
}
extern "C" int64_t juno_dbg_tiled_bytes(int type, int64_t rows, int64_t cols) {
    if (cols % 256 || !tile_bytes(type)) return -1;
    return ((rows + 15) / 16) * (cols / 256) * (int64_t)tile_bytes(type);
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

extern "C" int juno_dbg_dequant_tiled_host(int type, const uint8_t *tiles, int64_t rows, int64_t cols, float *out) {
    if (cols % 256 || !tile_bytes(type)) return JUNO_ERR_INVALID_ARG;
    int64_t nb = cols / 256;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) {
            const uint8_t *tile = tiles + ((r >> 4) * nb + (c >> 8)) * (int64_t)tile_bytes(type);
            out[r * cols + c] = tile_elem_value(type, tile, (int)(r & 15), (int)(c & 255));
        }
    return JUNO_OK;
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
