// Batched dequant-GEMM for decode batches above eight sequences (and for prompt chunks): Y[b][r] = sum_c w(r,c) x[b][c]
// in ONE pass over the quantised weights.
//
// Where the GEMV kernel (qgemv.cu) spends three int8 limb columns per sequence to keep the products exact, this kernel
// treats the batch as a real dense contraction: a warp owns one 16-row tile of the weights for the whole of K, turns
// each 16x256 quantised tile in registers into FP16 A fragments (w = (d*sc)*q - dmin*m, scale and min in FP16, the
// integer q exact), and multiplies it with mma.sync.m16n8k16 (f16 in, f32 accumulate) against the activations, one
// FP16 column per sequence, staged in shared memory slab by slab (256 columns of K at a time, cp.async, three
// stages, shared by the eight warps of the CTA).  Activations are pre-scaled per row by a power of two so that they
// sit well inside the FP16 range; the factor is multiplied back in the epilogue.  Rounding weights and activations
// to FP16 costs about 3e-4 relative on the products (the tolerance of this path is 1e-3).
#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>

#include "gemv.cuh"
#include "layout.cuh"
#include "tile_math.cuh"

namespace juno {

constexpr int kGemmWarps = 8, kGemmThreads = kGemmWarps * 32, kGemmStages = 3;

struct GemmParams {
    const uint8_t *w;     // tiled weights of one block format
    float *out;           // [batch][ld_out]
    int rows, total_rt;
    int K, nb;            // nb = K / 256 slabs
    int batch, NC;        // NC = batch rounded up to a multiple of 8
    int ld_out, epi;
    const uint8_t *ximg;  // FP16 staged activation [K/16][NC][4][4]
    const float *xscale;  // [batch]: factor to multiply the products with
    const float *resid;   // EPI_RESID_NORM here means just out = resid + y (no image, no sums of squares)
    int ldx;
    int n_tasks;          // groups of kGemmWarps >> kin_log2 row tiles
    int kin_log2;         // 1 << kin_log2 warps share a row tile, each taking its share of every tile's four 64-column quarters
};

__device__ __forceinline__ void mma16816_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t v, uint32_t c) {
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&v), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t v, uint32_t c) {
    __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&v), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t h2_dup(float v) {
    __half2 r = __float2half2_rn(v);
    return *reinterpret_cast<uint32_t *>(&r);
}
constexpr uint32_t kH1024 = 0x64006400u;  // (1024, 1024): 0x6400 | n is the FP16 number 1024 + n for n < 1024
constexpr uint32_t kH1056 = 0x64206420u;  // (1056, 1056)
constexpr uint32_t kH1152 = 0x64806480u;  // (1152, 1152)

// B fragment of n-tile nt for 16-column group s16 of the slab: (b0, b1) of column nt*8 + lane/4.
struct SlabView {
    const unsigned short *lane_base;  // slab + ((lane/4) * 4 + lane%4) * 4
    int NC;
    __device__ __forceinline__ uint2 b(int nt, int s16) const {
        return *reinterpret_cast<const uint2 *>(lane_base + ((size_t)s16 * NC + nt * 8) * 16);
    }
};

// ── Q4_K ────────────────────────────────────────────────────────────────────────────────────
// (scale, -min) of one row for the lane's two sub-blocks 2c, 2c+1, each as an FP16 pair packed in one word.
__device__ __forceinline__ void q4_header_f16(uint32_t dm, uint32_t sm, uint32_t &p0, uint32_t &p1) {
    const float d = f16bits_to_f32(dm), dmin = f16bits_to_f32(dm >> 16);
    const float s0 = d * (float)(sm & 0xFFu), s1 = d * (float)((sm >> 8) & 0xFFu);
    const float m0 = dmin * (float)((sm >> 16) & 0xFFu), m1 = dmin * (float)(sm >> 24);
    __half2 a = __floats2half2_rn(s0, -m0), b = __floats2half2_rn(s1, -m1);
    p0 = *reinterpret_cast<uint32_t *>(&a);
    p1 = *reinterpret_cast<uint32_t *>(&b);
}

template <int NT>
__device__ __forceinline__ void gemm_tile(const TileRegs<12> &R, int q0, int q1, const SlabView &xv, int lane, float (&acc)[NT][4]) {
    uint32_t pr0, pr1, pq0, pq1;  // (scale, -min) pairs: row r8 / r8+8, sub-blocks 2c / 2c+1
    q4_header_f16(R.dm0, R.sm0, pr0, pr1);
    q4_header_f16(R.dm1, R.sm1, pq0, pq1);
    uint32_t M4 = 0x000F000Fu, K = kH1024;
    asm volatile("" : "+r"(M4), "+r"(K));
#pragma unroll
    for (int g = 0; g < 4; g++) {
        if (g < q0 || g >= q1) continue;  // warp-uniform: the 64-column quarters of the tile this warp works on
        const int src = (lane & ~3) | g;  // quad lane g owns sub-blocks 2g and 2g+1
        const uint32_t r0 = __shfl_sync(0xffffffffu, pr0, src), r1 = __shfl_sync(0xffffffffu, pr1, src);
        const uint32_t q0 = __shfl_sync(0xffffffffu, pq0, src), q1 = __shfl_sync(0xffffffffu, pq1, src);
        // (s, s) and (-m, -m) for rows r / q and for the low-nibble (2g) / high-nibble (2g+1) sub-block
        const uint32_t sr0 = __byte_perm(r0, 0, 0x1010), mr0 = __byte_perm(r0, 0, 0x3232);
        const uint32_t sr1 = __byte_perm(r1, 0, 0x1010), mr1 = __byte_perm(r1, 0, 0x3232);
        const uint32_t sq0 = __byte_perm(q0, 0, 0x1010), mq0 = __byte_perm(q0, 0, 0x3232);
        const uint32_t sq1 = __byte_perm(q1, 0, 0x1010), mq1 = __byte_perm(q1, 0, 0x3232);
        uint32_t la[4], lb[4], ha[4], hb[4];  // index: word x, y, z, w of the group
        q4_unpack(R.q[g].x, M4, K, la[0], lb[0], ha[0], hb[0]);
        q4_unpack(R.q[g].y, M4, K, la[1], lb[1], ha[1], hb[1]);
        q4_unpack(R.q[g].z, M4, K, la[2], lb[2], ha[2], hb[2]);
        q4_unpack(R.q[g].w, M4, K, la[3], lb[3], ha[3], hb[3]);
        // words x, y belong to row r8, words z, w to row r8+8
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t s_lo = (i < 2) ? sr0 : sq0, m_lo = (i < 2) ? mr0 : mq0;
            const uint32_t s_hi = (i < 2) ? sr1 : sq1, m_hi = (i < 2) ? mr1 : mq1;
            la[i] = h2_fma(h2_sub(la[i], K), s_lo, m_lo);
            lb[i] = h2_fma(h2_sub(lb[i], K), s_lo, m_lo);
            ha[i] = h2_fma(h2_sub(ha[i], K), s_hi, m_hi);
            hb[i] = h2_fma(h2_sub(hb[i], K), s_hi, m_hi);
        }
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            uint2 b = xv.b(nt, 4 * g + 0);
            mma16816_f16(acc[nt], la[0], la[2], lb[0], lb[2], b.x, b.y);
            b = xv.b(nt, 4 * g + 1);
            mma16816_f16(acc[nt], la[1], la[3], lb[1], lb[3], b.x, b.y);
            b = xv.b(nt, 4 * g + 2);
            mma16816_f16(acc[nt], ha[0], ha[2], hb[0], hb[2], b.x, b.y);
            b = xv.b(nt, 4 * g + 3);
            mma16816_f16(acc[nt], ha[1], ha[3], hb[1], hb[3], b.x, b.y);
        }
    }
}

// ── Q6_K ────────────────────────────────────────────────────────────────────────────────────
template <int NT>
__device__ __forceinline__ void gemm_tile(const TileRegs<14> &R, int q0, int q1, const SlabView &xv, int lane, float (&acc)[NT][4]) {
    const float d_r = f16bits_to_f32(R.d01), d_q = f16bits_to_f32(R.d01 >> 16);
    uint32_t s_r[4], s_q[4];  // FP16 pairs (s, s) of sub-blocks 4c..4c+3 for rows r8 and r8+8
#pragma unroll
    for (int k = 0; k < 4; k++) {
        s_r[k] = h2_dup(d_r * i8_to_f32(R.sc0, k));
        s_q[k] = h2_dup(d_q * i8_to_f32(R.sc1, k));
    }
    uint32_t NIB = 0x0F0F0F0Fu, HI = 0x30303030u;
    asm volatile("" : "+r"(NIB), "+r"(HI));
#pragma unroll
    for (int m = 0; m < 4; m++) {
        if (m < q0 || m >= q1) continue;
        const uint32_t WA_r = R.ql[m].x, WB_r = R.ql[m].y, WA_q = R.ql[m].z, WB_q = R.ql[m].w;
        const uint4 hq = R.qh[m >> 1];
        const uint32_t H_r = (m & 1) ? hq.y : hq.x, H_q = (m & 1) ? hq.w : hq.z;
        uint32_t V_r[4], V_q[4];  // four 6-bit values per word, for sub-blocks 4m+0..3
        V_r[0] = and_or(WA_r, NIB, H_r & HI);
        V_r[1] = and_or(WA_r >> 4, NIB, (H_r >> 2) & HI);
        V_r[2] = and_or(WB_r, NIB, (H_r << 2) & HI);
        V_r[3] = and_or(WB_r >> 4, NIB, (H_r << 4) & HI);
        V_q[0] = and_or(WA_q, NIB, H_q & HI);
        V_q[1] = and_or(WA_q >> 4, NIB, (H_q >> 2) & HI);
        V_q[2] = and_or(WB_q, NIB, (H_q << 2) & HI);
        V_q[3] = and_or(WB_q >> 4, NIB, (H_q << 4) & HI);
        const int src = (lane & ~3) | m;  // quad lane m owns the scales of sub-blocks 4m..4m+3
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t sr = __shfl_sync(0xffffffffu, s_r[k], src), sq = __shfl_sync(0xffffffffu, s_q[k], src);
            const uint32_t a0 = h2_mul(h2_sub(__byte_perm(V_r[k], 0x64646464u, 0x4140), kH1056), sr);
            const uint32_t a2 = h2_mul(h2_sub(__byte_perm(V_r[k], 0x64646464u, 0x4342), kH1056), sr);
            const uint32_t a1 = h2_mul(h2_sub(__byte_perm(V_q[k], 0x64646464u, 0x4140), kH1056), sq);
            const uint32_t a3 = h2_mul(h2_sub(__byte_perm(V_q[k], 0x64646464u, 0x4342), kH1056), sq);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 b = xv.b(nt, 4 * m + k);
                mma16816_f16(acc[nt], a0, a1, a2, a3, b.x, b.y);
            }
        }
    }
}

// ── Q8_0 ────────────────────────────────────────────────────────────────────────────────────
template <int NT>
__device__ __forceinline__ void gemm_tile(const TileRegs<8> &R, int q0, int q1, const SlabView &xv, int /*lane*/, float (&acc)[NT][4]) {
    const uint32_t dr[4] = {R.d0.x, R.d0.y, R.d0.z, R.d0.w}, dq[4] = {R.d1.x, R.d1.y, R.d1.z, R.d1.w};
    uint32_t SGN = 0x80808080u;
    asm volatile("" : "+r"(SGN));
#pragma unroll
    for (int j = 0; j < 8; j++) {
        if ((j >> 1) < q0 || (j >> 1) >= q1) continue;
        const uint32_t d_r = __byte_perm(dr[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);  // (d, d) as stored FP16 bits
        const uint32_t d_q = __byte_perm(dq[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);
        const uint32_t w4[4] = {R.q[j].x ^ SGN, R.q[j].y ^ SGN, R.q[j].z ^ SGN, R.q[j].w ^ SGN};  // int8 + 128
        uint32_t a[4][2];  // [word][bytes (0,2) | bytes (1,3)]
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t d = (i == 0 || i == 1) ? d_r : d_q;
            a[i][0] = h2_mul(h2_sub(__byte_perm(w4[i], 0x64646464u, 0x4240), kH1152), d);
            a[i][1] = h2_mul(h2_sub(__byte_perm(w4[i], 0x64646464u, 0x4341), kH1152), d);
        }
        // words x, y: row r8 (16-column groups 2j, 2j+1); words z, w: row r8+8
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            uint2 b = xv.b(nt, 2 * j);
            mma16816_f16(acc[nt], a[0][0], a[2][0], a[0][1], a[2][1], b.x, b.y);
            b = xv.b(nt, 2 * j + 1);
            mma16816_f16(acc[nt], a[1][0], a[3][0], a[1][1], a[3][1], b.x, b.y);
        }
    }
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One CTA = 8 >> kin_log2 consecutive row tiles, all of K, slab by slab; the 1 << kin_log2 warps of a row tile split
// every tile by 64-column quarters and their partial sums are added (in warp order) through shared memory.
template <int TYPE, int NT>
__global__ void __launch_bounds__(kGemmThreads, (NT > 4 ? 1 : 2)) gemm_kernel(const GemmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NC = p.NC;
    const size_t slab_bytes = (size_t)16 * NC * 32;  // 16 groups of 16 columns, NC sequences, 2 bytes
    const int n16 = (int)(slab_bytes >> 4);
    SlabView xv;
    xv.NC = NC;
    for (int task = blockIdx.x; task < p.n_tasks; task += gridDim.x) {
        const int kl = p.kin_log2, kin = 1 << kl, kq = warp & (kin - 1);
        const int R = task * (kGemmWarps >> kl) + (warp >> kl);
        const int q0 = kq * (4 >> kl), q1 = q0 + (4 >> kl);
        const bool have = R < p.total_rt;
        const uint8_t *wrow = p.w + (size_t)(have ? R : 0) * p.nb * tile_bytes(TYPE);
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        TileRegs<TYPE> bufA, bufB;
        if (have) load_tile<TYPE>(bufA, wrow, lane);
        // prologue: slabs 0 .. stages-2
#pragma unroll
        for (int s = 0; s < kGemmStages - 1; s++) {
            if (s < p.nb) {
                const uint4 *src = reinterpret_cast<const uint4 *>(p.ximg + (size_t)s * slab_bytes);
                uint4 *dst = reinterpret_cast<uint4 *>(smem + (size_t)s * slab_bytes);
                for (int i = tid; i < n16; i += kGemmThreads) cp_async16(dst + i, src + i);
            }
            cp_async_commit();
        }
        for (int sb = 0; sb < p.nb; sb++) {
            cp_async_wait<kGemmStages - 2>();  // slab sb has landed (for this thread's copies)
            __syncthreads();                    // ... for everybody's; and everybody is done with slab sb-1
            {
                const int s = sb + kGemmStages - 1;
                if (s < p.nb) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(p.ximg + (size_t)s * slab_bytes);
                    uint4 *dst = reinterpret_cast<uint4 *>(smem + (size_t)(s % kGemmStages) * slab_bytes);
                    for (int i = tid; i < n16; i += kGemmThreads) cp_async16(dst + i, src + i);
                }
                cp_async_commit();
            }
            xv.lane_base = reinterpret_cast<const unsigned short *>(smem + (size_t)(sb % kGemmStages) * slab_bytes) +
                           ((lane >> 2) * 4 + (lane & 3)) * 4;
            if (have) {
                if (sb & 1) {
                    if (sb + 1 < p.nb) load_tile<TYPE>(bufA, wrow + (size_t)(sb + 1) * tile_bytes(TYPE), lane);
                    gemm_tile<NT>(bufB, q0, q1, xv, lane, acc);
                } else {
                    if (sb + 1 < p.nb) load_tile<TYPE>(bufB, wrow + (size_t)(sb + 1) * tile_bytes(TYPE), lane);
                    gemm_tile<NT>(bufA, q0, q1, xv, lane, acc);
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();  // the stages are reused (by the reduction below and by the next task)
        if (kin > 1) {
            float *red = reinterpret_cast<float *>(smem);  // [warp][NT*4][32]
            if (kq != 0) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) red[((size_t)warp * NT * 4 + nt * 4 + i) * 32 + lane] = acc[nt][i];
            }
            __syncthreads();
            if (kq == 0) {
                for (int k2 = 1; k2 < kin; k2++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int i = 0; i < 4; i++) acc[nt][i] += red[((size_t)(warp + k2) * NT * 4 + nt * 4 + i) * 32 + lane];
            }
            __syncthreads();  // before the next task's copies land in the same memory
        }
        if (!have || kq != 0) continue;
        // epilogue: this thread holds rows r8, r8+8 of the tile for columns nt*8 + 2c, +1
        const int r8 = lane >> 2, c = lane & 3;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int b = nt * 8 + 2 * c + j;
                if (b >= p.batch) continue;
                const float sc = p.xscale ? p.xscale[b] : 1.f;
                const float lo = acc[nt][j] * sc, hi = acc[nt][2 + j] * sc;
                if (p.epi == EPI_SILU_PAIR) {  // rows 0-7 of a tile are gate rows, rows 8-15 the matching up rows
                    const int orow = R * 8 + r8;
                    if (orow < p.rows) p.out[(size_t)b * p.ld_out + orow] = __fmul_rn(silu_ref(lo), hi);
                } else {
                    const int row0 = R * 16 + r8, row1 = row0 + 8;
                    if (p.epi == EPI_RESID_NORM) {
                        if (row0 < p.rows) p.out[(size_t)b * p.ld_out + row0] = __fadd_rn(p.resid[(size_t)b * p.ldx + row0], lo);
                        if (row1 < p.rows) p.out[(size_t)b * p.ld_out + row1] = __fadd_rn(p.resid[(size_t)b * p.ldx + row1], hi);
                    } else {
                        if (row0 < p.rows) p.out[(size_t)b * p.ld_out + row0] = lo;
                        if (row1 < p.rows) p.out[(size_t)b * p.ld_out + row1] = hi;
                    }
                }
            }
        }
    }
}

// ───────────────────────────── FP16 staging ───────────────────────────────────────────────
// One CTA per image column: columns below `batch` hold one sequence (optionally residual add + RMSNorm), scaled by
// a power of two so that its largest magnitude lands in [256, 512); the remaining columns are zero.
struct StageF16Params {
    int mode;
    const float *x;
    int ldx;
    const float *x_add, *normw;
    float *x_out;
    float eps;
    int K, batch, NC;
    uint8_t *img;
    float *xscale;
    uint8_t *img_tc;  // optional second copy, chunk-major [K/8][N][8] for the tcgen05 kernel (gemm_tc.cu)
    int N_tc;
};

__global__ void __launch_bounds__(256) stage_f16_kernel(const StageF16Params p) {
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned short *xb = reinterpret_cast<unsigned short *>(p.img);
    const int K = p.K, NC = p.NC;
    __shared__ float red[8], redm[8];
    unsigned short *xt = reinterpret_cast<unsigned short *>(p.img_tc);
    auto tc_dst = [&](int i4) {  // where columns i4..i4+3 go in the chunk-major image (see gemm_tc.cu)
        const int s16 = i4 >> 4, c = (i4 >> 2) & 3, slab = s16 >> 4, t = s16 & 15;
        const int chunk = slab * 32 + ((t >> 2) * 2 + ((t >> 1) & 1)) * 4 + c;
        return ((size_t)chunk * p.N_tc + b) * 8 + (size_t)(t & 1) * 4;
    };
    if (b >= p.batch) {
        for (int i4 = tid * 4; i4 < K; i4 += 256 * 4) {
            const int s16 = i4 >> 4, c = (i4 >> 2) & 3;
            if (b < NC) *reinterpret_cast<uint2 *>(xb + ((size_t)(s16 * NC + b) * 4 + c) * 4) = make_uint2(0u, 0u);
            if (xt && b < p.N_tc) *reinterpret_cast<uint2 *>(xt + tc_dst(i4)) = make_uint2(0u, 0u);
        }
        return;
    }
    const float *xrow = p.x + (size_t)b * p.ldx;
    const float *arow = p.x_add ? p.x_add + (size_t)b * p.ldx : nullptr;
    float scale = 1.f;
    if (p.mode == STAGE_RMSNORM) {
        float part = 0.f;
        for (int i = tid; i < K; i += 256) {
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
        for (int w8 = 0; w8 < 8; w8++) ss += red[w8];
        scale = __fdiv_rn(1.f, (float)sqrt((double)__fadd_rn(__fdiv_rn(ss, (float)K), p.eps)));
    }
    // pass 1: the values (kept in FP32) and their largest magnitude
    float vmax = 0.f;
    for (int i = tid; i < K; i += 256) {
        float r = xrow[i];
        if (p.mode == STAGE_RMSNORM) {
            if (arow) r = __fadd_rn(r, arow[i]);
            if (p.x_out) p.x_out[(size_t)b * p.ldx + i] = r;
            r = __fmul_rn(__fmul_rn(p.normw[i], r), scale);
        }
        vmax = fmaxf(vmax, fabsf(r));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    if (lane == 0) redm[warp] = vmax;
    __syncthreads();
    vmax = redm[0];
#pragma unroll
    for (int w8 = 1; w8 < 8; w8++) vmax = fmaxf(vmax, redm[w8]);
    // power of two that brings vmax into [256, 512) (1 for an all-zero or non-finite row)
    float down = 1.f, up = 1.f;
    if (vmax > 0.f && vmax < 3.0e38f) {
        int e;
        frexpf(vmax, &e);  // vmax = f * 2^e, f in [0.5, 1)
        down = ldexpf(1.f, 9 - e);
        up = ldexpf(1.f, e - 9);
    }
    if (tid == 0) p.xscale[b] = up;
    // pass 2: write the column
    for (int i4 = tid * 4; i4 < K; i4 += 256 * 4) {
        float v[4];
        const float4 xv = *reinterpret_cast<const float4 *>(xrow + i4);
        v[0] = xv.x; v[1] = xv.y; v[2] = xv.z; v[3] = xv.w;
        if (p.mode == STAGE_RMSNORM) {
            if (arow) {
                const float4 av = *reinterpret_cast<const float4 *>(arow + i4);
                v[0] = __fadd_rn(v[0], av.x); v[1] = __fadd_rn(v[1], av.y);
                v[2] = __fadd_rn(v[2], av.z); v[3] = __fadd_rn(v[3], av.w);
            }
            const float4 wv = *reinterpret_cast<const float4 *>(p.normw + i4);
            v[0] = __fmul_rn(__fmul_rn(wv.x, v[0]), scale);
            v[1] = __fmul_rn(__fmul_rn(wv.y, v[1]), scale);
            v[2] = __fmul_rn(__fmul_rn(wv.z, v[2]), scale);
            v[3] = __fmul_rn(__fmul_rn(wv.w, v[3]), scale);
        }
        unsigned short h[4];
#pragma unroll
        for (int t = 0; t < 4; t++) h[t] = __half_as_ushort(__float2half_rn(v[t] * down));
        const int s16 = i4 >> 4, c = (i4 >> 2) & 3;
        uint2 w;  // feed order: columns (4c, 4c+2 | 4c+1, 4c+3)
        w.x = (uint32_t)h[0] | ((uint32_t)h[2] << 16);
        w.y = (uint32_t)h[1] | ((uint32_t)h[3] << 16);
        *reinterpret_cast<uint2 *>(xb + ((size_t)(s16 * NC + b) * 4 + c) * 4) = w;
        if (xt) *reinterpret_cast<uint2 *>(xt + tc_dst(i4)) = w;  // same (x0, x2, x1, x3) packing
    }
}

// ───────────────────────────── host ───────────────────────────────────────────────────────
int gemm_min_batch() {
    static const int v = [] {
        const char *e = getenv("JUNO_GEMM_MIN_BATCH");
        const int n = (e && *e) ? atoi(e) : 9;
        return std::max(2, n);
    }();
    return v;
}

int gemm_padded_batch(int batch) { return (batch + 7) / 8 * 8; }
size_t gemm_image_bytes(int K, int batch) { return (size_t)K * gemm_padded_batch(batch) * 2; }

int launch_stage_f16(juno_ctx *ctx, const StageArgs &a, float *xscale, cudaStream_t st, uint8_t *img_tc) {
    JUNO_REQUIRE(a.K > 0 && a.K % 256 == 0 && a.batch >= 1 && a.batch <= kGemmMaxBatch && a.x && a.img && xscale,
                 "stage (fp16): bad arguments (K=%d, batch=%d)", a.K, a.batch);
    JUNO_REQUIRE(a.ldx % 4 == 0, "stage: row stride %d must be a multiple of 4", a.ldx);
    StageF16Params p;
    p.mode = a.mode;
    p.x = a.x;
    p.ldx = a.ldx;
    p.x_add = a.x_add;
    p.normw = a.normw;
    p.x_out = a.x_out;
    p.eps = a.eps;
    p.K = a.K;
    p.batch = a.batch;
    p.NC = gemm_padded_batch(a.batch);
    p.img = a.img;
    p.xscale = xscale;
    p.img_tc = img_tc;
    p.N_tc = gemm_tc_padded_batch(a.batch);
    ProfScope prof(ctx, st, PROF_OTHER, 0);
    stage_f16_kernel<<<img_tc ? std::max(p.NC, p.N_tc) : p.NC, 256, 0, st>>>(p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

template <int TYPE, int NT>
static int gemm_launch_inst(juno_ctx *ctx, const GemmParams &p, cudaStream_t st) {
    const size_t smem = (size_t)kGemmStages * 16 * p.NC * 32;
    static std::mutex mu;
    static bool configured[16] = {false};
    {
        std::lock_guard<std::mutex> g(mu);
        const int dev = ctx->device & 15;
        if (!configured[dev]) {
            JUNO_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<TYPE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 16 * 64 * 32));
            configured[dev] = true;
        }
    }
    const int grid = std::max(1, std::min(p.n_tasks, (NT > 4 ? 1 : 2) * ctx->sm_count));
    gemm_kernel<TYPE, NT><<<grid, kGemmThreads, smem, st>>>(p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

template <int TYPE>
static int gemm_launch_type(juno_ctx *ctx, const GemmParams &p, cudaStream_t st) {
    switch (p.NC / 8) {
    case 1: return gemm_launch_inst<TYPE, 1>(ctx, p, st);
    case 2: return gemm_launch_inst<TYPE, 2>(ctx, p, st);
    case 3: return gemm_launch_inst<TYPE, 3>(ctx, p, st);
    case 4: return gemm_launch_inst<TYPE, 4>(ctx, p, st);
    case 5: return gemm_launch_inst<TYPE, 5>(ctx, p, st);
    case 6: return gemm_launch_inst<TYPE, 6>(ctx, p, st);
    case 7: return gemm_launch_inst<TYPE, 7>(ctx, p, st);
    case 8: return gemm_launch_inst<TYPE, 8>(ctx, p, st);
    default: break;
    }
    set_error("gemm: batch %d is not supported (1..%d)", p.batch, kGemmMaxBatch);
    return JUNO_ERR_UNSUPPORTED;
}

// One launch per segment (each segment has a single block format).
int launch_gemm(juno_ctx *ctx, const GemvArgs &a, cudaStream_t st) {
    JUNO_REQUIRE(a.batch >= 1 && a.batch <= kGemmMaxBatch, "gemm: batch %d outside [1, %d]", a.batch, kGemmMaxBatch);
    JUNO_REQUIRE(a.K > 0 && a.K % 256 == 0 && a.ximg && a.xscale, "gemm: bad arguments (K=%d)", a.K);
    JUNO_REQUIRE(a.epi != EPI_RESID_NORM || (a.resid && a.nseg == 1), "gemm: residual epilogue needs resid and one segment");
    for (int s = 0; s < a.nseg; s++) {
        const int t = a.seg[s].type ? a.seg[s].type : a.type;
        JUNO_REQUIRE(t == 12 || t == 14 || t == 8, "gemm: type %d has no tiled kernel", t);
        if (a.ximg_tc && a.tc_err && a.epi != EPI_RESID_NORM && gemm_tc_enabled() && gemm_tc_shape_ok(ctx, a.seg[s].row_tiles, a.batch)) {
            JUNO_REQUIRE(a.seg[s].out, "gemm: segment %d has no output", s);
            JUNO_TRY(launch_gemm_tc(ctx, a.seg[s].w, t, a.seg[s].rows, a.seg[s].row_tiles, a.K, a.batch, a.ximg_tc, a.xscale, a.seg[s].out,
                                    a.ld_out, a.epi, a.tc_err, st));
            continue;
        }
        GemmParams p;
        memset(&p, 0, sizeof(p));
        p.w = a.seg[s].w;
        p.out = a.epi == EPI_RESID_NORM ? a.x_out : a.seg[s].out;
        JUNO_REQUIRE(p.out, "gemm: segment %d has no output", s);
        p.rows = a.seg[s].rows;
        p.total_rt = a.seg[s].row_tiles;
        p.K = a.K;
        p.nb = a.K / 256;
        p.batch = a.batch;
        p.NC = gemm_padded_batch(a.batch);
        p.ld_out = a.epi == EPI_RESID_NORM ? a.ldx : a.ld_out;
        p.epi = a.epi;
        p.ximg = a.ximg;
        p.xscale = a.xscale;
        p.resid = a.resid;
        p.ldx = a.ldx;
        // warps per row tile: one, unless that leaves more than half of the SMs without a CTA (each extra warp on a
        // tile re-reads it from L1/L2 and repeats the header arithmetic: measured slower as soon as the SMs are busy)
        p.kin_log2 = 0;
        while (p.kin_log2 < 2 && (p.total_rt + (kGemmWarps >> p.kin_log2) - 1) / (kGemmWarps >> p.kin_log2) < ctx->sm_count / 2) p.kin_log2++;
        if (const char *e = getenv("JUNO_GEMM_KIN")) p.kin_log2 = std::max(0, std::min(2, atoi(e)));
        p.n_tasks = (p.total_rt + (kGemmWarps >> p.kin_log2) - 1) / (kGemmWarps >> p.kin_log2);
        const double bpw = t == 12 ? 144.0 / 256 : t == 14 ? 210.0 / 256 : 34.0 / 32;
        const double algo = (double)a.seg[s].rows * a.K * bpw * (a.epi == EPI_SILU_PAIR ? 2 : 1) + (double)a.batch * a.K * 4 +
                            (double)a.batch * a.seg[s].rows * 4;
        ProfScope prof(ctx, st, t == 12 ? PROF_GEMV_Q4K : t == 14 ? PROF_GEMV_Q6K : PROF_GEMV_Q80, algo);
        int rc = t == 12 ? gemm_launch_type<12>(ctx, p, st) : t == 14 ? gemm_launch_type<14>(ctx, p, st) : gemm_launch_type<8>(ctx, p, st);
        JUNO_TRY(rc);
    }
    return JUNO_OK;
}

}  // namespace juno
