// Batched dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), for matrices with many row tiles.
//
// One CTA works on 128 weight rows (eight 16-row tiles) for all of K, slab by slab (256 columns):
//   * sixteen warps dequantise: two warps per row tile turn the quantised 16x256 tile into FP16 values in registers
//     (the arithmetic of gemm.cu) and store them into the slab's A operand in shared memory, laid out as the
//     canonical K-major "core matrices" of a shared-memory matrix descriptor without swizzle: 8 rows x 16 bytes
//     contiguous, row groups 128 bytes apart, the two 16-byte K chunks of an MMA 2048 bytes apart.  The order of the
//     256 columns inside a slab is free as long as both operands use it: here a 16-byte chunk is exactly the eight
//     values ONE lane holds for one row and one 32-column sub-block quarter, so every store is a 128-bit store;
//   * one thread copies the slab of the activation (one FP16 column per sequence, already stored chunk-major in the
//     same K order) with one cp.async.bulk;
//   * one thread issues sixteen tcgen05.mma (M = 128, N = padded batch, K = 16, FP16 in, FP32 accumulate in TMEM) per
//     slab and commits them to the mbarrier that releases the stage;
//   * after the last slab four warps read the accumulator with tcgen05.ld (lane = weight row, column = sequence),
//     scale by the activation's power-of-two factor and store / apply the SiLU pair epilogue.
// Two shared-memory stages; every mbarrier wait is bounded and reports through an error word; TMEM is freed on
// every path.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "gemv.cuh"
#include "layout.cuh"
#include "tile_math.cuh"

namespace juno {

constexpr int kTcDequantWarps = 16, kTcThreads = (kTcDequantWarps + 1) * 32, kTcStages = 2;
constexpr int kTcRows = 128;
// A chunk (8 K values of all 128 rows) is 2048 bytes; the 32-byte pad between chunks spreads the four chunks a warp
// writes at once (one per lane % 4) over all shared-memory banks.
constexpr unsigned kTcChunkStride = kTcRows * 16 + 32;
constexpr unsigned kTcASlabBytes = 32 * kTcChunkStride;  // 65 KB

struct TcParams {
    const uint8_t *w;
    float *out;
    int rows, total_rt;
    int K, nb;
    int batch, N;          // N = batch rounded up to a multiple of 16 (the MMA's N)
    int ld_out, epi;
    const uint8_t *ximg;   // chunk-major FP16 image [K/8][N][8]
    const float *xscale;
    int n_tasks;
    unsigned *err;         // device word: first wait that gave up (0 = none)
    int type;
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_test(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (about 0.2 s of SM clock); false = gave up or the CTA is already in the failed state.
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, unsigned parity, volatile unsigned *err_s, unsigned *err_g, unsigned code) {
    if (tc_mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (tc_mbar_test(bar, parity)) return true;
        if (*err_s) return false;
        if (clock64() - t0 > 400000000ll) break;
    }
    *err_s = code;
    atomicCAS(err_g, 0u, code | (blockIdx.x << 8));
    return false;
}
__device__ __forceinline__ void tc_bulk_g2s(uint32_t dst, const void *src, unsigned bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// K-major operand without swizzle: start address, byte distance between the two K chunks of an MMA (leading
// dimension) and between 8-row groups (stride dimension), descriptor version 1.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

__device__ __forceinline__ uint32_t tc_h2_sub(uint32_t v, uint32_t c) {
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&v), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t tc_h2_mul(uint32_t v, uint32_t c) {
    __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&v), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t tc_h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b), *reinterpret_cast<__half2 *>(&c));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t tc_h2_dup(float v) {
    __half2 r = __float2half2_rn(v);
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ void tc_sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }

// K order inside a slab (both operands): chunk index = (quarter * 2 + half) * 4 + c, where quarter = 64-column quarter
// of the slab, half = first / second 32 columns of the quarter, c = lane % 4; the chunk's eight values are columns
// 64*quarter + 32*half + {4c, 4c+2, 4c+1, 4c+3, 16+4c, 16+4c+2, 16+4c+1, 16+4c+3} -- what lane c holds for one row as
// the A fragments of two consecutive 16-column steps.  One 128-bit store per (row, chunk).
__device__ __forceinline__ void tc_sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// a_row = shared address of row r8 of this tile inside chunk 0; rows r8 and r8+8 of chunk (quarter, half, c).
__device__ __forceinline__ void tc_store_chunk(uint32_t a_row, int quarter, int half, int c, const uint32_t (&lo)[4],
                                               const uint32_t (&hi)[4]) {
    const uint32_t base = a_row + (uint32_t)((quarter * 2 + half) * 4 + c) * kTcChunkStride;
    tc_sts128(base, lo[0], lo[1], lo[2], lo[3]);
    tc_sts128(base + 8u * 16u, hi[0], hi[1], hi[2], hi[3]);
}

// Dequantise quarters [q0, q1) of a tile (64 columns each) into the A operand.  a_row = shared address of
// (row r8 of this tile, byte 4*c) inside chunk 0.
__device__ __forceinline__ void tc_dequant(const TileRegs<12> &R, int q0, int q1, uint32_t a_row, int lane) {
    const int c = lane & 3;
    const float d_r = f16bits_to_f32(R.dm0), m_r = f16bits_to_f32(R.dm0 >> 16);
    const float d_q = f16bits_to_f32(R.dm1), m_q = f16bits_to_f32(R.dm1 >> 16);
    // (scale, -min) of sub-blocks 2c, 2c+1 for rows r8 / r8+8, packed as FP16 pairs
    __half2 t;
    t = __floats2half2_rn(d_r * (float)(R.sm0 & 0xFFu), -(m_r * (float)((R.sm0 >> 16) & 0xFFu)));
    const uint32_t pr0 = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2half2_rn(d_r * (float)((R.sm0 >> 8) & 0xFFu), -(m_r * (float)(R.sm0 >> 24)));
    const uint32_t pr1 = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2half2_rn(d_q * (float)(R.sm1 & 0xFFu), -(m_q * (float)((R.sm1 >> 16) & 0xFFu)));
    const uint32_t pq0 = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2half2_rn(d_q * (float)((R.sm1 >> 8) & 0xFFu), -(m_q * (float)(R.sm1 >> 24)));
    const uint32_t pq1 = *reinterpret_cast<uint32_t *>(&t);
    uint32_t M4 = 0x000F000Fu, K = 0x64006400u;
    asm volatile("" : "+r"(M4), "+r"(K));
#pragma unroll
    for (int g = 0; g < 4; g++) {
        if (g < q0 || g >= q1) continue;
        const int src = (lane & ~3) | g;
        const uint32_t r0 = __shfl_sync(0xffffffffu, pr0, src), r1 = __shfl_sync(0xffffffffu, pr1, src);
        const uint32_t qq0 = __shfl_sync(0xffffffffu, pq0, src), qq1 = __shfl_sync(0xffffffffu, pq1, src);
        const uint32_t sr0 = __byte_perm(r0, 0, 0x1010), mr0 = __byte_perm(r0, 0, 0x3232);
        const uint32_t sr1 = __byte_perm(r1, 0, 0x1010), mr1 = __byte_perm(r1, 0, 0x3232);
        const uint32_t sq0 = __byte_perm(qq0, 0, 0x1010), mq0 = __byte_perm(qq0, 0, 0x3232);
        const uint32_t sq1 = __byte_perm(qq1, 0, 0x1010), mq1 = __byte_perm(qq1, 0, 0x3232);
        uint32_t la[4], lb[4], ha[4], hb[4];
        q4_unpack(R.q[g].x, M4, K, la[0], lb[0], ha[0], hb[0]);
        q4_unpack(R.q[g].y, M4, K, la[1], lb[1], ha[1], hb[1]);
        q4_unpack(R.q[g].z, M4, K, la[2], lb[2], ha[2], hb[2]);
        q4_unpack(R.q[g].w, M4, K, la[3], lb[3], ha[3], hb[3]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t s_lo = (i < 2) ? sr0 : sq0, m_lo = (i < 2) ? mr0 : mq0;
            const uint32_t s_hi = (i < 2) ? sr1 : sq1, m_hi = (i < 2) ? mr1 : mq1;
            la[i] = tc_h2_fma(tc_h2_sub(la[i], K), s_lo, m_lo);
            lb[i] = tc_h2_fma(tc_h2_sub(lb[i], K), s_lo, m_lo);
            ha[i] = tc_h2_fma(tc_h2_sub(ha[i], K), s_hi, m_hi);
            hb[i] = tc_h2_fma(tc_h2_sub(hb[i], K), s_hi, m_hi);
        }
        // words x, y (index 0, 1) are row r8, words z, w (2, 3) row r8+8; low nibbles = first 32 columns of the quarter
        {
            const uint32_t r_lo[4] = {la[0], lb[0], la[1], lb[1]}, q_lo[4] = {la[2], lb[2], la[3], lb[3]};
            const uint32_t r_hi[4] = {ha[0], hb[0], ha[1], hb[1]}, q_hi[4] = {ha[2], hb[2], ha[3], hb[3]};
            tc_store_chunk(a_row, g, 0, c, r_lo, q_lo);
            tc_store_chunk(a_row, g, 1, c, r_hi, q_hi);
        }
    }
}

__device__ __forceinline__ void tc_dequant(const TileRegs<14> &R, int q0, int q1, uint32_t a_row, int lane) {
    const int c = lane & 3;
    const float d_r = f16bits_to_f32(R.d01), d_q = f16bits_to_f32(R.d01 >> 16);
    uint32_t s_r[4], s_q[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        s_r[k] = tc_h2_dup(d_r * i8_to_f32(R.sc0, k));
        s_q[k] = tc_h2_dup(d_q * i8_to_f32(R.sc1, k));
    }
    uint32_t NIB = 0x0F0F0F0Fu, HI = 0x30303030u;
    asm volatile("" : "+r"(NIB), "+r"(HI));
#pragma unroll
    for (int m = 0; m < 4; m++) {
        if (m < q0 || m >= q1) continue;
        const uint32_t WA_r = R.ql[m].x, WB_r = R.ql[m].y, WA_q = R.ql[m].z, WB_q = R.ql[m].w;
        const uint4 hq = R.qh[m >> 1];
        const uint32_t H_r = (m & 1) ? hq.y : hq.x, H_q = (m & 1) ? hq.w : hq.z;
        uint32_t V_r[4], V_q[4];
        V_r[0] = and_or(WA_r, NIB, H_r & HI);
        V_r[1] = and_or(WA_r >> 4, NIB, (H_r >> 2) & HI);
        V_r[2] = and_or(WB_r, NIB, (H_r << 2) & HI);
        V_r[3] = and_or(WB_r >> 4, NIB, (H_r << 4) & HI);
        V_q[0] = and_or(WA_q, NIB, H_q & HI);
        V_q[1] = and_or(WA_q >> 4, NIB, (H_q >> 2) & HI);
        V_q[2] = and_or(WB_q, NIB, (H_q << 2) & HI);
        V_q[3] = and_or(WB_q >> 4, NIB, (H_q << 4) & HI);
        const int src = (lane & ~3) | m;
        uint32_t ar[4][2], aq[4][2];  // [16-column step k of the quarter][fragment k 2c.. | 2c+8..] for rows r8 / r8+8
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t sr = __shfl_sync(0xffffffffu, s_r[k], src), sq = __shfl_sync(0xffffffffu, s_q[k], src);
            ar[k][0] = tc_h2_mul(tc_h2_sub(__byte_perm(V_r[k], 0x64646464u, 0x4140), 0x64206420u), sr);
            ar[k][1] = tc_h2_mul(tc_h2_sub(__byte_perm(V_r[k], 0x64646464u, 0x4342), 0x64206420u), sr);
            aq[k][0] = tc_h2_mul(tc_h2_sub(__byte_perm(V_q[k], 0x64646464u, 0x4140), 0x64206420u), sq);
            aq[k][1] = tc_h2_mul(tc_h2_sub(__byte_perm(V_q[k], 0x64646464u, 0x4342), 0x64206420u), sq);
        }
        {
            const uint32_t r0[4] = {ar[0][0], ar[0][1], ar[1][0], ar[1][1]}, q0v[4] = {aq[0][0], aq[0][1], aq[1][0], aq[1][1]};
            const uint32_t r1[4] = {ar[2][0], ar[2][1], ar[3][0], ar[3][1]}, q1v[4] = {aq[2][0], aq[2][1], aq[3][0], aq[3][1]};
            tc_store_chunk(a_row, m, 0, c, r0, q0v);
            tc_store_chunk(a_row, m, 1, c, r1, q1v);
        }
    }
}

__device__ __forceinline__ void tc_dequant(const TileRegs<8> &R, int q0, int q1, uint32_t a_row, int lane) {
    const int c = lane & 3;
    const uint32_t dr[4] = {R.d0.x, R.d0.y, R.d0.z, R.d0.w}, dq[4] = {R.d1.x, R.d1.y, R.d1.z, R.d1.w};
    uint32_t SGN = 0x80808080u;
    asm volatile("" : "+r"(SGN));
#pragma unroll
    for (int j = 0; j < 8; j++) {
        if ((j >> 1) < q0 || (j >> 1) >= q1) continue;
        const uint32_t d_r = __byte_perm(dr[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);
        const uint32_t d_q = __byte_perm(dq[j >> 1], 0, (j & 1) ? 0x3232 : 0x1010);
        const uint32_t w4[4] = {R.q[j].x ^ SGN, R.q[j].y ^ SGN, R.q[j].z ^ SGN, R.q[j].w ^ SGN};
        uint32_t a[4][2];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t d = (i == 0 || i == 1) ? d_r : d_q;
            a[i][0] = tc_h2_mul(tc_h2_sub(__byte_perm(w4[i], 0x64646464u, 0x4240), 0x64806480u), d);
            a[i][1] = tc_h2_mul(tc_h2_sub(__byte_perm(w4[i], 0x64646464u, 0x4341), 0x64806480u), d);
        }
        // block j = 32 columns = half (j & 1) of quarter j >> 1; words x, y: row r8; z, w: row r8+8
        {
            const uint32_t rr[4] = {a[0][0], a[0][1], a[1][0], a[1][1]}, qq[4] = {a[2][0], a[2][1], a[3][0], a[3][1]};
            tc_store_chunk(a_row, j >> 1, j & 1, c, rr, qq);
        }
    }
}

// The half of a tile one warp works on (quarters 2h, 2h+1): only those registers of TileRegs are loaded.
__device__ __forceinline__ void tc_load_half(TileRegs<12> &r, const uint8_t *tile, int lane, int h) {
    const uint32_t *t1 = reinterpret_cast<const uint32_t *>(tile);
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile + kQ4KQsOff);
    const int r8 = lane >> 2, c = lane & 3;
    r.dm0 = __ldcs(t1 + r8);
    r.dm1 = __ldcs(t1 + r8 + 8);
    r.sm0 = __ldcs(t1 + 16 + r8 * 4 + c);
    r.sm1 = __ldcs(t1 + 16 + (r8 + 8) * 4 + c);
    if (h == 0) {  // static register indices: a runtime index would push the tile into local memory
        r.q[0] = __ldcs(t4 + 0 * 32 + lane);
        r.q[1] = __ldcs(t4 + 1 * 32 + lane);
    } else {
        r.q[2] = __ldcs(t4 + 2 * 32 + lane);
        r.q[3] = __ldcs(t4 + 3 * 32 + lane);
    }
}
__device__ __forceinline__ void tc_load_half(TileRegs<14> &r, const uint8_t *tile, int lane, int h) {
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile);
    const int r8 = lane >> 2, c = lane & 3;
    if (h == 0) {
        r.ql[0] = __ldcs(t4 + 0 * 32 + lane);
        r.ql[1] = __ldcs(t4 + 1 * 32 + lane);
        r.qh[0] = __ldcs(t4 + 128 + lane);
    } else {
        r.ql[2] = __ldcs(t4 + 2 * 32 + lane);
        r.ql[3] = __ldcs(t4 + 3 * 32 + lane);
        r.qh[1] = __ldcs(t4 + 128 + 32 + lane);
    }
    const uint32_t *sc = reinterpret_cast<const uint32_t *>(tile + 3072);
    r.sc0 = __ldcs(sc + r8 * 4 + c);
    r.sc1 = __ldcs(sc + (r8 + 8) * 4 + c);
    const unsigned short *d = reinterpret_cast<const unsigned short *>(tile + 3328);
    r.d01 = (uint32_t)__ldcs(d + r8) | ((uint32_t)__ldcs(d + r8 + 8) << 16);
}
__device__ __forceinline__ void tc_load_half(TileRegs<8> &r, const uint8_t *tile, int lane, int h) {
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile);
    const int r8 = lane >> 2;
    if (h == 0) {
#pragma unroll
        for (int j = 0; j < 4; j++) r.q[j] = __ldcs(t4 + j * 32 + lane);
    } else {
#pragma unroll
        for (int j = 4; j < 8; j++) r.q[j] = __ldcs(t4 + j * 32 + lane);
    }
    r.d0 = __ldcs(t4 + 256 + r8);
    r.d1 = __ldcs(t4 + 256 + r8 + 8);
}

template <int TYPE>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned b_slab_bytes = (unsigned)p.N * 512u;  // 32 chunks x N rows x 16 bytes
    // [A stage 0 | A stage 1 | B stage 0 | B stage 1 | barriers | tmem base | error]
    const uint32_t a_s = tc_smem_u32(smem), b_s = a_s + kTcStages * kTcASlabBytes;
    uint8_t *tail = smem + kTcStages * kTcASlabBytes + kTcStages * b_slab_bytes;
    const uint32_t bars = tc_smem_u32(tail);  // full[2], free[2], acc_ready, acc_free
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(tail + 64);
    volatile unsigned *err_s = reinterpret_cast<volatile unsigned *>(tail + 72);
    float *xs_s = reinterpret_cast<float *>(tail + 128);  // the activation's per-row factors, read once
    if (tid < kGemmMaxBatch) xs_s[tid] = (tid < p.batch && p.xscale) ? p.xscale[tid] : 1.f;
    const uint32_t full0 = bars, free0 = bars + 16, acc_ready = bars + 32, acc_free = bars + 40;
    const int tmem_cols = p.N <= 32 ? 32 : 64;
    if (tid == 0) {
        for (int s = 0; s < kTcStages; s++) {
            tc_mbar_init(full0 + 8 * s, kTcDequantWarps + 1);  // sixteen warps + the thread that posts the activation copy
            tc_mbar_init(free0 + 8 * s, 1);                     // one tcgen05.commit
        }
        tc_mbar_init(acc_ready, 1);
        tc_mbar_init(acc_free, 4);  // four epilogue warps
        *err_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTcDequantWarps) {  // the MMA warp owns the TMEM allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32((const void *)tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // instruction descriptor: D = F32, A = B = F16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    const uint32_t idesc = (1u << 4) | ((uint32_t)(p.N >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);

    unsigned it = 0;  // slabs issued so far by this CTA (stage = it % 2, use = it / 2)
    int task_no = 0;
    for (int task = blockIdx.x; task < p.n_tasks; task += gridDim.x, task_no++) {
        if (warp < kTcDequantWarps) {
            // ── dequantise: two warps per row tile, each the two 64-column quarters q0, q0+1 of every tile ──
            const int rt_local = warp >> 1, q0 = (warp & 1) * 2, q1 = q0 + 2;
            const int R = task * 8 + rt_local;
            const bool have = R < p.total_rt;
            const uint8_t *wrow = p.w + (size_t)(have ? R : 0) * p.nb * tile_bytes(TYPE);
            TileRegs<TYPE> buf0, buf1, buf2;  // this warp's half of the tiles sb, sb+1, sb+2 (two tiles in flight)
            const int h = warp & 1;
            const size_t tb = (size_t)tile_bytes(TYPE);
            if (have) tc_load_half(buf0, wrow, lane, h);
            if (have && p.nb > 1) tc_load_half(buf1, wrow + tb, lane, h);
            const int r8 = lane >> 2;
            const uint32_t row_off = (uint32_t)(rt_local * 16 + r8) * 16u;
            unsigned my_it = it;
            for (int sb = 0; sb < p.nb; sb++, my_it++) {
                const unsigned stage = my_it % kTcStages, use = my_it / kTcStages;
                // the MMAs that read this stage two slabs ago are done
                tc_mbar_wait(free0 + 8 * stage, (use & 1u) ^ 1u, err_s, p.err, 1);
                if (tid == 0) {  // activation slab: one contiguous copy
                    tc_mbar_expect_tx(full0 + 8 * stage, b_slab_bytes);
                    tc_bulk_g2s(b_s + stage * b_slab_bytes, p.ximg + (size_t)sb * b_slab_bytes, b_slab_bytes, full0 + 8 * stage);
                }
                const uint32_t a_row = a_s + stage * kTcASlabBytes + row_off;
                const bool pre = have && sb + 2 < p.nb;
                const uint8_t *nxt = wrow + (size_t)(sb + 2) * tb;
                const int which = sb % 3;
                if (which == 0) {
                    if (pre) tc_load_half(buf2, nxt, lane, h);
                    if (have) tc_dequant(buf0, q0, q1, a_row, lane);
                } else if (which == 1) {
                    if (pre) tc_load_half(buf0, nxt, lane, h);
                    if (have) tc_dequant(buf1, q0, q1, a_row, lane);
                } else {
                    if (pre) tc_load_half(buf1, nxt, lane, h);
                    if (have) tc_dequant(buf2, q0, q1, a_row, lane);
                }
                if (!have) {  // rows past the end of the matrix: zeros
                    const uint32_t z[4] = {0u, 0u, 0u, 0u};
                    for (int q = q0; q < q1; q++) {
                        tc_store_chunk(a_row, q, 0, lane & 3, z, z);
                        tc_store_chunk(a_row, q, 1, lane & 3, z, z);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic stores -> visible to the tensor core
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(full0 + 8 * stage);
            }
        } else if (lane == 0) {
            // ── issue the MMAs ──
            if (task_no > 0) tc_mbar_wait(acc_free, (unsigned)(task_no - 1) & 1u, err_s, p.err, 2);  // epilogue of the previous task has drained TMEM
            tc_fence_after();
            unsigned my_it = it;
            for (int sb = 0; sb < p.nb; sb++, my_it++) {
                const unsigned stage = my_it % kTcStages, use = my_it / kTcStages;
                const bool ok = tc_mbar_wait(full0 + 8 * stage, use & 1u, err_s, p.err, 3);
                tc_fence_after();
                if (ok) {
#pragma unroll 4
                    for (int s16 = 0; s16 < 16; s16++) {
                        const uint64_t ad = tc_smem_desc(a_s + stage * kTcASlabBytes + (uint32_t)(2 * s16) * kTcChunkStride, kTcChunkStride, 128u);
                        const uint64_t bd = tc_smem_desc(b_s + stage * b_slab_bytes + (uint32_t)(2 * s16) * ((uint32_t)p.N * 16u), (uint32_t)p.N * 16u, 128u);
                        tc_mma_f16(tmem_base, ad, bd, idesc, (sb > 0 || s16 > 0) ? 1u : 0u);
                    }
                }
                tc_commit(free0 + 8 * stage);  // arrives when the MMAs above have read the stage
            }
            tc_commit(acc_ready);  // arrives when the whole accumulation is in TMEM
        }
        it += (unsigned)p.nb;
        // ── epilogue: warps 0..3, TMEM lanes 32*warp .. +31 = weight rows of the CTA tile ──
        if (warp < 4) {
            const bool ok = tc_mbar_wait(acc_ready, (unsigned)task_no & 1u, err_s, p.err, 4);
            tc_fence_after();
            const int row_in_cta = warp * 32 + lane;
            for (int c0 = 0; c0 < p.N; c0 += 16) {
                uint32_t v[16];
                tc_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int b = c0 + j;
                    float y = __uint_as_float(v[j]);
                    y *= xs_s[b];
                    if (p.epi == EPI_SILU_PAIR) {
                        const float up = __shfl_down_sync(0xffffffffu, y, 8);  // rows 8..15 of a tile are the up rows
                        const int orow = (task * 8 + (row_in_cta >> 4)) * 8 + (row_in_cta & 7);
                        if (ok && b < p.batch && (row_in_cta & 8) == 0 && orow < p.rows) p.out[(size_t)b * p.ld_out + orow] = __fmul_rn(silu_ref(y), up);
                    } else {
                        const int orow = task * kTcRows + row_in_cta;
                        if (ok && b < p.batch && orow < p.rows) p.out[(size_t)b * p.ld_out + orow] = y;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(acc_free);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kTcDequantWarps) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ───────────────────────────── chunk-major FP16 staging ────────────────────────────────────
// Image [K/8][N][8] in the slab K order described above (tc_store_chunk): the four consecutive columns 16*s16 + 4c ..
// + 3 of a sequence go, as (x0, x2, x1, x3), to half of the chunk (quarter, half, c) with quarter = (s16 % 16) / 4,
// half = (s16 / 2) % 2, and to its first or second 8 bytes for even / odd s16.
struct StageTcParams {
    const float *x;
    int ldx;
    int K, batch, N;
    uint8_t *img;
    float *xscale;
};

__global__ void __launch_bounds__(256) stage_tc_kernel(const StageTcParams p) {
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned short *img = reinterpret_cast<unsigned short *>(p.img);
    const int K = p.K, N = p.N;
    __shared__ float redm[8];
    auto chunk_of = [&](int i4) {  // destination (in halfs) of columns i4..i4+3
        const int s16 = i4 >> 4, c = (i4 >> 2) & 3, slab = s16 >> 4, t = s16 & 15;
        const int chunk = slab * 32 + ((t >> 2) * 2 + ((t >> 1) & 1)) * 4 + c;
        return ((size_t)chunk * N + b) * 8 + (size_t)(t & 1) * 4;
    };
    if (b >= p.batch) {
        for (int i4 = tid * 4; i4 < K; i4 += 256 * 4) *reinterpret_cast<uint2 *>(img + chunk_of(i4)) = make_uint2(0u, 0u);
        return;
    }
    const float *xrow = p.x + (size_t)b * p.ldx;
    float vmax = 0.f;
    for (int i = tid; i < K; i += 256) vmax = fmaxf(vmax, fabsf(xrow[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    if (lane == 0) redm[warp] = vmax;
    __syncthreads();
    vmax = redm[0];
#pragma unroll
    for (int w8 = 1; w8 < 8; w8++) vmax = fmaxf(vmax, redm[w8]);
    float down = 1.f, up = 1.f;
    if (vmax > 0.f && vmax < 3.0e38f) {
        int e;
        frexpf(vmax, &e);
        down = ldexpf(1.f, 9 - e);
        up = ldexpf(1.f, e - 9);
    }
    if (tid == 0) p.xscale[b] = up;
    for (int i4 = tid * 4; i4 < K; i4 += 256 * 4) {
        const float4 xv = *reinterpret_cast<const float4 *>(xrow + i4);
        const __half2 lo = __floats2half2_rn(xv.x * down, xv.z * down);  // columns 4c, 4c+2
        const __half2 hi = __floats2half2_rn(xv.y * down, xv.w * down);  // columns 4c+1, 4c+3
        uint2 w;
        w.x = *reinterpret_cast<const uint32_t *>(&lo);
        w.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(img + chunk_of(i4)) = w;
    }
}

// ───────────────────────────── host ───────────────────────────────────────────────────────
bool gemm_tc_enabled() {
    static const bool on = [] {
        const char *e = getenv("JUNO_GEMM_TCGEN05");  // JUNO_GEMM_TCGEN05=0: keep every batched product on mma.sync
        return !(e && *e == '0');
    }();
    return on;
}
int gemm_tc_padded_batch(int batch) { return (batch + 15) / 16 * 16; }
size_t gemm_tc_image_bytes(int K, int batch) { return (size_t)K * gemm_tc_padded_batch(batch) * 2; }
// Shapes this kernel takes: enough 128-row blocks to occupy the GPU, and a batch from which it measured faster than the
// mma.sync kernel (its time hardly depends on the batch: 185-209 us on 128256 x 4096 Q4_K for 16-64 sequences, against
// 138-294 us).
bool gemm_tc_shape_ok(const juno_ctx *ctx, int row_tiles, int batch) {
    static const int min_batch = [] {
        const char *e = getenv("JUNO_GEMM_TC_MIN_BATCH");
        return (e && *e) ? atoi(e) : 48;
    }();
    return batch >= min_batch && batch <= kGemmMaxBatch && (row_tiles + 7) / 8 >= ctx->sm_count / 2;
}

int launch_stage_tc(juno_ctx *ctx, const float *x, int ldx, int K, int batch, uint8_t *img, float *xscale, cudaStream_t st) {
    JUNO_REQUIRE(K > 0 && K % 256 == 0 && batch >= 1 && batch <= kGemmMaxBatch && x && img && xscale && ldx % 4 == 0,
                 "stage (tcgen05): bad arguments (K=%d, batch=%d)", K, batch);
    StageTcParams p;
    p.x = x;
    p.ldx = ldx;
    p.K = K;
    p.batch = batch;
    p.N = gemm_tc_padded_batch(batch);
    p.img = img;
    p.xscale = xscale;
    ProfScope prof(ctx, st, PROF_OTHER, 0);
    stage_tc_kernel<<<p.N, 256, 0, st>>>(p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

template <int TYPE>
static int gemm_tc_launch_type(juno_ctx *ctx, const TcParams &p, cudaStream_t st) {
    const size_t smem = (size_t)kTcStages * kTcASlabBytes + (size_t)kTcStages * p.N * 512 + 128 + kGemmMaxBatch * 4;
    static std::mutex mu;
    static bool configured[16] = {false};
    {
        std::lock_guard<std::mutex> g(mu);
        const int dev = ctx->device & 15;
        if (!configured[dev]) {
            JUNO_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin));
            configured[dev] = true;
        }
    }
    JUNO_REQUIRE(smem <= ctx->smem_optin, "gemm (tcgen05): %zu bytes of shared memory needed", smem);
    const int grid = std::max(1, std::min(p.n_tasks, ctx->sm_count));
    gemm_tc_kernel<TYPE><<<grid, kTcThreads, smem, st>>>(p);
    JUNO_CUDA_TRY(cudaGetLastError());
    ctx->kernel_launches++;
    return JUNO_OK;
}

// One matrix (one block format), EPI_STORE or EPI_SILU_PAIR.  `err` is a device word that stays zero unless a wait
// inside the kernel gave up.
int launch_gemm_tc(juno_ctx *ctx, const uint8_t *w, int type, int rows, int row_tiles, int K, int batch, const uint8_t *ximg,
                   const float *xscale, float *out, int ld_out, int epi, unsigned *err, cudaStream_t st) {
    JUNO_REQUIRE(type == 12 || type == 14 || type == 8, "gemm (tcgen05): type %d has no tiled kernel", type);
    JUNO_REQUIRE(epi == EPI_STORE || epi == EPI_SILU_PAIR, "gemm (tcgen05): epilogue %d is not supported", epi);
    TcParams p;
    memset(&p, 0, sizeof(p));
    p.w = w;
    p.out = out;
    p.rows = rows;
    p.total_rt = row_tiles;
    p.K = K;
    p.nb = K / 256;
    p.batch = batch;
    p.N = gemm_tc_padded_batch(batch);
    p.ld_out = ld_out;
    p.epi = epi;
    p.ximg = ximg;
    p.xscale = xscale;
    p.n_tasks = (row_tiles + 7) / 8;
    p.err = err;
    p.type = type;
    const double bpw = type == 12 ? 144.0 / 256 : type == 14 ? 210.0 / 256 : 34.0 / 32;
    const double algo = (double)rows * K * bpw * (epi == EPI_SILU_PAIR ? 2 : 1) + (double)batch * K * 4 + (double)batch * rows * 4;
    ProfScope prof(ctx, st, type == 12 ? PROF_GEMV_Q4K : type == 14 ? PROF_GEMV_Q6K : PROF_GEMV_Q80, algo);
    ProfScope prof_tc(ctx, st, PROF_GEMM_TC, algo);
    return type == 12 ? gemm_tc_launch_type<12>(ctx, p, st) : type == 14 ? gemm_tc_launch_type<14>(ctx, p, st) : gemm_tc_launch_type<8>(ctx, p, st);
}

}  // namespace juno
