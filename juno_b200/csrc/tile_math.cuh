// Register-level arithmetic of the fused dequant-GEMV: one 16x256 weight tile (layout.cuh) held by a warp is
// unpacked into exact small-integer bf16 fragments and multiplied against the staged activation with
// mma.sync.m16n8k16.  Shared by the per-product GEMV kernel and by the persistent decode-step kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "layout.cuh"
#include "stage.cuh"

namespace juno {

// ───────────────────────────── device helpers ─────────────────────────────────────────────
__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }

// (a & b) | c in ONE logic instruction.  Written as lop3 with register operands: left to the compiler, a mask and
// a magic constant that are both immediates become two instructions on the half-rate integer pipe.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// ((a & b) ^ c) in one instruction.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t bf2_sub(uint32_t v, uint32_t c) {
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&v);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&c);
    __nv_bfloat162 r = __hsub2(a, b);
    return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

__device__ __forceinline__ float f16bits_to_f32(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)(bits & 0xFFFFu)));
}

constexpr uint32_t kBf128 = 0x43004300u;  // (128, 128)
constexpr uint32_t kBf160 = 0x43204320u;  // (160, 160)
constexpr uint32_t kBf384 = 0x43C043C0u;  // (384, 384)

// SiLU as LlamaTransformerHandler.silu (:1733-1735): x / (1f + (float) Math.exp(-x)).  The exponential is taken in
// FP32 (expf, <= 2 ulp) instead of binary64-then-cast: a binary64 exp on the few threads of a GEMV epilogue sat on the
// critical path of every CTA task.
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, __fadd_rn(1.f, expf(-x))); }

template <int TYPE>
struct TileRegs;
template <>
struct TileRegs<12> {
    uint32_t dm0, dm1, sm0, sm1;  // d|dmin and the lane's scale/min bytes for rows r8, r8+8
    uint4 q[4];
};
template <>
struct TileRegs<14> {
    uint4 ql[4], qh[2];
    uint32_t sc0, sc1;
    uint32_t d01;
};
template <>
struct TileRegs<8> {
    uint4 q[8], d0, d1;
};

template <int TYPE>
__device__ __forceinline__ void load_tile(TileRegs<TYPE> &r, const uint8_t *tile, int lane);

template <>
__device__ __forceinline__ void load_tile<12>(TileRegs<12> &r, const uint8_t *tile, int lane) {
    const uint32_t *t1 = reinterpret_cast<const uint32_t *>(tile);
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile + kQ4KQsOff);
    const int r8 = lane >> 2, c = lane & 3;
    r.dm0 = __ldcs(t1 + r8);
    r.dm1 = __ldcs(t1 + r8 + 8);
    r.sm0 = __ldcs(t1 + 16 + r8 * 4 + c);
    r.sm1 = __ldcs(t1 + 16 + (r8 + 8) * 4 + c);
#pragma unroll
    for (int g = 0; g < 4; g++) r.q[g] = ld_stream(t4 + g * 32 + lane);
}
template <>
__device__ __forceinline__ void load_tile<14>(TileRegs<14> &r, const uint8_t *tile, int lane) {
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile);
    int r8 = lane >> 2, c = lane & 3;
#pragma unroll
    for (int m = 0; m < 4; m++) r.ql[m] = ld_stream(t4 + m * 32 + lane);
#pragma unroll
    for (int p = 0; p < 2; p++) r.qh[p] = ld_stream(t4 + 128 + p * 32 + lane);
    const uint32_t *sc = reinterpret_cast<const uint32_t *>(tile + 3072);
    r.sc0 = __ldcs(sc + r8 * 4 + c);
    r.sc1 = __ldcs(sc + (r8 + 8) * 4 + c);
    const unsigned short *d = reinterpret_cast<const unsigned short *>(tile + 3328);
    r.d01 = (uint32_t)__ldcs(d + r8) | ((uint32_t)__ldcs(d + r8 + 8) << 16);
}
template <>
__device__ __forceinline__ void load_tile<8>(TileRegs<8> &r, const uint8_t *tile, int lane) {
    const uint4 *t4 = reinterpret_cast<const uint4 *>(tile);
    int r8 = lane >> 2;
#pragma unroll
    for (int j = 0; j < 8; j++) r.q[j] = ld_stream(t4 + j * 32 + lane);
    r.d0 = ld_stream(t4 + 256 + r8);
    r.d1 = ld_stream(t4 + 256 + r8 + 8);
}


// MMA whose accumulator input is zero (the register file's zero register), so no clears are issued.
__device__ __forceinline__ void mma16816_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma1688_z(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.f));
}

// Shared-memory view of the staged activation for one lane.  NC = 3*NB limb columns are compile-time, so every
// fetch below is a load with an immediate offset.  A lane whose fragment column does not exist (col >= NC) reads
// column NC-1 instead: it only feeds accumulator columns that are never read back.
template <int NC>
struct XView {
    const unsigned short *xb_lane[(NC + 7) / 8];  // xb + (colc*4 + c)*4 for each n-tile
    const uint32_t *xs_lane[(NC + 7) / 8];        // xs32 + colc*4 + c
    __device__ __forceinline__ uint2 b(int nt, int s16) const {
        return *reinterpret_cast<const uint2 *>(xb_lane[nt] + s16 * (NC * 16));
    }
    __device__ __forceinline__ uint32_t sums(int nt, int sb) const { return xs_lane[nt][sb * (NC * 4)]; }
};

// ── Q4_K tile ────────────────────────────────────────────────────────────────────────────
// Nibbles -> bf16 pairs holding 128 + q exactly (mask | magic in one instruction).  The bias is not removed here:
// sum((128+q)*x) = 128*sum(x) + sum(q*x), and the 128*scale*sum(x) part is subtracted once per tile together with
// the min term (both are "per-sub-block constant times sum of x over the sub-block").
__device__ __forceinline__ void q4_unpack(uint32_t w, uint32_t M, uint32_t K, uint32_t &lo_a, uint32_t &lo_b,
                                          uint32_t &hi_a, uint32_t &hi_b) {
    lo_a = and_or(w, M, K);        // (byte0.lo, byte2.lo)
    hi_a = and_or(w >> 4, M, K);   // (byte0.hi, byte2.hi)
    lo_b = and_or(w >> 8, M, K);   // (byte1.lo, byte3.lo)
    hi_b = and_or(w >> 12, M, K);  // (byte1.hi, byte3.hi)
}

__device__ __forceinline__ uint32_t bf2_mul(uint32_t v, uint32_t c) {
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162 *>(&v);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162 *>(&c);
    __nv_bfloat162 r = __hmul2(a, b);
    return *reinterpret_cast<uint32_t *>(&r);
}

// Decodes one row's header words for the lane's two sub-blocks 2c, 2c+1.
__device__ __forceinline__ void q4_header(uint32_t dm, uint32_t sm, float &sc0, float &sc1, uint32_t &mins_bf2,
                                          uint32_t &sc128_bf2, float &d, float &dmin) {
    d = f16bits_to_f32(dm);
    dmin = f16bits_to_f32(dm >> 16);
    sc0 = __fmul_rn(d, (float)(sm & 0xFFu));
    sc1 = __fmul_rn(d, (float)((sm >> 8) & 0xFFu));
    mins_bf2 = bf2_sub(__byte_perm(sm, 0x43434343u, 0x4342), kBf128);                          // bf16x2 (m0, m1)
    sc128_bf2 = bf2_mul(bf2_sub(__byte_perm(sm, 0x43434343u, 0x4140), kBf128), kBf128);       // (128*s0, 128*s1), exact
}

template <int NC>
__device__ __forceinline__ void compute_tile(const TileRegs<12> &R, int sb, const XView<NC> &xv, int lane,
                                             float (&acc)[(NC + 7) / 8][4], float (&macc)[(NC + 7) / 8][4]) {
    constexpr int NT = (NC + 7) / 8;
    float s_r[2], s_q[2], dmin_r, dmin_q, d_r, d_q;
    uint32_t mins_r, mins_q, off_r, off_q;
    q4_header(R.dm0, R.sm0, s_r[0], s_r[1], mins_r, off_r, d_r, dmin_r);
    q4_header(R.dm1, R.sm1, s_q[0], s_q[1], mins_q, off_q, d_q, dmin_q);
    const int s16base = sb * 16;
    // held in registers on purpose (see and_or)
    uint32_t M4 = 0x000F000Fu, K128 = kBf128;
    asm volatile("" : "+r"(M4), "+r"(K128));
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint32_t la_x, lb_x, ha_x, hb_x, la_y, lb_y, ha_y, hb_y, la_z, lb_z, ha_z, hb_z, la_w, lb_w, ha_w, hb_w;
        q4_unpack(R.q[g].x, M4, K128, la_x, lb_x, ha_x, hb_x);
        q4_unpack(R.q[g].y, M4, K128, la_y, lb_y, ha_y, hb_y);
        q4_unpack(R.q[g].z, M4, K128, la_z, lb_z, ha_z, hb_z);
        q4_unpack(R.q[g].w, M4, K128, la_w, lb_w, ha_w, hb_w);
        const int src = (lane & ~3) | g;  // quad lane g owns sub-blocks 2g and 2g+1
        const float sr0 = __shfl_sync(0xffffffffu, s_r[0], src), sr1 = __shfl_sync(0xffffffffu, s_r[1], src);
        const float sq0 = __shfl_sync(0xffffffffu, s_q[0], src), sq1 = __shfl_sync(0xffffffffu, s_q[1], src);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float ct[4], ch[4];
            uint2 b = xv.b(nt, s16base + 4 * g + 0);
            mma16816_z(ct, la_x, la_z, lb_x, lb_z, b.x, b.y);
            b = xv.b(nt, s16base + 4 * g + 1);
            mma16816(ct, la_y, la_w, lb_y, lb_w, b.x, b.y);
            b = xv.b(nt, s16base + 4 * g + 2);
            mma16816_z(ch, ha_x, ha_z, hb_x, hb_z, b.x, b.y);
            b = xv.b(nt, s16base + 4 * g + 3);
            mma16816(ch, ha_y, ha_w, hb_y, hb_w, b.x, b.y);
            acc[nt][0] = fmaf(sr0, ct[0], acc[nt][0]);
            acc[nt][1] = fmaf(sr0, ct[1], acc[nt][1]);
            acc[nt][2] = fmaf(sq0, ct[2], acc[nt][2]);
            acc[nt][3] = fmaf(sq0, ct[3], acc[nt][3]);
            acc[nt][0] = fmaf(sr1, ch[0], acc[nt][0]);
            acc[nt][1] = fmaf(sr1, ch[1], acc[nt][1]);
            acc[nt][2] = fmaf(sq1, ch[2], acc[nt][2]);
            acc[nt][3] = fmaf(sq1, ch[3], acc[nt][3]);
        }
    }
    // min term: sum_j (dmin*m_j) * sum_{c in sub-block j} x[c]
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        float cm[4], co[4];
        const uint32_t xsum = xv.sums(nt, sb);
        mma1688_z(cm, mins_r, mins_q, xsum);
        mma1688_z(co, off_r, off_q, xsum);  // sum_j 128*sc_j * sum(x over sub-block j): the bias of the nibbles
        macc[nt][0] = fmaf(dmin_r, cm[0], fmaf(d_r, co[0], macc[nt][0]));
        macc[nt][1] = fmaf(dmin_r, cm[1], fmaf(d_r, co[1], macc[nt][1]));
        macc[nt][2] = fmaf(dmin_q, cm[2], fmaf(d_q, co[2], macc[nt][2]));
        macc[nt][3] = fmaf(dmin_q, cm[3], fmaf(d_q, co[3], macc[nt][3]));
    }
}

// ── Q6_K tile ────────────────────────────────────────────────────────────────────────────
__device__ __forceinline__ float i8_to_f32(uint32_t w, int k) { return (float)(int)(signed char)((w >> (8 * k)) & 0xFFu); }

template <int NC>
__device__ __forceinline__ void compute_tile(const TileRegs<14> &R, int sb, const XView<NC> &xv, int lane,
                                             float (&acc)[(NC + 7) / 8][4], float (& /*macc*/)[(NC + 7) / 8][4]) {
    constexpr int NT = (NC + 7) / 8;
    const float d_r = f16bits_to_f32(R.d01), d_q = f16bits_to_f32(R.d01 >> 16);
    float s_r[4], s_q[4];  // scales of sub-blocks 4c..4c+3 for rows r8 and r8+8
#pragma unroll
    for (int k = 0; k < 4; k++) {
        s_r[k] = __fmul_rn(d_r, i8_to_f32(R.sc0, k));
        s_q[k] = __fmul_rn(d_q, i8_to_f32(R.sc1, k));
    }
    const int s16base = sb * 16;
    uint32_t NIB = 0x0F0F0F0Fu, HI = 0x30303030u;
    asm volatile("" : "+r"(NIB), "+r"(HI));
#pragma unroll
    for (int m = 0; m < 4; m++) {
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
            const float sr = __shfl_sync(0xffffffffu, s_r[k], src), sq = __shfl_sync(0xffffffffu, s_q[k], src);
            const uint32_t a0 = bf2_sub(__byte_perm(V_r[k], 0x43434343u, 0x4140), kBf160);
            const uint32_t a2 = bf2_sub(__byte_perm(V_r[k], 0x43434343u, 0x4342), kBf160);
            const uint32_t a1 = bf2_sub(__byte_perm(V_q[k], 0x43434343u, 0x4140), kBf160);
            const uint32_t a3 = bf2_sub(__byte_perm(V_q[k], 0x43434343u, 0x4342), kBf160);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float ct[4];
                const uint2 b = xv.b(nt, s16base + 4 * m + k);
                mma16816_z(ct, a0, a1, a2, a3, b.x, b.y);
                acc[nt][0] = fmaf(sr, ct[0], acc[nt][0]);
                acc[nt][1] = fmaf(sr, ct[1], acc[nt][1]);
                acc[nt][2] = fmaf(sq, ct[2], acc[nt][2]);
                acc[nt][3] = fmaf(sq, ct[3], acc[nt][3]);
            }
        }
    }
}

// ── Q8_0 tile: int8 q = 16*h + l, both nibble planes exact in bf16 ────────────────────────
__device__ __forceinline__ void q8_unpack(uint32_t w, uint32_t M, uint32_t K, uint32_t MH, uint32_t KH, uint32_t &l_a,
                                          uint32_t &l_b, uint32_t &h_a, uint32_t &h_b) {
    l_a = bf2_sub(and_or(w, M, K), K);          // (b0&15, b2&15)
    l_b = bf2_sub(and_or(w >> 8, M, K), K);     // (b1&15, b3&15)
    h_a = bf2_sub(and_xor(w >> 1, MH, KH), KH); // 16*(b0>>4), 16*(b2>>4)  (arithmetic >>)
    h_b = bf2_sub(and_xor(w >> 9, MH, KH), KH); // 16*(b1>>4), 16*(b3>>4)
}

template <int NC>
__device__ __forceinline__ void compute_tile(const TileRegs<8> &R, int sb, const XView<NC> &xv, int /*lane*/,
                                             float (&acc)[(NC + 7) / 8][4], float (& /*macc*/)[(NC + 7) / 8][4]) {
    constexpr int NT = (NC + 7) / 8;
    const int s16base = sb * 16;
    const uint32_t dr[4] = {R.d0.x, R.d0.y, R.d0.z, R.d0.w}, dq[4] = {R.d1.x, R.d1.y, R.d1.z, R.d1.w};
    uint32_t M4 = 0x000F000Fu, K128 = kBf128, MH = 0x00780078u, KH = kBf384;
    asm volatile("" : "+r"(M4), "+r"(K128), "+r"(MH), "+r"(KH));
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float d_r = f16bits_to_f32(dr[j >> 1] >> ((j & 1) * 16)), d_q = f16bits_to_f32(dq[j >> 1] >> ((j & 1) * 16));
        uint32_t la_x, lb_x, ha_x, hb_x, la_y, lb_y, ha_y, hb_y, la_z, lb_z, ha_z, hb_z, la_w, lb_w, ha_w, hb_w;
        q8_unpack(R.q[j].x, M4, K128, MH, KH, la_x, lb_x, ha_x, hb_x);
        q8_unpack(R.q[j].y, M4, K128, MH, KH, la_y, lb_y, ha_y, hb_y);
        q8_unpack(R.q[j].z, M4, K128, MH, KH, la_z, lb_z, ha_z, hb_z);
        q8_unpack(R.q[j].w, M4, K128, MH, KH, la_w, lb_w, ha_w, hb_w);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float ct[4];
            uint2 b = xv.b(nt, s16base + 2 * j);
            mma16816_z(ct, la_x, la_z, lb_x, lb_z, b.x, b.y);
            mma16816(ct, ha_x, ha_z, hb_x, hb_z, b.x, b.y);
            b = xv.b(nt, s16base + 2 * j + 1);
            mma16816(ct, la_y, la_w, lb_y, lb_w, b.x, b.y);
            mma16816(ct, ha_y, ha_w, hb_y, hb_w, b.x, b.y);
            acc[nt][0] = fmaf(d_r, ct[0], acc[nt][0]);
            acc[nt][1] = fmaf(d_r, ct[1], acc[nt][1]);
            acc[nt][2] = fmaf(d_q, ct[2], acc[nt][2]);
            acc[nt][3] = fmaf(d_q, ct[3], acc[nt][3]);
        }
    }
}

// ── mixed launches: Q4_K and Q6_K segments in one grid (the fused Q,K,V projection of a Q4_K_M model) ─────────
// TYPE 0 keeps a tile in a format-neutral register image and dispatches per task on the segment's block format
// (warp-uniform: a warp works on one row tile at a time).
template <>
struct TileRegs<0> {
    uint4 v[6];
    uint32_t s[4];
};
template <int TYPE>
__device__ __forceinline__ void load_tile_t(TileRegs<TYPE> &r, const uint8_t *tile, int lane, int /*type*/) {
    load_tile<TYPE>(r, tile, lane);
}
template <>
__device__ __forceinline__ void load_tile_t<0>(TileRegs<0> &r, const uint8_t *tile, int lane, int type) {
    if (type == 12) {
        TileRegs<12> t;
        load_tile<12>(t, tile, lane);
#pragma unroll
        for (int g = 0; g < 4; g++) r.v[g] = t.q[g];
        r.s[0] = t.dm0; r.s[1] = t.dm1; r.s[2] = t.sm0; r.s[3] = t.sm1;
    } else {
        TileRegs<14> t;
        load_tile<14>(t, tile, lane);
#pragma unroll
        for (int m = 0; m < 4; m++) r.v[m] = t.ql[m];
        r.v[4] = t.qh[0]; r.v[5] = t.qh[1];
        r.s[0] = t.sc0; r.s[1] = t.sc1; r.s[2] = t.d01;
    }
}
template <int TYPE, int NC>
__device__ __forceinline__ void compute_tile_t(const TileRegs<TYPE> &R, int /*type*/, int sb, const XView<NC> &xv, int lane,
                                               float (&acc)[(NC + 7) / 8][4], float (&macc)[(NC + 7) / 8][4]) {
    compute_tile<NC>(R, sb, xv, lane, acc, macc);
}
template <int NC>
__device__ __forceinline__ void compute_tile_mixed(const TileRegs<0> &R, int type, int sb, const XView<NC> &xv, int lane,
                                                   float (&acc)[(NC + 7) / 8][4], float (&macc)[(NC + 7) / 8][4]) {
    if (type == 12) {
        TileRegs<12> t;
#pragma unroll
        for (int g = 0; g < 4; g++) t.q[g] = R.v[g];
        t.dm0 = R.s[0]; t.dm1 = R.s[1]; t.sm0 = R.s[2]; t.sm1 = R.s[3];
        compute_tile<NC>(t, sb, xv, lane, acc, macc);
    } else {
        TileRegs<14> t;
#pragma unroll
        for (int m = 0; m < 4; m++) t.ql[m] = R.v[m];
        t.qh[0] = R.v[4]; t.qh[1] = R.v[5];
        t.sc0 = R.s[0]; t.sc1 = R.s[1]; t.d01 = R.s[2];
        compute_tile<NC>(t, sb, xv, lane, acc, macc);
    }
}

}  // namespace juno
