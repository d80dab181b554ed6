// Fused dequant-GEMV for GGUF Q4_K / Q6_K / Q8_0 weights on integer tensor-core MMAs, 1..8 decode sequences.
//
// y[b][r] = sum_c w(r,c) * x[b][c] with w as LlamaTransformerHandler.matVecQ4Kraw / matVecQ6Kraw / matVecQ8_0raw
// define it (LlamaTransformerHandler.java:1428-1508, 1587-1638), accumulated in a different order.
//
// Arithmetic.  The activation of every 256-column slice is turned into block floating point: q = round(v * 2^-e)
// with |q| <= 2^22 and e chosen from the slice's largest magnitude, q split into three signed bytes
// (q = l0 + 256 l1 + 65536 l2).  The 4-, 6- and 8-bit weight fields are used as 8-bit integers as they are
// (a nibble is one AND away from a byte), so one mma.sync.m16n8k32 (s32 += u8 x s8) multiplies 16 rows x 32 columns
// of weights with the limbs of two sequences, exactly.  Per 32-column sub-block the s32 results are combined with the
// integer sub-block scales; one conversion per 256-column tile applies d * 2^e in FP32.  The Q4_K min term and the
// Q6_K offset of 32 are one more integer MMA per tile against per-sub-block sums of q.
//
// Data flow.  CTAs of 16 warps, one or two per SM.  A CTA owns a contiguous range of row tiles (the ranges differ by
// at most one row tile across the grid); its tiles form one flat sequence that the sixteen warps split evenly
// (QCursor below), and the partial sums of a row tile are added through shared memory in warp order (bitwise
// repeatable).  Weights go HBM -> shared memory through a ring of tile slots per warp: each slot is filled by ONE
// cp.async.bulk that the warp issues itself (completion on an mbarrier, L2 evict-first) and re-issues as soon as it
// has used the tile.  The ring is filled before the kernel waits for its predecessor (programmatic dependent launch).  The activation operand is built by
// every CTA from the FP32 rows after that wait: the only data that depends on the predecessor.
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "gemv.cuh"
#include "layout.cuh"
#include "qgemv.cuh"
#include "qsplit.cuh"

namespace juno {

constexpr int kQThreads = 512;
constexpr int kQWarps = kQThreads / 32;

struct QParams {
    const uint8_t *w[3];
    float *out[3];
    int rows[3];
    int seg_type[3];
    int rt_begin[4];
    int nseg, total_rt;
    int K, NB;
    int ld_out, epi, bc;
    const float *x;
    int ldx;
    const float *add[kQMaxAdd];
    int n_add;
    float *x_store;
    const float *normw;
    float eps;
    int ring;       // tile slots per warp
    int slot_bytes; // bytes of one slot (largest tile of the launch)
    int wait_ns;             // suspend hint of a wait on a weight tile
    // tensor-parallel push all-reduce (see QGemvArgs)
    int n_peers;
    float *peer_out[kQMaxAdd];
    int tagged_adds;
    int n_red;                       // TAGGED kernels: pre-reduction of the ranks' inbox slots by the first CTAs
    const float *red_src[kQMaxAdd];
    float *red_dst;
    const unsigned *epoch;
    unsigned *peer_failed;
    unsigned *err;  // device word: a wait on a weight tile gave up (code | warp << 8 | block << 16)
};

// ───────────────────────────── shared-memory operand ──────────────────────────────────────
// One block per (sequence, 256-column slice):
//   nat  [3 limbs][256 B]  bytes in MMA "B" fragment order for k32 steps: lane (limb j, t) owns 64 bytes = four 16-byte
//                          chunks; chunk q = { sub-block 2q: k 4t..4t+3, k 16+4t..; sub-block 2q+1: same }.
//                          Chunks are XOR-swizzled so that the 128-bit reads of a quarter warp hit 32 distinct banks.
//   perm [3 limbs][256 B]  the same with the four bytes of every word in the order (0,2,1,3): the column order of
//                          the Q6_K tile words.
//   xs32 [4 limbs][4 t]    words (0, 0, S(2t), S(2t+1)): limbs of the sums of q over 32-column sub-blocks, placed
//                          against the Q4_K header word (scale, scale, min, min) of the same lane
//   xs16 [4 limbs][4 t]    words S16(4t..4t+3): limbs of the sums over 16 columns, against the Q6_K scale words
//   scale                  2^e as FP32
template <int TYPE>
struct XBlk {
    static constexpr bool kNat = TYPE != 14, kPerm = TYPE == 14 || TYPE == 0;
    static constexpr bool kXs32 = TYPE == 12 || TYPE == 0, kXs16 = TYPE == 14 || TYPE == 0;
    static constexpr int nat_off = 0;
    static constexpr int perm_off = kNat ? 768 : 0;
    static constexpr int xs32_off = perm_off + (kPerm ? 768 : 0);
    static constexpr int xs16_off = xs32_off + (kXs32 ? 64 : 0);
    static constexpr int scale_off = xs16_off + (kXs16 ? 64 : 0);
    static constexpr int bytes = scale_off + 16;
};
static int xblk_bytes(int type_mix) {
    return type_mix == 12 ? XBlk<12>::bytes : type_mix == 14 ? XBlk<14>::bytes : type_mix == 8 ? XBlk<8>::bytes : XBlk<0>::bytes;
}

__device__ __forceinline__ int swz_key(int t, int j) { return (t >> 1) | ((j & 1) << 1); }

// ───────────────────────────── integer MMAs ───────────────────────────────────────────────
__device__ __forceinline__ void imma_k32_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_k32_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_k16_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void imma_k16_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)(bits & 0xFFFFu))); }
__device__ __forceinline__ int ubyte(uint32_t w, int k) { return (int)__byte_perm(w, 0, 0x4440 | k); }
__device__ __forceinline__ int sbyte(uint32_t w, int k) {  // sign-extended byte k: selector nibbles 8|k replicate its sign bit
    int d;                                                 // (the __byte_perm intrinsic only honours three bits per nibble)
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(0), "r"(((8 | k) << 12) | ((8 | k) << 8) | ((8 | k) << 4) | k));
    return d;
}
__device__ __forceinline__ uint32_t pick4(const uint4 &v, int t) { return (t & 2) ? ((t & 1) ? v.w : v.z) : ((t & 1) ? v.y : v.x); }
// SiLU as LlamaTransformerHandler.silu (:1733-1735): x / (1f + (float) Math.exp(-x)), exponential in FP32 (<= 2 ulp).
__device__ __forceinline__ float silu_f(float x) { return __fdiv_rn(x, __fadd_rn(1.f, expf(-x))); }

// ───────────────────────────── one weight tile against the operand ────────────────────────
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
    uint32_t v;
    asm volatile("{\n.reg .u16 h;\nld.shared.u16 h, [%1];\ncvt.u32.u16 %0, h;\n}\n" : "=r"(v) : "r"(a));
    return v;
}

// Per-lane constants of the operand fetch and of the limb recombination.  Lane (g, t) FEEDS the limb column g of the
// MMA (limb g%4 of sequence g/4 of the n-tile) and HOLDS the accumulator columns 2t, 2t+1 (limbs 0,1 or 2,- of
// sequence t/2).
template <int NT>
struct LaneX {
    int boff[NT];    // operand offset of the sequence the lane feeds: b * NB * block bytes
    int soff[NT];    // operand offset of the sequence the lane holds
    int coff[4];     // offset of the lane's chunk q inside nat / perm: j*256 + t*64 + ((q ^ key) << 4)
    int xoff;        // (j4*4 + t)*4 inside xs32 / xs16
    float wA, wB;    // weights of the two accumulator columns: limbs (0,1) -> (1, 256); limbs (2,-) -> (65536, 0)
    float vA, vB;    // the same for the four limbs of the sums: (1, 256) or (65536, 16777216)
    int g, t;
};

// `tile` is the shared-memory address of a ring slot (layout.cuh), `xs` the shared-memory address of the operand
// blocks of this 256-column slice (sequence 0).
// ── Q4_K ─────────────────────────────────────────────────────────────────────────────────
template <int XT, int NT>
__device__ __forceinline__ void qcompute12(uint32_t tile, uint32_t xs, int lane, const LaneX<NT> &L, float (&facc)[NT][2]) {
    using B = XBlk<XT>;
    int lo[NT][4], hi[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) lo[nt][i] = hi[nt][i] = 0;
    const uint32_t ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
    const uint32_t hdrA = tile + 64 + L.g * 16, hdrB = hdrA + 128;  // (scale, scale, min, min) words of rows g, g+8
#pragma unroll
    for (int g4 = 0; g4 < 4; g4++) {
        // word x = row g k 4t.., y = row g k 16+4t.., z, w = the same of row g+8
        const uint4 w = lds128(tile + kQ4KQsOff + (g4 * 32 + lane) * 16);
        // lo nibbles: sub-block 2*g4; hi nibbles, left in place (16*q as an unsigned byte): sub-block 2*g4+1
        const uint32_t l0 = w.x & ML, l1 = w.z & ML, l2 = w.y & ML, l3 = w.w & ML;
        const uint32_t h0 = w.x & MH, h1 = w.z & MH, h2 = w.y & MH, h3 = w.w & MH;
        const uint32_t wa = lds32(hdrA + g4 * 4), wb = lds32(hdrB + g4 * 4);
        const int sa0 = ubyte(wa, 0), sa1 = ubyte(wa, 1), sb0 = ubyte(wb, 0), sb1 = ubyte(wb, 1);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint4 bb = lds128(xs + L.boff[nt] + B::nat_off + L.coff[g4]);
            int c[4];
            imma_k32_u8s8(c, l0, l1, l2, l3, bb.x, bb.y);
            lo[nt][0] += sa0 * c[0]; lo[nt][1] += sa0 * c[1]; lo[nt][2] += sb0 * c[2]; lo[nt][3] += sb0 * c[3];
            imma_k32_u8s8(c, h0, h1, h2, h3, bb.z, bb.w);
            hi[nt][0] += sa1 * c[0]; hi[nt][1] += sa1 * c[1]; hi[nt][2] += sb1 * c[2]; hi[nt][3] += sb1 * c[3];
        }
    }
    const uint32_t dm0 = lds32(tile + L.g * 4), dm1 = lds32(tile + (L.g + 8) * 4);
    // d/16: the accumulators below carry 16x the sum (lo*16 + hi)
    const float d_a = h2f(dm0) * 0.0625f, dmin_a = h2f(dm0 >> 16), d_b = h2f(dm1) * 0.0625f, dmin_b = h2f(dm1 >> 16);
    const uint32_t ma = lds32(hdrA + L.t * 4), mb = lds32(hdrB + L.t * 4);
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const float sx = __uint_as_float(lds32(xs + L.soff[nt] + B::scale_off));
        int cm[4];
        imma_k16_u8s8(cm, ma, mb, lds32(xs + L.boff[nt] + B::xs32_off + L.xoff));
        const float f0 = (float)(lo[nt][0] * 16 + hi[nt][0]), f1 = (float)(lo[nt][1] * 16 + hi[nt][1]);
        const float f2 = (float)(lo[nt][2] * 16 + hi[nt][2]), f3 = (float)(lo[nt][3] * 16 + hi[nt][3]);
        const float pa = fmaf(f1, L.wB, f0 * L.wA), pb = fmaf(f3, L.wB, f2 * L.wA);
        const float qa = fmaf((float)cm[1], L.vB, (float)cm[0] * L.vA), qb = fmaf((float)cm[3], L.vB, (float)cm[2] * L.vA);
        facc[nt][0] += sx * (d_a * pa - dmin_a * qa);
        facc[nt][1] += sx * (d_b * pb - dmin_b * qb);
    }
}

// ── Q6_K ─────────────────────────────────────────────────────────────────────────────────
template <int XT, int NT>
__device__ __forceinline__ void qcompute14(uint32_t tile, uint32_t xs, int lane, const LaneX<NT> &L, float (&facc)[NT][2]) {
    using B = XBlk<XT>;
    int tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) tot[nt][i] = 0;
    const uint32_t NIB = 0x0F0F0F0Fu, HI = 0x30303030u;
    const uint32_t scA = tile + 3072 + L.g * 16, scB = scA + 128;  // the 16 int8 scales of rows g, g+8
#pragma unroll
    for (int m = 0; m < 4; m++) {
        const uint4 ql = lds128(tile + (m * 32 + lane) * 16);
        const uint32_t WA_r = ql.x, WB_r = ql.y, WA_q = ql.z, WB_q = ql.w;
        const uint2 hq = (m & 1) ? make_uint2(lds32(tile + 2048 + ((m >> 1) * 32 + lane) * 16 + 4), lds32(tile + 2048 + ((m >> 1) * 32 + lane) * 16 + 12))
                                 : make_uint2(lds32(tile + 2048 + ((m >> 1) * 32 + lane) * 16), lds32(tile + 2048 + ((m >> 1) * 32 + lane) * 16 + 8));
        const uint32_t H_r = hq.x, H_q = hq.y;
        uint32_t V_r[4], V_q[4];  // four unsigned 6-bit values (q + 32) per word, for the 16-column groups 4m+0..3
        V_r[0] = (WA_r & NIB) | (H_r & HI);
        V_r[1] = ((WA_r >> 4) & NIB) | ((H_r >> 2) & HI);
        V_r[2] = (WB_r & NIB) | ((H_r << 2) & HI);
        V_r[3] = ((WB_r >> 4) & NIB) | ((H_r << 4) & HI);
        V_q[0] = (WA_q & NIB) | (H_q & HI);
        V_q[1] = ((WA_q >> 4) & NIB) | ((H_q >> 2) & HI);
        V_q[2] = (WB_q & NIB) | ((H_q << 2) & HI);
        V_q[3] = ((WB_q >> 4) & NIB) | ((H_q << 4) & HI);
        const uint32_t sa = lds32(scA + m * 4), sb = lds32(scB + m * 4);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint4 bb = lds128(xs + L.boff[nt] + B::perm_off + L.coff[m]);
            const uint32_t bw[4] = {bb.x, bb.y, bb.z, bb.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                int c[4];
                imma_k16_u8s8(c, V_r[k], V_q[k], bw[k]);
                const int s_r = sbyte(sa, k), s_q = sbyte(sb, k);
                tot[nt][0] += s_r * c[0]; tot[nt][1] += s_r * c[1]; tot[nt][2] += s_q * c[2]; tot[nt][3] += s_q * c[3];
            }
        }
    }
    const float d_a = h2f(lds16(tile + 3328 + L.g * 2)), d_b = h2f(lds16(tile + 3328 + (L.g + 8) * 2));
    const uint32_t ca = lds32(scA + L.t * 4), cb = lds32(scB + L.t * 4);
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const float sx = __uint_as_float(lds32(xs + L.soff[nt] + B::scale_off));
        int co[4];  // sum over 16-column groups of scale * sum(q): the offset of 32 in every 6-bit value
        imma_k16_s8s8(co, ca, cb, lds32(xs + L.boff[nt] + B::xs16_off + L.xoff));
        const float pa = fmaf((float)tot[nt][1], L.wB, (float)tot[nt][0] * L.wA), pb = fmaf((float)tot[nt][3], L.wB, (float)tot[nt][2] * L.wA);
        const float qa = fmaf((float)co[1], L.vB, (float)co[0] * L.vA), qb = fmaf((float)co[3], L.vB, (float)co[2] * L.vA);
        facc[nt][0] += (sx * d_a) * fmaf(qa, -32.f, pa);
        facc[nt][1] += (sx * d_b) * fmaf(qb, -32.f, pb);
    }
}

// ── Q8_0 ─────────────────────────────────────────────────────────────────────────────────
template <int XT, int NT>
__device__ __forceinline__ void qcompute8(uint32_t tile, uint32_t xs, int lane, const LaneX<NT> &L, float (&facc)[NT][2]) {
    using B = XBlk<XT>;
    float fa[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) fa[nt][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint4 w = lds128(tile + (j * 32 + lane) * 16);  // x = row g k 4t.., y = row g k 16+4t.., z, w = row g+8
        const float d_a = h2f(lds16(tile + 4096 + L.g * 16 + j * 2)), d_b = h2f(lds16(tile + 4096 + (L.g + 8) * 16 + j * 2));
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint32_t ba = xs + L.boff[nt] + B::nat_off + L.coff[j >> 1] + (j & 1) * 8;
            int c[4];
            imma_k32_s8s8(c, w.x, w.z, w.y, w.w, lds32(ba), lds32(ba + 4));
            fa[nt][0] = fmaf(d_a, (float)c[0], fa[nt][0]);
            fa[nt][1] = fmaf(d_a, (float)c[1], fa[nt][1]);
            fa[nt][2] = fmaf(d_b, (float)c[2], fa[nt][2]);
            fa[nt][3] = fmaf(d_b, (float)c[3], fa[nt][3]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const float sx = __uint_as_float(lds32(xs + L.soff[nt] + B::scale_off));
        facc[nt][0] += sx * fmaf(fa[nt][1], L.wB, fa[nt][0] * L.wA);
        facc[nt][1] += sx * fmaf(fa[nt][3], L.wB, fa[nt][2] * L.wA);
    }
}

template <int TYPE, int NT>
__device__ __forceinline__ void qcompute(int type, uint32_t tile, uint32_t xs, int lane, const LaneX<NT> &L, float (&facc)[NT][2]) {
    if constexpr (TYPE == 12)
        qcompute12<TYPE, NT>(tile, xs, lane, L, facc);
    else if constexpr (TYPE == 14)
        qcompute14<TYPE, NT>(tile, xs, lane, L, facc);
    else if constexpr (TYPE == 8)
        qcompute8<TYPE, NT>(tile, xs, lane, L, facc);
    else if (type == 12)  // launches that mix Q4_K and Q6_K row tiles: warp-uniform branch
        qcompute12<TYPE, NT>(tile, xs, lane, L, facc);
    else
        qcompute14<TYPE, NT>(tile, xs, lane, L, facc);
}

// ───────────────────────────── building the operand ───────────────────────────────────────
// Packs byte `j` of four biased integers into one word and removes the bias (byte ^ 0x80 is the signed limb).
__device__ __forceinline__ uint32_t pack_limb(uint32_t a, uint32_t b, uint32_t c, uint32_t d, int j) {
    const uint32_t sel = (uint32_t)j | ((uint32_t)(4 + j) << 4);
    const uint32_t lo = __byte_perm(a, b, sel), hi = __byte_perm(c, d, sel);
    return __byte_perm(lo, hi, 0x5410) ^ 0x80808080u;
}

// Where the input rows of a product come from (a register-resident copy of the launch parameters that matter here).
struct QSrc {
    const float *x;
    const float *add0, *add1, *add2, *add3, *add4, *add5, *add6, *add7;  // partial products to add, null from the first unused one on
    const float *normw;
    float *x_store;
    int ldx;
    unsigned tag;      // non-zero: the addends are (value, step number) pairs stored by other GPUs; wait for this number
    unsigned *failed;  // the word a wait that ran out sets (later waits give up at once), and the error word
    unsigned *err;
};
// The eight values of one lane (columns sb*256 + lane*8 .. +7 of row b) on their way to the operand.
struct QIn {
    float v[8];   // residual row (or the plain input)
    float s[8];   // sum of the partial products to add
};
__device__ __forceinline__ void ld8(const float *p, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p), c = *reinterpret_cast<const float4 *>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = c.x; o[5] = c.y; o[6] = c.z; o[7] = c.w;
}
// A wait for another rank's partial products gives up after about a second (the rank may have failed).
constexpr long long kQPeerWaitLimitClk = 2000000000ll;
// Eight (value, step number) pairs that another GPU stores with one 8-byte store each: the data is its own flag, so
// the consumer needs no fence and no separate signal - it re-reads until every pair carries this step's number.  The
// wait is bounded; a wait that runs out sets the failure word, which ends every later wait at once.
__device__ __forceinline__ uint4 ld_pairs(const uint4 *p) {
    uint4 r;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void st_pair(float *slot, size_t idx, float v, unsigned tag) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | ((unsigned long long)tag << 32);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long *>(slot) + idx), "l"(w) : "memory");
}
__device__ __forceinline__ void ld4_tagged(const uint4 *p, unsigned want, unsigned *failed, unsigned *err, unsigned code, float *o) {
    uint4 a, b;
    long long t0 = 0;
    for (int spin = 0;; spin++) {
        a = ld_pairs(p);
        b = ld_pairs(p + 1);
        if (a.y == want && a.w == want && b.y == want && b.w == want) break;
        if (*reinterpret_cast<volatile unsigned *>(failed) != 0u) break;
        if (spin == 0) {
            t0 = clock64();
        } else if (clock64() - t0 > kQPeerWaitLimitClk) {  // about a second: the rank may have failed
            *reinterpret_cast<volatile unsigned *>(failed) = 1u;
            *reinterpret_cast<volatile unsigned *>(err) = code;
            break;
        }
    }
    o[0] = __uint_as_float(a.x);
    o[1] = __uint_as_float(a.z);
    o[2] = __uint_as_float(b.x);
    o[3] = __uint_as_float(b.z);
}
__device__ __forceinline__ void ld8_tagged(const float *slot, size_t idx, unsigned want, unsigned *failed, unsigned *err, unsigned code,
                                           float (&o)[8]) {
    const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint2 *>(slot) + idx);
    ld4_tagged(p, want, failed, err, code, o);
    ld4_tagged(p + 2, want, failed, err, code, o + 4);
}
// Issues the loads of one (row, slice) pair; nothing here waits for them (unless there are several addends).
template <bool TAGGED>
__device__ __forceinline__ void quantize_fetch(const QSrc &q, int b, int sb, int lane, QIn &in) {
    const size_t roff = (size_t)b * q.ldx + sb * 256 + lane * 8;
    ld8(q.x + roff, in.v);
    if (q.add0) {
        // partial products are summed first, in the order given (TensorParallelPipelineClient.allReduceSum :244-272 adds
        // rank 0..N-1), then added to the residual row (LlamaTransformerHandler.add :1738-1743)
        if (TAGGED)
            ld8_tagged(q.add0, roff, q.tag, q.failed, q.err, 3u, in.s);
        else
            ld8(q.add0 + roff, in.s);
        const float *more[7] = {q.add1, q.add2, q.add3, q.add4, q.add5, q.add6, q.add7};
#pragma unroll
        for (int k = 0; k < 7; k++) {
            if (!more[k]) break;
            float t[8];
            if (TAGGED)
                ld8_tagged(more[k], roff, q.tag, q.failed, q.err, 3u | ((unsigned)(k + 1) << 8), t);
            else
                ld8(more[k] + roff, t);
#pragma unroll
            for (int i = 0; i < 8; i++) in.s[i] = __fadd_rn(in.s[i], t[i]);
        }
    }
}

// nw: the RMSNorm weights of the lane's columns.
template <int TYPE>
__device__ __forceinline__ void quantize_slice(const QSrc &q, int b, int sb, int lane, const QIn &in, const float (&nw)[8],
                                               uint8_t *blk, float &ss_out) {
    using B = XBlk<TYPE>;
    const int c0 = sb * 256 + lane * 8;
    const size_t roff = (size_t)b * q.ldx + c0;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = in.v[i];
    if (q.add0) {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fadd_rn(v[i], in.s[i]);
    }
    if (q.x_store && blockIdx.x == 0) {
        float *dst = q.x_store + roff;
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (q.normw) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) ss = fmaf(v[i], v[i], ss);
        ss_out += ss;
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(nw[i], v[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // amax < 2^(E-126); q = round(v * 2^(148-E)) has |q| <= 2^22
    int E = (int)(__float_as_uint(amax) >> 23);
    E = min(max(E, 21), 254);
    const float inv_s = __uint_as_float((uint32_t)(275 - E) << 23), s = __uint_as_float((uint32_t)(E - 21) << 23);
    uint32_t tq[8];
    int sum8 = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int q = __float2int_rn(v[i] * inv_s);
        sum8 += q;
        tq[i] = (uint32_t)(q + 0x808080);
    }
    // words of the lane: 32-column sub-block sub = lane/4, k = 8*(lane%4) .. +7
    const int sub = lane >> 2, tp = lane & 3, wsel = tp >> 1, tt = (tp & 1) << 1;
    const int q4 = sub >> 1, wic = ((sub & 1) << 1) | wsel;
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const uint32_t w0 = pack_limb(tq[0], tq[1], tq[2], tq[3], j), w1 = pack_limb(tq[4], tq[5], tq[6], tq[7], j);
        const int o0 = j * 256 + tt * 64 + ((q4 ^ swz_key(tt, j)) << 4) + wic * 4;
        const int o1 = j * 256 + (tt + 1) * 64 + ((q4 ^ swz_key(tt + 1, j)) << 4) + wic * 4;
        if (B::kNat) {
            *reinterpret_cast<uint32_t *>(blk + B::nat_off + o0) = w0;
            *reinterpret_cast<uint32_t *>(blk + B::nat_off + o1) = w1;
        }
        if (B::kPerm) {
            *reinterpret_cast<uint32_t *>(blk + B::perm_off + o0) = __byte_perm(w0, 0, 0x3120);
            *reinterpret_cast<uint32_t *>(blk + B::perm_off + o1) = __byte_perm(w1, 0, 0x3120);
        }
    }
    // sums over 16 and 32 columns (exact integers, |S32| <= 2^27)
    const int s16 = sum8 + __shfl_xor_sync(0xffffffffu, sum8, 1);
    if (B::kXs16) {
        // lane 8t collects the sums of the 16-column groups 4t..4t+3 (lanes 8t, 8t+2, 8t+4, 8t+6)
        const uint32_t a = (uint32_t)s16 + 0x80808080u;
        const uint32_t b1 = __shfl_down_sync(0xffffffffu, a, 2), c1 = __shfl_down_sync(0xffffffffu, a, 4), d1 = __shfl_down_sync(0xffffffffu, a, 6);
        if ((lane & 7) == 0) {
            const int t = lane >> 3;
#pragma unroll
            for (int j = 0; j < 4; j++) *reinterpret_cast<uint32_t *>(blk + B::xs16_off + (j * 4 + t) * 4) = pack_limb(a, b1, c1, d1, j);
        }
    }
    if (B::kXs32) {
        const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
        const uint32_t a = (uint32_t)s32 + 0x80808080u;
        const uint32_t b1 = __shfl_down_sync(0xffffffffu, a, 4);  // the odd sub-block of the pair
        if ((lane & 7) == 0) {
            const int t = lane >> 3;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t sel = ((uint32_t)j << 8) | ((uint32_t)(4 + j) << 12);  // bytes 2, 3 = a.byte j, b1.byte j
                *reinterpret_cast<uint32_t *>(blk + B::xs32_off + (j * 4 + t) * 4) = (__byte_perm(a, b1, sel) ^ 0x80800000u) & 0xFFFF0000u;
            }
        }
    }
    if (lane == 0) *reinterpret_cast<float *>(blk + B::scale_off) = s;
}

// ───────────────────────────── the kernel ─────────────────────────────────────────────────
__device__ __forceinline__ int qseg_of(const QParams &p, int R) {
    int s = 0;
    if (p.nseg > 1 && R >= p.rt_begin[1]) s = 1;
    if (p.nseg > 2 && R >= p.rt_begin[2]) s = 2;
    return s;
}
template <int TYPE>
__device__ __forceinline__ const uint8_t *qtile_addr(const QParams &p, int R, int sb, int &type) {
    const int s = qseg_of(p, R);
    type = (TYPE == 0) ? p.seg_type[s] : TYPE;
    return p.w[s] + ((size_t)(R - p.rt_begin[s]) * p.NB + sb) * (size_t)tile_bytes(type);
}

// ── mbarrier / bulk-copy primitives ──────────────────────────────────────────────────────
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One attempt.  ns == 0: a plain test.  Otherwise the hardware may park the warp for up to about `ns` nanoseconds when
// the phase is not complete yet (fewer issue slots than polling, but it wakes late when the hint is long).
__device__ __forceinline__ bool mbar_test(uint32_t bar, unsigned parity, unsigned ns) {
    unsigned ok;
    if (ns == 0)
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
    else
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(ns)
            : "memory");
    return ok != 0;
}
// Weight tiles are read once per step: they are requested with the evict-first policy, so that the gigabytes streamed
// through the L2 do not push out what every kernel start needs again (activations, norm weights, instructions).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, unsigned bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(pol)
                 : "memory");
}
// A wait on a weight tile gives up after this many SM cycles (about a fifth of a second); after the first give-up
// of a warp its later waits are short, so that the kernel still drains the copies it has in flight and returns.
constexpr long long kQWaitLimitClk = 400000000ll, kQWaitLimitAfterFail = 2000000ll;
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, unsigned parity, unsigned ns, unsigned *err, bool &failed) {
    if (mbar_test(bar, parity, 0)) return;
    const long long t0 = clock64(), limit = failed ? kQWaitLimitAfterFail : kQWaitLimitClk;
    while (!mbar_test(bar, parity, ns)) {
        if (clock64() - t0 > limit) {
            if (!failed && (threadIdx.x & 31) == 0) *reinterpret_cast<volatile unsigned *>(err) = 1u | ((threadIdx.x >> 5) << 8) | (blockIdx.x << 16);
            failed = true;
            return;
        }
    }
}

constexpr int kQBufs = 2;  // buffers of partial sums (one CTA barrier per chunk)

// A CTA owns the row tiles [c * RT / grid, (c+1) * RT / grid) and walks them in chunks of at most kQChunk row tiles.
// Inside a chunk the tiles (row tile, 256-column block) form one flat sequence of T = row tiles x NB tiles, which is
// also one contiguous stretch of memory; warp w takes the tiles [w*T/16, (w+1)*T/16).  So the sixteen warps carry the
// same load whatever the shape (no power-of-two split of K, no idle warps), and because a warp's share is at most NB
// tiles long it touches at most two row tiles, whose partial sums it leaves in two slots of shared memory.
struct QCursor {
    int k;        // chunk
    int f, fend;  // flat tile range still to request inside chunk k
    int R, sb;    // row tile and block of tile f
};

// TAGGED: the addends are (value, step number) pairs from other GPUs (a kernel of its own, so that the polling loads
// cost the single-GPU kernels no registers).
template <int TYPE, int NT, int OCC, bool TAGGED>
__global__ void __launch_bounds__(kQThreads, OCC) qgemv_kernel(const QParams p) {
    using B = XBlk<TYPE>;
    constexpr int NSEQ = 2 * NT;
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NB = p.NB;
    // [ring: 16 warps x ring x slot_bytes][operand: bc x NB blocks][partials: kQBufs x 16 warps x 2 row tiles x 16 rows x NSEQ][ssw][rs][mbarriers]
    const size_t ring_bytes = (size_t)kQWarps * p.ring * p.slot_bytes;
    uint8_t *xop = smem + ring_bytes;
    float *red = reinterpret_cast<float *>(xop + (size_t)p.bc * NB * B::bytes);
    float *ssw = red + kQBufs * kQWarps * 2 * 16 * NSEQ;  // [16 warps][8] sums of squares of the slices a warp converted
    float *rs_s = ssw + kQWarps * 8;                  // [8] 1/rms per sequence
    const uint32_t my_ring = smem_u32(smem) + (uint32_t)(warp * p.ring * p.slot_bytes);
    int *wr_s = reinterpret_cast<int *>(rs_s + 16);   // [kQBufs][kQChunk] first | last << 8 warp of a row tile of the chunk
    const uint32_t my_bars = smem_u32(wr_s + kQBufs * kQChunk) + (uint32_t)(warp * p.ring * 8);

    int rt0, rtc;
    qsplit_cta((int)blockIdx.x, (int)gridDim.x, p.total_rt, rt0, rtc);
    const int n_chunks = qsplit_chunks(rtc);
    auto chunk_lo = [&](int k) { return qsplit_chunk_lo(rt0, rtc, n_chunks, k); };

    // Fill the ring: weights do not depend on the producer of x.  Lane 0 owns the warp's barriers and copies.
    QCursor pc{0, 0, 0, 0, 0};
    const uint8_t *pc_src = nullptr;  // source of the next copy
    unsigned pc_bytes = 0;
    bool pc_fresh = true;             // the address has to be worked out (first tile of a chunk or of a row tile)
    auto cursor_seek = [&](int k) {   // first chunk from k on in which this warp has tiles
        for (; k < n_chunks; k++) {
            const int lo = chunk_lo(k), T = (chunk_lo(k + 1) - lo) * NB;
            int f0, f1;
            qsplit_warp(warp, T, f0, f1);
            if (f0 < f1) {
                const int l = f0 / NB;
                pc = QCursor{k, f0, f1, lo + l, f0 - l * NB};
                pc_fresh = true;
                return;
            }
        }
        pc.k = n_chunks;
    };
    const uint64_t l2_pol = l2_evict_first_policy();
    auto produce = [&](int slot) {  // lane 0 only
        if (pc.k >= n_chunks) return;
        if (pc_fresh) {  // consecutive tiles of a row tile are contiguous; the next row tile may belong to another matrix
            int ty;
            pc_src = qtile_addr<TYPE>(p, pc.R, pc.sb, ty);
            pc_bytes = (unsigned)tile_bytes(ty);
            pc_fresh = false;
        }
        mbar_expect_tx(my_bars + slot * 8, pc_bytes);
        bulk_g2s(my_ring + slot * p.slot_bytes, pc_src, pc_bytes, my_bars + slot * 8, l2_pol);
        pc_src += pc_bytes;
        if (++pc.f == pc.fend) {
            cursor_seek(pc.k + 1);
        } else if (++pc.sb == NB) {
            pc.sb = 0;
            pc.R++;
            pc_fresh = true;
        }
    };
    if (lane == 0) cursor_seek(0);
    if (lane == 0) {
        for (int sl = 0; sl < p.ring; sl++) mbar_init(my_bars + sl * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");
        for (int sl = 0; sl < p.ring; sl++) produce(sl);
    }
    __syncwarp();

    // The RMSNorm weights are model data: those of the warp's first slice are requested before the wait, so that their
    // trip to DRAM overlaps the end of the producing kernel.
    float w8[8];
    if (p.normw && warp < p.bc * NB) ld8(p.normw + (warp % NB) * 256 + lane * 8, w8);
    pdl_wait();  // everything below reads what earlier kernels of the stream wrote
    bool failed = false;
    const unsigned step_no = (p.tagged_adds || p.n_peers) ? *reinterpret_cast<const volatile unsigned *>(p.epoch) : 0u;
    if (TAGGED && p.n_red > 0 && warp == 0) {
        // The first CTAs add the ranks' partial products of one (sequence, slice) each, in rank order, and publish the
        // sums as (value, step number) pairs; all CTAs (these too) then poll one vector instead of n_red.
        for (int pr = blockIdx.x; pr < p.bc * NB; pr += gridDim.x) {
            const int b = pr / NB, sb = pr - b * NB;
            const size_t roff = (size_t)b * p.ldx + sb * 256 + lane * 8;
            float acc[8];
            ld8_tagged(p.red_src[0], roff, step_no, p.peer_failed, p.err, 3u, acc);
            for (int k = 1; k < p.n_red; k++) {
                float t[8];
                ld8_tagged(p.red_src[k], roff, step_no, p.peer_failed, p.err, 3u | ((unsigned)k << 8), t);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[i] = __fadd_rn(acc[i], t[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) st_pair(p.red_dst, roff + i, acc[i], step_no);
        }
    }
    // operand: every warp converts (sequence, slice) pairs warp, warp+16, ...
    {
        const QSrc q{p.x, p.n_add > 0 ? p.add[0] : nullptr, p.n_add > 1 ? p.add[1] : nullptr, p.n_add > 2 ? p.add[2] : nullptr, p.n_add > 3 ? p.add[3] : nullptr,
                     p.n_add > 4 ? p.add[4] : nullptr, p.n_add > 5 ? p.add[5] : nullptr, p.n_add > 6 ? p.add[6] : nullptr, p.n_add > 7 ? p.add[7] : nullptr,
                     p.normw, p.x_store, p.ldx, p.tagged_adds ? step_no : 0u, p.peer_failed, p.err};
        float ss[8];
#pragma unroll
        for (int b = 0; b < 8; b++) ss[b] = 0.f;
        const int pairs = p.bc * NB;
        for (int pr = warp; pr < pairs; pr += kQWarps) {
            const int b = pr / NB, sb = pr - b * NB;
            QIn t;
            quantize_fetch<TAGGED>(q, b, sb, lane, t);
            if (q.normw && pr != warp) ld8(q.normw + sb * 256 + lane * 8, w8);
            float part = 0.f;
            quantize_slice<TYPE>(q, b, sb, lane, t, w8, xop + (size_t)pr * B::bytes, part);
#pragma unroll
            for (int bb = 0; bb < 8; bb++)
                if (bb == b) ss[bb] += part;
        }
        if (p.normw) {
            for (int b = 0; b < p.bc; b++) {
                float s = 0.f;
#pragma unroll
                for (int bb = 0; bb < 8; bb++)
                    if (bb == b) s = ss[bb];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) ssw[warp * 8 + b] = s;
            }
        }
    }
    __syncthreads();
    if (tid < 8) {
        float sc = 1.f;
        if (p.normw) {
            float s = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < kQWarps; w8++) s += ssw[w8 * 8 + tid];
            // rmsNorm (:818-828): 1f / (float) Math.sqrt(ss / n + eps)
            // (float) Math.sqrt((double) v) is the correctly rounded single-precision root of v: 53 bits are more than
            // twice 24 + 2, so the second rounding cannot change the result
            sc = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s, (float)p.K), p.eps)));
        }
        rs_s[tid] = sc;  // read when the outputs of a chunk are finished: ordered by the chunk barrier
    }

    LaneX<NT> L;
    {
        const int g = lane >> 2, t = lane & 3, j4 = g & 3, j = min(j4, 2);
        L.g = g;
        L.t = t;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            L.boff[nt] = min(2 * nt + (g >> 2), p.bc - 1) * NB * B::bytes;
            L.soff[nt] = min(2 * nt + (t >> 1), p.bc - 1) * NB * B::bytes;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) L.coff[q] = j * 256 + t * 64 + ((q ^ swz_key(t, j)) << 4);
        L.xoff = (j4 * 4 + t) * 4;
        L.wA = (t & 1) ? 65536.f : 1.f;
        L.wB = (t & 1) ? 0.f : 256.f;
        L.vA = L.wA;
        L.vB = (t & 1) ? 16777216.f : 256.f;
    }

    float facc[NT][2];
    const uint32_t xop_s = smem_u32(xop);
    int slot = 0;
    unsigned parity = 0;
    for (int k = 0; k < n_chunks; k++) {
        const int lo = chunk_lo(k), crt = chunk_lo(k + 1) - lo, T = crt * NB;
        int f0, f1;
        qsplit_warp(warp, T, f0, f1);
        const int l_first = f0 / NB;
        float *cred = red + (size_t)(k & (kQBufs - 1)) * (kQWarps * 2 * 16 * NSEQ);
        float *myred = cred + warp * (2 * 16 * NSEQ);
        int f = f0;
#pragma unroll 1
        for (int j = 0; j < 2; j++) {  // the (at most two) row tiles this warp's tiles belong to
            const int l = l_first + j, fe = min(f1, (l + 1) * NB);
            if (f >= fe) continue;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) facc[nt][0] = facc[nt][1] = 0.f;
            const int type = (TYPE == 0) ? p.seg_type[qseg_of(p, lo + l)] : TYPE;
            for (int sb = f - l * NB; f < fe; f++, sb++) {
                mbar_wait_bounded(my_bars + slot * 8, parity, (unsigned)p.wait_ns, p.err, failed);
                qcompute<TYPE, NT>(type, my_ring + slot * p.slot_bytes, xop_s + (uint32_t)(sb * B::bytes), lane, L, facc);
                __syncwarp();  // every lane has used the slot's bytes before lane 0 overwrites them
                if (lane == 0) produce(slot);
                if (++slot == p.ring) {
                    slot = 0;
                    parity ^= 1u;
                }
            }
            // lanes t and t^1 hold the two halves (limbs 0,1 / limb 2) of a (row, sequence) value
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float a = facc[nt][0] + __shfl_xor_sync(0xffffffffu, facc[nt][0], 1);
                const float c = facc[nt][1] + __shfl_xor_sync(0xffffffffu, facc[nt][1], 1);
                if ((lane & 1) == 0) {
                    const int seq = 2 * nt + (L.t >> 1);
                    myred[(j * 16 + L.g) * NSEQ + seq] = a;
                    myred[(j * 16 + L.g + 8) * NSEQ + seq] = c;
                }
            }
        }
        if (tid < crt) {  // the warps whose tiles reach into row tile `tid` of the chunk
            int w_lo, w_hi;
            qsplit_row_tile_warps(tid, NB, T, w_lo, w_hi);
            wr_s[(k & (kQBufs - 1)) * kQChunk + tid] = w_lo | (w_hi << 8);
        }
        // One CTA barrier per chunk.  Two buffers of partial sums: a buffer is rewritten two barriers later, when every
        // thread has finished reading it.
        __syncthreads();
        // K spans of a row in warp order (a fixed order: results are bitwise repeatable), then the output transform
        const int rows_sh = (p.epi == QEPI_SILU_PAIR) ? 3 : 4, rows_out = 1 << rows_sh;
        const int per_b = crt << rows_sh, total = per_b * p.bc;
        for (int idx = tid; idx < total; idx += kQThreads) {
            const int b = (p.bc == 1) ? 0 : idx / per_b, rg = idx - b * per_b, l = rg >> rows_sh, row = rg & (rows_out - 1);
            const int tlo = l * NB, wr = wr_s[(k & (kQBufs - 1)) * kQChunk + l];
            float v = 0.f, v2 = 0.f;
            for (int w = wr & 255; w <= (wr >> 8); w++) {
                int wf0, wf1;
                qsplit_warp(w, T, wf0, wf1);
                if (wf0 >= wf1) continue;  // with fewer than sixteen tiles in the chunk some warps have none
                // a warp that started in the row tile before has this one in its second slot
                const float *cr = cred + w * (2 * 16 * NSEQ) + (wf0 < tlo ? 16 * NSEQ : 0) + b;
                v += cr[row * NSEQ];
                if (p.epi == QEPI_SILU_PAIR) v2 += cr[(row + 8) * NSEQ];
            }
            const int Rg = lo + l;
            const int s = qseg_of(p, Rg);
            const int orow = (Rg - p.rt_begin[s]) * rows_out + row;
            if (orow >= p.rows[s]) continue;
            const float sc = rs_s[b];
            v = __fmul_rn(v, sc);
            if (p.epi == QEPI_SILU_PAIR) v = __fmul_rn(silu_f(v), __fmul_rn(v2, sc));
            if (p.n_peers) {
                // one 8-byte (value, step number) store per rank over NVLink: the consumer polls the data itself
                for (int d = 0; d < p.n_peers; d++) st_pair(p.peer_out[d], (size_t)b * p.ld_out + orow, v, step_no);
            } else {
                p.out[s][(size_t)b * p.ld_out + orow] = v;
            }
        }
    }
}

// ───────────────────────────── host: launch ───────────────────────────────────────────────
static int q_env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

constexpr int kQMinRing = 2, kQMaxRing = 6;
static int q_slot_bytes(int type_mix) { return type_mix == 12 ? kQ4KTileBytes : type_mix == 8 ? kQ80TileBytes : kQ6KTileBytes; }
// Shared memory of a launch without its weight ring.
static size_t qgemv_fixed_smem(int K, int type_mix, int bc) {
    const int nt = (bc + 1) / 2;
    return (size_t)bc * (K / 256) * xblk_bytes(type_mix) + (size_t)kQBufs * kQWarps * 2 * 16 * 2 * nt * 4 + (size_t)kQWarps * 8 * 4 + 64 + (size_t)kQBufs * kQChunk * 4 +
           (size_t)kQWarps * kQMaxRing * 8 + 128;
}
// Ring slots per warp that fit when `occ` CTAs share an SM (each CTA also pays 1 KB of system shared memory).
static int qgemv_ring_slots(const juno_ctx *ctx, int K, int type_mix, int bc, int occ = 1) {
    const size_t avail = occ == 1 ? ctx->smem_optin : (ctx->smem_optin + 1024) / occ - 1024;
    const size_t fixed = qgemv_fixed_smem(K, type_mix, bc);
    if (fixed >= avail) return 0;
    const int fit = (int)((avail - fixed) / ((size_t)kQWarps * q_slot_bytes(type_mix)));
    return std::min(fit, kQMaxRing);
}

int qgemv_batch_chunk(const juno_ctx *ctx, int K, int type_mix, int batch) {
    int bc = std::min(batch, 8);
    while (bc > 1 && qgemv_ring_slots(ctx, K, type_mix, bc) < kQMinRing) bc--;
    return bc;
}

template <int TYPE, int NT, int OCC, bool TAGGED>
static int qlaunch_inst(juno_ctx *ctx, const QParams &p, int grid, size_t smem, cudaStream_t st) {
    static std::mutex mu;
    static bool configured[64] = {false};
    {
        std::lock_guard<std::mutex> g(mu);
        const int dev = ctx->device & 63;
        if (!configured[dev]) {
            JUNO_CUDA_TRY(cudaFuncSetAttribute(qgemv_kernel<TYPE, NT, OCC, TAGGED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin));
            configured[dev] = true;
        }
    }
    JUNO_CUDA_TRY(launch_pdl(qgemv_kernel<TYPE, NT, OCC, TAGGED>, dim3(grid), dim3(kQThreads), smem, st, p));
    ctx->kernel_launches++;
    return JUNO_OK;
}
template <int TYPE>
static int qlaunch_type(juno_ctx *ctx, const QParams &p, int occ, int grid, size_t smem, cudaStream_t st) {
    const bool tg = p.tagged_adds != 0;
    switch ((p.bc + 1) / 2) {
    case 1:
        if (occ == 2) return tg ? qlaunch_inst<TYPE, 1, 2, true>(ctx, p, grid, smem, st) : qlaunch_inst<TYPE, 1, 2, false>(ctx, p, grid, smem, st);
        return tg ? qlaunch_inst<TYPE, 1, 1, true>(ctx, p, grid, smem, st) : qlaunch_inst<TYPE, 1, 1, false>(ctx, p, grid, smem, st);
    case 2: return tg ? qlaunch_inst<TYPE, 2, 1, true>(ctx, p, grid, smem, st) : qlaunch_inst<TYPE, 2, 1, false>(ctx, p, grid, smem, st);
    case 3: return tg ? qlaunch_inst<TYPE, 3, 1, true>(ctx, p, grid, smem, st) : qlaunch_inst<TYPE, 3, 1, false>(ctx, p, grid, smem, st);
    case 4: return tg ? qlaunch_inst<TYPE, 4, 1, true>(ctx, p, grid, smem, st) : qlaunch_inst<TYPE, 4, 1, false>(ctx, p, grid, smem, st);
    default: break;
    }
    set_error("qgemv: unsupported batch chunk %d", p.bc);
    return JUNO_ERR_UNSUPPORTED;
}

int launch_qgemv(juno_ctx *ctx, const QGemvArgs &a, cudaStream_t st) {
    JUNO_REQUIRE(a.nseg >= 1 && a.nseg <= 3, "qgemv: nseg %d", a.nseg);
    JUNO_REQUIRE(a.K > 0 && a.K % 256 == 0, "qgemv: K=%d must be a multiple of 256", a.K);
    JUNO_REQUIRE(a.batch >= 1 && a.x && a.ldx % 4 == 0 && a.ldx >= a.K, "qgemv: bad activation (batch %d, ldx %d)", a.batch, a.ldx);
    JUNO_REQUIRE(a.n_add >= 0 && a.n_add <= kQMaxAdd, "qgemv: %d addends", a.n_add);
    int type_mix = a.seg[0].type, total_rt = 0;
    for (int s = 0; s < a.nseg; s++) {
        const int t = a.seg[s].type;
        JUNO_REQUIRE(t == 12 || t == 14 || t == 8, "qgemv: type %d has no tiled kernel", t);
        if (t != type_mix) type_mix = 0;
        total_rt += a.seg[s].row_tiles;
    }
    if (type_mix == 0)
        for (int s = 0; s < a.nseg; s++) JUNO_REQUIRE(a.seg[s].type != 8, "qgemv: mixed launches take Q4_K and Q6_K segments only");
    JUNO_REQUIRE(qgemv_ring_slots(ctx, a.K, type_mix, 1) >= kQMinRing, "qgemv: K=%d does not fit shared memory", a.K);

    double algo_bytes = (double)a.batch * a.K * 4;
    int rt = 0;
    QParams p;
    memset(&p, 0, sizeof(p));
    for (int s = 0; s < a.nseg; s++) {
        const int t = a.seg[s].type;
        const double bpw = t == 12 ? 144.0 / 256 : t == 14 ? 210.0 / 256 : 34.0 / 32;
        // every stored row is read: the paired gate/up matrix holds twice the rows it emits
        const double stored_rows = a.epi == QEPI_SILU_PAIR ? 2.0 * a.seg[s].rows : (double)a.seg[s].rows;
        algo_bytes += stored_rows * a.K * bpw + (double)a.batch * a.seg[s].rows * 4;
        p.w[s] = a.seg[s].w;
        p.rows[s] = a.seg[s].rows;
        p.seg_type[s] = t;
        p.rt_begin[s] = rt;
        rt += a.seg[s].row_tiles;
    }
    for (int s = a.nseg; s < 4; s++) p.rt_begin[s] = rt;
    ProfScope prof(ctx, st, (type_mix == 12 || type_mix == 0) ? PROF_GEMV_Q4K : type_mix == 14 ? PROF_GEMV_Q6K : PROF_GEMV_Q80, algo_bytes);
    p.nseg = a.nseg;
    p.total_rt = total_rt;
    p.K = a.K;
    p.NB = a.K / 256;
    const int bc_full = qgemv_batch_chunk(ctx, a.K, type_mix, a.batch);
    // two CTAs per SM (64 registers per thread, half the ring each) when the launch is a single n-tile and still gets a ring
    int occ = q_env_int("JUNO_QGEMV_OCC", 2);
    if (occ != 2 || bc_full > 2 || qgemv_ring_slots(ctx, a.K, type_mix, bc_full, 2) < kQMinRing) occ = 1;
    // one CTA per slot of the GPU, each with its share of the row tiles (never more CTAs than row tiles)
    const int grid = std::max(1, std::min(ctx->sm_count * occ, total_rt));
    p.ld_out = a.ld_out;
    p.epi = a.epi;
    p.ldx = a.ldx;
    p.n_add = a.n_add;
    p.normw = a.normw;
    p.eps = a.eps;
    p.slot_bytes = q_slot_bytes(type_mix);
    p.err = ctx->gemv_scratch.qerr;
    p.wait_ns = q_env_int("JUNO_QGEMV_WAIT_NS", 0);
    p.n_peers = a.n_peers;
    for (int d = 0; d < a.n_peers; d++) {
        p.peer_out[d] = a.peer_out[d];
    }
    p.tagged_adds = a.tagged_adds ? 1 : 0;
    p.n_red = a.tagged_adds ? a.n_red : 0;
    for (int k = 0; k < p.n_red; k++) p.red_src[k] = a.red_src[k];
    p.red_dst = a.red_dst;
    if (p.n_red) JUNO_REQUIRE(a.red_dst && a.n_add == 1 && a.add[0] == a.red_dst, "qgemv: with a pre-reduction the only addend is its result");
    p.epoch = a.epoch;
    p.peer_failed = a.peer_failed;
    if (a.n_peers) JUNO_REQUIRE(a.nseg == 1 && a.epoch && a.epi == QEPI_STORE, "qgemv: a pushed product is one matrix with a plain store");
    if (a.tagged_adds) JUNO_REQUIRE(a.peer_failed && a.epoch && a.n_add > 0, "qgemv: a consumer of pushed products needs the step number and the failure word");
    if (a.n_peers || a.tagged_adds) JUNO_REQUIRE(a.batch <= 8, "qgemv: peer exchange carries at most 8 sequences per launch");
    for (int b0 = 0; b0 < a.batch; b0 += bc_full) {
        p.bc = std::min(bc_full, a.batch - b0);
        for (int s = 0; s < a.nseg; s++) p.out[s] = a.seg[s].out + (size_t)b0 * a.ld_out;
        p.x = a.x + (size_t)b0 * a.ldx;
        for (int k = 0; k < a.n_add; k++) p.add[k] = a.add[k] + (size_t)b0 * a.ldx;
        p.x_store = a.x_store ? a.x_store + (size_t)b0 * a.ldx : nullptr;
        // Two slots per warp, although more would fit: with 16-32 warps per SM the copies in flight already cover the
        // bandwidth-delay product, and every further slot only lengthens the queue in front of the loads of x (the
        // decode step measured 2.5-5 % slower with four to eight slots).
        p.ring = std::max(kQMinRing, std::min(qgemv_ring_slots(ctx, a.K, type_mix, p.bc, occ), q_env_int("JUNO_QGEMV_RING", 2)));
        const size_t smem = qgemv_fixed_smem(a.K, type_mix, p.bc) + (size_t)kQWarps * p.ring * p.slot_bytes;
        int rc;
        if (type_mix == 0)
            rc = qlaunch_type<0>(ctx, p, occ, grid, smem, st);
        else if (type_mix == 12)
            rc = qlaunch_type<12>(ctx, p, occ, grid, smem, st);
        else if (type_mix == 14)
            rc = qlaunch_type<14>(ctx, p, occ, grid, smem, st);
        else
            rc = qlaunch_type<8>(ctx, p, occ, grid, smem, st);
        JUNO_TRY(rc);
    }
    return JUNO_OK;
}

}  // namespace juno
