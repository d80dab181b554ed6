// Register image of one 16x256 weight tile (layout.cuh) and small helpers, shared by the batched dequant-GEMM
// kernels (gemm.cu, gemm_tc.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "layout.cuh"

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

__device__ __forceinline__ float f16bits_to_f32(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)(bits & 0xFFFFu)));
}

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


// Nibbles of one word as four register pairs: (w & mask) | magic in one instruction each.
__device__ __forceinline__ void q4_unpack(uint32_t w, uint32_t M, uint32_t K, uint32_t &lo_a, uint32_t &lo_b,
                                          uint32_t &hi_a, uint32_t &hi_b) {
    lo_a = and_or(w, M, K);        // (byte0.lo, byte2.lo)
    hi_a = and_or(w >> 4, M, K);   // (byte0.hi, byte2.hi)
    lo_b = and_or(w >> 8, M, K);   // (byte1.lo, byte3.lo)
    hi_b = and_or(w >> 12, M, K);  // (byte1.hi, byte3.hi)
}
__device__ __forceinline__ float i8_to_f32(uint32_t w, int k) { return (float)(int)(signed char)((w >> (8 * k)) & 0xFFu); }

}  // namespace juno
