// Bit-exact element dequantisation, shared by the dequantise, embedding and fallback kernels.
// Formulas and rounding order of LlamaTransformerHandler.dequantizeQ4K/Q6K/Q8_0 (:1017-1050,
// :1095-1135, :895-913): every product and difference is rounded separately (no FMA).
#pragma once
#if defined(__CUDACC__)
#include <cuda_fp16.h>
#endif
#include <string.h>

#include "layout.cuh"

#if defined(__CUDACC__)
#define JDQ __host__ __device__ inline
#else
#define JDQ inline
#endif

namespace juno {

JDQ float dq_f16(const uint8_t *p) {
    uint32_t bits = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half((unsigned short)bits));
#else
    // host mirror of GgufReader.f16ToF32 (:1248-1271)
    int s = (bits >> 15) & 1, e = (bits >> 10) & 0x1F, m = bits & 0x3FF;
    uint32_t f;
    if (e == 0) {
        if (m == 0)
            f = (uint32_t)s << 31;
        else {
            int ex = -14;
            while ((m & 0x400) == 0) {
                m <<= 1;
                ex--;
            }
            m &= 0x3FF;
            f = ((uint32_t)s << 31) | ((uint32_t)(ex + 127) << 23) | ((uint32_t)m << 13);
        }
    } else if (e == 31)
        f = ((uint32_t)s << 31) | 0x7F800000u | ((uint32_t)m << 13);
    else
        f = ((uint32_t)s << 31) | ((uint32_t)(e - 15 + 127) << 23) | ((uint32_t)m << 13);
    float o;
    memcpy(&o, &f, 4);
    return o;
#endif
}

#if defined(__CUDA_ARCH__)
#define JMUL(a, b) __fmul_rn((a), (b))
#define JSUB(a, b) __fsub_rn((a), (b))
#else
#define JMUL(a, b) ((a) * (b))
#define JSUB(a, b) ((a) - (b))
#endif

JDQ float tile_elem_value(int type, const uint8_t *tile, int row16, int e) {
    if (type == 12) {
        const uint8_t *dm = tile + row16 * 4;
        float d = dq_f16(dm), dmin = dq_f16(dm + 2);
        int s = e >> 5;
        const uint8_t *sm = tile + 64 + (row16 * 4 + (s >> 1)) * 4;
        float scale = JMUL(d, (float)sm[s & 1]);
        float mn = JMUL(dmin, (float)sm[2 + (s & 1)]);
        int off, hi;
        q4k_elem_loc(row16, e, off, hi);
        int q = hi ? (tile[off] >> 4) : (tile[off] & 15);
        return JSUB(JMUL(scale, (float)q), mn);
    } else if (type == 14) {
        Q6Loc L = q6k_elem_loc(row16, e);
        uint32_t W = (uint32_t)tile[L.w_off] | ((uint32_t)tile[L.w_off + 1] << 8) | ((uint32_t)tile[L.w_off + 2] << 16) |
                     ((uint32_t)tile[L.w_off + 3] << 24);
        uint32_t H = (uint32_t)tile[L.h_off] | ((uint32_t)tile[L.h_off + 1] << 8) | ((uint32_t)tile[L.h_off + 2] << 16) |
                     ((uint32_t)tile[L.h_off + 3] << 24);
        int u6 = (int)((W >> (4 * L.nu)) & 15u) | (int)(((H >> L.h_bit) & 3u) << 4);
        float d = dq_f16(tile + L.d_off);
        float ds = JMUL(d, (float)(int)(signed char)tile[L.sc_off]);
        return JMUL(ds, (float)(u6 - 32));
    } else {
        int off, doff;
        q80_elem_loc(row16, e, off, doff);
        return JMUL(dq_f16(tile + doff), (float)(int)(signed char)tile[off]);
    }
}

#if defined(__CUDACC__)
__device__ inline float raw_elem_value(int type, const uint8_t *rowp, int64_t c) {
    if (type == 0) return reinterpret_cast<const float *>(rowp)[c];
    if (type == 8) {
        const uint8_t *b = rowp + (c >> 5) * 34;
        return __fmul_rn(dq_f16(b), (float)(int)(signed char)b[2 + (c & 31)]);
    }
    if (type == 12) {
        const uint8_t *b = rowp + (c >> 8) * 144;
        int e = (int)(c & 255), s = e >> 5;
        float scale = __fmul_rn(dq_f16(b), (float)q4k_scale6(b + 4, s));
        float mn = __fmul_rn(dq_f16(b + 2), (float)q4k_min6(b + 4, s));
        int byte = b[16 + (e >> 6) * 32 + (e & 31)];
        int q = ((e >> 5) & 1) ? (byte >> 4) : (byte & 15);
        return __fsub_rn(__fmul_rn(scale, (float)q), mn);
    }
    const uint8_t *b = rowp + (c >> 8) * 210;
    int e = (int)(c & 255);
    float ds = __fmul_rn(dq_f16(b + 208), (float)(int)(signed char)b[192 + (e >> 4)]);
    return __fmul_rn(ds, (float)(q6k_raw_u6(b, e) - 32));
}

#endif

}  // namespace juno
