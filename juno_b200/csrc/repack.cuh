// Repack of raw GGUF blocks into the 16x256 tile layout (layout.cuh), one 32-bit output word at a time.
// __host__ __device__: the same index maps drive the device repack kernels (gemv.cu) and the host-side layout
// tests, which build them with the C++ compiler alone.
#pragma once
#include <stdint.h>

#include "layout.cuh"

#if defined(__CUDACC__)
#define JRP __host__ __device__ inline
#else
#define JRP inline
#endif

namespace juno {

// raw: rows [0,nrows) of the source tensor, row stride raw_row_bytes; R: row tile; sb_abs: super-block of the row.
JRP uint32_t q4k_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
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

JRP uint32_t q6k_tile_word(const uint8_t *blk_row /* raw block of (row, sb) or null */, int w,
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

JRP uint32_t q6k_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
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

JRP uint32_t q80_out_word(const uint8_t *raw, size_t raw_row_bytes, int nrows, int sb_abs, int R,
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

}  // namespace juno
