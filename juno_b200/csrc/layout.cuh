// Tile layouts of the resident quantised matrices.
//
// A matrix of GGUF blocks (row-major, rows x cols/256 super-blocks) is repacked at
// upload into TILES of 16 rows x 256 columns.  Tiles are stored [row_tile][super_block]
// so a warp that walks along K for one row tile reads one contiguous stream.  Inside a
// tile the bytes are arranged so that lane L = (r8 = L>>2, c = L&3) of a warp fetches,
// with 128-bit loads that are contiguous across the warp, exactly the weights of the
// m16n8k16 MMA "A" fragment rows r8 and r8+8.  One MMA k-step covers 16 consecutive
// columns ("s16" sub-block); inside it lane c owns columns 4c..4c+3, fed in the order
// (4c, 4c+2 | 4c+1, 4c+3).
//
// The maps below are __host__ __device__ so the same code drives the device repack
// kernels, the bit-exact dequantisation kernels and the host-side layout tests.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define JHD __host__ __device__ __forceinline__
#else
#define JHD inline
#endif

namespace juno {

constexpr int kTileRows = 16;
constexpr int kTileCols = 256;
constexpr int kQ4KTileBytes = 2368;  // 16 x 148: scales and mins widened to bytes
constexpr int kQ6KTileBytes = 3360;  // 16 x 210
constexpr int kQ80TileBytes = 4352;  // 16 x 8 x 34

JHD int tile_bytes(int ggml_type) {
    return ggml_type == 12 ? kQ4KTileBytes : ggml_type == 14 ? kQ6KTileBytes : ggml_type == 8 ? kQ80TileBytes : 0;
}
JHD int raw_block_bytes(int ggml_type) { return ggml_type == 12 ? 144 : ggml_type == 14 ? 210 : ggml_type == 8 ? 34 : 4; }
JHD int raw_block_elems(int ggml_type) { return ggml_type == 8 ? 32 : ggml_type == 0 ? 1 : 256; }

// Position of column-in-s16 t (0..3 inside a lane's group of four) in MMA feed order.
JHD int feed_pos(int t) { return ((t & 1) << 1) | (t >> 1); }

// ── Q4_K tile (2368 B) ──────────────────────────────────────────────────────────
//   [0,64)     dm[row16]      : d:f16 | dmin:f16 << 16
//   [64,320)   sm[row16][c4]  : the two sub-blocks 2c, 2c+1 that lane column c decodes, widened from 6 bits to bytes:
//                               scale(2c) | scale(2c+1) << 8 | min(2c) << 16 | min(2c+1) << 24
//   [320,2368) qs[g4][lane32] 16 B : word0 = row r8   raw qs[32g+4c .. +4)      (cols 64g+4c..   lo nibble, 64g+32+4c.. hi nibble)
//                                    word1 = row r8   raw qs[32g+16+4c .. +4)
//                                    word2 = row r8+8 raw qs[32g+4c .. +4)
//                                    word3 = row r8+8 raw qs[32g+16+4c .. +4)
constexpr int kQ4KQsOff = 320;
// Source of qs output word v (0..511): row in tile and byte offset inside that row's raw block.
JHD void q4k_qs_word_src(int v, int &row16, int &raw_off) {
    int g = v >> 7, lane = (v >> 2) & 31, k = v & 3;
    row16 = (lane >> 2) + 8 * (k >> 1);
    raw_off = 16 + 32 * g + 16 * (k & 1) + 4 * (lane & 3);
}
// Location of element (row16, e in 0..255) in the tile: byte offset of its qs byte, and which nibble.
JHD void q4k_elem_loc(int row16, int e, int &byte_off, int &hi_nibble) {
    int g = e >> 6, idx = e & 31;
    hi_nibble = (e >> 5) & 1;
    int half16 = idx >> 4, c = (idx >> 2) & 3, bw = idx & 3;
    int lane = ((row16 & 7) << 2) | c, k = 2 * (row16 >> 3) + half16;
    byte_off = kQ4KQsOff + g * 512 + lane * 16 + k * 4 + bw;
}
// 6-bit scale / min j of the 12 packed bytes (LlamaTransformerHandler.java:1471-1482).
JHD int q4k_scale6(const uint8_t *sc, int j) {
    return j < 4 ? (sc[j] & 0x3F) : (((sc[j + 4] & 0x0F) | ((sc[j - 4] & 0xC0) >> 2)) & 0x3F);
}
JHD int q4k_min6(const uint8_t *sc, int j) {
    return j < 4 ? (sc[j + 4] & 0x3F) : (((sc[j + 4] >> 4) | ((sc[j] & 0xC0) >> 2)) & 0x3F);
}

// ── Q6_K tile (3360 B) ──────────────────────────────────────────────────────────
//   [0,2048)    ql[m4][lane32] 16 B : words (row r8: W[2m], W[2m+1]; row r8+8: W[2m], W[2m+1])
//   [2048,3072) qh[p2][lane32] 16 B : words (row r8: H[2p], H[2p+1]; row r8+8: H[2p], H[2p+1])
//   [3072,3328) sc[row16][16] int8  (index = column/16)
//   [3328,3360) d[row16] f16
// For one lane-row, W[j] (j=0..7) holds the low nibbles of s16 sub-blocks 2j and 2j+1, columns 4c..4c+3;
// column t of sub-block 2j+odd sits in nibble nu = 2*feed_pos(t) + odd.  H[i] (i=0..3) holds the 2 high
// bits for W[2i] ("A") and W[2i+1] ("B"): for nibble nu the field is in byte nu/2 at bit
//   A even:4  A odd:6  B even:2  B odd:0
// so that (W & 0x0F0F0F0F) | (H & 0x30303030) etc. yields four 6-bit values in four bytes.
JHD int q6k_field_bit(int isB, int nu) {
    int inbyte = isB ? ((nu & 1) ? 0 : 2) : ((nu & 1) ? 6 : 4);
    return 8 * (nu >> 1) + inbyte;
}
struct Q6Loc {
    int w_off;   // byte offset of the ql word
    int nu;      // nibble index in that word
    int h_off;   // byte offset of the qh word
    int h_bit;   // bit position of the 2-bit field
    int sc_off;  // byte offset of the int8 scale
    int d_off;   // byte offset of d
};
JHD Q6Loc q6k_elem_loc(int row16, int e) {
    int s = e >> 4, within = e & 15, c = within >> 2, t = within & 3;
    int lane = ((row16 & 7) << 2) | c, rowsel = row16 >> 3;
    int j = s >> 1, odd = s & 1;
    Q6Loc L;
    L.nu = 2 * feed_pos(t) + odd;
    int m = j >> 1;
    L.w_off = m * 512 + lane * 16 + ((rowsel << 1) | (j & 1)) * 4;
    int i = j >> 1, isB = j & 1, p = i >> 1;
    L.h_off = 2048 + p * 512 + lane * 16 + ((rowsel << 1) | (i & 1)) * 4;
    L.h_bit = q6k_field_bit(isB, L.nu);
    L.sc_off = 3072 + row16 * 16 + s;
    L.d_off = 3328 + row16 * 2;
    return L;
}
// Raw Q6_K block: ql[128] qh[64] sc[16] d (LlamaTransformerHandler.java:1095-1135).
// 6-bit value (0..63, i.e. q+32) of element e of a raw block.
JHD int q6k_raw_u6(const uint8_t *blk, int e) {
    int hf = e >> 7, j = e & 127, tq = j >> 5, l = j & 31;
    int qlb = blk[hf * 64 + l + (tq & 1) * 32];
    int nib = (tq >= 2) ? (qlb >> 4) : (qlb & 15);
    int hb = (blk[128 + hf * 32 + l] >> (2 * tq)) & 3;
    return nib | (hb << 4);
}

// ── Q8_0 tile (4352 B): 16 rows x 8 blocks of 32 ────────────────────────────────
//   [0,4096)    q[j8][lane32] 16 B : word0 = row r8 block j bytes [4c,4c+4), word1 = row r8 bytes [16+4c,..),
//                                    word2/3 = same for row r8+8
//   [4096,4352) d[row16][8] f16
JHD void q80_elem_loc(int row16, int e, int &byte_off, int &d_off) {
    int j = e >> 5, idx = e & 31, half16 = idx >> 4, c = (idx >> 2) & 3, bw = idx & 3;
    int lane = ((row16 & 7) << 2) | c, k = 2 * (row16 >> 3) + half16;
    byte_off = j * 512 + lane * 16 + k * 4 + bw;
    d_off = 4096 + row16 * 16 + j * 2;
}

}  // namespace juno
