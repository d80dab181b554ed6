// Test-only host build of the tile-layout index maps (repack.cuh, dequant.cuh): the same code the device kernels run,
// compiled with the C++ compiler so that the layout tests need no GPU.  Not part of the product library.
#include <stdint.h>

#include "../../juno_b200/csrc/dequant.cuh"
#include "../../juno_b200/csrc/layout.cuh"
#include "../../juno_b200/csrc/repack.cuh"

using namespace juno;

extern "C" int64_t layout_tiled_bytes(int type, int64_t rows, int64_t cols) {
    if (cols % 256 || !tile_bytes(type)) return -1;
    return ((rows + 15) / 16) * (cols / 256) * (int64_t)tile_bytes(type);
}

extern "C" int layout_repack(int type, const uint8_t *raw, int64_t rows, int64_t cols, uint8_t *out) {
    if (cols % 256 || rows < 1 || !tile_bytes(type)) return -1;
    const int nsb = (int)(cols / 256), RT = (int)((rows + 15) / 16);
    const size_t rrb = (size_t)nsb * (type == 12 ? 144 : type == 14 ? 210 : 8 * 34);
    const int wpt = tile_bytes(type) / 4;
    uint32_t *o = reinterpret_cast<uint32_t *>(out);
    for (int R = 0; R < RT; R++)
        for (int b = 0; b < nsb; b++)
            for (int w = 0; w < wpt; w++)
                o[((size_t)R * nsb + b) * wpt + w] = type == 12   ? q4k_out_word(raw, rrb, (int)rows, b, R, w)
                                                     : type == 14 ? q6k_out_word(raw, rrb, (int)rows, b, R, w)
                                                                  : q80_out_word(raw, rrb, (int)rows, b, R, w);
    return 0;
}

extern "C" int layout_dequant_tiled(int type, const uint8_t *tiles, int64_t rows, int64_t cols, float *out) {
    if (cols % 256 || !tile_bytes(type)) return -1;
    const int64_t nb = cols / 256;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++)
            out[r * cols + c] = tile_elem_value(type, tiles + ((r >> 4) * nb + (c >> 8)) * (int64_t)tile_bytes(type), (int)(r & 15), (int)(c & 255));
    return 0;
}

// ── work split of the fused dequant-GEMV (qsplit.cuh) ────────────────────────────────────
#include <vector>

#include "../../juno_b200/csrc/qsplit.cuh"

// Walks the split exactly as the kernel does - the producer cursor of every warp, the consumer loop with its two
// partial-sum slots, the finisher's view - for a grid of `grid` CTAs over `total_rt` row tiles of NB tiles each.
// Returns 0 if every (row tile, block) is computed exactly once, every warp requests the tiles in the order it uses
// them, and the finisher adds, for every row tile, exactly the partial sums that were written, from the right slot;
// otherwise a code naming the first violated property.  *max_tiles_per_warp reports the load of the busiest warp.
extern "C" int qsplit_check(int total_rt, int NB, int grid, int *max_tiles_per_warp) {
    std::vector<uint8_t> seen((size_t)total_rt * NB, 0);
    int busiest = 0;
    for (int c = 0; c < grid; c++) {
        int rt0, rtc;
        qsplit_cta(c, grid, total_rt, rt0, rtc);
        const int nch = qsplit_chunks(rtc);
        for (int w = 0; w < kQSplitWarps; w++) {
            std::vector<int> prod, cons;
            // producer cursor (QCursor in qgemv.cu)
            for (int k = 0; k < nch; k++) {
                const int lo = qsplit_chunk_lo(rt0, rtc, nch, k), T = (qsplit_chunk_lo(rt0, rtc, nch, k + 1) - lo) * NB;
                int f0, f1;
                qsplit_warp(w, T, f0, f1);
                int R = lo + f0 / NB, sb = f0 % NB;
                for (int f = f0; f < f1; f++) {
                    prod.push_back(R * NB + sb);
                    if (++sb == NB) {
                        sb = 0;
                        R++;
                    }
                }
            }
            // consumer loop + finisher bookkeeping
            int tiles = 0;
            for (int k = 0; k < nch; k++) {
                const int lo = qsplit_chunk_lo(rt0, rtc, nch, k), crt = qsplit_chunk_lo(rt0, rtc, nch, k + 1) - lo, T = crt * NB;
                if (crt > kQChunk || crt < 1) return 1;
                int f0, f1;
                qsplit_warp(w, T, f0, f1);
                const int l_first = f0 / NB;
                int slot_of[kQChunk];
                for (int l = 0; l < kQChunk; l++) slot_of[l] = -1;
                int f = f0;
                for (int j = 0; j < 2; j++) {
                    const int l = l_first + j, fe = f1 < (l + 1) * NB ? f1 : (l + 1) * NB;
                    if (f >= fe) continue;
                    for (int sb = f - l * NB; f < fe; f++, sb++) {
                        cons.push_back((lo + l) * NB + sb);
                        tiles++;
                    }
                    slot_of[l] = j;
                }
                if (f != f1) return 2;  // a warp's share reached into a third row tile
                for (int l = 0; l < crt; l++) {
                    int w_lo, w_hi, wf0, wf1;
                    qsplit_row_tile_warps(l, NB, T, w_lo, w_hi);
                    qsplit_warp(w, T, wf0, wf1);
                    const bool read = w >= w_lo && w <= w_hi && wf0 < wf1;
                    if (read != (slot_of[l] >= 0)) return 3;  // the finisher reads a slot nobody wrote, or misses one
                    if (read && (wf0 < l * NB ? 1 : 0) != slot_of[l]) return 4;
                }
            }
            if (prod != cons) return 5;
            for (int t : cons) {
                if (t < 0 || t >= total_rt * NB || seen[(size_t)t]) return 6;
                seen[(size_t)t] = 1;
            }
            if (tiles > busiest) busiest = tiles;
        }
    }
    for (uint8_t s : seen)
        if (!s) return 7;
    if (max_tiles_per_warp) *max_tiles_per_warp = busiest;
    return 0;
}
