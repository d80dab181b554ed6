// Work split of the fused dequant-GEMV (qgemv.cu): which row tiles a CTA owns, how they are cut into chunks, which
// tiles of a chunk a warp computes and which warps contributed to a row tile.  Plain integer functions shared by the
// kernel and by a host-side test build (tests/native), so that coverage and bookkeeping are checked without a GPU.
#pragma once
#include "layout.cuh"

namespace juno {

constexpr int kQSplitWarps = 16;  // warps of a GEMV CTA
constexpr int kQChunk = 16;       // most row tiles per chunk: a warp's share is then at most NB tiles = two row tiles

// Row tiles [rt0, rt0 + rtc) of CTA c out of `grid`: the counts differ by at most one across the grid.
JHD void qsplit_cta(int c, int grid, int total_rt, int &rt0, int &rtc) {
    rt0 = (int)(((long long)c * total_rt) / grid);
    rtc = (int)(((long long)(c + 1) * total_rt) / grid) - rt0;
}
JHD int qsplit_chunks(int rtc) { return (rtc + kQChunk - 1) / kQChunk; }
// First row tile of chunk k (k = n_chunks gives the end): chunks of equal size up to one row tile.
JHD int qsplit_chunk_lo(int rt0, int rtc, int n_chunks, int k) { return rt0 + (k * rtc) / n_chunks; }
// Tiles [f0, f1) of warp w in a chunk of T = row tiles x NB tiles (flat index = local row tile * NB + block).
JHD void qsplit_warp(int w, int T, int &f0, int &f1) {
    f0 = (w * T) >> 4;
    f1 = ((w + 1) * T) >> 4;
}
// Warps whose tiles reach into local row tile l: the first with f1 > l*NB and the last with f0 < (l+1)*NB.  Warps in
// between with an empty range (fewer than sixteen tiles in the chunk) are skipped by the caller.
JHD void qsplit_row_tile_warps(int l, int NB, int T, int &w_lo, int &w_hi) {
    const int tlo = l * NB, thi = tlo + NB;
    w_lo = (16 * (tlo + 1) + T - 1) / T - 1;
    w_hi = (16 * thi + T - 1) / T - 1;
    if (w_hi > kQSplitWarps - 1) w_hi = kQSplitWarps - 1;
}

}  // namespace juno
