// Fused dequant-GEMV on integer tensor-core MMAs (decode batches of 1..8 sequences): device-level interface.
//
// The activation arrives as plain FP32 rows.  Every CTA builds its own operand from it: optional residual
// adds (x + partial products, summed in a fixed order), optional RMSNorm weights, then a block-floating-point
// split of every 256-column slice into three signed 8-bit limbs (q = round(v / 2^e), q = l0 + 256 l1 + 65536 l2),
// so that the products against the 4/6/8-bit weights are exact integers (qgemv.cu).
#pragma once
#include "common.cuh"

namespace juno {

enum QEpilogue {
    QEPI_STORE = 0,      // out[b][row] = y
    QEPI_SILU_PAIR = 1,  // tile rows 0-7 are gate rows, 8-15 the matching up rows: out[b][8*tile+row] = silu(gate)*up
};

constexpr int kQMaxAdd = 8;

struct QSeg {
    const uint8_t *w = nullptr;  // tiled weights (layout.cuh)
    float *out = nullptr;        // [batch][ld_out]
    int rows = 0;                // valid output rows (after pairing, for QEPI_SILU_PAIR)
    int row_tiles = 0;
    int type = 0;                // 12 / 14 / 8
};

struct QGemvArgs {
    QSeg seg[3];
    int nseg = 1;
    int K = 0;
    int batch = 1;
    int ld_out = 0;
    int epi = QEPI_STORE;
    // input rows: v = x (+ (add[0] + add[1] + ...)), each [batch][ldx]
    const float *x = nullptr;
    int ldx = 0;
    const float *add[kQMaxAdd] = {nullptr};
    int n_add = 0;
    float *x_store = nullptr;       // optional: the summed input rows are written here (by one CTA)
    const float *normw = nullptr;   // optional RMSNorm (LlamaTransformerHandler.rmsNorm :818-828): operand = normw*v,
    float eps = 0.f;                //   outputs multiplied by 1/sqrt(mean(v^2) + eps)

    // Tensor parallelism without a collective library call (one rank per GPU, peer memory mapped at load time).  The
    // exchanged unit is an 8-byte (value, step number) pair written with ONE store, so the data is its own flag:
    // no fence, no counter and no separate signal on either side.
    // Producer side (row-parallel products): the outputs go into every rank's inbox instead of seg[0].out
    // (peer_out[d]: this rank's slot in rank d's inbox, [batch][ld_out] pairs), tagged with the step number `*epoch`.
    int n_peers = 0;
    float *peer_out[kQMaxAdd] = {nullptr};
    // Consumer side: with tagged_adds the addends add[0..n_add) are inbox slots ([batch][ldx] pairs) written by the
    // ranks 0..n_add-1; every load re-reads until the pairs carry `*epoch` (bounded: about a second, then
    // *peer_failed is set, the error word says which rank, and every later wait gives up at once).
    bool tagged_adds = false;
    // With many ranks every CTA reading every inbox costs more than the smaller matrices save (the L2 reads grow with
    // CTAs x ranks).  With n_red > 0 the first CTAs of the grid first add the inbox slots red_src[0..n_red) of one
    // 256-column slice each, in rank order, and publish the sums as pairs in `red_dst` (local memory, same layout as an
    // inbox slot); add[0] must then be red_dst, which every CTA polls as its single addend.
    int n_red = 0;
    const float *red_src[kQMaxAdd] = {nullptr};
    float *red_dst = nullptr;
    const unsigned *epoch = nullptr;
    unsigned *peer_failed = nullptr;
};

// Most sequences one launch can take for this K and block format mix (shared memory), at most 8.
int qgemv_batch_chunk(const juno_ctx *ctx, int K, int type_mix, int batch);
// Enqueues the product (several launches when the batch exceeds one chunk).  All pointers are device pointers.
int launch_qgemv(juno_ctx *ctx, const QGemvArgs &a, cudaStream_t stream);

}  // namespace juno
