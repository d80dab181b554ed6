// Paged KV cache and GQA decode attention: device-level interface.
#pragma once
#include <vector>

#include "common.cuh"

// Page layout (both K and V): [layer][page][kv_head][page_tokens=16][head_dim], FP16 or FP32.
struct juno_kvpool {
    uint32_t magic;
    juno_ctx *ctx;
    int n_layers, n_kv_heads, head_dim, n_pages, dtype;  // dtype 0 = f16, 1 = f32
    int page_tokens;
    int elem_bytes;
    void *k, *v;
    std::vector<int> free_pages;
    std::vector<int> page_refs;  // sequences holding each page (0 = free): pages of a shared prefix are counted per holder
    // page table for sequences with a slot: [max_slots][max_pages_per_seq] on the device, mirrored in pinned host memory
    int max_slots, max_pages_per_seq;
    int32_t *d_table, *h_table;
    std::vector<int> free_slots;
    int owned_by_model;
};

struct juno_seq {
    uint32_t magic;
    juno_kvpool *pool;
    int max_tokens;
    int len;   // positions written so far (highest position + 1)
    int slot;  // row of the pool's page table
    std::vector<int> pages;
};

namespace juno {

constexpr int kPageTokens = 16;

struct AttnArgs {
    const juno_kvpool *pool;
    int layer;
    int n;               // sequences
    int n_heads;         // query heads (local)
    const float *q;      // [n][ldq], heads contiguous inside a row
    int ldq = 0;         // 0 = n_heads*hd
    float *out;          // [n][n_heads*hd]
    const int32_t *slots;     // [n] rows of the page table
    const int32_t *seq_lens;  // [n] number of positions to attend (pos+1)
    int n_splits;
    float *part_o;       // [n][n_heads][n_splits][hd]
    float *part_ml;      // [n][n_heads][n_splits][2]
    double algo_bytes = 0;  // K+V bytes the call has to read (for the profiler)
    // optional: fused RoPE + KV append.  q [n][ldq] is unrotated, knew/vnew [n][ldkv] hold this step's k and v,
    // rope_cs the table of launch_rope_table; the newest position (seq_lens-1) is rotated, rounded and appended.
    const float2 *rope_cs = nullptr;
    const float *knew = nullptr, *vnew = nullptr;
    int ldkv = 0;
};
size_t attn_scratch_floats(int n, int n_heads, int hd, int n_splits);
int attn_pick_splits(const juno_ctx *ctx, int n, int n_kv_heads, int max_len);
int launch_attn(juno_ctx *ctx, const AttnArgs &a, cudaStream_t st);

// RoPE on q and k (adjacent pairs, LlamaTransformerHandler.rope :1657-1671) and append of k, v at
// position pos[i] of each sequence.  cs_table: [n][hd/2] (cos, sin) from launch_rope_table.
int launch_rope_table(juno_ctx *ctx, const int32_t *positions, int n, int hd, float theta, float2 *table,
                      cudaStream_t st);
int launch_rope_append(juno_ctx *ctx, const juno_kvpool *pool, int layer, int n, int n_heads, float *q, int ldq,
                       const float *k, const float *v, int ldkv, const int32_t *slots, const int32_t *positions,
                       const float2 *cs_table, cudaStream_t st);

int kvpool_create(juno_ctx *ctx, int n_layers, int n_kv_heads, int head_dim, int n_pages, int dtype, int max_slots,
                  int max_pages_per_seq, juno_kvpool **out);
int kvpool_destroy(juno_kvpool *p);
int seq_create(juno_kvpool *p, int max_tokens, juno_seq **out);
// Makes sure pages exist for positions [0, upto) and that the device page table row is current (stream-ordered).
// Makes the positions [from, upto) of the sequence writable: allocates missing pages and gives the sequence a private
// copy of every page of the range that it shares with another sequence (copy-on-write, ordered on `st`).
int seq_reserve(juno_seq *s, int from, int upto, cudaStream_t st);

}  // namespace juno
