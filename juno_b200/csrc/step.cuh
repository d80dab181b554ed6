// The persistent decode-step kernel: every per-layer product and the attention of one decode step run as phases
// of ONE cooperative launch (one CTA per SM), separated by grid-wide barriers, with the quantised weights
// streamed through a shared-memory ring by bulk asynchronous copies that run ahead of the barriers.
//
// The host side records the phases: while a recorder is installed on the context, launch_gemv / launch_attn
// append a phase description instead of launching a kernel.
#pragma once
#include <vector>

#include "attn.cuh"
#include "gemv.cuh"
#include "gemv_params.cuh"

namespace juno {

enum StepPhaseKind { STEP_GEMV = 1, STEP_ATTN = 2 };

constexpr int kStepWarps = 16;
constexpr int kStepConsumers = kStepWarps * 32;
constexpr int kStepThreads = kStepConsumers;
constexpr int kStepRingDepth = 2;                           // tiles in flight per warp
constexpr int kStepRingSlots = kStepRingDepth * kStepWarps;
constexpr unsigned kStepFragBufs = 4;                       // partial-sum buffers per warp (tasks in flight per group)
constexpr unsigned kStepClaimRing = 4;                      // claimed CTA tasks in flight between warp 0 and the others
constexpr int kStepFinishLag = 2;                           // a task's rows are finished this many tasks later

// Attention of one layer inside the step kernel.  Work item = (sequence, kv head, group of GE query heads, context
// chunk); the last chunk of an item group to finish merges the chunks (no barrier between the two halves).
struct StepAttn {
    const void *k, *v;
    void *kw, *vw;
    const int32_t *table;
    int max_pages_per_seq, n_pages, n_kv_heads, n_heads, layer;
    int n;            // sequences
    int chunks;       // context chunks per (sequence, kv head, head group), <= 64
    int head_groups;  // (n_heads / n_kv_heads) / GE
    const float *q;   // unrotated, [n][ldq]
    int ldq;
    const float *knew, *vnew;  // this step's k and v rows, [n][ldkv]
    int ldkv;
    const int32_t *slots, *seq_lens;
    const float2 *rope_cs;
    float *part_o, *part_ml;  // [n][n_heads][chunks][hd], [n][n_heads][chunks][2]
    unsigned *counters;       // [n][n_kv_heads][head_groups], zero between uses
    float *out;               // optional [n][n_heads*hd]
    StageImage stage;         // optional: the output as the staged activation of the next product
};

struct alignas(16) StepPhase {
    int kind;
    int rot;      // STEP_GEMV: CTA (blockIdx + grid - rot) % grid takes CTA task 0, so consecutive phases start
                  // where the previous one stopped handing out work
    int need_xs;  // STEP_GEMV: some segment is Q4_K (32-column sums of x are needed)
    int pad;
    GemvParams g;
    StepAttn a;
};

struct StepRecorder {
    std::vector<StepPhase> phases;
    int grid = 0;  // CTAs of the step kernel
    int n = 0;     // sequences of the step
    int next_rot = 0;
};

// Device-resident plan of one step shape (built once, replayed by every launch of that shape).
struct StepPlan {
    StepPhase *d_phases = nullptr;
    int n_phases = 0;
    unsigned *d_sync = nullptr;  // {barrier arrivals, error code, one task counter per phase}
    unsigned *h_err = nullptr;   // pinned mirror of the error code
    size_t smem = 0;
    int slot_bytes = 0;
    unsigned img_cap = 0;
    int grid = 0;
    int kv_f32 = 0, hd = 0, ge = 0, nb = 0;
    double algo_bytes = 0;
    unsigned long long *d_timeline = nullptr;  // JUNO_STEP_TIMELINE=1: per-phase time stamps of CTA 0
    int timeline_period = 0;                   // phases per layer, for the printed summary
};

// CTA-task geometry inside the step kernel (16 warps, static assignment).
void step_task_geometry(int grid, int K, int total_rt, int *kin, int *tpt, int *n_ctasks);
// Whether the step kernel can run this shape at all (head layout, batch, shared memory).
bool step_supported(const juno_ctx *ctx, int n, int hd, int n_heads, int n_kv_heads, int max_K, int max_tile_bytes);
int step_record_gemv(juno_ctx *ctx, const GemvArgs &a);
int step_record_attn(juno_ctx *ctx, const AttnArgs &a);
int step_plan_build(juno_ctx *ctx, const StepRecorder &rec, int kv_f32, int hd, int group, StepPlan *plan);
void step_plan_free(StepPlan *plan);
int launch_step(juno_ctx *ctx, const StepPlan &plan, cudaStream_t st);
// Error code left by the last completed launch of the plan (0 = none); call after a stream synchronise.
unsigned step_plan_error(const StepPlan &plan);

}  // namespace juno
