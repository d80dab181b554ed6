/*
 * juno_oracle.c — CPU restatement of Juno's quantised LLaMA decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA engine: it is
 * compiled into liboracle.so and called from the test-suite, from the smoke test
 * and from the CPU-baseline leg of the benchmark.  The product library never
 * links, loads or calls it.
 *
 * Parity pin: checked against the reference's own known-answer tests
 * (GgufReaderTest f16/Q6_K golden block/Q4_K/Q8_0 cases, PhiQuantizedMatVecTest
 * one-block dot products) transcribed into tests/golden/; the reference is Java
 * and cannot run here, so attention / RoPE / RMSNorm are pinned by line-by-line
 * restatement only ("parity unpinned" for those three, pinned for the quant path).
 *
 * Every function cites the reference lines it follows; paths are relative to
 * node/src/main/java/cab/ml/juno/node/ unless stated.  Arithmetic rules kept from
 * the Java source: `float` stays binary32, `Math.*` calls are binary64 with a
 * (float) cast, no fused multiply-add (build with -ffp-contract=off), one
 * sequential accumulator per output row.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define JO_TYPE_F32 0
#define JO_TYPE_Q8_0 8
#define JO_TYPE_Q4_K 12
#define JO_TYPE_Q6_K 14

/* ── f16 → f32 : GgufReader.java:1248-1271 ─────────────────────────────────── */
float jo_f16_to_f32(uint16_t bits) {
    int s = (bits >> 15) & 1;
    int e = (bits >> 10) & 0x1F;
    int m = bits & 0x3FF;
    uint32_t f;
    if (e == 0) {
        if (m == 0) {
            f = (uint32_t)s << 31;
        } else { /* subnormal: normalise */
            int exp = -14;
            while ((m & 0x400) == 0) {
                m <<= 1;
                exp--;
            }
            m &= 0x3FF;
            f = ((uint32_t)s << 31) | ((uint32_t)(exp + 127) << 23) | ((uint32_t)m << 13);
        }
    } else if (e == 31) {
        f = ((uint32_t)s << 31) | 0x7F800000u | ((uint32_t)m << 13);
    } else {
        f = ((uint32_t)s << 31) | ((uint32_t)(e - 15 + 127) << 23) | ((uint32_t)m << 13);
    }
    float out;
    memcpy(&out, &f, 4);
    return out;
}

/* f32 → f16 round-to-nearest-even.  Not on the reference path (its KV cache is
 * FP32); used only when the oracle is asked to model an FP16 KV cache. */
uint16_t jo_f32_to_f16(float v) {
    uint32_t x;
    memcpy(&x, &v, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0));
    if (ax >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) /* < 2^-25 (or exactly 2^-25: ties to even -> 0) */
        return (uint16_t)sign;
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1)))
        q++;
    return (uint16_t)(sign | (base + q));
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ── Q4_K 6-bit scale / min : LlamaTransformerHandler.java:1471-1482,
 *    GgufReader.java:708-721 ─────────────────────────────────────────────── */
static inline int q4k_scale(const uint8_t *sc, int j) {
    if (j < 4)
        return sc[j] & 0x3F;
    return ((sc[j + 4] & 0x0F) | ((sc[j - 4] & 0xC0) >> 2)) & 0x3F;
}
static inline int q4k_min(const uint8_t *sc, int j) {
    if (j < 4)
        return sc[j + 4] & 0x3F;
    return ((sc[j + 4] >> 4) | ((sc[j] & 0xC0) >> 2)) & 0x3F;
}
int jo_q4k_scale(const uint8_t *sc12, int j) { return q4k_scale(sc12, j); }
int jo_q4k_min(const uint8_t *sc12, int j) { return q4k_min(sc12, j); }

/* ── row-wise dequantisation ───────────────────────────────────────────────
 * Q4_K: LlamaTransformerHandler.java:1017-1050 (≡ GgufReader.java:603-641)
 * Q6_K: :1095-1135 (≡ GgufReader.java:726-791)
 * Q8_0: :895-913  (≡ GgufReader.java:434-448)
 * F32 : :888-893 */
static void deq_row_q4k(const uint8_t *row, int cols, float *out) {
    int nb = cols / 256;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 144;
        const uint8_t *sc = bo + 4, *qs = bo + 16;
        float d = jo_f16_to_f32(rd16(bo));
        float dmin = jo_f16_to_f32(rd16(bo + 2));
        int qi = 0;
        for (int g = 0; g < 256; g += 64) {
            int s0 = g / 32, s1 = s0 + 1;
            float scale0 = d * (float)q4k_scale(sc, s0);
            float min0 = dmin * (float)q4k_min(sc, s0);
            float scale1 = d * (float)q4k_scale(sc, s1);
            float min1 = dmin * (float)q4k_min(sc, s1);
            float *o = out + b * 256 + g;
            for (int i = 0; i < 32; i++)
                o[i] = scale0 * (float)(qs[qi + i] & 0x0F) - min0;
            for (int i = 0; i < 32; i++)
                o[32 + i] = scale1 * (float)(qs[qi + i] >> 4) - min1;
            qi += 32;
        }
    }
}

static void deq_row_q6k(const uint8_t *row, int cols, float *out) {
    int nb = cols / 256;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 210;
        float d = jo_f16_to_f32(rd16(bo + 208));
        for (int half = 0; half < 2; half++) {
            const uint8_t *ql = bo + half * 64;
            const uint8_t *qh = bo + 128 + half * 32;
            const int8_t *sc = (const int8_t *)(bo + 192 + half * 8);
            float *o = out + b * 256 + half * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int qlL = ql[l], qlL2 = ql[l + 32], qhL = qh[l];
                int q1 = ((qlL & 0x0F) | (((qhL >> 0) & 3) << 4)) - 32;
                int q2 = ((qlL2 & 0x0F) | (((qhL >> 2) & 3) << 4)) - 32;
                int q3 = ((qlL >> 4) | (((qhL >> 4) & 3) << 4)) - 32;
                int q4 = ((qlL2 >> 4) | (((qhL >> 6) & 3) << 4)) - 32;
                float d1 = d * (float)sc[is];
                float d2 = d * (float)sc[is + 2];
                float d3 = d * (float)sc[is + 4];
                float d4 = d * (float)sc[is + 6];
                o[l] = d1 * (float)q1;
                o[l + 32] = d2 * (float)q2;
                o[l + 64] = d3 * (float)q3;
                o[l + 96] = d4 * (float)q4;
            }
        }
    }
}

static void deq_row_q8_0(const uint8_t *row, int cols, float *out) {
    int nb = cols / 32;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 34;
        float scale = jo_f16_to_f32(rd16(bo));
        const int8_t *q = (const int8_t *)(bo + 2);
        for (int i = 0; i < 32; i++)
            out[b * 32 + i] = scale * (float)q[i];
    }
}

/* bytes per row for a GGML type: GgufReader.java:347-360 */
int64_t jo_row_bytes(int type, int64_t cols) {
    switch (type) {
    case JO_TYPE_F32:
        return cols * 4;
    case JO_TYPE_Q8_0:
        return cols / 32 * 34;
    case JO_TYPE_Q4_K:
        return cols / 256 * 144;
    case JO_TYPE_Q6_K:
        return cols / 256 * 210;
    default:
        return -1;
    }
}

static int deq_row(int type, const uint8_t *row, int cols, float *out) {
    switch (type) {
    case JO_TYPE_F32:
        memcpy(out, row, (size_t)cols * 4);
        return 0;
    case JO_TYPE_Q8_0:
        deq_row_q8_0(row, cols, out);
        return 0;
    case JO_TYPE_Q4_K:
        deq_row_q4k(row, cols, out);
        return 0;
    case JO_TYPE_Q6_K:
        deq_row_q6k(row, cols, out);
        return 0;
    default:
        return -1;
    }
}

/* dequantize(t, rows, cols): LlamaTransformerHandler.java:873-885 */
int jo_dequantize(int type, const uint8_t *raw, int64_t rows, int64_t cols, float *out) {
    int64_t rb = jo_row_bytes(type, cols);
    if (rb < 0)
        return -1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        deq_row(type, raw + r * rb, (int)cols, out + r * cols);
    return 0;
}

/* ── quantised mat-vec, one sequential accumulator per row ─────────────────
 * Q4_K: LlamaTransformerHandler.java:1428-1468   Q6_K: :1587-1638
 * Q8_0: :1486-1508                               F32 : :1152-1172 */
static float dot_row_q4k(const uint8_t *row, const float *x, int cols) {
    int nb = cols / 256;
    float acc = 0.f;
    int xBase = 0;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 144;
        const uint8_t *sc = bo + 4, *qs = bo + 16;
        float d = jo_f16_to_f32(rd16(bo));
        float dmin = jo_f16_to_f32(rd16(bo + 2));
        int qi = 0;
        for (int g = 0; g < 256; g += 64) {
            int s0 = g / 32, s1 = s0 + 1;
            float scale0 = d * (float)q4k_scale(sc, s0);
            float min0 = dmin * (float)q4k_min(sc, s0);
            float scale1 = d * (float)q4k_scale(sc, s1);
            float min1 = dmin * (float)q4k_min(sc, s1);
            for (int i = 0; i < 32; i++)
                acc += (scale0 * (float)(qs[qi + i] & 0x0F) - min0) * x[xBase + g + i];
            for (int i = 0; i < 32; i++)
                acc += (scale1 * (float)(qs[qi + i] >> 4) - min1) * x[xBase + g + 32 + i];
            qi += 32;
        }
        xBase += 256;
    }
    return acc;
}

static float dot_row_q6k(const uint8_t *row, const float *x, int cols) {
    int nb = cols / 256;
    float acc = 0.f;
    int xBase = 0;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 210;
        float d = jo_f16_to_f32(rd16(bo + 208));
        for (int half = 0; half < 2; half++) {
            const uint8_t *ql = bo + half * 64;
            const uint8_t *qh = bo + 128 + half * 32;
            const int8_t *sc = (const int8_t *)(bo + 192 + half * 8);
            int xOff = xBase + half * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int qlL = ql[l], qlL2 = ql[l + 32], qhL = qh[l];
                int q1 = ((qlL & 0x0F) | (((qhL >> 0) & 3) << 4)) - 32;
                int q2 = ((qlL2 & 0x0F) | (((qhL >> 2) & 3) << 4)) - 32;
                int q3 = ((qlL >> 4) | (((qhL >> 4) & 3) << 4)) - 32;
                int q4 = ((qlL2 >> 4) | (((qhL >> 6) & 3) << 4)) - 32;
                float d1 = d * (float)sc[is];
                float d2 = d * (float)sc[is + 2];
                float d3 = d * (float)sc[is + 4];
                float d4 = d * (float)sc[is + 6];
                acc += d1 * (float)q1 * x[xOff + l];
                acc += d2 * (float)q2 * x[xOff + l + 32];
                acc += d3 * (float)q3 * x[xOff + l + 64];
                acc += d4 * (float)q4 * x[xOff + l + 96];
            }
        }
        xBase += 256;
    }
    return acc;
}

static float dot_row_q8_0(const uint8_t *row, const float *x, int cols) {
    int nb = cols / 32;
    float acc = 0.f;
    int xBase = 0;
    for (int b = 0; b < nb; b++) {
        const uint8_t *bo = row + (size_t)b * 34;
        float scale = jo_f16_to_f32(rd16(bo));
        const int8_t *q = (const int8_t *)(bo + 2);
        for (int i = 0; i < 32; i++)
            acc += scale * (float)q[i] * x[xBase + i];
        xBase += 32;
    }
    return acc;
}

static float dot_row_f32(const uint8_t *row, const float *x, int cols) {
    const float *a = (const float *)row;
    float acc = 0.f;
    for (int c = 0; c < cols; c++)
        acc += a[c] * x[c];
    return acc;
}

/* matVec(QuantizedTensor A, x, rowStart, rowEnd, cols): :1200-1245.  Rows are
 * split across threads as IntStream.range(0,rows).parallel() does (:1436); the
 * per-row arithmetic does not depend on the split. */
int jo_matvec(int type, const uint8_t *raw, const float *x, int64_t rowStart, int64_t rowEnd,
              int64_t cols, float *y) {
    int64_t rb = jo_row_bytes(type, cols);
    if (rb < 0 || rowEnd < rowStart)
        return -1;
    int64_t rows = rowEnd - rowStart;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        const uint8_t *row = raw + (rowStart + r) * rb;
        float v;
        switch (type) {
        case JO_TYPE_Q4_K:
            v = dot_row_q4k(row, x, (int)cols);
            break;
        case JO_TYPE_Q6_K:
            v = dot_row_q6k(row, x, (int)cols);
            break;
        case JO_TYPE_Q8_0:
            v = dot_row_q8_0(row, x, (int)cols);
            break;
        default:
            v = dot_row_f32(row, x, (int)cols);
            break;
        }
        y[r] = v;
    }
    return 0;
}

/* The reference has no batched product (InferencePipeline.java:62-69 loops over
 * requests); a batch is `batch` independent calls. */
int jo_matvec_batch(int type, const uint8_t *raw, const float *x, int batch, int64_t rows,
                    int64_t cols, float *y) {
    for (int b = 0; b < batch; b++) {
        int rc = jo_matvec(type, raw, x + (int64_t)b * cols, 0, rows, cols, y + (int64_t)b * rows);
        if (rc)
            return rc;
    }
    return 0;
}

/* ── elementwise primitives ────────────────────────────────────────────────── */
/* rmsNorm: LlamaTransformerHandler.java:818-828 */
void jo_rmsnorm(const float *x, const float *w, int n, float eps, float *out) {
    float ss = 0.f;
    for (int i = 0; i < n; i++)
        ss += x[i] * x[i];
    float scale = 1.f / (float)sqrt((double)(ss / (float)n + eps));
    for (int i = 0; i < n; i++)
        out[i] = w[i] * x[i] * scale;
}

/* rope: :1657-1671 (adjacent pairs; pow/cos/sin in binary64) */
void jo_rope(float *x, int pos, int nHeads, int headDim, float theta) {
    for (int h = 0; h < nHeads; h++) {
        int base = h * headDim;
        for (int i = 0; i < headDim / 2; i++) {
            double freq = 1.0 / pow((double)theta, (2.0 * i) / headDim);
            double angle = pos * freq;
            float c = (float)cos(angle), s = (float)sin(angle);
            float x0 = x[base + 2 * i], x1 = x[base + 2 * i + 1];
            x[base + 2 * i] = x0 * c - x1 * s;
            x[base + 2 * i + 1] = x0 * s + x1 * c;
        }
    }
}

/* softmax: :1718-1730 */
void jo_softmax(float *s, int n) {
    float max = -INFINITY;
    for (int i = 0; i < n; i++)
        if (s[i] > max)
            max = s[i];
    float sum = 0.f;
    for (int i = 0; i < n; i++) {
        s[i] = (float)exp((double)(s[i] - max));
        sum += s[i];
    }
    for (int i = 0; i < n; i++)
        s[i] /= sum;
}

/* silu: :1733-1735 */
float jo_silu(float x) { return x / (1.f + (float)exp((double)(-x))); }

/* gqa: :1678-1715.  K and V are position-major `seqLen × kvDim` FP32 arrays. */
void jo_gqa(const float *q, const float *K, const float *V, int seqLen, int nHeads, int nKvHeads,
            int headDim, float *out, float *scores /* scratch[seqLen] */) {
    int g = nHeads / nKvHeads, kvDim = nKvHeads * headDim;
    float scale = (float)(1.0 / sqrt((double)headDim));
    for (int i = 0; i < nHeads * headDim; i++)
        out[i] = 0.f;
    for (int h = 0; h < nHeads; h++) {
        int kvHead = h / g, qBase = h * headDim, kBase = kvHead * headDim;
        for (int t = 0; t < seqLen; t++) {
            float dot = 0.f;
            const float *k = K + (size_t)t * kvDim + kBase;
            for (int d = 0; d < headDim; d++)
                dot += q[qBase + d] * k[d];
            scores[t] = dot * scale;
        }
        jo_softmax(scores, seqLen);
        for (int t = 0; t < seqLen; t++) {
            const float *v = V + (size_t)t * kvDim + kBase;
            float w = scores[t];
            for (int d = 0; d < headDim; d++)
                out[qBase + d] += w * v[d];
        }
    }
}

/* Greedy pick: SoftmaxStep.java:36-59 then SampleStep.java:51-58 (first strict
 * maximum of the probabilities).  `probs` is scratch[n]. */
int jo_greedy(const float *logits, int n, float *probs) {
    float max = -INFINITY;
    for (int i = 0; i < n; i++)
        if (logits[i] > max)
            max = logits[i];
    float sum = 0.f;
    for (int i = 0; i < n; i++) {
        probs[i] = (float)exp((double)(logits[i] - max));
        sum += probs[i];
    }
    if (sum > 0.f)
        for (int i = 0; i < n; i++)
            probs[i] /= sum;
    int best = 0;
    for (int i = 1; i < n; i++)
        if (probs[i] > probs[best])
            best = i;
    return best;
}

/* ── model ─────────────────────────────────────────────────────────────────── */
enum { JO_T_TOKEN_EMBD = 0, JO_T_OUTPUT_NORM, JO_T_OUTPUT, JO_T_ATTN_NORM, JO_T_FFN_NORM,
       JO_T_ATTN_Q, JO_T_ATTN_K, JO_T_ATTN_V, JO_T_ATTN_OUT, JO_T_FFN_GATE, JO_T_FFN_UP,
       JO_T_FFN_DOWN, JO_T_ATTN_Q_BIAS, JO_T_ATTN_K_BIAS, JO_T_ATTN_V_BIAS, JO_T_COUNT };

typedef struct {
    const uint8_t *data; /* borrowed */
    int type;
    int64_t rows, cols;
} jo_tensor;

typedef struct {
    int hidden, layers, heads, kv_heads, head_dim, inter, vocab;
    float eps, theta;
    int kv_f16;   /* 0: FP32 KV as the reference; 1: K and V rounded to binary16 on append */
    int max_seq;  /* the reference caps at 2048 (:103); lifted here, caller chooses */
} jo_cfg;

typedef struct {
    jo_cfg cfg;
    jo_tensor glob[3];
    jo_tensor *layer; /* [layers][JO_T_COUNT] (entries 0..2 unused) */
} jo_model;

typedef struct {
    float *K, *V; /* [layers][max_seq][kvDim] */
} jo_seq;

jo_model *jo_model_create(const jo_cfg *cfg) {
    jo_model *m = (jo_model *)calloc(1, sizeof(jo_model));
    m->cfg = *cfg;
    m->layer = (jo_tensor *)calloc((size_t)cfg->layers * JO_T_COUNT, sizeof(jo_tensor));
    return m;
}
void jo_model_free(jo_model *m) {
    if (!m)
        return;
    free(m->layer);
    free(m);
}
/* tensor names → kinds: LlamaTransformerHandler.java:238-275 */
int jo_model_set_tensor(jo_model *m, int kind, int layer, const uint8_t *data, int type,
                        int64_t rows, int64_t cols) {
    jo_tensor t = {data, type, rows, cols};
    if (kind < 0 || kind >= JO_T_COUNT)
        return -1;
    if (kind <= JO_T_OUTPUT)
        m->glob[kind] = t;
    else {
        if (layer < 0 || layer >= m->cfg.layers)
            return -1;
        m->layer[(size_t)layer * JO_T_COUNT + kind] = t;
    }
    return 0;
}
jo_seq *jo_seq_create(const jo_model *m) {
    jo_seq *s = (jo_seq *)calloc(1, sizeof(jo_seq));
    size_t n = (size_t)m->cfg.layers * m->cfg.max_seq * m->cfg.kv_heads * m->cfg.head_dim;
    s->K = (float *)calloc(n, sizeof(float));
    s->V = (float *)calloc(n, sizeof(float));
    return s;
}
void jo_seq_free(jo_seq *s) {
    if (!s)
        return;
    free(s->K);
    free(s->V);
    free(s);
}

/* Benchmark helper (not part of the reference): fills positions [0, n_pos) of every layer's K and V with a
 * deterministic pseudo-random pattern in [-1, 1), so that a timed decode step attends over a context of that length
 * without running the n_pos forward passes that would normally produce it. */
void jo_seq_fill(jo_seq *s, const jo_model *m, int n_pos, unsigned seed) {
    const size_t kvDim = (size_t)m->cfg.kv_heads * m->cfg.head_dim, per_layer = (size_t)m->cfg.max_seq * kvDim;
    unsigned state = seed * 2654435761u + 12345u;
    for (int l = 0; l < m->cfg.layers; l++)
        for (size_t i = 0; i < (size_t)n_pos * kvDim; i++) {
            state = state * 1664525u + 1013904223u;
            s->K[l * per_layer + i] = (float)(int)(state >> 8) * (1.0f / 8388608.0f) - 1.0f;
            state = state * 1664525u + 1013904223u;
            s->V[l * per_layer + i] = (float)(int)(state >> 8) * (1.0f / 8388608.0f) - 1.0f;
        }
}

static void mv(const jo_tensor *t, const float *x, float *y) {
    jo_matvec(t->type, t->data, x, 0, t->rows, t->cols, y);
}

/* forward(): LlamaTransformerHandler.java:602-628 with getInitialActivation
 * :651-667, runLayers :670-717, transformerLayer :744-784, ffn :787-800,
 * outputProjection :803-810.  Returns 0, or -1 when pos >= max_seq.
 * `hidden_out` (optional) receives the residual stream after the last layer. */
int jo_forward(const jo_model *m, jo_seq *s, int token, int pos, float *logits, float *hidden_out) {
    const jo_cfg *c = &m->cfg;
    int H = c->hidden, kvDim = c->kv_heads * c->head_dim, I = c->inter;
    if (pos < 0 || pos >= c->max_seq)
        return -1;
    float *x = (float *)malloc(sizeof(float) * H), *xn = (float *)malloc(sizeof(float) * H);
    float *q = (float *)malloc(sizeof(float) * H), *k = (float *)malloc(sizeof(float) * kvDim);
    float *v = (float *)malloc(sizeof(float) * kvDim), *att = (float *)malloc(sizeof(float) * H);
    float *proj = (float *)malloc(sizeof(float) * H), *gate = (float *)malloc(sizeof(float) * I);
    float *up = (float *)malloc(sizeof(float) * I), *scores = (float *)malloc(sizeof(float) * (pos + 1));

    /* embedding row of the eagerly dequantised token_embd (:651-660) */
    int tok = token < 0 ? 0 : (token > c->vocab - 1 ? c->vocab - 1 : token);
    const jo_tensor *te = &m->glob[JO_T_TOKEN_EMBD];
    deq_row(te->type, te->data + (int64_t)tok * jo_row_bytes(te->type, te->cols), H, x);

    for (int li = 0; li < c->layers; li++) {
        const jo_tensor *L = m->layer + (size_t)li * JO_T_COUNT;
        float *Kc = s->K + (size_t)li * c->max_seq * kvDim, *Vc = s->V + (size_t)li * c->max_seq * kvDim;
        jo_rmsnorm(x, (const float *)L[JO_T_ATTN_NORM].data, H, c->eps, xn);
        mv(&L[JO_T_ATTN_Q], xn, q);
        mv(&L[JO_T_ATTN_K], xn, k);
        mv(&L[JO_T_ATTN_V], xn, v);
        if (L[JO_T_ATTN_Q_BIAS].data) { /* optional attn_{q,k,v}.bias, added before the rotation (:758-762) */
            const float *bq = (const float *)L[JO_T_ATTN_Q_BIAS].data, *bk = (const float *)L[JO_T_ATTN_K_BIAS].data,
                        *bv = (const float *)L[JO_T_ATTN_V_BIAS].data;
            for (int i = 0; i < H; i++) q[i] = q[i] + bq[i];
            for (int i = 0; i < kvDim; i++) {
                k[i] = k[i] + bk[i];
                v[i] = v[i] + bv[i];
            }
        }
        jo_rope(q, pos, c->heads, c->head_dim, c->theta);
        jo_rope(k, pos, c->kv_heads, c->head_dim, c->theta);
        for (int i = 0; i < kvDim; i++) {
            float kk = k[i], vv = v[i];
            if (c->kv_f16) {
                kk = jo_f16_to_f32(jo_f32_to_f16(kk));
                vv = jo_f16_to_f32(jo_f32_to_f16(vv));
            }
            Kc[(size_t)pos * kvDim + i] = kk;
            Vc[(size_t)pos * kvDim + i] = vv;
        }
        jo_gqa(q, Kc, Vc, pos + 1, c->heads, c->kv_heads, c->head_dim, att, scores);
        mv(&L[JO_T_ATTN_OUT], att, proj);
        for (int i = 0; i < H; i++)
            x[i] = x[i] + proj[i];
        jo_rmsnorm(x, (const float *)L[JO_T_FFN_NORM].data, H, c->eps, xn);
        mv(&L[JO_T_FFN_GATE], xn, gate);
        mv(&L[JO_T_FFN_UP], xn, up);
        for (int i = 0; i < I; i++)
            gate[i] = jo_silu(gate[i]) * up[i];
        mv(&L[JO_T_FFN_DOWN], gate, proj);
        for (int i = 0; i < H; i++)
            x[i] = x[i] + proj[i];
    }
    if (hidden_out)
        memcpy(hidden_out, x, sizeof(float) * H);
    if (logits) {
        jo_rmsnorm(x, (const float *)m->glob[JO_T_OUTPUT_NORM].data, H, c->eps, xn);
        /* tied-embedding fallback: :463-470 */
        const jo_tensor *out = m->glob[JO_T_OUTPUT].data ? &m->glob[JO_T_OUTPUT] : te;
        mv(out, xn, logits);
    }
    free(x); free(xn); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up);
    free(scores);
    return 0;
}

/* Decode driver: coordinator/.../GenerationLoop.java:306-334 — forward at
 * positions 0..P-2 on the prompt (logits discarded), then step s feeds the last
 * token at position P-1+s, picks greedily and appends.  `margins` (optional,
 * [steps]) receives logit(top1) - logit(top2) per step. */
int jo_generate_greedy(const jo_model *m, jo_seq *s, const int32_t *prompt, int P, int steps,
                       int32_t *out_ids, float *margins) {
    int V = m->cfg.vocab;
    float *logits = (float *)malloc(sizeof(float) * V), *probs = (float *)malloc(sizeof(float) * V);
    for (int p = 0; p < P - 1; p++)
        if (jo_forward(m, s, prompt[p], p, NULL, NULL))
            return -1;
    int last = prompt[P - 1];
    for (int st = 0; st < steps; st++) {
        if (jo_forward(m, s, last, P - 1 + st, logits, NULL))
            return -1;
        int best = jo_greedy(logits, V, probs);
        if (margins) {
            float second = -INFINITY;
            for (int i = 0; i < V; i++)
                if (i != best && logits[i] > second)
                    second = logits[i];
            margins[st] = logits[best] - second;
        }
        out_ids[st] = best;
        last = best;
    }
    free(logits);
    free(probs);
    return 0;
}

/* element-wise rank-ordered sum: juno-player/.../TensorParallelPipelineClient.java:244-272 */
void jo_allreduce_sum(const float *parts, int n_ranks, int n, float *out) {
    for (int i = 0; i < n; i++)
        out[i] = 0.f;
    for (int r = 0; r < n_ranks; r++)
        for (int i = 0; i < n; i++)
            out[i] += parts[(size_t)r * n + i];
}

int jo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void jo_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
