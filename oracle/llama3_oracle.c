/*
 * TEST INFRASTRUCTURE ONLY: CPU restatement of the reference forward loop.  See
 * llama3_oracle.h for the contract and the parity status.  Every function cites the
 * reference lines (paths inside abhisheknair10/LLM.cu) whose arithmetic it follows.
 *
 * Build: gcc -O3 -fopenmp -mavx2 -mfma -mf16c -ffp-contract=off -shared -fPIC.
 * Contraction is off so that each FMA below is an explicit decision: nvcc fuses
 * `acc += a * b` into one FMA; where the product is exact in FP32 (FP16 x FP16) that makes
 * no difference, where it is not (softmax weight x V, RoPE) fmaf() is written out.
 */
#include "llama3_oracle.h"

#include <float.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../include/llm_b200_synth.h"

static inline float h2f(uint16_t h) {
    _Float16 x;
    memcpy(&x, &h, 2);
    return (float)x;
}
/* __float2half / __float2half_rn: round to nearest even. */
static inline uint16_t f2h(float f) {
    _Float16 x = (_Float16)f;
    uint16_t h;
    memcpy(&h, &x, 2);
    return h;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* llama3.cu:240-254 */
void oracle_bf16_to_fp16(const uint16_t *bf16, uint16_t *fp16, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint32_t bits = (uint32_t)bf16[i] << 16;
        float f;
        memcpy(&f, &bits, 4);
        fp16[i] = f2h(f);
    }
}

/* ------------------------------------------------------------------------------------ */
/* Strict-order building blocks                                                          */
/* ------------------------------------------------------------------------------------ */

/*
 * inference.cu:393-449 (kernel_standard_tiled_gemm): O[t][n] = sum_k X[t][k] * W[n][k], FP32
 * accumulator, k strictly ascending (tiles of 32 k, low half then high half of each half2).
 * Returns the raw FP32 accumulators; the caller rounds (inference.cu:445) or feeds SwiGLU
 * (inference.cu:515).  Tokens sit in the SIMD lanes so every (t, n) chain keeps its order.
 */
#define TB 64
static void matmul_strict(const uint16_t *X, const uint16_t *W, int T, int N, int K, float *out) {
    int Tp = (T + TB - 1) / TB * TB;
    float *XT = (float *)aligned_alloc(64, (size_t)K * Tp * sizeof(float));
    for (int k = 0; k < K; ++k)
        for (int t = 0; t < Tp; ++t) XT[(size_t)k * Tp + t] = t < T ? h2f(X[(size_t)t * K + k]) : 0.0f;
#pragma omp parallel for schedule(dynamic, 16)
    for (int n = 0; n < N; ++n) {
        const uint16_t *w = W + (size_t)n * K;
        for (int t0 = 0; t0 < Tp; t0 += TB) {
            float acc[TB];
            for (int j = 0; j < TB; ++j) acc[j] = 0.0f;
            for (int k = 0; k < K; ++k) {
                float wf = h2f(w[k]);
                const float *x = XT + (size_t)k * Tp + t0;
                for (int j = 0; j < TB; ++j) acc[j] += wf * x[j]; /* product exact in FP32 */
            }
            for (int j = 0; j < TB && t0 + j < T; ++j) out[(size_t)(t0 + j) * N + n] = acc[j];
        }
    }
    free(XT);
}

static int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

/* The reduction order of a 1024-slot shared-memory tree followed by __shfl_down
 * (inference.cu:321-344, :829-834, :862-867): buf[i] += buf[i + offset], offset halving. */
static float tree_sum(float *buf, int n_pow2) {
    for (int off = n_pow2 / 2; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) buf[i] += buf[i + off];
    return buf[0];
}

/*
 * inference.cu:293-363 (kernel_compute_rms_norm), in place on one row.  One "thread" per four
 * consecutive elements; sum of squares left to right, then the tree.  `1e-5 + ...` is a double
 * addition in the reference (the literal is a double), narrowed for sqrtf.
 * The reference fixes d = 4096 (1024 threads); other d use d/4 threads padded to a power of 2.
 */
static void rmsnorm_row(uint16_t *x, const uint16_t *g, int d, double eps) {
    int nt = d / 4, np = next_pow2(nt);
    float *buf = (float *)alloca(sizeof(float) * np);
    for (int t = 0; t < np; ++t) {
        if (t < nt) {
            float a = h2f(x[4 * t]), b = h2f(x[4 * t + 1]), c = h2f(x[4 * t + 2]), e = h2f(x[4 * t + 3]);
            buf[t] = ((a * a + b * b) + c * c) + e * e;
        } else {
            buf[t] = 0.0f;
        }
    }
    float sum = tree_sum(buf, np);
    float rms = sqrtf((float)(eps + (double)(sum / (float)d)));
    for (int i = 0; i < d; ++i) x[i] = f2h(h2f(x[i]) * h2f(g[i]) / rms);
}

/* inference.cu:377-390 (kernel_add_norm): X = half(float(X) + float(PN_X)). */
static void add_rows(uint16_t *x, const uint16_t *r, size_t n) {
    for (size_t i = 0; i < n; ++i) x[i] = f2h(h2f(x[i]) + h2f(r[i]));
}

/*
 * inference.cu:640-695 (kernel_rope_scaling) with the stray parenthesis of line 673 removed:
 * interleaved pairs (x[2i], x[2i+1]), i = pair index inside the head, angle = pos * theta^(-2i/hd),
 * FP32 powf/cosf/sinf, in place, rounded to FP16.  a*b - c*d and a*b + c*d are written the way
 * nvcc contracts them: the first product is fused into the add.
 */
static void rope_row(uint16_t *row, int n_heads, int hd, int pos, float theta) {
    int half = hd / 2;
    for (int p = 0; p < n_heads * half; ++p) {
        int i = p % half;
        float even = h2f(row[2 * p]), odd = h2f(row[2 * p + 1]);
        float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)hd);
        float angle = (float)pos * freq;
        float c = cosf(angle), s = sinf(angle);
        float re = fmaf(c, even, -(s * odd));
        float ro = fmaf(s, even, c * odd);
        row[2 * p] = f2h(re);
        row[2 * p + 1] = f2h(ro);
    }
}

/* inference.cu:451-453 */
static inline float silu(float x) { return x / (1.0f + expf(-x)); }

/*
 * inference.cu:698-947: scores = (q . k) / sqrtf(hd) over FP16 inputs in FP32, ascending d
 * (:776-778, :784); causal mask + max-subtracted softmax with the 1024-thread tree sums
 * (:790-890); out = sum_t P[t] * V[t] ascending t with FMA (:934-938), rounded to FP16 (:945).
 * KV head of query head h is h / group (:752, :908).  `out` rows are [T][n_q*hd].
 */
static void attention_strict(const OracleConfig *c, const uint16_t *Q, const uint16_t *Kc, const uint16_t *Vc,
                             int T, uint16_t *out) {
    int hd = c->head_dim, nq = c->n_q_heads, nkv = c->n_kv_heads, group = nq / nkv;
    float inv_den = sqrtf((float)hd);
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int h = 0; h < nq; ++h) {
        for (int r = 0; r < T; ++r) {
            int g = h / group;
            int n = r + 1;
            float *s = (float *)malloc(sizeof(float) * (size_t)(n + 1024));
            float *buf = s + n;
            const uint16_t *q = Q + (size_t)r * nq * hd + (size_t)h * hd;
            float maxv = -FLT_MAX;
            for (int col = 0; col < n; ++col) {
                const uint16_t *k = Kc + (size_t)col * nkv * hd + (size_t)g * hd;
                float v = 0.0f;
                for (int d = 0; d < hd; ++d) v += h2f(q[d]) * h2f(k[d]);
                v = v / inv_den;
                s[col] = v;
                if (v > maxv) maxv = v;
            }
            for (int t = 0; t < 1024; ++t) buf[t] = 0.0f;
            for (int col = 0; col < n; ++col) { /* thread t owns cols t, t+1024, ... in order */
                float e = expf(s[col] - maxv);
                s[col] = e;
                buf[col & 1023] += e;
            }
            float den = tree_sum(buf, 1024);
            float acc[512];
            for (int d = 0; d < hd; ++d) acc[d] = 0.0f;
            for (int t = 0; t < n; ++t) {
                float p = s[t] / den;
                const uint16_t *v = Vc + (size_t)t * nkv * hd + (size_t)g * hd;
                for (int d = 0; d < hd; ++d) acc[d] = fmaf(p, h2f(v[d]), acc[d]);
            }
            uint16_t *o = out + (size_t)r * nq * hd + (size_t)h * hd;
            for (int d = 0; d < hd; ++d) o[d] = f2h(acc[d]);
            free(s);
        }
    }
}

static void round_rows(const float *acc, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = f2h(acc[i]);
}

int oracle_forward(const OracleConfig *c, const uint16_t *const *w, const int32_t *tokens, int T,
                   int first_logit_row, uint16_t *logits, uint16_t *hidden) {
    int d = c->d_model, hd = c->head_dim, nq = c->n_q_heads, nkv = c->n_kv_heads, F = c->ffn, V = c->vocab;
    if (T <= 0 || d % 4 || hd > 512 || nq % nkv || first_logit_row < 0 || first_logit_row > T) return 1;
    int dq = nq * hd, dkv = nkv * hd;
    size_t big = (size_t)T * (size_t)(F > dq ? (F > d ? F : d) : (dq > d ? dq : d));
    uint16_t *X = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * d);
    uint16_t *PN = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * d);
    uint16_t *Q = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * dq);
    uint16_t *Kb = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * dkv);
    uint16_t *Vb = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * dkv);
    uint16_t *A = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * dq);
    uint16_t *H = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)T * F);
    float *acc = (float *)malloc(sizeof(float) * big);
    float *acc2 = (float *)malloc(sizeof(float) * (size_t)T * F);
    if (!X || !PN || !Q || !Kb || !Vb || !A || !H || !acc || !acc2) return 2;

    /* inference.cu:209-223: X[t] = Embed[token[t]] */
    for (int t = 0; t < T; ++t) {
        if (tokens[t] < 0) return 3;
        memcpy(X + (size_t)t * d, w[ORC_EMBED] + (size_t)tokens[t] * d, sizeof(uint16_t) * d);
    }
    if (hidden) memcpy(hidden, X, sizeof(uint16_t) * (size_t)T * d);

    for (int l = 0; l < c->n_layers; ++l) {
        const uint16_t *const *lw = w + ORC_LAYER0 + ORC_PER_LAYER * l;
        /* :159-160 snapshot + input_layernorm */
        memcpy(PN, X, sizeof(uint16_t) * (size_t)T * d);
        for (int t = 0; t < T; ++t) rmsnorm_row(X + (size_t)t * d, lw[ORC_INPUT_LAYERNORM], d, c->eps);
        /* :163 q, k, v, each rounded to FP16 (:445) */
        matmul_strict(X, lw[ORC_Q], T, dq, d, acc);
        round_rows(acc, Q, (size_t)T * dq);
        matmul_strict(X, lw[ORC_K], T, dkv, d, acc);
        round_rows(acc, Kb, (size_t)T * dkv);
        matmul_strict(X, lw[ORC_V], T, dkv, d, acc);
        round_rows(acc, Vb, (size_t)T * dkv);
        /* :166 RoPE on Q and K, position = row index */
        for (int t = 0; t < T; ++t) {
            rope_row(Q + (size_t)t * dq, nq, hd, t, c->rope_theta);
            rope_row(Kb + (size_t)t * dkv, nkv, hd, t, c->rope_theta);
        }
        /* :169 attention into X; :172 o_proj; :175 residual add */
        attention_strict(c, Q, Kb, Vb, T, A);
        matmul_strict(A, lw[ORC_O], T, d, dq, acc);
        round_rows(acc, X, (size_t)T * d);
        add_rows(X, PN, (size_t)T * d);
        /* :178-179 snapshot + post_attention_layernorm */
        memcpy(PN, X, sizeof(uint16_t) * (size_t)T * d);
        for (int t = 0; t < T; ++t) rmsnorm_row(X + (size_t)t * d, lw[ORC_POST_LAYERNORM], d, c->eps);
        /* :182 feed-forward: half(SiLU(gate_f32) * up_f32) (:515), then down (:973), :185 add */
        matmul_strict(X, lw[ORC_GATE], T, F, d, acc);
        matmul_strict(X, lw[ORC_UP], T, F, d, acc2);
        for (size_t i = 0; i < (size_t)T * F; ++i) H[i] = f2h(silu(acc[i]) * acc2[i]);
        matmul_strict(H, lw[ORC_DOWN], T, d, F, acc);
        round_rows(acc, X, (size_t)T * d);
        add_rows(X, PN, (size_t)T * d);
        if (hidden) memcpy(hidden + (size_t)(l + 1) * T * d, X, sizeof(uint16_t) * (size_t)T * d);
    }
    /* :188 final norm (all rows), :1014-1018 lm_head on the wanted rows, FP16 logits */
    int rows = T - first_logit_row;
    if (rows > 0 && logits) {
        for (int t = first_logit_row; t < T; ++t) rmsnorm_row(X + (size_t)t * d, w[ORC_NORM], d, c->eps);
        float *lacc = (float *)malloc(sizeof(float) * (size_t)rows * V);
        if (!lacc) return 2;
        matmul_strict(X + (size_t)first_logit_row * d, w[ORC_LM_HEAD], rows, V, d, lacc);
        round_rows(lacc, logits, (size_t)rows * V);
        free(lacc);
    }
    free(X); free(PN); free(Q); free(Kb); free(Vb); free(A); free(H); free(acc); free(acc2);
    return 0;
}

int oracle_argmax_fp16(const uint16_t *logits, int n) {
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < n; ++i) {
        float v = h2f(logits[i]);
        if (v > bv) { bv = v; best = i; }
    }
    return best;
}

/*
 * inference.cu:1030-1161 (sample_next_token and its helpers), statement by statement, on a full
 * sorted copy of the distribution.  Two things are pinned down that the reference leaves open:
 * ties in the descending order go to the lower index (its qsort comparator returns 0 for them),
 * and the uniform number is an argument (it calls an unseeded rand()).  The top-k pass still
 * renormalises the first k entries in place before the top-p pass reads them; its own pick is
 * discarded there and not computed here.
 */
typedef struct { float probability; int index; } OracleProbIndex;

static int cmp_prob_desc(const void *a, const void *b) {
    const OracleProbIndex *x = (const OracleProbIndex *)a, *y = (const OracleProbIndex *)b;
    if (x->probability < y->probability) return 1;
    if (x->probability > y->probability) return -1;
    return (x->index > y->index) - (x->index < y->index);
}

int oracle_sample(const uint16_t *logits, int vocab, float temperature, int top_k, float top_p, float u) {
    OracleProbIndex *d = (OracleProbIndex *)malloc(sizeof(OracleProbIndex) * (size_t)vocab);
    float *t = (float *)malloc(sizeof(float) * (size_t)vocab);
    if (!d || !t) { free(d); free(t); return -1; }
    float cumsum = 0.0f;
    for (int i = 0; i < vocab; ++i) { /* :1044-1050 */
        float scaled = h2f(logits[i]) / temperature;
        t[i] = expf(scaled);
        cumsum += t[i];
    }
    for (int i = 0; i < vocab; ++i) { /* :1052-1057 */
        t[i] /= cumsum;
        d[i].probability = t[i];
        d[i].index = i;
    }
    qsort(d, (size_t)vocab, sizeof(OracleProbIndex), cmp_prob_desc); /* :1059 */
    int k = top_k > vocab ? vocab : top_k; /* :1083-1085 */
    float sum = 0.0f;
    for (int i = 0; i < k; ++i) sum += d[i].probability;  /* :1088-1091 */
    for (int i = 0; i < k; ++i) d[i].probability /= sum;  /* :1094-1096 */
    float p = top_p > 1.0f ? 1.0f : top_p; /* :1124-1126 */
    float cumulative = 0.0f;
    int cutoff = 0;
    for (; cutoff < vocab; ++cutoff) { /* :1131-1136 */
        cumulative += d[cutoff].probability;
        if (cumulative >= p) break;
    }
    sum = cumulative;
    if (cutoff >= vocab) cutoff = vocab - 1; /* :1140-1143 */
    for (int i = 0; i <= cutoff; ++i) d[i].probability /= sum; /* :1146-1148 */
    int token = d[0].index; /* :1159-1160 */
    cumulative = 0.0f;
    for (int i = 0; i <= cutoff; ++i) { /* :1154-1158 */
        cumulative += d[i].probability;
        if (u < cumulative) { token = d[i].index; break; }
    }
    free(d);
    free(t);
    return token;
}

float oracle_sampler_uniform(uint64_t seed, uint64_t draw) {
    return llmb_synth_uniform(llmb_stream_key(seed, LLMB_SID_SAMPLER), draw);
}

/* ------------------------------------------------------------------------------------ */
/* KV-cached decoder (timed CPU baseline; same rounding points, vectorised sums)         */
/* ------------------------------------------------------------------------------------ */

struct OracleDecoder {
    OracleConfig c;
    const uint16_t *const *w;
    int max_pos, pos;
    uint16_t *kc, *vc; /* [layer][pos][kv_head][hd] */
    uint16_t *x, *pn, *q, *a, *h, *lg;
    float *xf;
};

static float dot16(const uint16_t *w, const float *x, int K) {
    float acc[16];
    for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
    int k = 0;
    for (; k + 16 <= K; k += 16)
        for (int j = 0; j < 16; ++j) acc[j] += h2f(w[k + j]) * x[k + j];
    float s = 0.0f;
    for (int j = 0; j < 16; ++j) s += acc[j];
    for (; k < K; ++k) s += h2f(w[k]) * x[k];
    return s;
}

static void gemv_fast(const uint16_t *W, const uint16_t *x, float *xf, int N, int K, float *out) {
    for (int k = 0; k < K; ++k) xf[k] = h2f(x[k]);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n) out[n] = dot16(W + (size_t)n * K, xf, K);
}

OracleDecoder *oracle_decoder_new(const OracleConfig *cfg, const uint16_t *const *weights, int max_pos) {
    OracleDecoder *dec = (OracleDecoder *)calloc(1, sizeof(OracleDecoder));
    if (!dec) return NULL;
    dec->c = *cfg;
    dec->w = weights;
    dec->max_pos = max_pos;
    int dkv = cfg->n_kv_heads * cfg->head_dim, dq = cfg->n_q_heads * cfg->head_dim;
    size_t kvn = (size_t)cfg->n_layers * max_pos * dkv;
    int widest = cfg->ffn > cfg->d_model ? cfg->ffn : cfg->d_model;
    if (dq > widest) widest = dq;
    dec->kc = (uint16_t *)calloc(kvn, 2);
    dec->vc = (uint16_t *)calloc(kvn, 2);
    dec->x = (uint16_t *)calloc(cfg->d_model, 2);
    dec->pn = (uint16_t *)calloc(cfg->d_model, 2);
    dec->q = (uint16_t *)calloc(dq, 2);
    dec->a = (uint16_t *)calloc(dq, 2);
    dec->h = (uint16_t *)calloc(cfg->ffn, 2);
    dec->lg = (uint16_t *)calloc(cfg->vocab, 2);
    dec->xf = (float *)calloc((size_t)widest, 4);
    return dec;
}

void oracle_decoder_free(OracleDecoder *dec) {
    if (!dec) return;
    free(dec->kc); free(dec->vc); free(dec->x); free(dec->pn); free(dec->q); free(dec->a);
    free(dec->h); free(dec->lg); free(dec->xf); free(dec);
}

void oracle_decoder_reset(OracleDecoder *dec) { dec->pos = 0; }

int oracle_decoder_step(OracleDecoder *dec, int32_t token, uint16_t *logits) {
    const OracleConfig *c = &dec->c;
    int d = c->d_model, hd = c->head_dim, nq = c->n_q_heads, nkv = c->n_kv_heads, F = c->ffn, V = c->vocab;
    int dq = nq * hd, dkv = nkv * hd, group = nq / nkv, pos = dec->pos;
    if (pos >= dec->max_pos) return -1;
    int widest = F > V ? F : V;
    if (dq > widest) widest = dq;
    float *acc = (float *)malloc(sizeof(float) * (size_t)widest * 2);
    float *acc2 = acc + widest;
    memcpy(dec->x, dec->w[ORC_EMBED] + (size_t)token * d, 2 * (size_t)d);
    for (int l = 0; l < c->n_layers; ++l) {
        const uint16_t *const *lw = dec->w + ORC_LAYER0 + ORC_PER_LAYER * l;
        uint16_t *kl = dec->kc + ((size_t)l * dec->max_pos) * dkv;
        uint16_t *vl = dec->vc + ((size_t)l * dec->max_pos) * dkv;
        memcpy(dec->pn, dec->x, 2 * (size_t)d);
        rmsnorm_row(dec->x, lw[ORC_INPUT_LAYERNORM], d, c->eps);
        gemv_fast(lw[ORC_Q], dec->x, dec->xf, dq, d, acc);
        round_rows(acc, dec->q, dq);
        gemv_fast(lw[ORC_K], dec->x, dec->xf, dkv, d, acc);
        round_rows(acc, kl + (size_t)pos * dkv, dkv);
        gemv_fast(lw[ORC_V], dec->x, dec->xf, dkv, d, acc);
        round_rows(acc, vl + (size_t)pos * dkv, dkv);
        rope_row(dec->q, nq, hd, pos, c->rope_theta);
        rope_row(kl + (size_t)pos * dkv, nkv, hd, pos, c->rope_theta);
        float scale_den = sqrtf((float)hd);
#pragma omp parallel for schedule(static)
        for (int h = 0; h < nq; ++h) {
            int g = h / group, n = pos + 1;
            float *s = (float *)malloc(sizeof(float) * (size_t)n);
            float qf[512], o[512];
            for (int i = 0; i < hd; ++i) { qf[i] = h2f(dec->q[h * hd + i]); o[i] = 0.0f; }
            float maxv = -FLT_MAX, den = 0.0f;
            for (int t = 0; t < n; ++t) {
                s[t] = dot16(kl + (size_t)t * dkv + (size_t)g * hd, qf, hd) / scale_den;
                if (s[t] > maxv) maxv = s[t];
            }
            for (int t = 0; t < n; ++t) { s[t] = expf(s[t] - maxv); den += s[t]; }
            for (int t = 0; t < n; ++t) {
                float p = s[t] / den;
                const uint16_t *v = vl + (size_t)t * dkv + (size_t)g * hd;
                for (int i = 0; i < hd; ++i) o[i] = fmaf(p, h2f(v[i]), o[i]);
            }
            for (int i = 0; i < hd; ++i) dec->a[h * hd + i] = f2h(o[i]);
            free(s);
        }
        gemv_fast(lw[ORC_O], dec->a, dec->xf, d, dq, acc);
        round_rows(acc, dec->x, d);
        add_rows(dec->x, dec->pn, d);
        memcpy(dec->pn, dec->x, 2 * (size_t)d);
        rmsnorm_row(dec->x, lw[ORC_POST_LAYERNORM], d, c->eps);
        gemv_fast(lw[ORC_GATE], dec->x, dec->xf, F, d, acc);
        gemv_fast(lw[ORC_UP], dec->x, dec->xf, F, d, acc2);
        for (int i = 0; i < F; ++i) dec->h[i] = f2h(silu(acc[i]) * acc2[i]);
        gemv_fast(lw[ORC_DOWN], dec->h, dec->xf, d, F, acc);
        round_rows(acc, dec->x, d);
        add_rows(dec->x, dec->pn, d);
    }
    rmsnorm_row(dec->x, dec->w[ORC_NORM], d, c->eps);
    gemv_fast(dec->w[ORC_LM_HEAD], dec->x, dec->xf, V, d, acc);
    round_rows(acc, dec->lg, V);
    if (logits) memcpy(logits, dec->lg, 2 * (size_t)V);
    free(acc);
    dec->pos = pos + 1;
    return oracle_argmax_fp16(dec->lg, V);
}

/* ------------------------------------------------------------------------------------ */
/* Synthetic data                                                                        */
/* ------------------------------------------------------------------------------------ */

void oracle_synth_bf16(uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n, uint16_t *out) {
    uint64_t key = llmb_stream_key(seed, sid);
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; ++i) out[i] = llmb_synth_bf16(key, first + i, std);
}

void oracle_synth_fp16(uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n, uint16_t *out) {
    uint64_t key = llmb_stream_key(seed, sid);
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; ++i) out[i] = llmb_synth_fp16(key, first + i, std);
}

void oracle_synth_tokens(uint64_t seed, uint64_t sid, int32_t vocab, uint64_t first, uint64_t n, int32_t *out) {
    uint64_t key = llmb_stream_key(seed, sid);
    for (uint64_t i = 0; i < n; ++i) out[i] = llmb_synth_token(key, first + i, vocab);
}

void oracle_fill_u16(uint16_t value, uint64_t n, uint16_t *out) {
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; ++i) out[i] = value;
}
