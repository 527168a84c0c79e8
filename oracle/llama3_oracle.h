/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's per-token forward loop
 * (abhisheknair10/LLM.cu, src/inference/inference.cu and src/llama3/llama3.cu).  It is the
 * checker for the CUDA engine and the timed CPU baseline; nothing in the product path may
 * link or call it.
 *
 * Parity status: the reference's own tests hold no golden vectors for this path
 * (tests/gemm.cu and tests/llama3.py assert nothing), so this restatement is pinned against
 * outputs of the reference itself: the patched reference CUDA build (oracle/_ref) run on a
 * B200 on seeded weights, committed as tests/golden/ref_*.npz.
 */
#ifndef LLAMA3_ORACLE_H
#define LLAMA3_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int n_layers;
    int d_model;
    int n_q_heads;
    int n_kv_heads;
    int head_dim;
    int ffn;
    int vocab;
    float rope_theta; /* 500000 in the reference (inference.cu:673) */
    double eps;       /* 1e-5: a double literal in the reference (inference.cu:351), added in double */
} OracleConfig;

/* Index of each tensor in the flat weight-pointer array handed to the oracle. */
enum {
    ORC_EMBED = 0,
    ORC_LM_HEAD = 1,
    ORC_NORM = 2,
    ORC_LAYER0 = 3, /* then 9 per layer, in the reference's Llama3Layer field order */
    ORC_INPUT_LAYERNORM = 0,
    ORC_DOWN = 1,
    ORC_GATE = 2,
    ORC_UP = 3,
    ORC_POST_LAYERNORM = 4,
    ORC_K = 5,
    ORC_O = 6,
    ORC_Q = 7,
    ORC_V = 8,
    ORC_PER_LAYER = 9
};

/* llama3.cu:240-254  BF16 -> FP32 (shift) -> FP16 RN. */
void oracle_bf16_to_fp16(const uint16_t *bf16, uint16_t *fp16, size_t n);

/*
 * One causal pass over `n_tokens` tokens (inference.cu:149-193 with h_NUM_TOKENS = n_tokens),
 * every FP16 rounding point and FP32 summation order of the reference kept.  Because the
 * reference recomputes the whole sequence on each call and its row r never depends on rows
 * > r, row r of this pass equals the last row of the reference's call with r+1 tokens:
 * teacher-forced logits for all steps come from one pass.
 *
 * weights   : 3 + 9*n_layers pointers to FP16 bit patterns, row-major [out,in].
 * logits    : FP16 bits, [n_tokens - first_logit_row][vocab] (rows first_logit_row..n_tokens-1).
 * hidden    : optional (may be NULL) FP16 bits [n_layers + 1][n_tokens][d_model]: the residual
 *             stream after the embedding and after each layer.
 * Returns 0 on success.
 */
int oracle_forward(const OracleConfig *cfg, const uint16_t *const *weights, const int32_t *tokens,
                   int n_tokens, int first_logit_row, uint16_t *logits, uint16_t *hidden);

/* First maximum over FP16 logits (NaN never wins), the tie-break the engine must match. */
int oracle_argmax_fp16(const uint16_t *logits, int n);
/* inference.cu:1030-1161 with ties to the lower index and the uniform number as an argument. */
int oracle_sample(const uint16_t *logits, int vocab, float temperature, int top_k, float top_p, float u);
float oracle_sampler_uniform(uint64_t seed, uint64_t draw);

/*
 * KV-cached decode used as the timed CPU baseline: same rounding points, but dot products are
 * summed in 16 interleaved FP32 lanes (not strictly ascending k) so they vectorise.
 */
typedef struct OracleDecoder OracleDecoder;
OracleDecoder *oracle_decoder_new(const OracleConfig *cfg, const uint16_t *const *weights, int max_pos);
void oracle_decoder_free(OracleDecoder *dec);
void oracle_decoder_reset(OracleDecoder *dec);
/* Feed one token at the next position; writes FP16 logits (may be NULL); returns argmax. */
int oracle_decoder_step(OracleDecoder *dec, int32_t token, uint16_t *logits);

/* Synthetic data (include/llm_b200_synth.h), OpenMP-parallel. */
void oracle_synth_bf16(uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n, uint16_t *out);
void oracle_synth_fp16(uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n, uint16_t *out);
void oracle_synth_tokens(uint64_t seed, uint64_t sid, int32_t vocab, uint64_t first, uint64_t n, int32_t *out);
void oracle_fill_u16(uint16_t value, uint64_t n, uint16_t *out);

int oracle_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
