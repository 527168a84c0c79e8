/*
 * Seeded synthetic weights and token ids, bit-identical on every host and device.
 *
 * The reference ships no weights (its model_weights/ directory is a placeholder), so every
 * test and benchmark draws random-init tensors "~N(0, 0.02)" from a seed.  To make the
 * same tensor reproducible in plain C, in numpy and inside a CUDA kernel, the draw uses
 * only integer arithmetic plus one IEEE fp32 multiply:
 *
 *   - two splitmix64 outputs per element give eight 16-bit uniforms;
 *   - their sum (Irwin-Hall, n = 8; variance 8/12 * 65536^2) is centred as an integer;
 *   - one fp32 multiply scales it to standard deviation `std`;
 *   - the fp32 value is rounded to BF16 or FP16 with round-to-nearest-even.
 *
 * Element `i` of tensor stream `sid` depends on (seed, sid, i) only, so any slice of any
 * tensor can be generated independently (tensor-parallel shards, device kernels).
 *
 * This header is plain C99 and also compiles as CUDA device code.
 */
#ifndef LLM_B200_SYNTH_H
#define LLM_B200_SYNTH_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define LLMB_HD __host__ __device__ __forceinline__
#else
#define LLMB_HD static inline
#endif

/* splitmix64 finaliser (public-domain constant set by Steele/Vigna). */
LLMB_HD uint64_t llmb_mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Key of one tensor stream: seed and stream id folded together. */
LLMB_HD uint64_t llmb_stream_key(uint64_t seed, uint64_t sid) {
    return llmb_mix64(seed * 0xD1342543DE82EF95ull + llmb_mix64(sid));
}

/* Approximately standard-normal fp32 value (Irwin-Hall n=8), exact on every platform. */
LLMB_HD float llmb_synth_unit(uint64_t key, uint64_t i) {
    uint64_t a = llmb_mix64(key + 2ull * i);
    uint64_t b = llmb_mix64(key + 2ull * i + 1ull);
    int32_t s = (int32_t)(a & 0xFFFF) + (int32_t)((a >> 16) & 0xFFFF) + (int32_t)((a >> 32) & 0xFFFF) +
                (int32_t)(a >> 48) + (int32_t)(b & 0xFFFF) + (int32_t)((b >> 16) & 0xFFFF) +
                (int32_t)((b >> 32) & 0xFFFF) + (int32_t)(b >> 48);
    s -= 4 * 65535; /* centre: mean of the sum is 8 * 32767.5 */
    /* 1 / (65536 * sqrt(8/12)) as an fp32 literal; one exact-by-IEEE multiply. */
    return (float)s * 1.8688567e-05f;
}

LLMB_HD uint32_t llmb_f32_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}

/* fp32 -> BF16 bits, round to nearest even (finite inputs only). */
LLMB_HD uint16_t llmb_f32_to_bf16(float f) {
    uint32_t u = llmb_f32_bits(f);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* fp32 -> FP16 bits, round to nearest even, subnormals and overflow handled. */
LLMB_HD uint16_t llmb_f32_to_fp16(float f) {
    uint32_t u = llmb_f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(sign | (a > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
    if (a < 0x33000001u) return (uint16_t)sign;               /* <= 2^-25 -> 0 (ties to even) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    if (e < -14) { /* subnormal half */
        uint32_t shift = (uint32_t)(-14 - e) + 13u;
        uint32_t q = m >> shift, r = m & ((1u << shift) - 1u), half = 1u << (shift - 1u);
        if (r > half || (r == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    uint32_t r = m & 0x1FFFu;
    if (r > 0x1000u || (r == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

/* One BF16 weight: N(0, std) draw, rounded to BF16. */
LLMB_HD uint16_t llmb_synth_bf16(uint64_t key, uint64_t i, float std) {
    return llmb_f32_to_bf16(llmb_synth_unit(key, i) * std);
}

/* One FP16 weight: N(0, std) draw, rounded to FP16. */
LLMB_HD uint16_t llmb_synth_fp16(uint64_t key, uint64_t i, float std) {
    return llmb_f32_to_fp16(llmb_synth_unit(key, i) * std);
}

/* Uniform token id in [0, vocab). */
LLMB_HD int32_t llmb_synth_token(uint64_t key, uint64_t i, int32_t vocab) {
    return (int32_t)(llmb_mix64(key + i) % (uint64_t)vocab);
}

/* Uniform fp32 in [0, 1) with 24 random bits: exact on every platform. */
LLMB_HD float llmb_synth_uniform(uint64_t key, uint64_t i) {
    return (float)(llmb_mix64(key + i) >> 40) * 5.9604644775390625e-08f; /* 2^-24 */
}

/*
 * Stream ids.  Layer tensors: 16 + 16 * layer + slot, slots in the order below.
 * The order of the slots is the field order of the reference's Llama3Layer struct
 * (src/llama3/llama3.cuh:28-39).
 */
enum {
    LLMB_SID_EMBED = 1,
    LLMB_SID_LM_HEAD = 2,
    LLMB_SID_NORM = 3,
    LLMB_SID_TOKENS = 4,
    LLMB_SID_SAMPLER = 5,
    LLMB_SLOT_INPUT_LAYERNORM = 0,
    LLMB_SLOT_DOWN = 1,
    LLMB_SLOT_GATE = 2,
    LLMB_SLOT_UP = 3,
    LLMB_SLOT_POST_LAYERNORM = 4,
    LLMB_SLOT_K = 5,
    LLMB_SLOT_O = 6,
    LLMB_SLOT_Q = 7,
    LLMB_SLOT_V = 8
};
#define LLMB_LAYER_SID(layer, slot) (16ull + 16ull * (uint64_t)(layer) + (uint64_t)(slot))

#endif /* LLM_B200_SYNTH_H */
