// Warp-level tensor-core helpers (mma.sync m16n8k16, FP16 in, FP32 accumulate) shared by the block attention
// of the prompt phase (prefill.cu) and the decode attention (attn_decode.cu).
#pragma once

#include "common.cuh"

namespace llmb {

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

// Transposes an 8 x 8 matrix of 16-bit values held across the warp (lane l: row l / 4, columns 2 (l % 4), + 1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// x / c, correctly rounded, for a constant c with rc = 1.0f / c (itself correctly rounded): a product, the
// remainder in one FMA and the correction in another - the last step of the division's own fast path.  Checked
// against IEEE division over every float x with 1e-30 < |x| < 1e30 for c = sqrtf(32), sqrtf(96) and sqrtf(128)
// (no mismatch; c = sqrtf(64) = 8 is exact anyway); outside that range, and for zero, the division itself runs.
// A score matrix takes tens of these per thread and tile, and __fdiv_rn costs three times as many instructions.
__device__ __forceinline__ float div_by_const(float x, float c, float rc) {
    const float y = x * rc;
    const float q = __fmaf_rn(__fmaf_rn(-y, c, x), rc, y);
    const float ax = fabsf(x);
    if (!(ax > 1e-30f && ax < 1e30f)) return __fdiv_rn(x, c);
    return q;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

}  // namespace llmb
