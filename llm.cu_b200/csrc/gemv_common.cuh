// Arithmetic helpers shared by the projection kernels: the per-stage dot products (mixed-precision
// FMA), the RMSNorm pieces, the multi-row warp reduction and the reference's SiLU.
#pragma once

#include "common.cuh"

namespace llmb {

// d += w.lo * x.lo (into a0) and w.hi * x.hi (into a1): FP16 x FP16 products are exact in FP32 and
// the sm_100 mixed-precision FMA rounds once, so this equals fmaf(float(w), float(x), acc) without
// the conversions.  Two accumulators per row keep two independent dependency chains.
__device__ __forceinline__ void fma2_f16(float &a0, float &a1, uint32_t w2, uint32_t x2) {
    asm("{\n\t.reg .f16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\t"
        "mov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
        : "+f"(a0), "+f"(a1)
        : "r"(w2), "r"(x2));
}

// Per-thread part of NR dot products over one ring stage: rows are `row_bytes` apart in shared
// memory, this thread owns the 16-byte chunks idx + stride * j (j < NJ, where have[j]); x holds the
// same chunks of the input row as packed FP16.  Loads for all rows are issued before the FMAs and
// the FMAs run row-interleaved, so NR * 2 independent chains are in flight.
template <int NR, int NJ, bool DUAL>
__device__ __forceinline__ void stage_dot_rows(const unsigned char *base, size_t row_bytes, int rows, int idx, int stride,
                                               const uint4 (&x)[NJ], const bool (&have)[NJ], float (&acc)[NR]) {
    constexpr int R = DUAL ? (NR > 1 ? NR / 2 : 1) : NR;
    constexpr int C = NR >= 4 ? 1 : 4 / NR;  // accumulator pairs per row: at least 8 chains in flight
    float a0[NR][C], a1[NR][C];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int c = 0; c < C; ++c) a0[r][c] = a1[r][c] = 0.0f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        if (have[j]) {
            uint4 w[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int rr = DUAL ? (r % R) : r;
                w[r] = (rr < rows) ? *reinterpret_cast<const uint4 *>(base + (size_t)r * row_bytes + (size_t)(idx + stride * j) * 16)
                                   : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int r = 0; r < NR; ++r) fma2_f16(a0[r][0 % C], a1[r][0 % C], w[r].x, x[j].x);
#pragma unroll
            for (int r = 0; r < NR; ++r) fma2_f16(a0[r][1 % C], a1[r][1 % C], w[r].y, x[j].y);
#pragma unroll
            for (int r = 0; r < NR; ++r) fma2_f16(a0[r][2 % C], a1[r][2 % C], w[r].z, x[j].z);
#pragma unroll
            for (int r = 0; r < NR; ++r) fma2_f16(a0[r][3 % C], a1[r][3 % C], w[r].w, x[j].w);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        float t0 = a0[r][0], t1 = a1[r][0];
#pragma unroll
        for (int c = 1; c < C; ++c) {
            t0 += a0[r][c];
            t1 += a1[r][c];
        }
        acc[r] = t0 + t1;
    }
}

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 t = __half22float2(h[e]);
        f[2 * e] = t.x;
        f[2 * e + 1] = t.y;
    }
}

// Sum of squares of 8 FP16 values as the two partials of the reference's RMSNorm reduction
// (inference.cu:309-313): one partial per four consecutive elements, left to right.
__device__ __forceinline__ void sumsq_partials(const uint4 &v, float &p0, float &p1) {
    float f[8];
    unpack8(v, f);
    p0 = __fmaf_rn(f[3], f[3], __fmaf_rn(f[2], f[2], __fmaf_rn(f[1], f[1], f[0] * f[0])));
    p1 = __fmaf_rn(f[7], f[7], __fmaf_rn(f[6], f[6], __fmaf_rn(f[5], f[5], f[4] * f[4])));
}

// half((x * g) / rms) for 8 values (inference.cu:355-358), repacked as FP16.
__device__ __forceinline__ uint4 rmsnorm_apply8(const uint4 &xv, const uint4 &gv, float rms) {
    float x[8], g[8];
    unpack8(xv, x);
    unpack8(gv, g);
    uint4 out;
    __half2 *o = reinterpret_cast<__half2 *>(&out);
#pragma unroll
    for (int e = 0; e < 4; ++e)
        o[e] = __halves2half2(__float2half_rn(__fdiv_rn(x[2 * e] * g[2 * e], rms)),
                              __float2half_rn(__fdiv_rn(x[2 * e + 1] * g[2 * e + 1], rms)));
    return out;
}

// Reduce NV per-lane values across the warp with NV-1 + (5 - log2 NV) shuffles.  Afterwards
// lane l holds the warp total of value index row_of_lane<NV>(l).
template <int NV>
__device__ __forceinline__ float warp_reduce_multi(float (&v)[NV], int lane) {
    int mask = 16;
#pragma unroll
    for (int step = NV / 2; step >= 1; step >>= 1) {
        bool hi = (lane & mask) != 0;
#pragma unroll
        for (int i = 0; i < step; ++i) {
            float send = hi ? v[i] : v[i + step];
            float keep = hi ? v[i + step] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
        }
        mask >>= 1;
    }
    float r = v[0];
    for (; mask >= 1; mask >>= 1) r += __shfl_xor_sync(0xffffffffu, r, mask);
    return r;
}

template <int NV>
__device__ __forceinline__ int row_of_lane(int lane) {
    int row = 0, mask = 16;
#pragma unroll
    for (int step = NV / 2; step >= 1; step >>= 1) {
        if (lane & mask) row += step;
        mask >>= 1;
    }
    return row;
}

// SiLU exactly as the reference writes it (inference.cu:451-453).
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

}  // namespace llmb
