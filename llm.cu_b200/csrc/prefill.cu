// Row-batched kernels of the prompt phase, beside the tensor-core projections (gemm_tc.cu):
//
//   rmsnorm_rows   RMSNorm of M rows (replaces kernel_compute_rms_norm + kernel_compute_norm_tensor,
//                  inference.cu:272-375, for M rows at once): same partials of four elements, same
//                  binary reduction tree, eps added in double, IEEE division, FP16 rounding.
//   attn_prefill   causal attention of M new rows against the KV cache (replaces compute_attention's
//                  three kernels, inference.cu:698-947): scores (q.k)/sqrtf(head_dim) in FP32 from
//                  FP16, softmax in FP32 (online, never materialising the N x N matrix), P.V in FP32,
//                  FP16 out.  K and V come from the cache rows the QKV projection just appended, so a
//                  chunk that starts at position pos0 > 0 attends to the earlier rows as well.
//   iota           positions pos0 .. pos0 + n - 1 for the embedding / RoPE-angle prologue.
//
// attn_prefill runs on the CUDA cores (32 query rows x one head per CTA, 32-row K/V tiles staged in
// shared memory); it is bound by FP32 FMA issue, not by memory.
#include "common.cuh"
#include "gemv_common.cuh"

namespace llmb {

constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_rows_kernel(const __half *__restrict__ x, const __half *__restrict__ gamma, __half *__restrict__ y, int d,
                    int n_pow2, double eps) {
    extern __shared__ float norm_part[];  // n_pow2 partials (d / 4 real ones, zero padded)
    __shared__ float rms_s;
    const int row = blockIdx.x, tid = threadIdx.x;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * d);
    const int nchunks = d >> 3;
    for (int c = tid; c < (n_pow2 >> 1); c += kNormThreads) {
        float p0 = 0.0f, p1 = 0.0f;
        if (c < nchunks) sumsq_partials(xr[c], p0, p1);
        norm_part[2 * c] = p0;
        norm_part[2 * c + 1] = p1;
    }
    __syncthreads();
    for (int off = n_pow2 >> 1; off >= 1; off >>= 1) {
        for (int t = tid; t < off; t += kNormThreads) norm_part[t] += norm_part[t + off];
        __syncthreads();
    }
    if (tid == 0) rms_s = sqrtf((float)(eps + (double)(norm_part[0] / (float)d)));
    __syncthreads();
    const float rms = rms_s;
    uint4 *yr = reinterpret_cast<uint4 *>(y + (size_t)row * d);
    const uint4 *gr = reinterpret_cast<const uint4 *>(gamma);
    for (int c = tid; c < nchunks; c += kNormThreads) yr[c] = rmsnorm_apply8(xr[c], __ldg(gr + c), rms);
}

constexpr int kPfRows = 32;     // query rows per CTA
constexpr int kPfTile = 32;     // K/V rows per shared-memory tile
constexpr int kPfThreads = 128; // 4 threads per query row

template <int HD>
__global__ void __launch_bounds__(kPfThreads)
attn_prefill_kernel(const __half *__restrict__ q, const __half *__restrict__ k_cache, const __half *__restrict__ v_cache,
                    __half *__restrict__ out, int m, int pos0, int n_q_heads, int n_kv_heads) {
    constexpr int KP = HD + 8;  // padded K row: the four key rows a quad reads fall in different banks
    constexpr int DQ = HD / 4;  // output columns per thread
    __shared__ __align__(16) __half k_s[kPfTile][KP];
    __shared__ __align__(16) __half v_s[kPfTile][HD];
    __shared__ float s_s[kPfRows][kPfTile + 1];

    const int tid = threadIdx.x, r = tid >> 2, qd = tid & 3;
    const int head = blockIdx.y, kvh = head / (n_q_heads / n_kv_heads);
    const int m0 = blockIdx.x * kPfRows;
    const int row = min(m0 + r, m - 1);        // tail rows repeat the last row and are not stored
    const int qpos = pos0 + row;               // keys 0 .. qpos are visible
    const int last_pos = pos0 + min(m0 + kPfRows, m) - 1;
    const int n_q = n_q_heads * HD, n_kv = n_kv_heads * HD;
    const float inv_sqrt = sqrtf((float)HD);

    __half2 qreg[HD / 2];
    {
        const uint4 *qr = reinterpret_cast<const uint4 *>(q + (size_t)row * n_q + (size_t)head * HD);
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4 *>(qreg)[i] = qr[i];
    }
    float acc[DQ];
#pragma unroll
    for (int i = 0; i < DQ; ++i) acc[i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;

    for (int kv0 = 0; kv0 <= last_pos; kv0 += kPfTile) {
        __syncthreads();  // the previous tile has been consumed
        constexpr int kChunks = HD / 8;
        for (int i = tid; i < kPfTile * kChunks; i += kPfThreads) {
            const int c = i / kChunks, part = i % kChunks;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (kv0 + c <= last_pos) {  // rows past the last visible key are never read from the cache
                const size_t off = (size_t)(kv0 + c) * n_kv + (size_t)kvh * HD;
                kv = reinterpret_cast<const uint4 *>(k_cache + off)[part];
                vv = reinterpret_cast<const uint4 *>(v_cache + off)[part];
            }
            *reinterpret_cast<uint4 *>(&k_s[c][part * 8]) = kv;
            *reinterpret_cast<uint4 *>(&v_s[c][part * 8]) = vv;
        }
        __syncthreads();
        // scores of this row against keys qd, qd + 4, ...
        float sc[kPfTile / 4];
        float tile_max = -INFINITY;
#pragma unroll
        for (int j = 0; j < kPfTile / 4; ++j) {
            const int c = qd + 4 * j;
            const __half2 *kr = reinterpret_cast<const __half2 *>(&k_s[c][0]);
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < HD / 2; ++i) {
                const float2 a = __half22float2(qreg[i]), b = __half22float2(kr[i]);
                dot = __fmaf_rn(a.x, b.x, dot);
                dot = __fmaf_rn(a.y, b.y, dot);
            }
            sc[j] = (kv0 + c <= qpos) ? __fdiv_rn(dot, inv_sqrt) : -INFINITY;
            tile_max = fmaxf(tile_max, sc[j]);
        }
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float m_new = fmaxf(m_run, tile_max);  // finite: key kv0 <= qpos is visible in every tile started
        const float scale = expf(m_run - m_new);     // expf(-inf) = 0 on the first tile
        float psum = 0.0f;
#pragma unroll
        for (int j = 0; j < kPfTile / 4; ++j) {
            const float pj = expf(sc[j] - m_new);
            s_s[r][qd + 4 * j] = pj;
            psum += pj;
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        l_run = l_run * scale + psum;
        m_run = m_new;
        __syncwarp();  // row r of s_s is written and read by the four threads of one quad only
#pragma unroll
        for (int i = 0; i < DQ; ++i) acc[i] *= scale;
#pragma unroll 4
        for (int c = 0; c < kPfTile; ++c) {
            const float pc = s_s[r][c];
            const __half2 *vr = reinterpret_cast<const __half2 *>(&v_s[c][qd * DQ]);
#pragma unroll
            for (int i = 0; i < DQ / 2; ++i) {
                const float2 vv = __half22float2(vr[i]);
                acc[2 * i] = __fmaf_rn(pc, vv.x, acc[2 * i]);
                acc[2 * i + 1] = __fmaf_rn(pc, vv.y, acc[2 * i + 1]);
            }
        }
        __syncwarp();
    }
    if (m0 + r < m) {
        __align__(16) __half o[DQ];
#pragma unroll
        for (int i = 0; i < DQ; ++i) o[i] = __float2half_rn(__fdiv_rn(acc[i], l_run));
        uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)row * n_q + (size_t)head * HD + qd * DQ);
#pragma unroll
        for (int i = 0; i < DQ / 8; ++i) dst[i] = reinterpret_cast<const uint4 *>(o)[i];
    }
}

__global__ void iota_kernel(int *dst, int first, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = first + i;
}

}  // namespace llmb

extern "C" int llmb_rmsnorm_rows(const uint16_t *d_x, const uint16_t *d_gamma, uint16_t *d_y, int m, int d, double eps,
                                 llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_x || !d_gamma || !d_y || m <= 0 || d <= 0) return LLMB_ERR_INVALID;
    if ((d & 7) || (((uintptr_t)d_x | (uintptr_t)d_gamma | (uintptr_t)d_y) & 15)) {
        set_last_error("llmb_rmsnorm_rows: d must be a multiple of 8 and the pointers 16-byte aligned");
        return LLMB_ERR_UNSUPPORTED;
    }
    int n_pow2 = 2;
    while (n_pow2 < d / 4) n_pow2 <<= 1;
    if ((size_t)n_pow2 * 4 > 40 * 1024) {
        set_last_error("llmb_rmsnorm_rows: d above 40960 is not supported");
        return LLMB_ERR_UNSUPPORTED;
    }
    rmsnorm_rows_kernel<<<m, kNormThreads, (size_t)n_pow2 * 4, static_cast<cudaStream_t>(stream_)>>>(
        reinterpret_cast<const __half *>(d_x), reinterpret_cast<const __half *>(d_gamma), reinterpret_cast<__half *>(d_y), d,
        n_pow2, eps);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_attn_prefill(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, int m, int pos0,
                                 int n_q_heads, int n_kv_heads, int head_dim, uint16_t *d_out, llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_q || !d_k_cache || !d_v_cache || !d_out || m <= 0 || pos0 < 0 || n_q_heads <= 0 || n_kv_heads <= 0 ||
        n_q_heads % n_kv_heads)
        return LLMB_ERR_INVALID;
    if (n_q_heads > 65535) return LLMB_ERR_UNSUPPORTED;
    const dim3 grid((m + kPfRows - 1) / kPfRows, n_q_heads);
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    const __half *q = reinterpret_cast<const __half *>(d_q), *kc = reinterpret_cast<const __half *>(d_k_cache),
                 *vc = reinterpret_cast<const __half *>(d_v_cache);
    __half *o = reinterpret_cast<__half *>(d_out);
    if (head_dim == 128) attn_prefill_kernel<128><<<grid, kPfThreads, 0, s>>>(q, kc, vc, o, m, pos0, n_q_heads, n_kv_heads);
    else if (head_dim == 64) attn_prefill_kernel<64><<<grid, kPfThreads, 0, s>>>(q, kc, vc, o, m, pos0, n_q_heads, n_kv_heads);
    else {
        set_last_error("llmb_attn_prefill: head_dim must be 64 or 128");
        return LLMB_ERR_UNSUPPORTED;
    }
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_iota_i32(int32_t *d_out, int first, int n, llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_out || n <= 0) return LLMB_ERR_INVALID;
    iota_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream_)>>>(d_out, first, n);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}
