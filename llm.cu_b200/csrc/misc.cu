// Small kernels around the projections: load-time BF16->FP16 conversion, synthetic weights,
// the step prologue (embedding row + RoPE angles) and the greedy-argmax step epilogue.
#include "common.cuh"

#include "../../include/llm_b200_synth.h"

namespace llmb {

// ---------------------------------------------------------------------------------------
// BF16 -> FP16 (src/llama3/llama3.cu:240-254): fp32 bits = bf16 << 16, then RN to FP16.
// Bound: HBM, 4 bytes per element.  128-bit loads/stores, grid-stride.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cvt_pair(uint32_t two_bf16) {
    float lo = __uint_as_float(two_bf16 << 16);
    float hi = __uint_as_float(two_bf16 & 0xFFFF0000u);
    __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void bf16_to_fp16_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, size_t n) {
    const size_t n8 = n / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        uint4 v = __ldcs(reinterpret_cast<const uint4 *>(in) + i);
        uint4 o;
        o.x = cvt_pair(v.x);
        o.y = cvt_pair(v.y);
        o.z = cvt_pair(v.z);
        o.w = cvt_pair(v.w);
        __stcs(reinterpret_cast<uint4 *>(out) + i, o);
    }
    // ragged tail (fewer than 8 elements)
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
        size_t i = n8 * 8 + threadIdx.x;
        out[i] = __half_as_ushort(__float2half_rn(__uint_as_float((uint32_t)in[i] << 16)));
    }
}

// Same conversion for pointers that are not 16-byte aligned.
__global__ void bf16_to_fp16_scalar_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __half_as_ushort(__float2half_rn(__uint_as_float((uint32_t)in[i] << 16)));
}

template <bool BF16>
__global__ void synth_kernel(uint16_t *out, uint64_t key, float std, uint64_t first, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = BF16 ? llmb_synth_bf16(key, first + i, std) : llmb_synth_fp16(key, first + i, std);
}

// 2-D window of a stream: out[r][c] = element first + r * row_stride + c (tensor-parallel shards).
template <bool BF16>
__global__ void synth_2d_kernel(uint16_t *out, uint64_t key, float std, uint64_t first, uint64_t row_stride, uint64_t rows,
                                uint64_t cols) {
    const uint64_t n = rows * cols;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t src = first + (i / cols) * row_stride + (i % cols);
        out[i] = BF16 ? llmb_synth_bf16(key, src, std) : llmb_synth_fp16(key, src, std);
    }
}

__global__ void fill_u16_kernel(uint16_t *out, uint16_t value, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}

// ---------------------------------------------------------------------------------------
// Step prologue: one CTA per row.  Copies the embedding row (inference.cu:209-223) and writes
// the (cos, sin) pairs of the row's position with the reference's FP32 formula
// (inference.cu:673-678): freq = 1 / powf(theta, 2 i / head_dim), angle = pos * freq.
// ---------------------------------------------------------------------------------------
__global__ void embed_rope_kernel(const __half *__restrict__ embed, const int *__restrict__ tokens,
                                  const int *__restrict__ pos, int d_model, int vocab, int head_dim, float theta,
                                  __half *__restrict__ x, float2 *__restrict__ rope_cs, int tokens_by_pos) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    int tok = tokens[tokens_by_pos ? pos[row] : row];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const uint4 *src = reinterpret_cast<const uint4 *>(embed + (size_t)tok * d_model);
    uint4 *dst = reinterpret_cast<uint4 *>(x + (size_t)row * d_model);
    for (int i = threadIdx.x; i < d_model / 8; i += blockDim.x) dst[i] = __ldg(src + i);
    const int half_dim = head_dim / 2;
    const float fpos = (float)pos[row];
    for (int i = threadIdx.x; i < half_dim; i += blockDim.x) {
        float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
        float angle = fpos * freq;
        rope_cs[(size_t)row * half_dim + i] = make_float2(cosf(angle), sinf(angle));
    }
}

// ---------------------------------------------------------------------------------------
// Greedy argmax over FP16 logits, first maximum wins, plus the step bookkeeping that lets a
// captured decode step be replayed without the host.  One CTA of 1024 threads: the logits
// (256 KB for a 128256-entry vocabulary) were just written and sit in L2.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) argmax_kernel(const __half *__restrict__ logits, int n, int *token_out,
                                                      int *pos_inout, int *history, int history_len) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait();
    // one CTA per row of logits (a single row unless the decode is batched)
    logits += (size_t)blockIdx.x * n;
    token_out += blockIdx.x;
    if (pos_inout) pos_inout += blockIdx.x;
    if (history) history += (size_t)blockIdx.x * history_len;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int n8 = n / 8;
    for (int c = threadIdx.x; c < n8; c += blockDim.x) {
        uint4 v = *(reinterpret_cast<const uint4 *>(logits) + c);
        const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float f = __half2float(h[e]);
            if (f > best) {  // ascending index inside a thread: first maximum kept
                best = f;
                best_i = c * 8 + e;
            }
        }
    }
    for (int i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) {
        float f = __half2float(logits[i]);
        if (f > best || (f == best && i < best_i)) {
            best = f;
            best_i = i;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, m);
        int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best || (ov == best && oi < best_i)) {
            best = ov;
            best_i = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        best_i = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, m);
            int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
            if (ov > best || (ov == best && oi < best_i)) {
                best = ov;
                best_i = oi;
            }
        }
        if (threadIdx.x == 0) {
            if (best_i == 0x7fffffff) best_i = 0;  // all NaN / -inf: the oracle returns index 0
            token_out[0] = best_i;
            if (pos_inout) {
                int np = pos_inout[0] + 1;
                pos_inout[0] = np;
                if (history && np >= 0 && np < history_len) history[np] = best_i;
            }
        }
    }
}

__global__ void advance_pos_kernel(int *pos) {
    pdl_launch_dependents();
    pdl_wait();
    *pos = *pos + 1;
}

static inline int grid_for(size_t work_items, int block) {
    size_t g = (work_items + block - 1) / block;
    size_t cap = (size_t)sm_count_cached() * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace llmb

using namespace llmb;

extern "C" int llmb_bf16_to_fp16(const uint16_t *d_bf16, uint16_t *d_fp16, size_t n, llmb_stream_t stream_) {
    if (!d_bf16 || !d_fp16) return n == 0 ? LLMB_OK : LLMB_ERR_INVALID;
    if (n == 0) return LLMB_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if ((((uintptr_t)d_bf16 | (uintptr_t)d_fp16) & 15) == 0) {
        bf16_to_fp16_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, stream>>>(d_bf16, d_fp16, n);
    } else {
        bf16_to_fp16_scalar_kernel<<<grid_for(n, 256), 256, 0, stream>>>(d_bf16, d_fp16, n);
    }
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_synth_bf16(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n,
                               llmb_stream_t stream_) {
    if (!d_out) return LLMB_ERR_INVALID;
    if (n == 0) return LLMB_OK;
    synth_kernel<true><<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        d_out, llmb_stream_key(seed, sid), std, first, n);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_synth_fp16(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n,
                               llmb_stream_t stream_) {
    if (!d_out) return LLMB_ERR_INVALID;
    if (n == 0) return LLMB_OK;
    synth_kernel<false><<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
        d_out, llmb_stream_key(seed, sid), std, first, n);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_synth_2d(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, int bf16, uint64_t first,
                             uint64_t row_stride, uint64_t rows, uint64_t cols, llmb_stream_t stream_) {
    if (!d_out) return LLMB_ERR_INVALID;
    if (rows == 0 || cols == 0) return LLMB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    const uint64_t key = llmb_stream_key(seed, sid);
    if (bf16) synth_2d_kernel<true><<<grid_for(rows * cols, 256), 256, 0, st>>>(d_out, key, std, first, row_stride, rows, cols);
    else synth_2d_kernel<false><<<grid_for(rows * cols, 256), 256, 0, st>>>(d_out, key, std, first, row_stride, rows, cols);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_fill_u16(uint16_t *d_out, uint16_t value, uint64_t n, llmb_stream_t stream_) {
    if (!d_out) return LLMB_ERR_INVALID;
    if (n == 0) return LLMB_OK;
    fill_u16_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(d_out, value, n);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}

extern "C" int llmb_embed_rope(const uint16_t *d_embed, const int32_t *d_tokens, const int32_t *d_pos, int n_rows,
                               int d_model, int vocab, int head_dim, float rope_theta, uint16_t *d_x,
                               float *d_rope_cs, int tokens_by_pos, int use_pdl, llmb_stream_t stream_) {
    if (!d_embed || !d_tokens || !d_pos || !d_x || !d_rope_cs) return LLMB_ERR_INVALID;
    if (n_rows <= 0 || d_model <= 0 || (d_model % 8) || head_dim <= 0 || (head_dim & 1) || vocab <= 0)
        return LLMB_ERR_INVALID;
    if ((((uintptr_t)d_embed | (uintptr_t)d_x) & 15) || ((uintptr_t)d_rope_cs & 7)) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(launch_pdl(embed_rope_kernel, dim3(n_rows), dim3(256), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0,
                            reinterpret_cast<const __half *>(d_embed), d_tokens, d_pos, d_model, vocab, head_dim,
                            rope_theta, reinterpret_cast<__half *>(d_x), reinterpret_cast<float2 *>(d_rope_cs),
                            tokens_by_pos));
    return LLMB_OK;
}

extern "C" int llmb_argmax_f16(const uint16_t *d_logits, int n, int32_t *d_token_out, int32_t *d_pos_inout,
                               int32_t *d_history, int history_len, int use_pdl, llmb_stream_t stream_) {
    if (!d_logits || !d_token_out || n <= 0 || ((uintptr_t)d_logits & 15)) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(launch_pdl(argmax_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0,
                            reinterpret_cast<const __half *>(d_logits), n, d_token_out, d_pos_inout, d_history,
                            history_len));
    return LLMB_OK;
}

extern "C" int llmb_argmax_rows_f16(const uint16_t *d_logits, int n, int rows, int32_t *d_token_out, int32_t *d_pos_inout,
                                    int32_t *d_history, int history_len, int use_pdl, llmb_stream_t stream_) {
    if (!d_logits || !d_token_out || n <= 0 || rows <= 0 || rows > 65535 || ((uintptr_t)d_logits & 15)) return LLMB_ERR_INVALID;
    if (rows > 1 && (n % 8)) return LLMB_ERR_UNSUPPORTED;  // every row must start on a 16-byte boundary
    LLMB_CUDA_OK(launch_pdl(argmax_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0,
                            reinterpret_cast<const __half *>(d_logits), n, d_token_out, d_pos_inout, d_history,
                            history_len));
    return LLMB_OK;
}

extern "C" int llmb_advance_pos(int32_t *d_pos, int use_pdl, llmb_stream_t stream_) {
    if (!d_pos) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(launch_pdl(advance_pos_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0,
                            d_pos));
    return LLMB_OK;
}
