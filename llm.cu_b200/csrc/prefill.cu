// Row-batched kernels of the prompt phase, beside the tensor-core projections (gemm_tc.cu):
//
//   rmsnorm_rows   RMSNorm of M rows (replaces kernel_compute_rms_norm + kernel_compute_norm_tensor,
//                  inference.cu:272-375, for M rows at once): same partials of four elements, same
//                  binary reduction tree, eps added in double, IEEE division, FP16 rounding.
//   attn_prefill   causal attention of M new rows against the KV cache (replaces compute_attention's
//                  three kernels, inference.cu:698-947): scores (q.k)/sqrtf(head_dim) in FP32 from
//                  FP16, softmax in FP32 (online, never materialising the N x N matrix), P.V with FP32
//                  accumulation, FP16 out.  K and V come from the cache rows the QKV projection just
//                  appended, so a chunk that starts at position pos0 > 0 attends to the earlier rows
//                  as well.
//   iota           positions pos0 .. pos0 + n - 1 for the embedding / RoPE-angle prologue.
#include "gemm_common.cuh"
#include "gemv_common.cuh"
#include "mma_common.cuh"

namespace llmb {

constexpr int kNormThreads = 256;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_rows_kernel(const __half *__restrict__ x, const __half *__restrict__ gamma, __half *__restrict__ y, int d,
                    int n_pow2, double eps) {
    extern __shared__ float norm_part[];  // n_pow2 partials (d / 4 real ones, zero padded)
    __shared__ float rms_s;
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();  // x is the previous kernel's output
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

// ---------------------------------------------------------------------------------------------
// Block attention on the tensor cores (warp-level mma.sync m16n8k16, FP16 in, FP32 accumulate).
// CTA = 64 query rows of one head, 4 warps x 16 rows; K/V tiles of 64 cache rows in shared memory,
// double-buffered, fetched as swizzled boxes through tensor maps.  Per tile and warp: S = Q K^T (fragments of Q live in registers for the whole kernel),
// scores / sqrtf(head_dim) and the online softmax in FP32 on the accumulator fragments, then
// O += P V with P split into an FP16 head and an FP16 remainder (two MMAs), so that the
// probabilities enter the product with ~22 bits as the reference's FP32 P does, not with 11.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaRows = 64;   // query rows per CTA
constexpr int kMmaTile = 64;   // cache rows per tile
constexpr int kMmaThreads = 128;

// Byte offset of 16-byte chunk `chunk` of row `row` in a K (or V) tile as the tensor-map loads leave it: boxes of
// 64 rows x 128 bytes in the 128-byte swizzle (chunk c of row r sits at chunk c ^ (r & 7)), one box per 64 dims.
__device__ __forceinline__ uint32_t box_off(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * (kMmaTile * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(kMmaThreads, 3)
attn_prefill_mma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __half *__restrict__ q, __half *__restrict__ out, int m, int pos0, int n_q_heads, int n_kv_heads,
                        int *status) {
    constexpr int KS = HD / 16;    // k-steps of Q K^T
    constexpr int NT = kMmaTile / 8;  // score n-tiles per tile
    constexpr int OT = HD / 8;     // output n-tiles
    // two K/V tile buffers in dynamic shared memory: tile t + 1 streams in while tile t is multiplied.  A tile
    // arrives as 64-row boxes through tensor maps of the K and V cache (rows 0 .. pos0 + m - 1 of this layer):
    // one instruction per box, where 16-byte cp.async pieces took 32 instructions and their addresses per thread.
    extern __shared__ __align__(16) unsigned char attn_smem_raw[];
    unsigned char *attn_smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(attn_smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) uint64_t tile_bar[2];
    constexpr size_t kTileBytes = (size_t)kMmaTile * HD * sizeof(__half);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
    const int head = blockIdx.y, kvh = head / (n_q_heads / n_kv_heads);
    const int m0 = blockIdx.x * kMmaRows;
    const int n_q = n_q_heads * HD;
    // this thread's two rows (tail rows repeat the last row and are not stored)
    const int r0 = m0 + warp * 16 + quad_row, r1 = r0 + 8;
    const int row0 = min(r0, m - 1), row1 = min(r1, m - 1);
    const int qpos0 = pos0 + row0, qpos1 = pos0 + row1;
    const int last_pos = pos0 + min(m0 + kMmaRows, m) - 1;
    static_assert(HD == 64 || HD == 128, "div_by_const is checked for sqrtf(64) and sqrtf(128)");
    const float sqrt_hd = sqrtf((float)HD), rsqrt_hd = __fdiv_rn(1.0f, sqrt_hd);

    uint32_t qf[KS][4];
    {
        const __half *q0 = q + (size_t)row0 * n_q + (size_t)head * HD + quad_col;
        const __half *q1 = q + (size_t)row1 * n_q + (size_t)head * HD + quad_col;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = *reinterpret_cast<const uint32_t *>(q0 + ks * 16);
            qf[ks][1] = *reinterpret_cast<const uint32_t *>(q1 + ks * 16);
            qf[ks][2] = *reinterpret_cast<const uint32_t *>(q0 + ks * 16 + 8);
            qf[ks][3] = *reinterpret_cast<const uint32_t *>(q1 + ks * 16 + 8);
        }
    }
    float o[OT][4];
#pragma unroll
    for (int t = 0; t < OT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    float m_run0 = -INFINITY, m_run1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;  // l: this thread's share of the row sum

    if (tid == 0) {
        mbar_init(&tile_bar[0], 1);
        mbar_init(&tile_bar[1], 1);
        fence_mbar_init();
    }
    __syncthreads();
    // Requests tile `t` (cache rows t * 64 ..) into buffer t & 1.  Rows past the last visible key are either
    // rows of this same block (written by the projection before this kernel: finite, and masked below) or past
    // the end of the tensor map (zero-filled).
    auto request_tile = [&](int t) {
        if (tid == 0) {
            unsigned char *kd = attn_smem + (size_t)(t & 1) * 2 * kTileBytes, *vd = kd + kTileBytes;
            mbar_arrive_expect_tx(&tile_bar[t & 1], (uint32_t)(2 * kTileBytes));
#pragma unroll
            for (int b = 0; b < HD / 64; ++b) {
                tma_load_2d(kd + (size_t)b * kMmaTile * 128, &map_k, kvh * HD + b * 64, t * kMmaTile, &tile_bar[t & 1]);
                tma_load_2d(vd + (size_t)b * kMmaTile * 128, &map_v, kvh * HD + b * 64, t * kMmaTile, &tile_bar[t & 1]);
            }
        }
    };
    const int n_tiles = last_pos / kMmaTile + 1;
    request_tile(0);
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int kv0 = tile * kMmaTile;
        // the next tile's buffer was released by the barrier that ended the previous iteration
        if (tile + 1 < n_tiles) request_tile(tile + 1);
        mbar_wait_warp(&tile_bar[tile & 1], (tile >> 1) & 1, status, 332, lane);
        const unsigned char *k_s = attn_smem + (size_t)(tile & 1) * 2 * kTileBytes, *v_s = k_s + kTileBytes;

        // S = Q K^T: B fragment of n-tile t, k-step ks = K[t * 8 + lane / 4][ks * 16 + 2 (lane % 4) (+ 8)]
        float sc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.0f;
        // (one ldmatrix.x4 = the B fragments of two n-tiles of one k-step: K rows are keys, and the MMA wants
        // the 16 dims of the k-step along k for each key column, which is how a K row lies in memory)
#pragma unroll
        for (int t = 0; t < NT; t += 2) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t kb[4];
                ldmatrix_x4(kb, k_s + box_off(t * 8 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                mma_16816(sc[t], qf[ks], kb[0], kb[1]);
                mma_16816(sc[t + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // scale, causal mask, tile maximum per row
        float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int key = kv0 + t * 8 + quad_col;
            sc[t][0] = key <= qpos0 ? div_by_const(sc[t][0], sqrt_hd, rsqrt_hd) : -INFINITY;
            sc[t][1] = key + 1 <= qpos0 ? div_by_const(sc[t][1], sqrt_hd, rsqrt_hd) : -INFINITY;
            sc[t][2] = key <= qpos1 ? div_by_const(sc[t][2], sqrt_hd, rsqrt_hd) : -INFINITY;
            sc[t][3] = key + 1 <= qpos1 ? div_by_const(sc[t][3], sqrt_hd, rsqrt_hd) : -INFINITY;
            tmax0 = fmaxf(tmax0, fmaxf(sc[t][0], sc[t][1]));
            tmax1 = fmaxf(tmax1, fmaxf(sc[t][2], sc[t][3]));
        }
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
        tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
        tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
        // key 0 is visible to every row, so the running maximum is finite from the first tile on
        const float mn0 = fmaxf(m_run0, tmax0), mn1 = fmaxf(m_run1, tmax1);
        const float scale0 = expf(m_run0 - mn0), scale1 = expf(m_run1 - mn1);
        m_run0 = mn0;
        m_run1 = mn1;
        l0 *= scale0;
        l1 *= scale1;
#pragma unroll
        for (int t = 0; t < OT; ++t) {
            o[t][0] *= scale0;
            o[t][1] *= scale0;
            o[t][2] *= scale1;
            o[t][3] *= scale1;
        }
        // probabilities as A fragments: two adjacent score n-tiles make one 16-key k-step
        uint32_t p_hi[NT / 2][4], p_lo[NT / 2][4];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float pr[4];
            pr[0] = expf(sc[t][0] - mn0);
            pr[1] = expf(sc[t][1] - mn0);
            pr[2] = expf(sc[t][2] - mn1);
            pr[3] = expf(sc[t][3] - mn1);
            l0 += pr[0] + pr[1];
            l1 += pr[2] + pr[3];
            const __half2 h01 = __floats2half2_rn(pr[0], pr[1]), h23 = __floats2half2_rn(pr[2], pr[3]);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const int j = t >> 1, base = (t & 1) * 2;
            p_hi[j][base] = *reinterpret_cast<const uint32_t *>(&h01);
            p_hi[j][base + 1] = *reinterpret_cast<const uint32_t *>(&h23);
            p_lo[j][base] = pack_half2(pr[0] - f01.x, pr[1] - f01.y);
            p_lo[j][base + 1] = pack_half2(pr[2] - f23.x, pr[3] - f23.y);
        }
        // O += P V: B fragments of V through ldmatrix.trans (V rows are keys, the MMA wants keys along k)
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
#pragma unroll
            for (int t2 = 0; t2 < OT / 2; ++t2) {
                uint32_t vb[4];
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(vb, v_s + box_off(j * 16 + (mat & 1) * 8 + rr, t2 * 2 + (mat >> 1)));
                mma_16816(o[2 * t2], p_hi[j], vb[0], vb[1]);
                mma_16816(o[2 * t2], p_lo[j], vb[0], vb[1]);
                mma_16816(o[2 * t2 + 1], p_hi[j], vb[2], vb[3]);
                mma_16816(o[2 * t2 + 1], p_lo[j], vb[2], vb[3]);
            }
        }
        __syncthreads();  // this tile has been consumed: its buffer may be refilled
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __half *o0 = out + (size_t)row0 * n_q + (size_t)head * HD + quad_col;
    __half *o1 = out + (size_t)row1 * n_q + (size_t)head * HD + quad_col;
#pragma unroll
    for (int t = 0; t < OT; ++t) {
        if (r0 < m) *reinterpret_cast<uint32_t *>(o0 + t * 8) = pack_half2(__fdiv_rn(o[t][0], l0), __fdiv_rn(o[t][1], l0));
        if (r1 < m) *reinterpret_cast<uint32_t *>(o1 + t * 8) = pack_half2(__fdiv_rn(o[t][2], l1), __fdiv_rn(o[t][3], l1));
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
    // launched with programmatic stream serialization: the kernel waits for its predecessor itself
    LLMB_CUDA_OK(launch_pdl(rmsnorm_rows_kernel, dim3(m), dim3(kNormThreads), (size_t)n_pow2 * 4, static_cast<cudaStream_t>(stream_),
                            true, reinterpret_cast<const __half *>(d_x), reinterpret_cast<const __half *>(d_gamma),
                            reinterpret_cast<__half *>(d_y), d, n_pow2, eps));
    return LLMB_OK;
}

extern "C" int llmb_attn_prefill(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, int m, int pos0,
                                 int n_q_heads, int n_kv_heads, int head_dim, uint16_t *d_out, llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_q || !d_k_cache || !d_v_cache || !d_out || m <= 0 || pos0 < 0 || n_q_heads <= 0 || n_kv_heads <= 0 ||
        n_q_heads % n_kv_heads)
        return LLMB_ERR_INVALID;
    if (n_q_heads > 65535) return LLMB_ERR_UNSUPPORTED;
    const dim3 grid((m + kMmaRows - 1) / kMmaRows, n_q_heads);
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    const __half *q = reinterpret_cast<const __half *>(d_q), *kc = reinterpret_cast<const __half *>(d_k_cache),
                 *vc = reinterpret_cast<const __half *>(d_v_cache);
    __half *o = reinterpret_cast<__half *>(d_out);
    if (head_dim != 64 && head_dim != 128) {
        set_last_error("llmb_attn_prefill: head_dim must be 64 or 128");
        return LLMB_ERR_UNSUPPORTED;
    }
    if ((((uintptr_t)d_k_cache | (uintptr_t)d_v_cache) & 15) || (long long)pos0 + m >= (1ll << 31)) {
        set_last_error("llmb_attn_prefill: the caches must be 16-byte aligned");
        return LLMB_ERR_UNSUPPORTED;
    }
    // tensor maps of the rows this launch can see: [pos0 + m][n_kv_heads * head_dim], boxes of 64 rows x 64 dims
    CUtensorMap mk, mv;
    int rc;
    if ((rc = make_map(&mk, kc, pos0 + m, n_kv_heads * head_dim, kMmaTile))) return rc;
    if ((rc = make_map(&mv, vc, pos0 + m, n_kv_heads * head_dim, kMmaTile))) return rc;
    int *status = device_status_ptr();
    if (!status) return LLMB_ERR_CUDA;
    // two buffers x (K tile + V tile) of 64 rows, 1024-byte aligned for the swizzle
    const size_t smem = (size_t)4 * kMmaTile * head_dim * sizeof(__half) + 1024;
    static size_t attr_set[2][kMaxDevices] = {};  // per instantiation and device
    if (head_dim == 128) {
        LLMB_CUDA_OK(ensure_dynamic_smem(attn_prefill_mma_kernel<128>, attr_set[0], smem));
        attn_prefill_mma_kernel<128><<<grid, kMmaThreads, smem, s>>>(mk, mv, q, o, m, pos0, n_q_heads, n_kv_heads, status);
    } else {
        LLMB_CUDA_OK(ensure_dynamic_smem(attn_prefill_mma_kernel<64>, attr_set[1], smem));
        attn_prefill_mma_kernel<64><<<grid, kMmaThreads, smem, s>>>(mk, mv, q, o, m, pos0, n_q_heads, n_kv_heads, status);
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
