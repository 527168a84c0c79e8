// Prompt-phase projections: C[M][N] = A[M][K] . B[N][K]^T on the 5th-generation tensor cores.
//
// Replaces kernel_standard_tiled_gemm / kernel_standard_tiled_gemm_ffn_swiglu of the reference
// (inference.cu:393-519) for M > 1 rows, with the same FP16 inputs, FP32 accumulation and FP16
// rounding points, and the neighbouring element-wise kernels fused into the epilogue.
//
// Bound: tensor pipe (2 * M * N * K flops); A and B are both K-major, which is how the
// activations and the checkpoint's [out][in] weights already sit in memory.
//
//   tile     128 x BN output per CTA (BN = 128, 64 or 32: the widest that still gives every SM a CTA),
//            K in steps of 64 (one 128-byte swizzle span of FP16); two CTAs share an SM, so one's
//            epilogue overlaps the other's main loop
//   warp 0   producer: TMA (cp.async.bulk.tensor.2d, 128B swizzle, no multicast) fills a shared-memory
//            ring, completion on mbarriers; 3 stages (SwiGLU: 2) when CTAs share an SM, up to 8 when
//            the grid is a single partial wave and only the ring can hide the copy latency
//   warp 1   allocates tensor memory and issues tcgen05.mma (kind::f16, M = 128, N = BN, K = 16)
//            from one elected lane; tcgen05.commit releases ring stages and signals the epilogue
//   warps 2-5 epilogue: tcgen05.ld the FP32 accumulators (one output row per thread), apply
//            store / residual add / RoPE + KV-cache append / SiLU(gate) * up, write FP16
// The SwiGLU variant keeps two accumulators (gate and up, 2 x BN TMEM columns) fed by two B tiles.
// Rows of A beyond M are zero-filled by TMA and masked in the epilogue; N and K must be multiples
// of 128 and 64.  Every mbarrier wait is bounded (status word, see llmb_device_status).
// A launch with few output tiles and a caller-provided workspace splits K over blockIdx.z: partial
// accumulators are written to the workspace in FP32, and the last CTA of a tile to arrive adds them in
// slice order and runs the epilogue.
#include "gemm_common.cuh"

namespace llmb {

template <bool DUAL, int kBN>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b2, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char gemm_smem[];
    __shared__ __align__(8) uint64_t full_bar[kGemmMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kGemmMaxStages];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int prior_status;
    __shared__ int split_last;

    const int kGemmStages = p.stages;
    constexpr uint32_t kBTileBytes = kBN * kBK * 2;
    constexpr uint32_t kStageBytes = gemm_stage_bytes(DUAL, kBN);  // every tile a multiple of 1024 bytes
    constexpr uint32_t kTmemCols = (DUAL ? 2 : 1) * kBN < 32 ? 32 : (DUAL ? 2 : 1) * kBN;
    // kind::f16: D = F32 (bit 4), A = B = F16 (0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

    // the dynamic shared memory window is only 16-byte aligned by contract: align the ring to 1024 bytes
    unsigned char *ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(gemm_smem) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row tiles vary fastest across the grid: the CTAs that share a weight tile run together and it
    // comes from DRAM once
    const int m0 = blockIdx.x * kBM, n0 = blockIdx.y * kBN;
    const int k_tiles = p.K / kBK;
    const int kt_begin = (int)((long long)blockIdx.z * k_tiles / p.splits);
    const int kt_end = (int)((long long)(blockIdx.z + 1) * k_tiles / p.splits);

    // a wait that gave up earlier (here or in another kernel) leaves the status word set: do not queue
    // up more bounded waits behind it
    if (threadIdx.x == 0) prior_status = *reinterpret_cast<volatile int *>(p.status);
    __syncthreads();
    if (prior_status != 0) return;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {  // one warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            for (int kt = kt_begin, i = 0; kt < kt_end && ok; ++kt, ++i) {
                const int s = i % kGemmStages;
                if (i >= kGemmStages) ok = mbar_wait(&empty_bar[s], ((i / kGemmStages) - 1) & 1, p.status, 301);
                if (!ok) break;
                unsigned char *st = ring + (size_t)s * kStageBytes;
                mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
                tma_load_2d(st, &map_a, kt * kBK, m0, &full_bar[s]);
                tma_load_2d(st + kATileBytes, &map_b, kt * kBK, n0, &full_bar[s]);
                if (DUAL) tma_load_2d(st + kATileBytes + kBTileBytes, &map_b2, kt * kBK, n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kt = kt_begin, i = 0; kt < kt_end && ok; ++kt, ++i) {
                const int s = i % kGemmStages;
                ok = mbar_wait(&full_bar[s], (i / kGemmStages) & 1, p.status, 302);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = ring + (size_t)s * kStageBytes;
                const uint64_t adesc = umma_desc(st), bdesc = umma_desc(st + kATileBytes);
                const uint64_t b2desc = DUAL ? umma_desc(st + kATileBytes + kBTileBytes) : 0;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    // 16 FP16 along K = 32 bytes = 2 descriptor address units inside the swizzle span
                    umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
                    if (DUAL) umma_f16(tmem_base + kBN, adesc + 2 * k, b2desc + 2 * k, kIdesc, acc);
                }
                umma_commit(&empty_bar[s]);  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(&acc_bar);  // arrives even after a failed wait, so the epilogue never waits forever
        }
    } else {
        // ---- epilogue: thread = one row of the tile, TMEM lanes (warp % 4) * 32 .. + 32 ----
        const bool ok = mbar_wait(&acc_bar, 0, p.status, 303);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int lane_group = (warp & 3) * 32;
        const int row = m0 + lane_group + lane;
        const bool row_ok = ok && row < p.M;
        constexpr int kAccCols = (DUAL ? 2 : 1) * kBN;
        const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        bool finish = true;  // this CTA runs the epilogue
        if (p.splits > 1) {
            float *mine = p.ws_part + (((size_t)tile_id * p.splits + blockIdx.z) * kBM + lane_group + lane) * kAccCols;
#pragma unroll 1
            for (int c = 0; c < kBN / 32; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)lane_group << 16) + (uint32_t)(c * 32);
                tmem_ld32(taddr, v);  // warp-collective: every lane takes part, rows past M are not stored
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        reinterpret_cast<uint4 *>(mine + c * 32)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
                if (DUAL) {
                    tmem_ld32(taddr + kBN, v);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<uint4 *>(mine + kBN + c * 32)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                }
            }
            __threadfence();  // this thread's partials are visible device-wide before the arrival is counted
            named_bar_sync(1, 128);
            if (threadIdx.x == 64) {
                const int arrived = atomicAdd(p.ws_count + tile_id, 1);
                split_last = (arrived == p.splits - 1) ? 1 : 0;
                if (split_last) p.ws_count[tile_id] = 0;  // ready for the next launch
                __threadfence();
            }
            named_bar_sync(1, 128);
            finish = split_last != 0;
        }
#pragma unroll 1
        for (int c = 0; c < kBN / 32 && finish; ++c) {
            uint32_t v[32], u[32];
            if (p.splits > 1) {
                if (!row_ok) continue;  // no collective below on this path
                // partial sums in slice order: the result does not depend on which CTA arrived last
                float fv[32], fu[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) fv[i] = fu[i] = 0.0f;
                for (int z = 0; z < p.splits; ++z) {
                    const float *part = p.ws_part + (((size_t)tile_id * p.splits + z) * kBM + lane_group + lane) * kAccCols + c * 32;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 t = __ldcg(reinterpret_cast<const float4 *>(part) + i);
                        fv[4 * i] += t.x; fv[4 * i + 1] += t.y; fv[4 * i + 2] += t.z; fv[4 * i + 3] += t.w;
                    }
                    if (DUAL) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 t = __ldcg(reinterpret_cast<const float4 *>(part + kBN) + i);
                            fu[4 * i] += t.x; fu[4 * i + 1] += t.y; fu[4 * i + 2] += t.z; fu[4 * i + 3] += t.w;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    v[i] = __float_as_uint(fv[i]);
                    u[i] = __float_as_uint(fu[i]);
                }
            } else {
                const uint32_t taddr = tmem_base + ((uint32_t)lane_group << 16) + (uint32_t)(c * 32);
                tmem_ld32(taddr, v);
                if (DUAL) tmem_ld32(taddr + kBN, u);
            }
            if (!row_ok) continue;
            const int col0 = n0 + c * 32;
            __align__(16) __half out[32];
            if (DUAL) {
#pragma unroll
                for (int i = 0; i < 32; ++i) out[i] = __float2half_rn(silu_gemm(__uint_as_float(v[i])) * __uint_as_float(u[i]));
                uint4 *dst = reinterpret_cast<uint4 *>(p.c + (size_t)row * p.N + col0);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = reinterpret_cast<const uint4 *>(out)[i];
            } else if (p.epilogue == LLMB_EPI_STORE) {
#pragma unroll
                for (int i = 0; i < 32; ++i) out[i] = __float2half_rn(__uint_as_float(v[i]));
                uint4 *dst = reinterpret_cast<uint4 *>(p.c + (size_t)row * p.N + col0);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = reinterpret_cast<const uint4 *>(out)[i];
            } else if (p.epilogue == LLMB_EPI_RESIDUAL) {
                uint4 *dst = reinterpret_cast<uint4 *>(p.c + (size_t)row * p.N + col0);
                __align__(16) __half res[32];
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<uint4 *>(res)[i] = dst[i];
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    out[i] = __float2half_rn(__half2float(__float2half_rn(__uint_as_float(v[i]))) + __half2float(res[i]));
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = reinterpret_cast<const uint4 *>(out)[i];
            } else {  // LLMB_EPI_ROPE_KV
                const int pos = p.row_pos ? __ldg(p.row_pos + row) : p.pos0 + row;
                const size_t cache_row = p.row_pos ? (size_t)row * (size_t)p.seq_stride + (size_t)pos : (size_t)pos;
                const int half_dim = p.head_dim >> 1;
                const bool is_v = col0 >= p.n_q + p.n_kv;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float e = __half2float(__float2half_rn(__uint_as_float(v[i])));
                    const float o = __half2float(__float2half_rn(__uint_as_float(v[i + 1])));
                    if (is_v) {
                        out[i] = __float2half_rn(__uint_as_float(v[i]));
                        out[i + 1] = __float2half_rn(__uint_as_float(v[i + 1]));
                    } else {
                        const int local = (col0 < p.n_q ? col0 : col0 - p.n_q) + i;
                        const float2 cs = p.rope_cs[(size_t)row * half_dim + ((local >> 1) % half_dim)];
                        out[i] = __float2half_rn(__fmaf_rn(cs.x, e, -__fmul_rn(cs.y, o)));
                        out[i + 1] = __float2half_rn(__fmaf_rn(cs.y, e, __fmul_rn(cs.x, o)));
                    }
                }
                __half *dstp = nullptr;
                if (col0 < p.n_q) dstp = p.c + (size_t)row * p.n_q + col0;
                else if (pos >= 0 && pos < p.max_pos)
                    dstp = (is_v ? p.v_cache + cache_row * p.n_kv + (col0 - p.n_q - p.n_kv)
                                 : p.k_cache + cache_row * p.n_kv + (col0 - p.n_q));
                if (dstp) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) reinterpret_cast<uint4 *>(dstp)[i] = reinterpret_cast<const uint4 *>(out)[i];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// [rows][k] FP16 row-major as a 2-D tensor map with a 64 x box_rows box and 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, int rows, int k, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from this driver");
        return LLMB_ERR_UNSUPPORTED;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed (base must be 16-byte aligned, k a multiple of 8)");
        return LLMB_ERR_INVALID;
    }
    return LLMB_OK;
}

}  // namespace llmb

extern "C" int llmb_gemm_f16(const LlmbGemmArgs *a, llmb_stream_t stream_) {
    using namespace llmb;
    if (!a || !a->a || !a->b || (!a->c && a->epilogue != LLMB_EPI_TP_SCATTER) || a->m <= 0 || a->n <= 0 || a->k <= 0) return LLMB_ERR_INVALID;
    const bool small_m = a->m <= 32 && a->tile_n == 0;
    // the weight-streaming kernel masks the tail of its last tile, so STORE / TP_SCATTER take any n there
    const bool any_n = small_m && (a->epilogue == LLMB_EPI_STORE || a->epilogue == LLMB_EPI_TP_SCATTER) && a->n % 8 == 0;
    if ((a->n % 128 && !any_n) || a->k % kBK) {
        set_last_error("llmb_gemm_f16: n must be a multiple of 128 and k a multiple of 64");
        return LLMB_ERR_UNSUPPORTED;
    }
    if (a->epilogue == LLMB_EPI_TP_SCATTER && !small_m) {
        set_last_error("llmb_gemm_f16: LLMB_EPI_TP_SCATTER needs m <= 32");
        return LLMB_ERR_UNSUPPORTED;
    }
    const bool dual = a->epilogue == LLMB_EPI_SWIGLU;
    if (dual && !a->b2) return LLMB_ERR_INVALID;
    if (a->epilogue == LLMB_EPI_ROPE_KV) {
        if (!a->rope_cs || !a->k_cache || !a->v_cache || a->head_dim <= 0 || (a->head_dim & 1) ||
            a->n != a->n_q + 2 * a->n_kv || a->n_q % 32 || a->n_kv % 32)
            return LLMB_ERR_INVALID;
    } else if (a->epilogue != LLMB_EPI_STORE && a->epilogue != LLMB_EPI_RESIDUAL && a->epilogue != LLMB_EPI_TP_SCATTER && !dual) {
        return LLMB_ERR_INVALID;
    }
    // A handful of rows (batched decode): the weight-streaming kernel with the operands swapped
    if (small_m) return launch_gemm_smallm(a, static_cast<cudaStream_t>(stream_));
    // Small grids: with a workspace, 128-wide tiles and K split across CTAs until the SMs are covered
    // (every CTA then streams its own weights and only its slice of the activations); without one, the
    // widest tile that still gives every SM a CTA.
    const int m_tiles = (a->m + kBM - 1) / kBM;
    const int sms = sm_count_cached();
    const bool have_ws = a->workspace && a->workspace_bytes > 4096 && (((uintptr_t)a->workspace) & 15) == 0;
    int bn = a->tile_n;
    if (bn == 0) {
        bn = 128;
        if (!have_ws)
            while (bn > 32 && (a->n / bn) * m_tiles < sms) bn >>= 1;
    }
    if (bn != 128 && bn != 64 && bn != 32) {
        set_last_error("llmb_gemm_f16: tile_n must be 0, 32, 64 or 128");
        return LLMB_ERR_INVALID;
    }
    CUtensorMap ma, mb, mb2;
    int rc;
    if ((rc = make_map(&ma, a->a, a->m, a->k, kBM))) return rc;
    if ((rc = make_map(&mb, a->b, a->n, a->k, bn))) return rc;
    if ((rc = make_map(&mb2, dual ? a->b2 : a->b, a->n, a->k, bn))) return rc;
    GemmParams p = {};
    p.c = reinterpret_cast<__half *>(a->c);
    p.rope_cs = reinterpret_cast<const float2 *>(a->rope_cs);
    p.k_cache = reinterpret_cast<__half *>(a->k_cache);
    p.v_cache = reinterpret_cast<__half *>(a->v_cache);
    p.status = device_status_ptr();
    if (!p.status) return LLMB_ERR_CUDA;
    p.M = a->m; p.N = a->n; p.K = a->k; p.epilogue = a->epilogue;
    p.n_q = a->n_q; p.n_kv = a->n_kv; p.head_dim = a->head_dim; p.pos0 = a->pos0; p.max_pos = a->max_pos;
    p.row_pos = a->row_pos;
    p.seq_stride = a->seq_stride;
    dim3 grid(m_tiles, a->n / bn);
    const int tiles = (int)(grid.x * grid.y), k_tiles = a->k / kBK;
    p.splits = 1;
    if (have_ws && tiles * 2 <= sms && tiles <= 1024) {
        int splits = sms / tiles;
        if (splits > 8) splits = 8;
        if (splits > k_tiles / 8) splits = k_tiles / 8;
        const size_t need = 4096 + (size_t)tiles * splits * kBM * (dual ? 2 : 1) * bn * sizeof(float);
        if (splits > 1 && need <= a->workspace_bytes) p.splits = splits;
    }
    p.ws_count = static_cast<int *>(a->workspace);
    p.ws_part = reinterpret_cast<float *>(static_cast<unsigned char *>(a->workspace) + 4096);
    grid.z = p.splits;
    p.stages = gemm_stages(dual);
    if (tiles * p.splits <= sms) {
        p.stages = (int)((size_t)200 * 1024 / gemm_stage_bytes(dual, bn));
        if (p.stages > kGemmMaxStages) p.stages = kGemmMaxStages;
    }
    const size_t smem = (size_t)p.stages * gemm_stage_bytes(dual, bn) + 1024;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    void (*kernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams) =
        dual ? (bn == 128 ? gemm_tc_kernel<true, 128> : bn == 64 ? gemm_tc_kernel<true, 64> : gemm_tc_kernel<true, 32>)
             : (bn == 128 ? gemm_tc_kernel<false, 128> : bn == 64 ? gemm_tc_kernel<false, 64> : gemm_tc_kernel<false, 32>);
    static size_t attr_set[2][3][kMaxDevices] = {};  // per instantiation and device
    LLMB_CUDA_OK(ensure_dynamic_smem(kernel, attr_set[dual ? 1 : 0][bn == 128 ? 0 : bn == 64 ? 1 : 2], smem));
    kernel<<<grid, kGemmThreads, smem, stream>>>(ma, mb, mb2, p);
    LLMB_CUDA_OK(cudaGetLastError());
    return LLMB_OK;
}
