// Projections for a handful of rows (batched decode: one new row per sequence, m <= 32):
// C[m][n] = X[m][k] . W[n][k]^T with the roles of the two operands swapped on the tensor cores.
//
// Replaces kernel_standard_tiled_gemm / kernel_standard_tiled_gemm_ffn_swiglu of the reference
// (inference.cu:393-519) at small m, with the same FP16 inputs, FP32 accumulation, FP16 rounding points and
// fused element-wise neighbours as gemm_tc.cu.
//
// Bound: HBM.  Every weight byte is streamed once per launch; the m activation rows (a few KB per K step)
// come from L2.  So the kernel is shaped as a weight stream, like the batch-1 projections, not as a GEMM:
//
//   operands  the WEIGHT tile is the 128-row (M) operand of tcgen05.mma, the activation rows are the 32-column
//             (N) operand: D[128 weight rows][32 activation rows] in 32 columns of tensor memory.  A ring stage
//             is 16 KB of weights + 4 KB of activations (32 KB + 4 KB for the gate/up pair), so nearly all of
//             the shared memory in flight is weight bytes, and an MMA step costs a quarter of the 128-wide one.
//   grid      x = 128-row weight tile, y = slice of K.  K is split until about two CTAs per SM exist (each
//             slice at least 8 K steps); partial accumulators (128 x 32 FP32 = 16 KB) meet in a workspace and
//             the last CTA of a tile adds them in slice order and runs the epilogue.
//   ring      about 100 KB per CTA, so that two CTAs share an SM: two of this launch, or the tail of this
//             launch and the head of the next one.
//   overlap   programmatic dependent launch: a CTA releases its dependents at entry and asks for its first
//             ring-full of WEIGHT tiles at once (weights never depend on an earlier kernel); only then does
//             it wait for the previous kernel (griddepcontrol.wait) and ask for the activation tiles.  The
//             epilogue warps wait too before they touch global memory.
//   warps     0 = TMA producer, 1 = MMA issuer (one lane) + tensor-memory owner, 2-5 = epilogue; thread =
//             tensor-memory lane = one weight row n, holding the values of all activation rows for it.
// Every mbarrier wait is bounded (status word, see llmb_device_status).
#include "gemm_common.cuh"
#include "tp_common.cuh"

namespace llmb {

constexpr int kNX = 32;                                   // activation rows per launch (N of the MMA)
constexpr uint32_t kWTileBytes = kBM * kBK * 2;           // 16 KB
constexpr uint32_t kXTileBytes = kNX * kBK * 2;           // 4 KB
constexpr int kSmallMaxStages = 8;
__host__ __device__ constexpr uint32_t small_stage_bytes(bool dual) { return (dual ? 2 : 1) * kWTileBytes + kXTileBytes; }

template <bool DUAL>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char small_smem[];
    __shared__ __align__(8) uint64_t full_bar[kSmallMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kSmallMaxStages];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int split_last;
    __shared__ int prior_status;

    constexpr uint32_t kStageBytes = small_stage_bytes(DUAL);
    constexpr uint32_t kXOff = (DUAL ? 2 : 1) * kWTileBytes;
    constexpr uint32_t kTmemCols = DUAL ? 2 * kNX : kNX;   // 32 is the smallest allocation
    constexpr int kAcc = DUAL ? 2 * kNX : kNX;
    // kind::f16: D = F32 (bit 4), A = B = F16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kNX >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

    unsigned char *ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(small_smem) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
    const int n0 = blockIdx.x * kBM;
    const int k_tiles = p.K / kBK;
    const int kt_begin = (int)((long long)blockIdx.y * k_tiles / p.splits);
    const int kt_end = (int)((long long)(blockIdx.y + 1) * k_tiles / p.splits);

    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    auto stamp = [&](int which) {
        if (p.trace) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            p.trace[(size_t)cta * 8 + which] = t;
        }
    };
    if (threadIdx.x == 0) stamp(0);  // entry
    // The next kernel may start its own weight stream as soon as an SM has room.  After a scattering projection
    // the next kernel is the gather, which takes no wait of its own and reads the exchange counter and the
    // residual rows at once: it is let go only after this kernel's wait, when every earlier kernel is complete.
    const bool scatter = !DUAL && p.epilogue == LLMB_EPI_TP_SCATTER;
    if (!scatter) pdl_launch_dependents();
    // a wait that gave up earlier (here or in another kernel) leaves the status word set: take no wait at all,
    // but still let the previous kernel finish first so that the order of the chain holds
    if (threadIdx.x == 0) prior_status = *reinterpret_cast<volatile int *>(p.status);
    __syncthreads();  // one read for the whole CTA: every thread takes the same way out
    if (prior_status != 0) {
        pdl_wait();
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) stamp(1);  // barriers and tensor memory ready

    if (warp == 0) {
        if (lane == 0) {
            // the head of the weight stream does not depend on the previous kernel: ask for it first
            const int head = min(stages, kt_end - kt_begin);
            for (int i = 0; i < head; ++i) {
                unsigned char *st = ring + (size_t)i * kStageBytes;
                mbar_arrive_expect_tx(&full_bar[i], kStageBytes);
                tma_load_2d(st, &map_w, (kt_begin + i) * kBK, n0, &full_bar[i]);
                if (DUAL) tma_load_2d(st + kWTileBytes, &map_w2, (kt_begin + i) * kBK, n0, &full_bar[i]);
            }
            pdl_wait();  // the activations are the previous kernel's output
            if (scatter) pdl_launch_dependents();
            stamp(2);    // previous kernel complete
            // a wait that gave up earlier leaves the status word set: do not queue more bounded waits behind it
            bool ok = *reinterpret_cast<volatile int *>(p.status) == 0;
            for (int i = 0; i < head; ++i)
                tma_load_2d(ring + (size_t)i * kStageBytes + kXOff, &map_x, (kt_begin + i) * kBK, 0, &full_bar[i]);
            for (int kt = kt_begin + head, i = head; kt < kt_end && ok; ++kt, ++i) {
                const int s = i % stages;
                ok = mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1, p.status, 311);
                if (!ok) break;
                unsigned char *st = ring + (size_t)s * kStageBytes;
                mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
                tma_load_2d(st, &map_w, kt * kBK, n0, &full_bar[s]);
                if (DUAL) tma_load_2d(st + kWTileBytes, &map_w2, kt * kBK, n0, &full_bar[s]);
                tma_load_2d(st + kXOff, &map_x, kt * kBK, 0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kt = kt_begin, i = 0; kt < kt_end && ok; ++kt, ++i) {
                const int s = i % stages;
                ok = mbar_wait(&full_bar[s], (i / stages) & 1, p.status, 312);
                if (!ok) break;
                if (i == 0) stamp(3);  // first stage landed
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = ring + (size_t)s * kStageBytes;
                const uint64_t wdesc = umma_desc(st), xdesc = umma_desc(st + kXOff);
                const uint64_t w2desc = DUAL ? umma_desc(st + kWTileBytes) : 0;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    umma_f16(tmem_base, wdesc + 2 * k, xdesc + 2 * k, kIdesc, acc);
                    if (DUAL) umma_f16(tmem_base + kNX, w2desc + 2 * k, xdesc + 2 * k, kIdesc, acc);
                }
                umma_commit(&empty_bar[s]);
            }
            stamp(4);  // last MMA issued
            umma_commit(&acc_bar);  // arrives even after a failed wait, so the epilogue never waits forever
        }
    } else {
        // ---- epilogue: thread = weight row n0 + lane_group + lane; v[b] = its value for activation row b ----
        const bool got = mbar_wait(&acc_bar, 0, p.status, 313);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (threadIdx.x == 64) stamp(5);  // accumulators complete
        pdl_wait();  // from here on global memory of earlier kernels is read and written
        const bool ok = got && *reinterpret_cast<volatile int *>(p.status) == 0;
        const int lane_group = (warp & 3) * 32;
        const int n = n0 + lane_group + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)lane_group << 16);
        uint32_t v[32], u[32];
        tmem_ld32(taddr, v);
        if (DUAL) tmem_ld32(taddr + kNX, u);
        bool finish = true;
        if (p.splits > 1) {
            float *mine = p.ws_part + (((size_t)blockIdx.x * p.splits + blockIdx.y) * kBM + lane_group + lane) * kAcc;
#pragma unroll
            for (int i = 0; i < 8; ++i) reinterpret_cast<uint4 *>(mine)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            if (DUAL) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    reinterpret_cast<uint4 *>(mine + kNX)[i] = make_uint4(u[4 * i], u[4 * i + 1], u[4 * i + 2], u[4 * i + 3]);
            }
            __threadfence();  // this thread's partials are visible device-wide before the arrival is counted
            named_bar_sync(1, 128);
            if (threadIdx.x == 64) {
                const int arrived = atomicAdd(p.ws_count + blockIdx.x, 1);
                split_last = (arrived == p.splits - 1) ? 1 : 0;
                if (split_last) p.ws_count[blockIdx.x] = 0;  // ready for the next launch
                __threadfence();
            }
            named_bar_sync(1, 128);
            if (threadIdx.x == 64) stamp(6);  // partials published, arrival counted
            finish = split_last != 0;
            if (finish) {
                // partial sums in slice order: the result does not depend on which CTA arrived last
                float fv[32], fu[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) fv[i] = fu[i] = 0.0f;
                for (int z = 0; z < p.splits; ++z) {
                    const float *part = p.ws_part + (((size_t)blockIdx.x * p.splits + z) * kBM + lane_group + lane) * kAcc;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 t = __ldcg(reinterpret_cast<const float4 *>(part) + i);
                        fv[4 * i] += t.x; fv[4 * i + 1] += t.y; fv[4 * i + 2] += t.z; fv[4 * i + 3] += t.w;
                    }
                    if (DUAL) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 t = __ldcg(reinterpret_cast<const float4 *>(part + kNX) + i);
                            fu[4 * i] += t.x; fu[4 * i + 1] += t.y; fu[4 * i + 2] += t.z; fu[4 * i + 3] += t.w;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    v[i] = __float_as_uint(fv[i]);
                    u[i] = __float_as_uint(fu[i]);
                }
            }
        }
        if (finish && ok && n < p.N) {  // the last weight tile may reach past N (its rows are zero-filled by TMA)
            // Output element (b, n): the 32 lanes of a warp hold 32 consecutive n, so each store of a warp is
            // one 64-byte run of row b.
            if (!DUAL && p.epilogue == LLMB_EPI_TP_SCATTER) {
                // tensor parallel: this rank's partial sums go, tagged, to every rank's receive buffer
                const unsigned int tag = __ldg(p.tp_seq) + (unsigned int)p.tp_index + 1u;
                const size_t slot0 = tp_rows_slot(p.tp_size, p.N, p.tp_index, p.tp_rank, 0, n);
#pragma unroll
                for (int b = 0; b < kNX; ++b) {
                    if (b < p.M) {
                        const size_t off = slot0 + (size_t)b * p.N * 8;
                        for (int r = 0; r < p.tp_size; ++r)
                            asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p.tp_peer[r] + off), "r"(v[b]), "r"(tag)
                                         : "memory");
                    }
                }
            } else if (DUAL) {
#pragma unroll
                for (int b = 0; b < kNX; ++b)
                    if (b < p.M) p.c[(size_t)b * p.N + n] = __float2half_rn(silu_gemm(__uint_as_float(v[b])) * __uint_as_float(u[b]));
            } else if (p.epilogue == LLMB_EPI_STORE) {
#pragma unroll
                for (int b = 0; b < kNX; ++b)
                    if (b < p.M) p.c[(size_t)b * p.N + n] = __float2half_rn(__uint_as_float(v[b]));
            } else if (p.epilogue == LLMB_EPI_RESIDUAL) {
                // all residual values first, then the stores: a load after a store to the same array would
                // have to wait for it, and 32 dependent round trips to L2 cost more than the whole weight stream
                __half res[kNX];
#pragma unroll
                for (int b = 0; b < kNX; ++b) res[b] = b < p.M ? __ldcg(p.c + (size_t)b * p.N + n) : __half(0);
#pragma unroll
                for (int b = 0; b < kNX; ++b)
                    if (b < p.M)
                        p.c[(size_t)b * p.N + n] = __float2half_rn(__half2float(__float2half_rn(__uint_as_float(v[b]))) + __half2float(res[b]));
            } else {  // LLMB_EPI_ROPE_KV: the pair (even n, n + 1) sits in neighbouring lanes
                const int half_dim = p.head_dim >> 1;
                const bool is_q = n < p.n_q, is_v = n >= p.n_q + p.n_kv;
                const int local = is_q ? n : (is_v ? n - p.n_q - p.n_kv : n - p.n_q);
                const int pair = (local >> 1) % half_dim;
                // angles and cache positions of all rows first (independent loads), then the stores
                float2 cs[kNX];
                int pos[kNX];
#pragma unroll
                for (int b = 0; b < kNX; ++b) {
                    cs[b] = (b < p.M && !is_v) ? __ldg(p.rope_cs + (size_t)b * half_dim + pair) : make_float2(1.0f, 0.0f);
                    pos[b] = b < p.M ? (p.row_pos ? __ldg(p.row_pos + b) : p.pos0 + b) : -1;
                }
#pragma unroll
                for (int b = 0; b < kNX; ++b) {
                    if (b < p.M) {  // uniform across the warp: the shuffle below is executed by all 32 lanes
                        const float mine = __half2float(__float2half_rn(__uint_as_float(v[b])));
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        __half out;
                        if (is_v) {
                            out = __float2half_rn(__uint_as_float(v[b]));
                        } else {
                            out = __float2half_rn((n & 1) ? __fmaf_rn(cs[b].y, other, __fmul_rn(cs[b].x, mine))
                                                          : __fmaf_rn(cs[b].x, mine, -__fmul_rn(cs[b].y, other)));
                        }
                        if (is_q) {
                            p.c[(size_t)b * p.n_q + n] = out;
                        } else {
                            const size_t cache_row = p.row_pos ? (size_t)b * (size_t)p.seq_stride + (size_t)pos[b] : (size_t)pos[b];
                            if (pos[b] >= 0 && pos[b] < p.max_pos) (is_v ? p.v_cache : p.k_cache)[cache_row * p.n_kv + local] = out;
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) stamp(7);  // epilogue done
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

int launch_gemm_smallm(const LlmbGemmArgs *a, cudaStream_t stream) {
    const bool dual = a->epilogue == LLMB_EPI_SWIGLU;
    CUtensorMap mw, mw2, mx;
    int rc;
    if ((rc = make_map(&mw, a->b, a->n, a->k, kBM))) return rc;
    if ((rc = make_map(&mw2, dual ? a->b2 : a->b, a->n, a->k, kBM))) return rc;
    if ((rc = make_map(&mx, a->a, a->m, a->k, kNX))) return rc;
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
    p.trace = reinterpret_cast<unsigned long long *>(a->trace);
    p.tp_seq = nullptr;
    if (a->epilogue == LLMB_EPI_TP_SCATTER) {
        if (dual || a->tp_size < 2 || a->tp_size > 8 || a->tp_rank < 0 || a->tp_rank >= a->tp_size || a->tp_index < 0) return LLMB_ERR_INVALID;
        for (int r = 0; r < a->tp_size; ++r) {
            if (!a->tp_peers[r]) return LLMB_ERR_INVALID;
            p.tp_peer[r] = static_cast<unsigned char *>(a->tp_peers[r]);
        }
        p.tp_rank = a->tp_rank; p.tp_size = a->tp_size; p.tp_index = a->tp_index;
        p.tp_seq = reinterpret_cast<const unsigned int *>(p.tp_peer[a->tp_rank] + tp_rows_seq_off(a->tp_size, a->n));
    }
    const int tiles = (a->n + kBM - 1) / kBM, k_tiles = a->k / kBK, sms = sm_count_cached();
    const int kacc = dual ? 2 * kNX : kNX;
    // K is split until about two CTAs per SM stream weights, each slice at least 8 K steps long
    p.splits = 1;
    const bool have_ws = a->workspace && a->workspace_bytes > 4096 && (((uintptr_t)a->workspace) & 15) == 0;
    // (the gate/up pair moves two weight tiles and 32 KB of partials per CTA: it is split only while the tiles
    // alone leave half of the SMs without a CTA)
    if (have_ws && tiles <= 1024 && (dual ? tiles * 2 <= sms : tiles < 2 * sms)) {
        int splits = 2 * sms / tiles;  // never more CTAs than can be resident at once
        if (splits > k_tiles / 8) splits = k_tiles / 8;
        if (splits > 16) splits = 16;
        while (splits > 1 && 4096 + (size_t)tiles * splits * kBM * kacc * sizeof(float) > a->workspace_bytes) --splits;
        if (splits > 1) p.splits = splits;
    }
    p.ws_count = static_cast<int *>(a->workspace);
    p.ws_part = have_ws ? reinterpret_cast<float *>(static_cast<unsigned char *>(a->workspace) + 4096) : nullptr;
    // about 100 KB of ring per CTA: two CTAs (of this launch, or of this and the next one) share an SM
    p.stages = dual ? 3 : 5;  // 108 KB / 100 KB
    if (dual && tiles * p.splits <= sms) p.stages = 5;  // one CTA per SM anyway: a deeper ring (180 KB)
    const size_t smem = (size_t)p.stages * small_stage_bytes(dual) + 1024;
    static size_t attr_set[2][kMaxDevices] = {};  // per instantiation and device
    if (dual) {
        LLMB_CUDA_OK(ensure_dynamic_smem(gemm_smallm_kernel<true>, attr_set[1], smem));
        LLMB_CUDA_OK(launch_pdl(gemm_smallm_kernel<true>, dim3(tiles, p.splits), dim3(kGemmThreads), smem, stream, a->use_pdl != 0, mw,
                                mw2, mx, p));
    } else {
        LLMB_CUDA_OK(ensure_dynamic_smem(gemm_smallm_kernel<false>, attr_set[0], smem));
        LLMB_CUDA_OK(launch_pdl(gemm_smallm_kernel<false>, dim3(tiles, p.splits), dim3(kGemmThreads), smem, stream, a->use_pdl != 0, mw,
                                mw2, mx, p));
    }
    return LLMB_OK;
}

}  // namespace llmb
