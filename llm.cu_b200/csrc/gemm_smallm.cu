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
//   grid      x = 128-row weight tile, y = slice of K.  K is split in 2, 4 or 8 until about two CTAs per SM
//             exist (each slice at least 8 K steps).  The CTAs of one tile form a thread-block cluster: each
//             leaves its partial accumulators (128 x 32 FP32 = 16 KB) in its own shared memory, and after a
//             cluster barrier CTA r adds the partials of activation rows r * 32/S .. through distributed
//             shared memory, in slice order, and runs the epilogue for those rows.  No workspace, no atomic,
//             no last CTA that reduces alone.
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

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Every thread of every CTA of the cluster arrives; returns when all have (a hardware barrier: no spin of ours).
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// The S slices' partial sums of element (activation row b, weight row nl) of accumulator `acc`, added in slice order.
// rbase[z] = shared-memory address, as seen from this CTA, of slice z's [accumulator][32][128] FP32 block.
__device__ __forceinline__ float gather_slices(const uint32_t (&rbase)[8], int n_slices, int acc, int b, int nl) {
    const uint32_t off = (uint32_t)(((acc * kNX + b) * kBM + nl) * 4);
    float t[8];
#pragma unroll
    for (int z = 0; z < 8; ++z) {
        t[z] = 0.0f;
        if (z < n_slices) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(t[z]) : "r"(rbase[z] + off) : "memory");
    }
    float sum = 0.0f;
#pragma unroll
    for (int z = 0; z < 8; ++z)
        if (z < n_slices) sum += t[z];
    return sum;
}

template <bool DUAL>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char small_smem[];
    __shared__ __align__(8) uint64_t full_bar[kSmallMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kSmallMaxStages];
    __shared__ __align__(8) uint64_t acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int prior_status;

    constexpr uint32_t kStageBytes = small_stage_bytes(DUAL);
    constexpr uint32_t kXOff = (DUAL ? 2 : 1) * kWTileBytes;
    constexpr uint32_t kTmemCols = DUAL ? 2 * kNX : kNX;   // 32 is the smallest allocation
    // kind::f16: D = F32 (bit 4), A = B = F16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kNX >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

    unsigned char *ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(small_smem) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stages = p.stages;
    const int n0 = blockIdx.x * kBM;
    const int k_tiles = p.K / kBK;
    const bool clustered = p.splits > 1;  // then the p.splits CTAs of a tile are one cluster along y
    const int slice = clustered ? (int)cluster_cta_rank() : 0;
    const int kt_begin = (int)((long long)slice * k_tiles / p.splits);
    const int kt_end = (int)((long long)(slice + 1) * k_tiles / p.splits);

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
        if (clustered) {  // the other CTAs of the cluster may still read this one's shared memory: leave with them
            cluster_sync_all();
            cluster_sync_all();
        }
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
    }
    // ---- epilogue: thread = weight row n0 + lane_group + lane.  The accumulators go to shared memory first (over
    // the ring), [accumulator][activation row b][weight row]; the rows are then finished four at a time in a loop
    // that is NOT unrolled over all 32 rows: a CTA runs its epilogue once, so every instruction of it is fetched
    // cold, and the fully unrolled form (five epilogues x 32 rows) cost 5-19 us of instruction fetch per launch.
    const int lane_group = (warp & 3) * 32;
    const int nl = lane_group + lane;
    const int n = n0 + nl;
    uint32_t *red_own = reinterpret_cast<uint32_t *>(ring);
    bool ok = false;
    if (warp >= 2) {
        const bool got = mbar_wait(&acc_bar, 0, p.status, 313);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (threadIdx.x == 64) stamp(5);  // accumulators complete
        pdl_wait();  // from here on global memory of earlier kernels is read and written
        ok = got && *reinterpret_cast<volatile int *>(p.status) == 0;
        const uint32_t taddr = tmem_base + ((uint32_t)lane_group << 16);
        // every load of the ring has landed and every MMA has read it (acc_bar): the ring is free
        uint32_t v[32];
        tmem_ld32(taddr, v);
#pragma unroll
        for (int b = 0; b < kNX; ++b) red_own[b * kBM + nl] = v[b];
        if (DUAL) {
            tmem_ld32(taddr + kNX, v);
#pragma unroll
            for (int b = 0; b < kNX; ++b) red_own[(kNX + b) * kBM + nl] = v[b];
        }
    }
    // Split K: CTA r of the cluster finishes activation rows r * 32/S ..; without a split a thread only reads back
    // what it wrote itself, so no barrier is needed.
    int b_lo = 0, nb = kNX;
    if (clustered) {
        cluster_sync_all();  // all slices of the tile are in shared memory
        nb = kNX / p.splits;
        b_lo = slice * nb;
    }
    if (threadIdx.x == 64) stamp(6);
    if (warp >= 2 && ok && n < p.N) {  // the last weight tile may reach past N (its rows are zero-filled by TMA)
        uint32_t rbase[8];
        const uint32_t red = smem_u32(ring);
#pragma unroll
        for (int z = 0; z < 8; ++z) {
            rbase[z] = red;
            if (clustered && z < p.splits) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbase[z]) : "r"(red), "r"(z));
        }
        const int n_slices = clustered ? p.splits : 1;
        const int b_hi = min(b_lo + nb, p.M);
        // Output element (b, n): the 32 lanes of a warp hold 32 consecutive n, so each store of a warp is one
        // 64-byte run of row b.  Loads of four rows first, then their stores.
        const int half_dim = p.head_dim >> 1;
        const bool is_q = n < p.n_q, is_v = n >= p.n_q + p.n_kv;
        const int local = is_q ? n : (is_v ? n - p.n_q - p.n_kv : n - p.n_q);
        const int pair = half_dim > 0 ? (local >> 1) % half_dim : 0;
        const unsigned int tag = p.epilogue == LLMB_EPI_TP_SCATTER ? __ldg(p.tp_seq) + (unsigned int)p.tp_index + 1u : 0u;
#pragma unroll 1
        for (int b0 = b_lo; b0 < b_hi; b0 += 4) {
            float val[4], val2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int b = min(b0 + i, b_hi - 1);
                val[i] = gather_slices(rbase, n_slices, 0, b, nl);
                val2[i] = DUAL ? gather_slices(rbase, n_slices, 1, b, nl) : 0.0f;
            }
            if (!DUAL && p.epilogue == LLMB_EPI_TP_SCATTER) {
                // tensor parallel: this rank's partial sums go, tagged, to every rank's receive buffer
                const size_t slot0 = tp_rows_slot(p.tp_size, p.N, p.tp_index, p.tp_rank, 0, n);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (b0 + i < b_hi) {
                        const size_t off = slot0 + (size_t)(b0 + i) * p.N * 8;
                        for (int r = 0; r < p.tp_size; ++r)
                            asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p.tp_peer[r] + off), "r"(__float_as_uint(val[i])),
                                         "r"(tag)
                                         : "memory");
                    }
                }
            } else if (DUAL) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (b0 + i < b_hi) p.c[(size_t)(b0 + i) * p.N + n] = __float2half_rn(silu_gemm(val[i]) * val2[i]);
            } else if (p.epilogue == LLMB_EPI_STORE) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (b0 + i < b_hi) p.c[(size_t)(b0 + i) * p.N + n] = __float2half_rn(val[i]);
            } else if (p.epilogue == LLMB_EPI_RESIDUAL) {
                // the residual values of the four rows first, then the stores: a load after a store to the same
                // array would have to wait for it
                __half res[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) res[i] = __ldcg(p.c + (size_t)min(b0 + i, b_hi - 1) * p.N + n);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (b0 + i < b_hi)
                        p.c[(size_t)(b0 + i) * p.N + n] = __float2half_rn(__half2float(__float2half_rn(val[i])) + __half2float(res[i]));
            } else {  // LLMB_EPI_ROPE_KV: the pair (even n, n + 1) sits in neighbouring lanes
                float2 cs[4];
                int pos[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int b = min(b0 + i, b_hi - 1);
                    cs[i] = is_v ? make_float2(1.0f, 0.0f) : __ldg(p.rope_cs + (size_t)b * half_dim + pair);
                    pos[i] = p.row_pos ? __ldg(p.row_pos + b) : p.pos0 + b;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int b = b0 + i;
                    // b and b_hi are the same in all lanes, so the shuffle is executed by the whole warp (N is a
                    // multiple of 32 whenever this epilogue is used: whole heads)
                    if (b < b_hi) {
                        const float mine = __half2float(__float2half_rn(val[i]));
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
                        __half out;
                        if (is_v) {
                            out = __float2half_rn(val[i]);
                        } else {
                            out = __float2half_rn((n & 1) ? __fmaf_rn(cs[i].y, other, __fmul_rn(cs[i].x, mine))
                                                          : __fmaf_rn(cs[i].x, mine, -__fmul_rn(cs[i].y, other)));
                        }
                        if (is_q) {
                            p.c[(size_t)b * p.n_q + n] = out;
                        } else {
                            const size_t cache_row = p.row_pos ? (size_t)b * (size_t)p.seq_stride + (size_t)pos[i] : (size_t)pos[i];
                            if (pos[i] >= 0 && pos[i] < p.max_pos) (is_v ? p.v_cache : p.k_cache)[cache_row * p.n_kv + local] = out;
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (clustered) cluster_sync_all();  // no CTA leaves while another may still read its partial sums
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
    // K is split (2, 4 or 8 slices = the CTAs of one cluster) until about two CTAs per SM stream weights, each
    // slice at least 8 K steps long.  The gate/up pair moves two weight tiles per CTA: it is split only while
    // the tiles alone leave half of the SMs without a CTA.
    p.splits = 1;
    if (tiles < 2 * sms) {
        int want = 2 * sms / tiles;  // never more CTAs than can be resident at once
        if (want > k_tiles / 8) want = k_tiles / 8;
        p.splits = want >= 8 ? 8 : want >= 4 ? 4 : want >= 2 ? 2 : 1;
    }
    p.ws_count = nullptr;
    p.ws_part = nullptr;
    // about 100 KB of ring per CTA: two CTAs (of this launch, or of this and the next one) share an SM
    p.stages = dual ? 3 : 5;  // 108 KB / 100 KB
    if (dual && tiles * p.splits <= sms) p.stages = 5;  // one CTA per SM anyway: a deeper ring (180 KB)
    const size_t smem = (size_t)p.stages * small_stage_bytes(dual) + 1024;
    static size_t attr_set[2][kMaxDevices] = {};  // per instantiation and device
    if (dual) {
        LLMB_CUDA_OK(ensure_dynamic_smem(gemm_smallm_kernel<true>, attr_set[1], smem));
        LLMB_CUDA_OK(launch_pdl_cluster(gemm_smallm_kernel<true>, dim3(tiles, p.splits), dim3(kGemmThreads), smem, stream, a->use_pdl != 0,
                                        dim3(1, p.splits, 1), mw, mw2, mx, p));
    } else {
        LLMB_CUDA_OK(ensure_dynamic_smem(gemm_smallm_kernel<false>, attr_set[0], smem));
        LLMB_CUDA_OK(launch_pdl_cluster(gemm_smallm_kernel<false>, dim3(tiles, p.splits), dim3(kGemmThreads), smem, stream, a->use_pdl != 0,
                                        dim3(1, p.splits, 1), mw, mw2, mx, p));
    }
    return LLMB_OK;
}

}  // namespace llmb
