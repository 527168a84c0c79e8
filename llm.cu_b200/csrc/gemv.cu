// Batch-1 projection kernel: y = W x, W [n][k] FP16 row-major, FP32 accumulation.
//
// Bound: HBM bandwidth.  Algorithmic bytes per launch = n * k * 2 (twice that for the
// gate/up pair); x, gamma and y are kilobytes.
//
// Shape of the kernel
//   grid   one CTA per SM (at most); CTA b owns a contiguous range of row groups, so the weight
//          bytes it needs form one contiguous span of HBM.
//   warps  0..7  consumers (256 threads), 8 = producer (one elected lane).
//   smem   ring of `stages` buffers, each NR rows x k halves, filled by 1-D bulk copies
//          (cp.async.bulk, completion on an mbarrier, L2 evict-first: weights are read once
//          per token and must not push the KV cache and activations out of L2).
//   x      lives in registers: thread t owns the 16-byte chunks t, t+256, ... of the row, so
//          one 128-bit shared-memory load feeds eight FMAs and x is never re-read.
//   sums   per-thread FP32 -> warp butterfly that reduces NR rows at once -> 8 warp partials
//          per row in shared memory, added in warp order (deterministic).
//   PDL    the producer starts streaming weights immediately; consumers wait for the previous
//          kernel (griddepcontrol.wait) only before they read x.  Every kernel releases its
//          dependents at entry, so the tail of one projection overlaps the head of the next.
//
// The element-wise neighbours of each projection are fused in (see include/llm_b200.h).
#include <cstdlib>

#include "gemv_common.cuh"

namespace llmb {

constexpr int kConsumers = 256;
constexpr int kThreads = 288;
constexpr int kMaxStages = 8;

struct GemvParams {
    const __half *w;
    const __half *w2;
    const __half *x;
    __half *y;
    const __half *gamma;
    const float2 *rope_cs;
    __half *k_cache;
    __half *v_cache;
    const int *pos;
    int *status;
    double eps;
    int n, k, prologue;
    int n_q, n_kv, head_dim, max_pos;
    int groups;        // ceil(n / rows per group)
    int stages;
    uint32_t stage_bytes;  // smem bytes per stage
};

template <int J, int NR, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvParams p) {
    constexpr bool DUAL = (EPI == LLMB_EPI_SWIGLU);
    constexpr int R = DUAL ? NR / 2 : NR;  // output rows per group
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
    __shared__ float red[2][NR][8];
    __shared__ float norm_buf[512];
    __shared__ float norm_rms;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();

    if (tid == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 8);
        }
        fence_mbar_init();
    }
    __syncthreads();

    // Row groups owned by this CTA.
    const int g_begin = (int)(((long long)p.groups * blockIdx.x) / gridDim.x);
    const int g_end = (int)(((long long)p.groups * (blockIdx.x + 1)) / gridDim.x);
    const size_t row_bytes = (size_t)p.k * 2;

    if (warp == 8) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            bool ok = true;
            for (int g = g_begin, i = 0; g < g_end && ok; ++g, ++i) {
                const int s = i % p.stages;
                if (i >= p.stages) ok = mbar_wait(&empty_bar[s], ((i / p.stages) - 1) & 1, p.status, 101);
                if (!ok) break;
                const int row0 = g * R;
                const int rows = min(R, p.n - row0);
                unsigned char *dst = smem_raw + (size_t)s * p.stage_bytes;
                const uint32_t bytes = (uint32_t)(rows * row_bytes);
                mbar_arrive_expect_tx(&full_bar[s], DUAL ? 2 * bytes : bytes);
                bulk_g2s(dst, reinterpret_cast<const unsigned char *>(p.w) + (size_t)row0 * row_bytes, bytes,
                         &full_bar[s], policy);
                if (DUAL)
                    bulk_g2s(dst + (size_t)R * row_bytes,
                             reinterpret_cast<const unsigned char *>(p.w2) + (size_t)row0 * row_bytes, bytes,
                             &full_bar[s], policy);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int nchunks = p.k >> 3;
    uint4 xh[J];  // this thread's chunks of the input row, packed FP16
    bool have[J];
#pragma unroll
    for (int j = 0; j < J; ++j) have[j] = (tid + kConsumers * j) < nchunks;

    // gamma does not depend on the previous kernel; x does.
    uint4 gv[J];
    if (p.prologue == LLMB_PRO_RMSNORM) {
#pragma unroll
        for (int j = 0; j < J; ++j)
            gv[j] = have[j] ? __ldg(reinterpret_cast<const uint4 *>(p.gamma) + tid + kConsumers * j)
                            : make_uint4(0, 0, 0, 0);
    }
    pdl_wait();
#pragma unroll
    for (int j = 0; j < J; ++j)
        xh[j] = have[j] ? *(reinterpret_cast<const uint4 *>(p.x) + tid + kConsumers * j) : make_uint4(0, 0, 0, 0);
    if (p.prologue == LLMB_PRO_RMSNORM) {
        // Sum of squares in the order of the reference's block reduction
        // (inference.cu:309-344): one partial per four consecutive elements, then a binary
        // tree whose offsets halve from (k/4)/2 down to 1.  Chunk c = tid + 256 j holds
        // partials 2c and 2c+1, so tree levels with offset >= 512 pair values of one thread.
        float p0[J], p1[J];
#pragma unroll
        for (int j = 0; j < J; ++j) sumsq_partials(xh[j], p0[j], p1[j]);
#pragma unroll
        for (int off = J / 2; off >= 1; off >>= 1) {
#pragma unroll
            for (int j = 0; j < off; ++j) {
                p0[j] += p0[j + off];
                p1[j] += p1[j + off];
            }
        }
        norm_buf[2 * tid] = p0[0];
        norm_buf[2 * tid + 1] = p1[0];
        named_bar_sync(1, kConsumers);
        if (warp == 0) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float *b = norm_buf + 2 * lane + e;
                v[e] = ((b[0] + b[256]) + (b[128] + b[384])) + ((b[64] + b[320]) + (b[192] + b[448]));
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                v[0] += __shfl_down_sync(0xffffffffu, v[0], off);
                v[1] += __shfl_down_sync(0xffffffffu, v[1], off);
            }
            if (lane == 0) {
                float total = v[0] + v[1];
                norm_rms = sqrtf((float)(p.eps + (double)(total / (float)p.k)));
            }
        }
        named_bar_sync(1, kConsumers);
        const float rms = norm_rms;
#pragma unroll
        for (int j = 0; j < J; ++j)
            if (have[j]) xh[j] = rmsnorm_apply8(xh[j], gv[j], rms);  // (0 * g) / rms would hit the division's slow path
    }

    bool ok = true;
    for (int g = g_begin, i = 0; g < g_end; ++g, ++i) {
        const int s = i % p.stages;
        if (ok) ok = mbar_wait_warp(&full_bar[s], (i / p.stages) & 1, p.status, 102, lane);
        const int row0 = g * R;
        const int rows = min(R, p.n - row0);
        float acc[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = 0.0f;
        if (ok)
            stage_dot_rows<NR, J, DUAL>(smem_raw + (size_t)s * p.stage_bytes, row_bytes, rows, tid, kConsumers, xh, have, acc);
        const float tot = warp_reduce_multi<NR>(acc, lane);
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&empty_bar[s]);  // all lanes' smem reads are done
        if ((lane & ((32 / NR) - 1)) == 0) red[i & 1][row_of_lane<NR>(lane)][warp] = tot;
        named_bar_sync(2, kConsumers);

        if (warp == (i & 7) && lane < NR) {
            const float *rp = red[i & 1][lane];
            float sum = ((rp[0] + rp[1]) + (rp[2] + rp[3])) + ((rp[4] + rp[5]) + (rp[6] + rp[7]));
            if (EPI == LLMB_EPI_SWIGLU) {
                float up = __shfl_down_sync((1u << NR) - 1u, sum, R);
                if (lane < rows) p.y[row0 + lane] = __float2half_rn(silu_ref(sum) * up);
            } else if (EPI == LLMB_EPI_STORE) {
                if (lane < rows) p.y[row0 + lane] = __float2half_rn(sum);
            } else if (EPI == LLMB_EPI_RESIDUAL) {
                if (lane < rows) {
                    float o = __half2float(__float2half_rn(sum));
                    float res = __half2float(p.y[row0 + lane]);
                    p.y[row0 + lane] = __float2half_rn(o + res);
                }
            } else {  // ROPE_KV
                const int row = row0 + lane;
                float v = __half2float(__float2half_rn(sum));  // projection output is FP16 (inference.cu:445)
                float other = __shfl_xor_sync((1u << NR) - 1u, v, 1);
                if (lane < rows) {
                    const int pos = *p.pos;
                    if (row < p.n_q + p.n_kv) {
                        const int local = row < p.n_q ? row : row - p.n_q;
                        const float2 cs = p.rope_cs[(local >> 1) % (p.head_dim >> 1)];
                        // (cos*even - sin*odd, sin*even + cos*odd), inference.cu:681-682
                        float outv = (row & 1) ? __fmaf_rn(cs.y, other, __fmul_rn(cs.x, v))
                                               : __fmaf_rn(cs.x, v, -__fmul_rn(cs.y, other));
                        __half hv = __float2half_rn(outv);
                        if (row < p.n_q) {
                            p.y[row] = hv;
                        } else if (pos >= 0 && pos < p.max_pos) {
                            p.k_cache[(size_t)pos * p.n_kv + local] = hv;
                        }
                    } else if (pos >= 0 && pos < p.max_pos) {
                        p.v_cache[(size_t)pos * p.n_kv + (row - p.n_q - p.n_kv)] = __float2half_rn(sum);
                    }
                }
            }
        }
    }
}

// Shared-memory budget of a CTA's weight ring (two CTAs share an SM) and CTAs per SM, from sweeps on B200.
constexpr int kGemvSmemKb = 100;
constexpr int kGemvCtasPerSm = 2;

template <int J, int NR, int EPI>
static int launch_gemv(const GemvParams &p0, int sm_count, bool pdl, cudaStream_t stream) {
    GemvParams p = p0;
    constexpr bool DUAL = (EPI == LLMB_EPI_SWIGLU);
    constexpr int R = DUAL ? NR / 2 : NR;
    const uint32_t kSmemBudget = (uint32_t)kGemvSmemKb * 1024;
    if (J < 8) sm_count *= kGemvCtasPerSm;  // the k > 8192 variant needs too many registers for two CTAs per SM
    p.stage_bytes = (uint32_t)((size_t)NR * p.k * 2);
    int stages = (int)(kSmemBudget / p.stage_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return LLMB_ERR_UNSUPPORTED;
    p.stages = stages;
    p.groups = (p.n + R - 1) / R;
    int grid = p.groups < sm_count ? p.groups : sm_count;
    size_t smem = (size_t)stages * p.stage_bytes;
    auto kern = gemv_kernel<J, NR, EPI>;
    static size_t attr_set[kMaxDevices] = {};  // per instantiation and device
    LLMB_CUDA_OK(ensure_dynamic_smem(kern, attr_set, kSmemBudget));
    LLMB_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(kThreads), smem, stream, pdl, p));
    return LLMB_OK;
}

template <int EPI>
static int dispatch_j(const GemvParams &p, int sm_count, bool pdl, cudaStream_t stream) {
    const int chunks = p.k / 8;
    if (chunks <= 256) return launch_gemv<1, 8, EPI>(p, sm_count, pdl, stream);
    if (chunks <= 512) return launch_gemv<2, 4, EPI>(p, sm_count, pdl, stream);
    if (chunks <= 1024) return launch_gemv<4, 2, EPI>(p, sm_count, pdl, stream);
    if constexpr (EPI == LLMB_EPI_STORE || EPI == LLMB_EPI_RESIDUAL) {
        if (chunks <= 2048) return launch_gemv<8, 1, EPI>(p, sm_count, pdl, stream);
    }
    return LLMB_ERR_UNSUPPORTED;
}

}  // namespace llmb

extern "C" int llmb_gemv_f16(const LlmbGemvArgs *a, llmb_stream_t stream_) {
    using namespace llmb;
    if (!a || !a->w || !a->x || !a->y || a->n <= 0 || a->k <= 0 || (a->k % 8) != 0) return LLMB_ERR_INVALID;
    if (a->prologue == LLMB_PRO_RMSNORM && !a->gamma) return LLMB_ERR_INVALID;
    if (a->prologue != LLMB_PRO_NONE && a->prologue != LLMB_PRO_RMSNORM) return LLMB_ERR_INVALID;
    if (((uintptr_t)a->w | (uintptr_t)a->x | (uintptr_t)a->w2 | (uintptr_t)a->gamma) & 15) return LLMB_ERR_INVALID;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GemvParams p = {};
    p.w = reinterpret_cast<const __half *>(a->w);
    p.w2 = reinterpret_cast<const __half *>(a->w2);
    p.x = reinterpret_cast<const __half *>(a->x);
    p.y = reinterpret_cast<__half *>(a->y);
    p.gamma = reinterpret_cast<const __half *>(a->gamma);
    p.rope_cs = reinterpret_cast<const float2 *>(a->rope_cs);
    p.k_cache = reinterpret_cast<__half *>(a->k_cache);
    p.v_cache = reinterpret_cast<__half *>(a->v_cache);
    p.pos = a->pos;
    p.status = device_status_ptr();
    p.eps = a->eps;
    p.n = a->n;
    p.k = a->k;
    p.prologue = a->prologue;
    p.n_q = a->n_q;
    p.n_kv = a->n_kv;
    p.head_dim = a->head_dim;
    p.max_pos = a->max_pos;
    if (!p.status) return LLMB_ERR_CUDA;
    const int sms = sm_count_cached();
    const bool pdl = a->use_pdl != 0;
    switch (a->epilogue) {
        case LLMB_EPI_STORE: return dispatch_j<LLMB_EPI_STORE>(p, sms, pdl, stream);
        case LLMB_EPI_RESIDUAL: return dispatch_j<LLMB_EPI_RESIDUAL>(p, sms, pdl, stream);
        case LLMB_EPI_SWIGLU:
            if (!a->w2) return LLMB_ERR_INVALID;
            return dispatch_j<LLMB_EPI_SWIGLU>(p, sms, pdl, stream);
        case LLMB_EPI_ROPE_KV:
            if (!a->rope_cs || !a->k_cache || !a->v_cache || !a->pos || a->head_dim <= 0 || (a->head_dim & 1) ||
                a->n != a->n_q + 2 * a->n_kv || (a->n_q & 1) || (a->n_kv & 1))
                return LLMB_ERR_INVALID;
            return dispatch_j<LLMB_EPI_ROPE_KV>(p, sms, pdl, stream);
        default: return LLMB_ERR_INVALID;
    }
}
