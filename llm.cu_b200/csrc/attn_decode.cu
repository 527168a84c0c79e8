// Decode attention over the KV cache (one query row, grouped-query heads), split along the
// sequence ("flash-decode").
//
// Bound: HBM/L2 bandwidth on the cached K and V rows: algorithmic bytes per launch =
// (pos + 1) * 2 * n_kv_heads * head_dim * 2.  At the context lengths of the benchmark configs
// this is 1-4 % of a layer's weight bytes, so the kernel is shaped for latency: many small
// CTAs, one pass, no N x N score buffer.
//
//   grid   (n_splits, n_kv_heads); CTA (s, g) handles cache rows [s*split_len, (s+1)*split_len)
//          of KV head g for all `G` query heads of that group, so K and V are read once per
//          group, not once per query head.
//   block  128 threads; tiles of 64 cache rows, two buffers: the next tile streams in (cp.async)
//          while this one is used.  Scores: thread t < 64 owns cache row t of the tile and computes
//          the G dot products in FP32 ascending d, the order of the reference (inference.cu:776-778),
//          from a 16-byte-chunk XOR-swizzled shared-memory tile (conflict-free row reads).
//          P.V: thread t owns output dimension t % head_dim.
//   merge  each CTA writes (max, sum, unnormalised out) per query head to scratch; the last
//          CTA to finish for a KV head (atomic counter) rescales and adds the partials in split
//          order, normalises and writes FP16 (inference.cu:945).  The counter is left at zero.
#include <mutex>

#include "common.cuh"

namespace llmb {

constexpr int kAttnThreads = 128;
constexpr int kTile = 64;  // cache rows per shared-memory tile; two tiles take turns (one streams in while the other is used)

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct AttnParams {
    const __half *q;
    const __half *k_cache;
    const __half *v_cache;
    const int *pos;
    __half *out;
    int *counters;   // [n_kv_heads]
    float *part_ml;  // [n_kv_heads][n_splits][G][2]
    float *part_o;   // [n_kv_heads][n_splits][G][HD]
    int n_kv_heads, n_splits, split_len;
    // batched decode: blockIdx.z is the sequence; q and out are [n_seqs][n_q], pos is [n_seqs], the caches of
    // consecutive sequences are seq_stride elements apart (0 for a single sequence)
    int n_q;
    size_t seq_stride;
};

template <int HD, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnParams p) {
    constexpr int CHUNKS = HD / 8;              // 16-byte chunks per row
    constexpr int DGROUPS = kAttnThreads / HD;  // thread groups that share one output dim
    constexpr int HPT = G / DGROUPS;            // query heads per thread in the P.V phase
    static_assert(G % DGROUPS == 0 && HPT >= 1, "group size must fill the block");
    extern __shared__ __align__(128) unsigned char attn_smem[];
    // two buffers of (K tile, V tile); a split of at most one tile needs only the first
    const int tile_rows = min(kTile, p.split_len);
    __shared__ __align__(16) float q_s[G * HD];
    __shared__ __align__(16) float p_s[kTile * G];
    __shared__ float red_max[4][G];
    __shared__ float red_sum[4][G];
    __shared__ int is_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, g = blockIdx.y, seq = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();

    const int len_total = p.pos[seq] + 1;
    const __half *q_seq = p.q + (size_t)seq * p.n_q;
    const __half *k_seq = p.k_cache + (size_t)seq * p.seq_stride;
    const __half *v_seq = p.v_cache + (size_t)seq * p.seq_stride;
    const int gs = seq * p.n_kv_heads + g;  // (sequence, KV head): index of the counter and of the partials
    const int begin = split * p.split_len;
    const int end = min(begin + p.split_len, len_total);
    const size_t row_stride = (size_t)p.n_kv_heads * HD;
    const float inv_den = sqrtf((float)HD);

    for (int i = tid; i < G * HD; i += kAttnThreads) q_s[i] = __half2float(q_seq[(size_t)g * G * HD + i]);

    float m_run[G], l_run[G], acc[HPT];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.0f;
    }
#pragma unroll
    for (int h = 0; h < HPT; ++h) acc[h] = 0.0f;
    const int my_d = tid % HD;
    const int my_h0 = (DGROUPS == 1) ? 0 : (tid / HD) * HPT;

    // Requests tile i of this split into buffer i & 1 (one cp.async group per tile and thread).
    auto request_tile = [&](int i) {
        const int t0 = begin + i * kTile, rows = min(kTile, end - t0);
        __half *kd = reinterpret_cast<__half *>(attn_smem) + (size_t)(i & 1) * 2 * tile_rows * HD;
        __half *vd = kd + tile_rows * HD;
        for (int c = tid; c < rows * CHUNKS; c += kAttnThreads) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const int sw = ch ^ (r & 7);
            const size_t goff = (size_t)(t0 + r) * row_stride + (size_t)g * HD + ch * 8;
            cp_async16(&kd[r * HD + sw * 8], k_seq + goff);
            cp_async16(&vd[r * HD + ch * 8], v_seq + goff);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = end > begin ? (end - begin + kTile - 1) / kTile : 0;
    if (n_tiles > 0) request_tile(0);
    for (int ti = 0; ti < n_tiles; ++ti) {
        const int t0 = begin + ti * kTile;
        const int rows = min(kTile, end - t0);
        // the next tile streams in while this one is used (its buffer was released by the barrier that ended
        // the previous iteration)
        if (ti + 1 < n_tiles) {
            request_tile(ti + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // every thread's pieces of this tile have landed (also publishes q_s)
        const __half *k_tile = reinterpret_cast<const __half *>(attn_smem) + (size_t)(ti & 1) * 2 * tile_rows * HD;
        const __half *v_tile = k_tile + tile_rows * HD;

        // scores for cache row t0 + tid
        float s[G];
        const bool active = tid < rows;
#pragma unroll
        for (int h = 0; h < G; ++h) s[h] = 0.0f;
        if (active) {
#pragma unroll
            for (int ch = 0; ch < CHUNKS; ++ch) {
                const uint4 kv = *reinterpret_cast<const uint4 *>(&k_tile[tid * HD + ((ch ^ (tid & 7)) * 8)]);
                const __half2 *kh = reinterpret_cast<const __half2 *>(&kv);
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float2 f = __half22float2(kh[e]);
                    kf[2 * e] = f.x;
                    kf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float4 qa = *reinterpret_cast<const float4 *>(&q_s[h * HD + ch * 8]);
                    const float4 qb = *reinterpret_cast<const float4 *>(&q_s[h * HD + ch * 8 + 4]);
                    s[h] = fmaf(qa.x, kf[0], s[h]);
                    s[h] = fmaf(qa.y, kf[1], s[h]);
                    s[h] = fmaf(qa.z, kf[2], s[h]);
                    s[h] = fmaf(qa.w, kf[3], s[h]);
                    s[h] = fmaf(qb.x, kf[4], s[h]);
                    s[h] = fmaf(qb.y, kf[5], s[h]);
                    s[h] = fmaf(qb.z, kf[6], s[h]);
                    s[h] = fmaf(qb.w, kf[7], s[h]);
                }
            }
#pragma unroll
            for (int h = 0; h < G; ++h) s[h] = __fdiv_rn(s[h], inv_den);  // inference.cu:784
        } else {
#pragma unroll
            for (int h = 0; h < G; ++h) s[h] = -INFINITY;
        }
        // tile maximum per head
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float mx = warp_max(s[h]);
            if (lane == 0) red_max[warp][h] = mx;
        }
        __syncthreads();
        float scale[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float mx = fmaxf(fmaxf(red_max[0][h], red_max[1][h]), fmaxf(red_max[2][h], red_max[3][h]));
            float m_new = fmaxf(m_run[h], mx);
            scale[h] = (m_run[h] == -INFINITY) ? 0.0f : expf(m_run[h] - m_new);
            m_run[h] = m_new;
            float pv = active ? expf(s[h] - m_new) : 0.0f;
            l_run[h] = l_run[h] * scale[h] + pv;  // per-thread partial of the softmax denominator
            if (tid < kTile) p_s[tid * G + h] = pv;   // threads past the tile hold no row
        }
        __syncthreads();
        // P.V for this tile
#pragma unroll
        for (int h = 0; h < HPT; ++h) acc[h] *= scale[my_h0 + h];
        for (int r = 0; r < rows; ++r) {
            const float vf = __half2float(v_tile[r * HD + my_d]);
#pragma unroll
            for (int h = 0; h < HPT; ++h) acc[h] = fmaf(p_s[r * G + my_h0 + h], vf, acc[h]);
        }
        __syncthreads();  // this tile's buffer and p_s are free for the tile after next
    }

    // CTA totals: denominators across threads, then publish the partial.
    __syncthreads();
#pragma unroll
    for (int h = 0; h < G; ++h) {
        float sm = warp_sum(l_run[h]);
        if (lane == 0) red_sum[warp][h] = sm;
    }
    __syncthreads();
    const size_t pbase = ((size_t)gs * p.n_splits + split) * G;
    if (tid < G) {
        const float l = (red_sum[0][tid] + red_sum[1][tid]) + (red_sum[2][tid] + red_sum[3][tid]);
        float m = -INFINITY;
#pragma unroll
        for (int h = 0; h < G; ++h)
            if (h == tid) m = m_run[h];
        p.part_ml[(pbase + tid) * 2] = m;
        p.part_ml[(pbase + tid) * 2 + 1] = l;
    }
#pragma unroll
    for (int h = 0; h < HPT; ++h) p.part_o[(pbase + my_h0 + h) * HD + my_d] = acc[h];
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[gs], 1);
        is_last = (prev == p.n_splits - 1);
        if (is_last) p.counters[gs] = 0;  // every split has arrived; ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    // Merge, in split order.
    const int n_used = min(p.n_splits, (len_total + p.split_len - 1) / p.split_len);
    const size_t gbase = (size_t)gs * p.n_splits * G;
#pragma unroll
    for (int h = 0; h < HPT; ++h) {
        const int head = my_h0 + h;
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_used; ++sidx)
            M = fmaxf(M, __ldcg(&p.part_ml[(gbase + (size_t)sidx * G + head) * 2]));
        float num = 0.0f, den = 0.0f;
        for (int sidx = 0; sidx < n_used; ++sidx) {
            const size_t pi = gbase + (size_t)sidx * G + head;
            const float m = __ldcg(&p.part_ml[pi * 2]);
            const float l = __ldcg(&p.part_ml[pi * 2 + 1]);
            const float wgt = (m == -INFINITY) ? 0.0f : expf(m - M);
            num = fmaf(wgt, __ldcg(&p.part_o[pi * HD + my_d]), num);
            den = fmaf(wgt, l, den);
        }
        p.out[(size_t)seq * p.n_q + ((size_t)g * G + head) * HD + my_d] = __float2half_rn(__fdiv_rn(num, den));
    }
}

template <int HD, int G>
static int launch_attn(const AttnParams &p, int n_seqs, bool pdl, cudaStream_t stream) {
    // (K tile, V tile) of min(64, split_len) rows, twice if the split has more than one tile
    const size_t smem = (size_t)(p.split_len > kTile ? 2 : 1) * 2 * (p.split_len < kTile ? p.split_len : kTile) * HD * sizeof(__half);
    static size_t attr_set[kMaxDevices] = {};  // per instantiation and device
    LLMB_CUDA_OK(ensure_dynamic_smem(attn_decode_kernel<HD, G>, attr_set, (size_t)4 * kTile * HD * sizeof(__half)));
    LLMB_CUDA_OK(launch_pdl(attn_decode_kernel<HD, G>, dim3(p.n_splits, p.n_kv_heads, n_seqs), dim3(kAttnThreads), smem,
                            stream, pdl, p));
    return LLMB_OK;
}

static size_t attn_counters_bytes(int n_kv_heads) { return ((size_t)n_kv_heads * 4 + 255) / 256 * 256; }

}  // namespace llmb

extern "C" size_t llmb_attn_decode_scratch_bytes(int n_q_heads, int n_kv_heads, int head_dim, int n_splits) {
    if (n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || n_splits <= 0) return 0;
    size_t ml = ((size_t)n_q_heads * n_splits * 2 * 4 + 255) / 256 * 256;
    size_t o = (size_t)n_q_heads * n_splits * head_dim * 4;
    return llmb::attn_counters_bytes(n_kv_heads) + ml + o;
}

static int attn_decode_impl(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int32_t *d_pos,
                            int n_seqs, size_t seq_stride_elems, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                            int split_len, uint16_t *d_out, void *d_scratch, int use_pdl, llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out || !d_scratch) return LLMB_ERR_INVALID;
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads || n_splits <= 0 || split_len <= 0 || n_seqs <= 0 || n_seqs > 65535)
        return LLMB_ERR_INVALID;
    if (((uintptr_t)d_scratch & 255) || ((uintptr_t)d_k_cache & 15) || ((uintptr_t)d_v_cache & 15) || (seq_stride_elems & 7))
        return LLMB_ERR_INVALID;
    AttnParams p;
    p.q = reinterpret_cast<const __half *>(d_q);
    p.k_cache = reinterpret_cast<const __half *>(d_k_cache);
    p.v_cache = reinterpret_cast<const __half *>(d_v_cache);
    p.pos = d_pos;
    p.out = reinterpret_cast<__half *>(d_out);
    // scratch of n_seqs sequences = the layout of one sequence with n_seqs times the heads
    unsigned char *sc = static_cast<unsigned char *>(d_scratch);
    p.counters = reinterpret_cast<int *>(sc);
    sc += attn_counters_bytes(n_kv_heads * n_seqs);
    p.part_ml = reinterpret_cast<float *>(sc);
    sc += ((size_t)n_q_heads * n_seqs * n_splits * 2 * 4 + 255) / 256 * 256;
    p.part_o = reinterpret_cast<float *>(sc);
    p.n_kv_heads = n_kv_heads;
    p.n_splits = n_splits;
    p.split_len = split_len;
    p.n_q = n_q_heads * head_dim;
    p.seq_stride = seq_stride_elems;
    const int G = n_q_heads / n_kv_heads;
    const bool pdl = use_pdl != 0;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (head_dim == 128) {
        switch (G) {
            case 1: return launch_attn<128, 1>(p, n_seqs, pdl, stream);
            case 2: return launch_attn<128, 2>(p, n_seqs, pdl, stream);
            case 4: return launch_attn<128, 4>(p, n_seqs, pdl, stream);
            case 8: return launch_attn<128, 8>(p, n_seqs, pdl, stream);
        }
    } else if (head_dim == 64) {
        switch (G) {
            case 2: return launch_attn<64, 2>(p, n_seqs, pdl, stream);
            case 4: return launch_attn<64, 4>(p, n_seqs, pdl, stream);
            case 8: return launch_attn<64, 8>(p, n_seqs, pdl, stream);
        }
    }
    return LLMB_ERR_UNSUPPORTED;
}

extern "C" int llmb_attn_decode(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                const int32_t *d_pos, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                                int split_len, uint16_t *d_out, void *d_scratch, int use_pdl, llmb_stream_t stream_) {
    return attn_decode_impl(d_q, d_k_cache, d_v_cache, d_pos, 1, 0, n_q_heads, n_kv_heads, head_dim, n_splits, split_len, d_out,
                            d_scratch, use_pdl, stream_);
}

extern "C" size_t llmb_attn_decode_batch_scratch_bytes(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int n_splits) {
    if (n_seqs <= 0) return 0;
    return llmb_attn_decode_scratch_bytes(n_q_heads * n_seqs, n_kv_heads * n_seqs, head_dim, n_splits);
}

extern "C" int llmb_attn_decode_batch(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                      const int32_t *d_pos, int n_seqs, size_t seq_stride_rows, int n_q_heads, int n_kv_heads,
                                      int head_dim, int n_splits, int split_len, uint16_t *d_out, void *d_scratch, int use_pdl,
                                      llmb_stream_t stream_) {
    if (n_kv_heads <= 0 || head_dim <= 0) return LLMB_ERR_INVALID;
    return attn_decode_impl(d_q, d_k_cache, d_v_cache, d_pos, n_seqs, seq_stride_rows * (size_t)n_kv_heads * head_dim, n_q_heads,
                            n_kv_heads, head_dim, n_splits, split_len, d_out, d_scratch, use_pdl, stream_);
}

// ---------------------------------------------------------------------------------------
// llmb_attn_decode_static: the same split-KV attention, for hosts that must not allocate.
//
// Some programs that embed this library cannot call cudaMalloc themselves: an inference
// server that handed the whole device to its own pool at start-up and treats any later
// driver allocation as a bug, a real-time loop that cannot take the device-wide
// synchronisation an allocation may imply, or a plug-in that only receives input and output
// buffers from its host and has nowhere to keep a workspace.  For them the partial results
// live in the fixed array below instead of a caller-provided workspace.
//
//  * Limit: n_q_heads * n_splits <= 4096, head_dim <= 128, n_kv_heads <= 64; the array is
//    2,130,176 bytes and every GPU that loads the library carries it until the process ends.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress:
//    in host code the array's name is only a handle, not something a kernel can dereference)
//    and remembers it; make that first call before starting any stream capture.  If the
//    library's device code has not been loaded on that device yet, this look-up is what makes
//    the CUDA runtime load it (the array and the kernels then take their place in device
//    memory), so make the first call at start-up, not inside the allocation-free region.
//  * All calls on a device share the one array and it keeps whatever the previous call
//    left, so the arrival counters are cleared on the stream before each launch; two calls
//    that can overlap on the GPU (different streams, no dependency) race on it.
//  * No cudaMalloc, cudaFree or allocating library routine is called.
// ---------------------------------------------------------------------------------------
namespace llmb {

constexpr int kStaticMaxHeadSplits = 4096;  // n_q_heads * n_splits
constexpr int kStaticMaxHeadDim = 128;
constexpr int kStaticMaxKvHeads = 64;
constexpr size_t kStaticCounterBytes = 256;
constexpr size_t kStaticMlBytes = (size_t)kStaticMaxHeadSplits * 2 * sizeof(float);
constexpr size_t kStaticScratchBytes =
    kStaticCounterBytes + kStaticMlBytes + (size_t)kStaticMaxHeadSplits * kStaticMaxHeadDim * sizeof(float);

static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

static std::mutex g_static_mu;
static void *g_static_ptr[64] = {};

// Device address of the array on the current device (looked up once per device).
static int static_scratch_ptr(void **out) {
    int dev = 0;
    LLMB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_last_error("llmb_attn_decode_static: device ordinal above 63");
        return LLMB_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *ptr = nullptr;
        LLMB_CUDA_OK(cudaGetSymbolAddress(&ptr, g_attn_static_scratch));
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return LLMB_OK;
}

}  // namespace llmb

extern "C" int llmb_attn_decode_static(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                                       const int32_t *d_pos, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                                       int split_len, uint16_t *d_out, int use_pdl, llmb_stream_t stream_) {
    using namespace llmb;
    if (n_q_heads <= 0 || n_kv_heads <= 0 || n_splits <= 0 || head_dim <= 0) return LLMB_ERR_INVALID;
    if ((long long)n_q_heads * n_splits > kStaticMaxHeadSplits || head_dim > kStaticMaxHeadDim ||
        n_kv_heads > kStaticMaxKvHeads) {
        set_last_error(
            "llmb_attn_decode_static: request exceeds the built-in workspace (n_q_heads * n_splits <= 4096, "
            "head_dim <= 128, n_kv_heads <= 64); use llmb_attn_decode with a caller-provided workspace");
        return LLMB_ERR_UNSUPPORTED;
    }
    // the argument checks llmb_attn_decode makes, here already: nothing is queued on the stream for a call
    // that is going to be refused
    if (!d_q || !d_k_cache || !d_v_cache || !d_pos || !d_out) return LLMB_ERR_INVALID;
    if (split_len <= 0 || n_q_heads % n_kv_heads) return LLMB_ERR_INVALID;
    if (((uintptr_t)d_k_cache & 15) || ((uintptr_t)d_v_cache & 15)) return LLMB_ERR_INVALID;
    void *scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    // Carve the array exactly as llmb_attn_decode carves a caller workspace of this request's size:
    // the layout depends on the request, not on the array's capacity, and fits by the check above.
    if (llmb_attn_decode_scratch_bytes(n_q_heads, n_kv_heads, head_dim, n_splits) > kStaticScratchBytes) {
        set_last_error("llmb_attn_decode_static: request exceeds the built-in workspace");
        return LLMB_ERR_UNSUPPORTED;
    }
    // The counters must start at zero; a finished call leaves them so, an interrupted one may not.
    LLMB_CUDA_OK(cudaMemsetAsync(scratch, 0, kStaticCounterBytes, static_cast<cudaStream_t>(stream_)));
    return llmb_attn_decode(d_q, d_k_cache, d_v_cache, d_pos, n_q_heads, n_kv_heads, head_dim, n_splits, split_len,
                            d_out, scratch, use_pdl, stream_);
}
