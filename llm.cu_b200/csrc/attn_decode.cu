// Decode attention over the KV cache (one query row, grouped-query heads), split along the
// sequence ("flash-decode").
//
// Bound: HBM/L2 bandwidth on the cached K and V rows: algorithmic bytes per launch =
// (pos + 1) * 2 * n_kv_heads * head_dim * 2.  At the context lengths of the benchmark configs
// this is 1-4 % of a layer's weight bytes at batch 1 and a quarter of a step's bytes at 32 sequences:
// one pass, no N x N score buffer, and the arithmetic on the tensor cores so that a CTA is bound by its
// loads, not by instruction issue.
//
//   grid   (n_splits, n_kv_heads, n_seqs); CTA (s, g, b) handles cache rows [s*split_len, (s+1)*split_len)
//          of KV head g of sequence b for all `G` query heads of that group, so K and V are read once
//          per group, not once per query head.
//   block  128 threads = 4 warps; tiles of 64 cache rows in padded shared memory, two buffers: the next
//          tile streams in (cp.async) while this one is used.  Warp w takes keys 16w..16w+15 of every
//          tile.  The G query heads are the first G rows of a 16-row mma.sync tile (m16n8k16, FP16 in,
//          FP32 accumulate): S = q K^T, scores / sqrtf(head_dim) (inference.cu:784), online softmax in
//          FP32 on the accumulator fragments, O += P V with P split into an FP16 head and an FP16
//          remainder (two MMAs) so that the probabilities enter the product with ~22 bits, as the
//          reference's FP32 P does.  The four warps' (max, sum, out) meet in shared memory.
//   merge  each CTA writes (max, sum, unnormalised out) per query head to scratch; the last
//          CTA to finish for a (sequence, KV head) (atomic counter) rescales and adds the partials in
//          split order, normalises and writes FP16 (inference.cu:945).  The counter is left at zero.
#include <mutex>

#include "common.cuh"
#include "mma_common.cuh"

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
    unsigned long long *trace;  // optional profiling aid: [CTA][8] global-timer stamps (llmb_attn_decode_trace)
};

template <int HD, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnParams p) {
    static_assert(G <= 8, "the query heads of a KV head are the first rows of one 16-row MMA tile");
    constexpr int KP = HD + 8;       // padded tile row: 16-byte aligned, 8 consecutive rows fall in distinct banks
    constexpr int KS = HD / 16;      // k-steps of q . k
    constexpr int OT = HD / 8;       // output n-tiles
    constexpr int CHUNKS = HD / 8;   // 16-byte pieces per cache row
    extern __shared__ __align__(16) unsigned char attn_smem[];
    typedef __half (*TilePtr)[KP];
    constexpr size_t kTileBytes = (size_t)kTile * KP * sizeof(__half);
    __shared__ float wm_s[4][8], wl_s[4][8];  // per warp and query head: running maximum and sum
    __shared__ int is_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad_row = lane >> 2, quad_col = (lane & 3) * 2;
    const int split = blockIdx.x, g = blockIdx.y, seq = blockIdx.z;
    const size_t cta = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    auto stamp = [&](int which) {
        if (p.trace && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t) :: "memory");
            p.trace[cta * 8 + which] = t;
        }
    };
    stamp(0);
    pdl_launch_dependents();
    pdl_wait();
    stamp(1);

    const int len_total = p.pos[seq] + 1;
    const int begin = split * p.split_len;
    // a split that starts past the sequence has nothing to add: the merge below only waits for the splits in use
    if (begin >= len_total) return;
    const int end = min(begin + p.split_len, len_total);
    const __half *q_seq = p.q + (size_t)seq * p.n_q + (size_t)g * G * HD;
    const __half *k_seq = p.k_cache + (size_t)seq * p.seq_stride;
    const __half *v_seq = p.v_cache + (size_t)seq * p.seq_stride;
    const size_t row_stride = (size_t)p.n_kv_heads * HD;
    const int gs = seq * p.n_kv_heads + g;  // (sequence, KV head): index of the counter and of the partials
    const float sqrt_hd = sqrtf((float)HD);

    // A operand: row r < G of the 16-row tile is query head g * G + r; the other rows are zero
    uint32_t qf[KS][4];
    {
        const bool real = quad_row < G;
        const __half *qr = q_seq + (size_t)(real ? quad_row : 0) * HD + quad_col;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = real ? *reinterpret_cast<const uint32_t *>(qr + ks * 16) : 0u;
            qf[ks][2] = real ? *reinterpret_cast<const uint32_t *>(qr + ks * 16 + 8) : 0u;
            qf[ks][1] = qf[ks][3] = 0u;
        }
    }
    float o[OT][4];
#pragma unroll
    for (int t = 0; t < OT; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;  // of row quad_row, over this warp's keys (l: this lane's share)

    // Requests tile i of this split into buffer i & 1; pieces of rows past the split's end are zero-filled.
    auto request_tile = [&](int i) {
        TilePtr kd = reinterpret_cast<TilePtr>(attn_smem + (size_t)(i & 1) * 2 * kTileBytes);
        TilePtr vd = reinterpret_cast<TilePtr>(attn_smem + (size_t)(i & 1) * 2 * kTileBytes + kTileBytes);
        const int t0 = begin + i * kTile;
        for (int c = tid; c < kTile * CHUNKS; c += kAttnThreads) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const bool valid = t0 + r < end;
            const size_t goff = (size_t)(valid ? t0 + r : begin) * row_stride + (size_t)g * HD + ch * 8;
            const uint32_t bytes = valid ? 16u : 0u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&kd[r][ch * 8])), "l"(k_seq + goff), "r"(bytes) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(&vd[r][ch * 8])), "l"(v_seq + goff), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = end > begin ? (end - begin + kTile - 1) / kTile : 0;
    if (n_tiles > 0) request_tile(0);
    for (int ti = 0; ti < n_tiles; ++ti) {
        // the next tile streams in while this one is used
        if (ti + 1 < n_tiles) {
            request_tile(ti + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // every thread's pieces of this tile have landed
        if (ti == 0) stamp(2);
        TilePtr k_s = reinterpret_cast<TilePtr>(attn_smem + (size_t)(ti & 1) * 2 * kTileBytes);
        TilePtr v_s = reinterpret_cast<TilePtr>(attn_smem + (size_t)(ti & 1) * 2 * kTileBytes + kTileBytes);
        const int key0 = begin + ti * kTile + warp * 16;  // this warp's 16 keys of the tile
        if (key0 < end) {
            // S = q K^T for 16 keys: two n-tiles of 8 keys
            float sc[2][4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.0f;
                const __half *kr = &k_s[warp * 16 + t * 8 + quad_row][quad_col];
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
                    mma_16816(sc[t], qf[ks], *reinterpret_cast<const uint32_t *>(kr + ks * 16),
                              *reinterpret_cast<const uint32_t *>(kr + ks * 16 + 8));
            }
            // scale (inference.cu:784), mask keys past the end, row maximum over the 16 keys
            float tmax = -INFINITY;
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const int key = key0 + t * 8 + quad_col;
                sc[t][0] = key < end ? __fdiv_rn(sc[t][0], sqrt_hd) : -INFINITY;
                sc[t][1] = key + 1 < end ? __fdiv_rn(sc[t][1], sqrt_hd) : -INFINITY;
                tmax = fmaxf(tmax, fmaxf(sc[t][0], sc[t][1]));
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(m_run, tmax);  // finite: key0 < end
            const float scale = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
            m_run = m_new;
            l_run *= scale;
#pragma unroll
            for (int t = 0; t < OT; ++t) {
                o[t][0] *= scale;
                o[t][1] *= scale;
            }
            // probabilities as the A operand of P V: an FP16 head and an FP16 remainder (two MMAs), so that
            // they enter the product with ~22 bits, as the reference's FP32 probabilities do
            uint32_t p_hi[4], p_lo[4];
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const float p0 = expf(sc[t][0] - m_new), p1 = expf(sc[t][1] - m_new);  // exp(-inf) = 0 for masked keys
                l_run += p0 + p1;
                const __half2 h01 = __floats2half2_rn(p0, p1);
                const float2 f01 = __half22float2(h01);
                p_hi[2 * t] = *reinterpret_cast<const uint32_t *>(&h01);
                p_lo[2 * t] = pack_half2(p0 - f01.x, p1 - f01.y);
                p_hi[2 * t + 1] = p_lo[2 * t + 1] = 0u;  // rows 8..15 of the tile are not query heads
            }
            // O += P V: B fragments of V through ldmatrix.trans (V rows are keys, the MMA wants keys along k)
#pragma unroll
            for (int t2 = 0; t2 < OT / 2; ++t2) {
                uint32_t vb[4];
                const int mat = lane >> 3, rr = lane & 7;
                ldmatrix_x4_trans(vb, &v_s[warp * 16 + (mat & 1) * 8 + rr][t2 * 16 + (mat >> 1) * 8]);
                mma_16816(o[2 * t2], p_hi, vb[0], vb[1]);
                mma_16816(o[2 * t2], p_lo, vb[0], vb[1]);
                mma_16816(o[2 * t2 + 1], p_hi, vb[2], vb[3]);
                mma_16816(o[2 * t2 + 1], p_lo, vb[2], vb[3]);
            }
        }
        __syncthreads();  // this tile's buffer is free for the tile after next
    }

    stamp(3);
    // ---- the four warps' states meet in shared memory (the tile buffers are idle now) ----
    float *wo_s = reinterpret_cast<float *>(attn_smem);  // [4 warps][G][HD]
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (quad_row < G) {
        if ((lane & 3) == 0) {
            wm_s[warp][quad_row] = m_run;
            wl_s[warp][quad_row] = l_run;
        }
#pragma unroll
        for (int t = 0; t < OT; ++t) {
            wo_s[((size_t)warp * G + quad_row) * HD + t * 8 + quad_col] = o[t][0];
            wo_s[((size_t)warp * G + quad_row) * HD + t * 8 + quad_col + 1] = o[t][1];
        }
    }
    __syncthreads();
    // CTA partial of (head h, dim d): warps combined in warp order
    const size_t pbase = ((size_t)gs * p.n_splits + split) * G;
    for (int e = tid; e < G * HD; e += kAttnThreads) {
        const int h = e / HD, dd = e % HD;
        const float M = fmaxf(fmaxf(wm_s[0][h], wm_s[1][h]), fmaxf(wm_s[2][h], wm_s[3][h]));
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float wgt = (wm_s[w][h] == -INFINITY) ? 0.0f : expf(wm_s[w][h] - M);
            num = fmaf(wgt, wo_s[((size_t)w * G + h) * HD + dd], num);
            den = fmaf(wgt, wl_s[w][h], den);
        }
        p.part_o[(pbase + h) * HD + dd] = num;
        if (dd == 0) {
            p.part_ml[(pbase + h) * 2] = M;
            p.part_ml[(pbase + h) * 2 + 1] = den;
        }
    }
    __threadfence();
    __syncthreads();
    const int n_used = min(p.n_splits, (len_total + p.split_len - 1) / p.split_len);
    if (tid == 0) {
        const int prev = atomicAdd(&p.counters[gs], 1);
        is_last = (prev == n_used - 1);
        if (is_last) p.counters[gs] = 0;  // every split in use has arrived; ready for the next launch
    }
    __syncthreads();
    stamp(4);
    if (!is_last) return;
    __threadfence();

    // Merge, in split order.
    const size_t gbase = (size_t)gs * p.n_splits * G;
    for (int e = tid; e < G * HD; e += kAttnThreads) {
        const int head = e / HD, dd = e % HD;
        float M = -INFINITY;
        for (int sidx = 0; sidx < n_used; ++sidx)
            M = fmaxf(M, __ldcg(&p.part_ml[(gbase + (size_t)sidx * G + head) * 2]));
        float num = 0.0f, den = 0.0f;
        for (int sidx = 0; sidx < n_used; ++sidx) {
            const size_t pi = gbase + (size_t)sidx * G + head;
            const float m = __ldcg(&p.part_ml[pi * 2]);
            const float l = __ldcg(&p.part_ml[pi * 2 + 1]);
            const float wgt = (m == -INFINITY) ? 0.0f : expf(m - M);
            num = fmaf(wgt, __ldcg(&p.part_o[pi * HD + dd]), num);
            den = fmaf(wgt, l, den);
        }
        p.out[(size_t)seq * p.n_q + ((size_t)g * G + head) * HD + dd] = __float2half_rn(__fdiv_rn(num, den));
    }
    stamp(5);
}

template <int HD, int G>
static int launch_attn(const AttnParams &p, int n_seqs, bool pdl, cudaStream_t stream) {
    // two buffers of (K tile, V tile), 64 padded rows each
    const size_t smem = (size_t)4 * kTile * (HD + 8) * sizeof(__half);
    static size_t attr_set[kMaxDevices] = {};  // per instantiation and device
    LLMB_CUDA_OK(ensure_dynamic_smem(attn_decode_kernel<HD, G>, attr_set, smem));
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

static unsigned long long *g_attn_trace = nullptr;

// Profiling aid: per-CTA global-timer stamps of the next launches (entry, previous kernel complete, first tile
// landed, tiles done, partial published, merge done) into a device buffer of 8 uint64 per CTA; NULL turns it off.
extern "C" int llmb_attn_decode_trace(void *d_trace) {
    g_attn_trace = static_cast<unsigned long long *>(d_trace);
    return LLMB_OK;
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
    p.trace = g_attn_trace;
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
