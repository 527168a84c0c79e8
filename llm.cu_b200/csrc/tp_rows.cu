// Tensor parallel, rows at once (m <= 32): the receiving half of the all-reduces that the small-M projection
// starts with LLMB_EPI_TP_SCATTER (gemm_smallm.cu), fused with what follows them in the layer.
//
// A tensor-parallel port of the reference would place a sum all-reduce of [m][d_model] after o_proj and after
// down_proj of every layer (the reference's compute_output / compute_feedforward, inference.cu:600-618 and
// :950-979, then add_norm :366-390 and the next compute_layer_norm :282-363).  Here the projection's epilogue
// has already stored every rank's FP32 partial sums, tagged, into every rank's exchange block over NVLink, so
// the all-reduce is finished by a local kernel:
//
//   tp_gather_rows   one CTA per row; starts while the scattering projection still runs (programmatic
//                    dependent launch without an upfront wait).  Polls (bounded) the tp_size (value, tag) pairs of each element, adds
//                    them in rank order (every rank gets the same bits), rounds to FP16 as the projection
//                    does (:445), adds the residual row in FP32 and rounds (:385-387), writes x, and - if a
//                    gain vector is given - the RMSNorm of the new row (same partials of four, same binary
//                    tree, eps added in double, IEEE division) as the input of the next projection.
//   tp_argmax_rows   one CTA per row.  First maximum of this rank's vocabulary slice, sent as tagged pairs
//                    to every rank; every rank then picks the same winner among the tp_size candidates
//                    (larger value, ties to the lower index) and advances token, position and history.
//   tp_advance       moves the exchange counter on at the end of a step.
//
// Bound: latency (a row is 16 KB of pairs per rank); the bytes are the partial sums that cross NVLink,
// tp_size * m * d_model * 8 per exchange and rank.  Every spin is bounded: on expiry the kernel records status
// 205 (llmb_device_status) and goes on with what it has.
#include "gemv_common.cuh"
#include "tp_common.cuh"

namespace llmb {

constexpr int kGatherThreads = 256;
constexpr uint32_t kRowsPollLimit = 1u << 20;

struct GatherParams {
    unsigned char *exchange;  // this rank's block
    __half *x;                // [m][d] residual rows, updated in place
    const __half *gamma;      // optional [d]
    __half *xn;               // [m][d] normalised rows (when gamma)
    int *status;
    double eps;
    int tp_size, tp_index, d, n_pow2;
    uint32_t poll_limit;
};

__global__ void __launch_bounds__(kGatherThreads) tp_gather_rows_kernel(const GatherParams p) {
    extern __shared__ float part_s[];  // n_pow2 partials of the RMSNorm tree
    __shared__ float rms_s;
    __shared__ int abort_s;
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_launch_dependents();
    if (tid == 0) abort_s = 0;
    __syncthreads();
    // No wait for the previous kernel here: the partial sums carry their own tags, so this kernel may start while
    // the projection that scatters them is still running and takes each chunk as soon as every rank's pair is there.
    // The residual row is read only after this rank's own tagged pair of the chunk has been seen: that pair was
    // stored by the projection's epilogue, which runs after the projection has waited for every earlier kernel -
    // the one that wrote the residual rows among them.
    const bool ok = *reinterpret_cast<volatile int *>(p.status) == 0;
    const unsigned int tag = *reinterpret_cast<const unsigned int *>(p.exchange + tp_rows_seq_off(p.tp_size, p.d)) +
                             (unsigned int)p.tp_index + 1u;
    const int nchunks = p.d >> 3;
    uint4 *xr = reinterpret_cast<uint4 *>(p.x + (size_t)row * p.d);
    for (int c = tid; c < (p.n_pow2 >> 1); c += kGatherThreads) {
        float p0 = 0.0f, p1 = 0.0f;
        if (c < nchunks) {
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
            // The eight elements of a chunk are four 16-byte loads per rank.  Two loads of every rank go out
            // together and are repeated together until all their tags are there (then the other two): one
            // round trip to L2 per half when the data has arrived, not one per rank.
            const unsigned char *src0 = p.exchange + tp_rows_slot(p.tp_size, p.d, p.tp_index, 0, row, c * 8);
            const size_t rank_stride = tp_rows_slot(p.tp_size, p.d, p.tp_index, 1, row, c * 8) - tp_rows_slot(p.tp_size, p.d, p.tp_index, 0, row, c * 8);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint4 q[8][2];
                uint32_t spins = 0;
                for (;;) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        if (r < p.tp_size) {
#pragma unroll
                            for (int u = 0; u < 2; ++u)
                                asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                             : "=r"(q[r][u].x), "=r"(q[r][u].y), "=r"(q[r][u].z), "=r"(q[r][u].w)
                                             : "l"(src0 + (size_t)r * rank_stride + 32 * half + 16 * u)
                                             : "memory");
                        }
                    }
                    bool all = true;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        if (r < p.tp_size)
                            all = all && q[r][0].y == tag && q[r][0].w == tag && q[r][1].y == tag && q[r][1].w == tag;
                    if (all || !ok) break;
                    if ((++spins & 63u) == 0) {
                        if (*reinterpret_cast<volatile int *>(&abort_s)) break;
                        if (spins > p.poll_limit) {
                            atomicExch(p.status, 205);
                            abort_s = 1;
                            break;
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    if (r < p.tp_size) {  // in rank order: every rank forms the same bits
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            acc[4 * half + 2 * u] += __uint_as_float(q[r][u].x);
                            acc[4 * half + 2 * u + 1] += __uint_as_float(q[r][u].z);
                        }
                    }
                }
            }
            float xf[8];
            unpack8(__ldcg(xr + c), xf);  // after the tags: see above
            uint4 xn;
            __half2 *o = reinterpret_cast<__half2 *>(&xn);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                o[e] = __halves2half2(__float2half_rn(__half2float(__float2half_rn(acc[2 * e])) + xf[2 * e]),
                                      __float2half_rn(__half2float(__float2half_rn(acc[2 * e + 1])) + xf[2 * e + 1]));
            xr[c] = xn;
            sumsq_partials(xn, p0, p1);
        }
        part_s[2 * c] = p0;
        part_s[2 * c + 1] = p1;
    }
    if (!p.gamma) {
        pdl_wait();  // keeps the chain of kernels ordered for the launches that follow
        return;
    }
    __syncthreads();  // also orders this CTA's stores of the row before the reads below
    for (int off = p.n_pow2 >> 1; off >= 1; off >>= 1) {
        for (int t = tid; t < off; t += kGatherThreads) part_s[t] += part_s[t + off];
        __syncthreads();
    }
    if (tid == 0) rms_s = sqrtf((float)(p.eps + (double)(part_s[0] / (float)p.d)));
    __syncthreads();
    const float rms = rms_s;
    uint4 *yr = reinterpret_cast<uint4 *>(p.xn + (size_t)row * p.d);
    const uint4 *gr = reinterpret_cast<const uint4 *>(p.gamma);
    for (int c = tid; c < nchunks; c += kGatherThreads) yr[c] = rmsnorm_apply8(xr[c], __ldg(gr + c), rms);
    pdl_wait();  // keeps the chain of kernels ordered for the launches that follow
}

struct TpArgmaxParams {
    unsigned char *peer[8];
    const __half *logits;  // [rows][n_local]
    int *token_out, *pos_inout, *history;
    int *status;
    int tp_rank, tp_size, d, tp_index, n_local, vocab_offset, history_len;
    uint32_t poll_limit;
};

__global__ void __launch_bounds__(1024) tp_argmax_rows_kernel(const TpArgmaxParams p) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const __half *logits = p.logits + (size_t)row * p.n_local;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int n8 = p.n_local / 8;
    for (int c = threadIdx.x; c < n8; c += blockDim.x) {
        const uint4 v = *(reinterpret_cast<const uint4 *>(logits) + c);
        const __half *h = reinterpret_cast<const __half *>(&v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float f = __half2float(h[e]);
            if (f > best) {  // ascending index inside a thread: first maximum kept
                best = f;
                best_i = c * 8 + e;
            }
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x >= 32) return;
    best = sv[threadIdx.x];
    best_i = si[threadIdx.x];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, m);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, m);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    // lane r < tp_size: sends this rank's candidate to rank r, then fetches rank r's candidate
    const int lane = threadIdx.x;
    const unsigned int tag = *reinterpret_cast<const unsigned int *>(p.peer[p.tp_rank] + tp_rows_seq_off(p.tp_size, p.d)) +
                             (unsigned int)p.tp_index + 1u;
    const int global_i = best_i == 0x7fffffff ? 0x7fffffff : best_i + p.vocab_offset;
    float cv = -INFINITY;
    int ci = 0x7fffffff;
    if (lane < p.tp_size) {
        unsigned char *dst = p.peer[lane] + tp_rows_best_off(p.tp_size, p.d) + ((size_t)p.tp_rank * kTpRows + row) * 16;
        asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(best)), "r"(tag),
                     "r"((unsigned int)global_i), "r"(tag)
                     : "memory");
        const unsigned char *src = p.peer[p.tp_rank] + tp_rows_best_off(p.tp_size, p.d) + ((size_t)lane * kTpRows + row) * 16;
        const bool ok = *reinterpret_cast<volatile int *>(p.status) == 0;
        uint4 q;
        uint32_t spins = 0;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                         : "l"(src)
                         : "memory");
            if ((q.y == tag && q.w == tag) || !ok) break;
            if (++spins > p.poll_limit) {
                atomicExch(p.status, 206);
                break;
            }
        }
        cv = __uint_as_float(q.x);
        ci = (int)q.z;
        if (!(cv == cv)) cv = -INFINITY;
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, cv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, ci, m);
        if (ov > cv || (ov == cv && oi < ci)) { cv = ov; ci = oi; }
    }
    if (lane == 0) {
        if (ci == 0x7fffffff) ci = 0;  // all NaN / -inf: the oracle returns index 0
        p.token_out[row] = ci;
        if (p.pos_inout) {
            const int np = p.pos_inout[row] + 1;
            p.pos_inout[row] = np;
            if (p.history && np >= 0 && np < p.history_len) p.history[(size_t)row * p.history_len + np] = ci;
        }
    }
}

__global__ void tp_advance_kernel(unsigned int *seq, unsigned int n) {
    pdl_launch_dependents();
    pdl_wait();
    *seq = *seq + n;
}

}  // namespace llmb

using namespace llmb;

extern "C" int llmb_tp_gather_rows(void *d_exchange, int tp_size, int tp_index, uint16_t *d_x, const uint16_t *d_gamma,
                                   uint16_t *d_xn, int m, int d, double eps, uint32_t poll_limit, int use_pdl, llmb_stream_t stream_) {
    if (!d_exchange || !d_x || m <= 0 || m > kTpRows || d <= 0 || (d & 7) || tp_size < 2 || tp_size > 8 || tp_index < 0 ||
        (d_gamma && !d_xn) || (((uintptr_t)d_x | (uintptr_t)d_gamma | (uintptr_t)d_xn | (uintptr_t)d_exchange) & 15))
        return LLMB_ERR_INVALID;
    GatherParams p;
    p.exchange = static_cast<unsigned char *>(d_exchange);
    p.x = reinterpret_cast<__half *>(d_x);
    p.gamma = reinterpret_cast<const __half *>(d_gamma);
    p.xn = reinterpret_cast<__half *>(d_xn);
    p.status = device_status_ptr();
    if (!p.status) return LLMB_ERR_CUDA;
    p.eps = eps;
    p.tp_size = tp_size;
    p.tp_index = tp_index;
    p.d = d;
    p.n_pow2 = 2;
    while (p.n_pow2 < d / 4) p.n_pow2 <<= 1;
    if ((size_t)p.n_pow2 * 4 > 40 * 1024) return LLMB_ERR_UNSUPPORTED;
    p.poll_limit = poll_limit ? poll_limit : kRowsPollLimit;
    LLMB_CUDA_OK(launch_pdl(tp_gather_rows_kernel, dim3(m), dim3(kGatherThreads), (size_t)p.n_pow2 * 4,
                            static_cast<cudaStream_t>(stream_), use_pdl != 0, p));
    return LLMB_OK;
}

extern "C" int llmb_tp_argmax_rows(void *const *d_peers, int tp_rank, int tp_size, int d_model, int tp_index, const uint16_t *d_logits,
                                   int n_local, int vocab_offset, int rows, int32_t *d_token_out, int32_t *d_pos_inout,
                                   int32_t *d_history, int history_len, uint32_t poll_limit, int use_pdl, llmb_stream_t stream_) {
    if (!d_peers || !d_logits || !d_token_out || rows <= 0 || rows > kTpRows || n_local <= 0 || (n_local & 7) || tp_size < 2 ||
        tp_size > 8 || tp_rank < 0 || tp_rank >= tp_size || ((uintptr_t)d_logits & 15))
        return LLMB_ERR_INVALID;
    TpArgmaxParams p;
    for (int r = 0; r < tp_size; ++r) {
        if (!d_peers[r]) return LLMB_ERR_INVALID;
        p.peer[r] = static_cast<unsigned char *>(d_peers[r]);
    }
    p.logits = reinterpret_cast<const __half *>(d_logits);
    p.token_out = d_token_out;
    p.pos_inout = d_pos_inout;
    p.history = d_history;
    p.status = device_status_ptr();
    if (!p.status) return LLMB_ERR_CUDA;
    p.tp_rank = tp_rank; p.tp_size = tp_size; p.d = d_model; p.tp_index = tp_index;
    p.n_local = n_local; p.vocab_offset = vocab_offset; p.history_len = history_len;
    p.poll_limit = poll_limit ? poll_limit : kRowsPollLimit;
    LLMB_CUDA_OK(launch_pdl(tp_argmax_rows_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0, p));
    return LLMB_OK;
}

extern "C" int llmb_tp_advance(void *d_exchange, int tp_size, int d_model, int n_exchanges, int use_pdl, llmb_stream_t stream_) {
    if (!d_exchange || tp_size < 2 || tp_size > 8 || d_model <= 0 || n_exchanges <= 0) return LLMB_ERR_INVALID;
    unsigned int *seq = reinterpret_cast<unsigned int *>(static_cast<unsigned char *>(d_exchange) + tp_rows_seq_off(tp_size, d_model));
    LLMB_CUDA_OK(launch_pdl(tp_advance_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0, seq,
                            (unsigned int)n_exchanges));
    return LLMB_OK;
}
