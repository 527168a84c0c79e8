// Temperature / top-k / top-p sampling on the device: the reference's host chain sample_next_token ->
// temperature_softmax -> top_k_sampling -> top_p_sampling (src/inference/inference.cu:1030-1161) as one
// kernel over the FP16 logits a decode step leaves in device memory, so that a sampled decode needs no
// 256 KB device-to-host copy of the logits per token.
//
//   t_i = expf(float(logit_i) / temperature);  p_i = t_i / sum(t)             (:1041-1061, no maximum subtracted)
//   order by p descending, ties to the lower index                            (:1059, qsort with ties unspecified)
//   the first top_k entries are renormalised to sum 1                         (:1088-1096; its own pick is discarded)
//   the shortest prefix whose running sum reaches top_p is renormalised       (:1131-1148)
//   the first entry whose running sum exceeds u is returned, entry 0 if none  (:1154-1160)
//
// One CTA of 1024 threads; thread t owns the vocabulary entries i = t (mod 1024).  The descending order is
// never built for the whole vocabulary: entries are taken one at a time by a block-wide argmax (the owner of
// the winner rescans its own entries), first top_k of them, then more only while the prefix has not reached
// top_p (at most kSamplerMaxSelect in all).  The sequential part runs on thread 0 with the reference's
// statements in the reference's order.  Different from the host code: the sum of the t_i is a tree over
// threads, not a loop in index order, and expf is CUDA's, so probabilities can differ from the host's by a
// few FP32 ulps; the token differs only if u lies within that distance of a boundary between two entries.
#include "common.cuh"
#include "../../include/llm_b200_synth.h"

namespace llmb {

constexpr int kSamplerThreads = 1024;
constexpr int kSamplerMaxSelect = 1024;

struct SamplerParams {
    const __half *logits;
    float *probs;   // [vocab] scratch
    int *token_out;
    int *pos;       // optional: history[*pos] = token (the position the decode step has already advanced to)
    int *history;
    int history_len;
    int *result;    // 0 ok, 1 overflow, 2 prefix longer than kSamplerMaxSelect
    int vocab, top_k;
    float temperature, top_p, u;
};

__device__ __forceinline__ bool before(float pa, int ia, float pb, int ib) { return pa > pb || (pa == pb && ia < ib); }

__global__ void __launch_bounds__(kSamplerThreads) sample_kernel(const SamplerParams p) {
    __shared__ float sel_p[kSamplerMaxSelect];
    __shared__ int sel_i[kSamplerMaxSelect];
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    __shared__ float total_s;
    __shared__ int more_s;     // thread 0 wants one more entry of the order
    __shared__ int winner_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch_dependents();
    pdl_wait();

    // ---- t_i and their sum ----
    float local = 0.0f;
    for (int i = tid; i < p.vocab; i += kSamplerThreads) {
        const float t = expf(__fdiv_rn(__half2float(p.logits[i]), p.temperature));
        p.probs[i] = t;
        local += t;
    }
    local = warp_sum(local);
    if (lane == 0) red_v[warp] = local;
    __syncthreads();
    if (warp == 0) {
        float v = red_v[lane];
        v = warp_sum(v);
        if (lane == 0) total_s = v;
    }
    __syncthreads();
    const float total = total_s;
    if (!(total > 0.0f) || isinf(total) || isnan(total)) {
        if (tid == 0) { p.token_out[0] = -1; p.result[0] = 1; }
        return;
    }
    // ---- p_i; every thread's best entry ----
    float best = -1.0f;
    int best_i = 0x7fffffff;
    for (int i = tid; i < p.vocab; i += kSamplerThreads) {
        const float pr = __fdiv_rn(p.probs[i], total);
        p.probs[i] = pr;
        if (before(pr, i, best, best_i)) { best = pr; best_i = i; }
    }
    // ---- the order, one entry at a time ----
    int n_sel = 0;
    float sum_k = 0.0f, cumulative = 0.0f;  // thread 0's running values
    int cutoff = -1;
    for (;;) {
        // block-wide argmax of the threads' best entries
        float v = best;
        int vi = best_i;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, m);
            const int oi = __shfl_xor_sync(0xffffffffu, vi, m);
            if (before(ov, oi, v, vi)) { v = ov; vi = oi; }
        }
        if (lane == 0) { red_v[warp] = v; red_i[warp] = vi; }
        __syncthreads();
        if (warp == 0) {
            v = red_v[lane];
            vi = red_i[lane];
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, m);
                const int oi = __shfl_xor_sync(0xffffffffu, vi, m);
                if (before(ov, oi, v, vi)) { v = ov; vi = oi; }
            }
            if (lane == 0) {
                sel_p[n_sel] = v;
                sel_i[n_sel] = vi;
                winner_s = vi;
                // does the sequential part need another entry after this one?
                int more = 1;
                const int have = n_sel + 1;
                if (have < p.top_k && have < p.vocab) {
                    more = 1;                       // still collecting the first top_k entries
                } else {
                    if (have == p.top_k || (have == p.vocab && have < p.top_k)) {
                        // top_k_sampling: renormalise the first k entries (inference.cu:1088-1096)
                        for (int i = 0; i < have; ++i) sum_k += sel_p[i];
                        for (int i = 0; i < have; ++i) sel_p[i] = __fdiv_rn(sel_p[i], sum_k);
                        // top_p_sampling: running sum over the (partly renormalised) order (:1131-1136)
                        for (int i = 0; i < have && cutoff < 0; ++i) {
                            cumulative += sel_p[i];
                            if (cumulative >= p.top_p) cutoff = i;
                        }
                    } else {  // an entry beyond the first k keeps its own probability
                        cumulative += sel_p[have - 1];
                        if (cumulative >= p.top_p) cutoff = have - 1;
                    }
                    more = (cutoff < 0 && have < p.vocab && have < kSamplerMaxSelect) ? 1 : 0;
                }
                more_s = more;
            }
        }
        __syncthreads();
        ++n_sel;
        if (!more_s) break;
        // the owner of the winner strikes it out and finds its next best entry
        const int w = winner_s;
        if ((w % kSamplerThreads) == tid) {
            p.probs[w] = -1.0f;
            best = -1.0f;
            best_i = 0x7fffffff;
            for (int i = tid; i < p.vocab; i += kSamplerThreads) {
                const float pr = p.probs[i];
                if (pr >= 0.0f && before(pr, i, best, best_i)) { best = pr; best_i = i; }
            }
        }
    }
    if (tid != 0) return;
    if (cutoff < 0) {
        if (n_sel < p.vocab) {  // the prefix ran past what this kernel orders: let the host sampler take the step
            p.token_out[0] = -1;
            p.result[0] = 2;
            return;
        }
        cutoff = p.vocab - 1;   // :1140-1143
    }
    const float sum = cumulative;  // :1138
    for (int i = 0; i <= cutoff; ++i) sel_p[i] = __fdiv_rn(sel_p[i], sum);  // :1146-1148
    int token = sel_i[0];          // :1159-1160
    float run = 0.0f;
    for (int i = 0; i <= cutoff; ++i) {  // :1154-1158
        run += sel_p[i];
        if (p.u < run) { token = sel_i[i]; break; }
    }
    p.token_out[0] = token;
    p.result[0] = 0;
    if (p.pos && p.history) {
        const int at = p.pos[0];
        if (at >= 0 && at < p.history_len) p.history[at] = token;
    }
}

}  // namespace llmb

extern "C" size_t llmb_sample_scratch_bytes(int vocab) { return vocab > 0 ? (size_t)vocab * sizeof(float) + 256 : 0; }

extern "C" int llmb_sample_logits(const uint16_t *d_logits, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
                                  uint64_t draw, void *d_scratch, int32_t *d_token_out, int32_t *d_pos, int32_t *d_history,
                                  int history_len, int use_pdl, llmb_stream_t stream_) {
    using namespace llmb;
    if (!d_logits || !d_scratch || !d_token_out || vocab <= 0 || !(temperature > 0.0f) || top_k < 1 || !(top_p > 0.0f) ||
        ((uintptr_t)d_scratch & 255)) {
        set_last_error("llmb_sample_logits: need temperature > 0, top_k >= 1, 0 < top_p, a 256-byte aligned scratch");
        return LLMB_ERR_INVALID;
    }
    if (top_p > 1.0f) top_p = 1.0f;    // inference.cu:1124-1126
    if (top_k > vocab) top_k = vocab;  // :1083-1085
    if (top_k > kSamplerMaxSelect) {
        set_last_error("llmb_sample_logits: top_k above 1024 is not ordered on the device; use llmb_sample_logits_host");
        return LLMB_ERR_UNSUPPORTED;
    }
    SamplerParams p;
    p.logits = reinterpret_cast<const __half *>(d_logits);
    p.result = static_cast<int *>(d_scratch);
    p.probs = reinterpret_cast<float *>(static_cast<unsigned char *>(d_scratch) + 256);
    p.token_out = d_token_out;
    p.pos = d_pos;
    p.history = d_history;
    p.history_len = history_len;
    p.vocab = vocab;
    p.top_k = top_k;
    p.temperature = temperature;
    p.top_p = top_p;
    p.u = llmb_synth_uniform(llmb_stream_key(seed, LLMB_SID_SAMPLER), draw);
    LLMB_CUDA_OK(launch_pdl(sample_kernel, dim3(1), dim3(kSamplerThreads), 0, static_cast<cudaStream_t>(stream_), use_pdl != 0, p));
    return LLMB_OK;
}
