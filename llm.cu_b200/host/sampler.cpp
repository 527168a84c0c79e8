// Host-side temperature / top-k / top-p sampling: the reference's sample_next_token chain
// (src/inference/inference.cu:1030-1161) without its full-vocabulary qsort.  Only the first top_k
// entries of the descending order can ever be drawn (the top-k pass renormalises them to sum 1, so
// the top-p prefix ends inside them), so the order is built with a partial sort and completed only
// if the prefix runs past top_k.
#include <algorithm>
#include <cmath>
#include <vector>

#include <cuda_fp16.h>

#include "../../include/llm_b200.h"
#include "../../include/llm_b200_synth.h"

namespace llmb {
void set_last_error(const char *msg);
}

namespace {

struct ProbIndex {
    float probability;
    int index;
};

// descending probability; equal probabilities keep index order (the reference's qsort comparator,
// inference.cu:1063-1074, returns 0 for ties and leaves their order to the library)
inline bool before(const ProbIndex &a, const ProbIndex &b) {
    return a.probability > b.probability || (a.probability == b.probability && a.index < b.index);
}

}  // namespace

extern "C" float llmb_sampler_uniform(uint64_t seed, uint64_t draw) {
    return llmb_synth_uniform(llmb_stream_key(seed, LLMB_SID_SAMPLER), draw);
}

extern "C" int llmb_sample_logits_host(const uint16_t *h_logits, int vocab, float temperature, int top_k, float top_p,
                                       float u, int32_t *token_out) {
    if (!h_logits || !token_out || vocab <= 0 || !(temperature > 0.0f) || top_k < 1 || !(top_p > 0.0f) ||
        !(u >= 0.0f && u < 1.0f)) {
        llmb::set_last_error("llmb_sample_logits_host: need temperature > 0, top_k >= 1, 0 < top_p <= 1, 0 <= u < 1");
        return LLMB_ERR_INVALID;
    }
    if (top_p > 1.0f) top_p = 1.0f;        // inference.cu:1124-1126
    if (top_k > vocab) top_k = vocab;      // :1083-1085
    const __half *logits = reinterpret_cast<const __half *>(h_logits);
    std::vector<ProbIndex> dist((size_t)vocab);
    // temperature_softmax (:1041-1061): no maximum is subtracted, the sum runs in index order in FP32
    float cumsum = 0.0f;
    for (int i = 0; i < vocab; ++i) {
        const float t = expf(__half2float(logits[i]) / temperature);
        dist[(size_t)i].probability = t;
        dist[(size_t)i].index = i;
        cumsum += t;
    }
    if (!std::isfinite(cumsum) || !(cumsum > 0.0f)) {
        // the reference subtracts no maximum, so expf overflows once logit / temperature passes ~88
        llmb::set_last_error("llmb_sample_logits_host: exp(logit / temperature) overflowed FP32 (the reference's softmax "
                             "subtracts no maximum); raise the temperature");
        return LLMB_ERR_UNSUPPORTED;
    }
    for (int i = 0; i < vocab; ++i) dist[(size_t)i].probability /= cumsum;
    std::partial_sort(dist.begin(), dist.begin() + top_k, dist.end(), before);
    // top_k_sampling (:1076-1113): the first k probabilities are renormalised in place; its pick is discarded
    float sum = 0.0f;
    for (int i = 0; i < top_k; ++i) sum += dist[(size_t)i].probability;
    for (int i = 0; i < top_k; ++i) dist[(size_t)i].probability /= sum;
    // top_p_sampling (:1115-1161): shortest prefix of the (partly renormalised) order that reaches p
    float cumulative = 0.0f;
    int cutoff = 0;
    bool tail_sorted = top_k == vocab;
    for (; cutoff < vocab; ++cutoff) {
        if (cutoff == top_k && !tail_sorted) {  // rounding left the first k just short of p: order the rest too
            std::sort(dist.begin() + top_k, dist.end(), before);
            tail_sorted = true;
        }
        cumulative += dist[(size_t)cutoff].probability;
        if (cumulative >= top_p) break;
    }
    if (cutoff >= vocab) cutoff = vocab - 1;
    sum = cumulative;
    for (int i = 0; i <= cutoff; ++i) dist[(size_t)i].probability /= sum;
    cumulative = 0.0f;
    for (int i = 0; i <= cutoff; ++i) {
        cumulative += dist[(size_t)i].probability;
        if (u < cumulative) {
            *token_out = dist[(size_t)i].index;
            return LLMB_OK;
        }
    }
    *token_out = dist[0].index;  // :1159-1160
    return LLMB_OK;
}
