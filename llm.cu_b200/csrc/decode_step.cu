// One decode step of the whole model as ONE persistent kernel (one CTA per SM, cooperative
// launch): the per-token forward loop of the reference (inference.cu:149-193) for a single new
// row, without a kernel boundary between its phases.
//
// Why: at batch 1 a layer is five dependent phases of 5-36 us each.  As separate kernels each
// boundary drains and refills the memory pipeline; here the weights of every projection stream, in
// program order, through one shared-memory ring of 1-D bulk copies that runs ahead of the math
// across phase boundaries, so HBM keeps working while the CTAs synchronise.  The phases are the
// fused operations of gemv.cu / attn_decode.cu:
//
//   per layer   QKV    RMSNorm(x) -> [q;k;v] rows -> RoPE -> q buffer / KV-cache row `pos`
//               ATTN   split-KV softmax(q K^T / sqrt(hd)) V, last CTA per KV head merges
//               O      o_proj + residual add into x
//               GU     RMSNorm(x) -> SiLU(gate) * up -> h
//               DOWN   down_proj + residual add into x
//   then        LM     RMSNorm(x) -> FP16 logits, per-CTA argmax; CTA 0 picks the first maximum,
//                      appends it to the history and advances `pos`
//
// Bound: HBM.  Algorithmic bytes per launch = all projection weights + lm_head + norm gains + one
// embedding row + (pos + 1) KV rows read + one KV row written.
//
// Roles inside a CTA (17 warps)
//   warps 0-15  two consumer groups of 8 warps; ring stage `it` belongs to group it % 2.  A thread
//               holds its 16-byte chunks of the input row in registers, multiplies them with the
//               stage's rows (mixed-precision FMA, FP32 accumulate), the warp reduces and leaves one
//               partial per row in shared memory, then moves on: consumer warps never wait for each
//               other, only for data.
//   warp 16     the stage finisher: waits until the 8 partials of a stage are there, adds them in
//               warp order, applies the epilogue (RoPE + cache append / residual add / SwiGLU /
//               logit + argmax) and refills the ring slot with the stage six ahead.
// Grid-wide order between phases: a monotonically increasing 64-bit arrival counter in global
// memory; the k-th wait of a launch needs base + k * gridDim.x arrivals, and CTA 0 stores the next
// launch's base at the end.  Every wait (mbarrier or counter) is bounded: on expiry the CTA records
// a status code, stops waiting for anything else and runs to the end.
#include <cstdlib>

#include "gemv_common.cuh"
#include "tp_common.cuh"

namespace llmb {

constexpr int kDsWarps = 16;                      // consumer warps
constexpr int kDsConsumers = kDsWarps * 32;       // 512
constexpr int kDsFinishers = 2;                   // stage finisher warps: finisher f takes the stages of consumer group f
constexpr int kDsThreads = kDsConsumers + 32 * kDsFinishers;
constexpr int kDsGroups = 2;
constexpr int kDsGWarps = kDsWarps / kDsGroups;   // 8
constexpr int kDsGThreads = kDsGWarps * 32;       // 256
constexpr int kDsSlots = 6;
constexpr uint32_t kDsSlotBytes = 32 * 1024;
constexpr int kDsJ = 8;                           // 16-byte chunks of x per thread: k <= 16384
constexpr int kDsTile = 32;                       // cache rows per attention tile
constexpr uint32_t kPollLimit = 1u << 22;
constexpr uint32_t kTagPollLimit = 1u << 20;  // default spins of a tagged wait: on the order of a second

struct DsLayer {
    const __half *wqkv, *wo, *wgate, *wup, *wdown, *g_in, *g_post;
    __half *k_cache, *v_cache;
};

struct DsParams {
    const DsLayer *layers;
    const __half *embed, *lm_head, *g_final;
    const int *history;
    int *pos;
    __half *x, *q, *attn, *h, *logits, *hidden;
    int *next_token;
    unsigned long long *bar;  // [0] arrival counter, [1] base of the next launch
    int *attn_counters;       // [n_kv_heads]
    float *part_ml, *part_o;  // attention partials
    float *amax_val;          // [gridDim]
    int *amax_idx;
    int *status;
    unsigned long long *trace;  // optional: [gridDim][phases][8] globaltimer stamps
    double eps;
    float rope_theta;
    int n_layers, d, nq, nkv, hd, ffn, vocab, embed_rows, max_pos;
    int n_splits, split_len, with_logits, history_len;
    uint32_t tag_poll_limit;    // spins a tagged wait may take before it gives up
    // tensor parallel: nq, nkv, ffn and vocab above are this rank's shares
    int tp_rank, tp_size, vocab_offset;
    __half *x_alt;              // second residual-stream buffer (ping-pong across all-reduces)
    unsigned char *peer[8];     // every rank's exchange block (own block at [tp_rank]); see TpBlock
};

enum { PH_QKV = 0, PH_O = 1, PH_GU = 2, PH_DOWN = 3, PH_LM = 4 };

struct GemvDesc {
    const __half *w, *w2, *x, *gamma, *res;
    __half *y, *hidden_row, *k_cache, *v_cache;
    int n, k, nr, R, kind;
    // tensor parallel: `reduce` >= 0 means the input row is x_old + sum over ranks of recv[reduce & 1]
    // (all-reduce number `reduce` of the step); `scatter` >= 0 means the output is a partial sum that
    // goes to every rank's recv[scatter & 1] instead of the residual stream.
    int reduce, scatter;
    const __half *x_old;
    __half *x_new;
};

__device__ __forceinline__ int rows_per_stage(int k) {
    const int fit = (int)(kDsSlotBytes / (uint32_t)(k * 2));
    return fit >= 8 ? 8 : (fit >= 4 ? 4 : (fit >= 2 ? 2 : 1));
}

// Projection number `ph` of the step: 4 * layer + {QKV, O, GU, DOWN}, then the lm_head.
// `emb` is the embedding row of this step's token.
template <bool kTp>
__device__ __forceinline__ GemvDesc gemv_desc(const DsParams &p, const DsLayer *layers, int ph, const __half *emb) {
    GemvDesc g;
    const int l = ph >> 2;
    const int kind = (ph < 4 * p.n_layers) ? (ph & 3) : PH_LM;
    g.kind = kind;
    g.w2 = nullptr;
    g.gamma = nullptr;
    g.res = nullptr;
    g.hidden_row = nullptr;
    g.k_cache = g.v_cache = nullptr;
    g.reduce = g.scatter = -1;
    g.x_old = nullptr;
    g.x_new = nullptr;
    const int nq = p.nq * p.hd, nkv = p.nkv * p.hd;
    if (kind == PH_LM) {
        g.w = p.lm_head; g.x = p.x; g.gamma = p.g_final; g.y = p.logits; g.n = p.vocab; g.k = p.d;
    } else {
        const DsLayer &L = layers[l];
        if (kind == PH_QKV) {
            g.w = L.wqkv; g.x = (l == 0) ? emb : p.x; g.gamma = L.g_in; g.y = p.q; g.n = nq + 2 * nkv; g.k = p.d;
            g.k_cache = L.k_cache; g.v_cache = L.v_cache;
        } else if (kind == PH_O) {
            g.w = L.wo; g.x = p.attn; g.res = (l == 0) ? emb : p.x; g.y = p.x; g.n = p.d; g.k = nq;
        } else if (kind == PH_GU) {
            g.w = L.wgate; g.w2 = L.wup; g.x = p.x; g.gamma = L.g_post; g.y = p.h; g.n = p.ffn; g.k = p.d;
        } else {
            g.w = L.wdown; g.x = p.h; g.res = p.x; g.y = p.x; g.n = p.d; g.k = p.ffn;
            if (p.hidden) g.hidden_row = p.hidden + (size_t)(l + 1) * p.d;
        }
    }
    if (kTp) {
        // all-reduce 2l follows o_proj of layer l, 2l + 1 follows its down_proj; the reduced row lands
        // in residual buffer (number & 1), the previous row is in the other one (or the embedding)
        __half *xb[2] = {p.x, p.x_alt};
        if (kind == PH_O) g.scatter = 2 * l;
        else if (kind == PH_DOWN) g.scatter = 2 * l + 1;
        else if (kind == PH_GU) g.reduce = 2 * l;
        else if (kind == PH_QKV && l > 0) g.reduce = 2 * l - 1;
        else if (kind == PH_LM) g.reduce = 2 * p.n_layers - 1;
        if (g.reduce >= 0) {
            g.x_old = g.reduce == 0 ? emb : xb[(g.reduce - 1) & 1];
            g.x_new = xb[g.reduce & 1];
            g.hidden_row = (p.hidden && (g.reduce & 1)) ? p.hidden + (size_t)((g.reduce >> 1) + 1) * p.d : nullptr;
        } else if (g.scatter >= 0) {
            g.hidden_row = nullptr;
        }
    }
    g.nr = rows_per_stage(g.k);
    g.R = (kind == PH_GU) ? g.nr / 2 : g.nr;
    return g;
}

__device__ __forceinline__ void cta_range(int groups, int &begin, int &end) {
    begin = (int)(((long long)groups * blockIdx.x) / gridDim.x);
    end = (int)(((long long)groups * (blockIdx.x + 1)) / gridDim.x);
}

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void cp_async16_ds(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all_ds() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct DsShared {
    uint64_t full_bar[kDsSlots];   // stage data has landed (bulk-copy byte count)
    uint64_t done_bar[kDsSlots];   // the 8 consumer warps of the stage have left their partials
    float red[kDsSlots][8][kDsGWarps];
    float res_s[kDsFinishers][128];  // this CTA's slice of the residual stream for the current projection (per finisher)
    float fin_best_val;              // finisher 1's best logit on its way to finisher 0
    int fin_best_idx;
    float norm_buf[kDsGroups][512];
    float2 rope_cs[64];
    float q_s[8 * 128];
    float p_s[8 * kDsTile];
    float scale_s[8];
    float m_s[8], l_s[8];
    float norm_rms[kDsGroups];
    int abort_flag;
    int is_last;
};

// Where the finisher's weight stream stands: the next ring stage to request.
struct DsCursor {
    const unsigned char *w, *w2;
    size_t row_bytes;
    int ph, rg, rg_end, n, R;
    uint32_t it;
};

// Walks the cursor on to the next ring stage in program order (through the projections of the step)
// and yields its source span(s).  False once the last stage of the step has been handed out.
template <bool kTp>
__device__ __forceinline__ bool cursor_next(const DsParams &p, const DsLayer *layers, const __half *emb, DsCursor &c, int n_gemv,
                                            const unsigned char *&src, const unsigned char *&src2, uint32_t &bytes) {
    while (c.rg >= c.rg_end) {
        if (c.ph + 1 >= n_gemv) { c.ph = n_gemv; return false; }
        ++c.ph;
        const GemvDesc g = gemv_desc<kTp>(p, layers, c.ph, emb);
        c.w = reinterpret_cast<const unsigned char *>(g.w);
        c.w2 = reinterpret_cast<const unsigned char *>(g.w2);
        c.row_bytes = (size_t)g.k * 2;
        c.n = g.n;
        c.R = g.R;
        cta_range((g.n + g.R - 1) / g.R, c.rg, c.rg_end);
    }
    const int row0 = c.rg * c.R;
    const int rows = min(c.R, c.n - row0);
    bytes = (uint32_t)(rows * c.row_bytes);
    src = c.w + (size_t)row0 * c.row_bytes;
    src2 = c.w2 ? c.w2 + (size_t)row0 * c.row_bytes : nullptr;
    ++c.rg;
    return true;
}

// Requests the next ring stage.
template <bool kTp>
__device__ __forceinline__ void issue_next_stage(const DsParams &p, const DsLayer *layers, const __half *emb, DsCursor &c, int n_gemv,
                                                 unsigned char *ring, uint64_t *full_bar, uint64_t policy) {
    const unsigned char *src, *src2;
    uint32_t bytes;
    if (!cursor_next<kTp>(p, layers, emb, c, n_gemv, src, src2, bytes)) return;
    const int s = c.it % kDsSlots;
    unsigned char *dst = ring + (size_t)s * kDsSlotBytes;
    mbar_arrive_expect_tx(&full_bar[s], src2 ? 2 * bytes : bytes);
    bulk_g2s(dst, src, bytes, &full_bar[s], policy);
    if (src2) bulk_g2s(dst + (size_t)c.R * c.row_bytes, src2, bytes, &full_bar[s], policy);
    ++c.it;
}

// Walks the cursor past one stage without requesting it (the other finisher's).
template <bool kTp>
__device__ __forceinline__ void skip_stage(const DsParams &p, const DsLayer *layers, const __half *emb, DsCursor &c, int n_gemv) {
    const unsigned char *src, *src2;
    uint32_t bytes;
    if (cursor_next<kTp>(p, layers, emb, c, n_gemv, src, src2, bytes)) ++c.it;
}

template <int NR>
__device__ __forceinline__ float stage_dot(const unsigned char *base, size_t row_bytes, int rows, bool dual,
                                           const uint4 (&xh)[kDsJ], const bool (&have)[kDsJ], int gtid, int lane) {
    // NR rows fit a 32 KB stage only if a row has at most 8 / NR chunks per thread, so the chunk loop
    // is bounded by NJ and no issue slot goes to chunks that cannot exist.
    constexpr int NJ = kDsJ / NR;
    uint4 xs[NJ];
    bool hs[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        xs[j] = xh[j];
        hs[j] = have[j];
    }
    float acc[NR];
    if (dual) stage_dot_rows<NR, NJ, true>(base, row_bytes, rows, gtid, kDsGThreads, xs, hs, acc);
    else stage_dot_rows<NR, NJ, false>(base, row_bytes, rows, gtid, kDsGThreads, xs, hs, acc);
    return warp_reduce_multi<NR>(acc, lane);
}

// kTp = false compiles every tensor-parallel branch out of the single-GPU kernel.
template <bool kTp>
__global__ void __launch_bounds__(kDsThreads, 1) decode_step_kernel(const DsParams p) {
    extern __shared__ __align__(128) unsigned char ds_smem[];
    unsigned char *ring = ds_smem;
    __half *k_tile = reinterpret_cast<__half *>(ds_smem + (size_t)kDsSlots * kDsSlotBytes);
    __half *v_tile = k_tile + kDsTile * 128;
    // the per-layer pointer table, copied once: phase switches must not wait on global memory
    DsLayer *layer_s = reinterpret_cast<DsLayer *>(v_tile + kDsTile * 128);
    __shared__ DsShared sh;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kDsSlots; ++s) {
            mbar_init(&sh.full_bar[s], 1);
            mbar_init(&sh.done_bar[s], kDsGWarps);
        }
        fence_mbar_init();
        sh.abort_flag = 0;
    }
    for (int i = threadIdx.x; i < p.n_layers * (int)(sizeof(DsLayer) / 8); i += kDsThreads)
        reinterpret_cast<unsigned long long *>(layer_s)[i] = reinterpret_cast<const unsigned long long *>(p.layers)[i];
    __syncthreads();

    const int pos = *p.pos;
    int tok = p.history[pos];
    tok = tok < 0 ? 0 : (tok >= p.embed_rows ? p.embed_rows - 1 : tok);
    const __half *emb = p.embed + (size_t)tok * p.d;
    const int n_gemv = 4 * p.n_layers + (p.with_logits ? 1 : 0);
    const int n_q = p.nq * p.hd, n_kv = p.nkv * p.hd;
    const unsigned long long bar_base = p.bar[1];
    unsigned long long n_bar = 0;  // grid-wide waits passed in this launch
    // A wait that gave up in an earlier launch leaves the status word set: until the host has read
    // and cleared it (llmb_device_status), every later launch skips all waits and just runs through,
    // so a lost peer or a wedged ring costs one bounded wait, not one per step.
    bool ok = *reinterpret_cast<volatile int *>(p.status) == 0;  // later only changes right after a barrier of all 17 warps

    // End of a phase for this CTA: all its global writes are ordered before the arrival.
    // the cross-GPU synchronisation number lives in this rank's exchange block (never reset locally)
    unsigned long long *tp_state = kTp ? reinterpret_cast<unsigned long long *>(p.peer[p.tp_rank] + 128) : nullptr;
    const unsigned long long tp_base = tp_state ? tp_state[0] : 0ULL;
    const unsigned int tag_base = tp_state ? (unsigned int)tp_state[1] : 0u;  // all-reduces done before this launch
    unsigned long long n_tp = 0;   // cross-GPU synchronisations passed in this launch
    auto grid_arrive = [&]() {
        named_bar_sync(3, kDsThreads);
        if (tid == 0) {
            // Device scope also under tensor parallelism: the arrival counter orders this GPU's CTAs only.  What goes
            // to the peers (the partial sums of o_proj / down_proj) carries its own tag in the same 8-byte store and is
            // never read on the strength of this counter; a system-scope fence here waited for NVLink in every phase.
            __threadfence();
            atomicAdd(p.bar, 1ULL);
        }
    };
    auto grid_wait = [&]() {
        ++n_bar;
        if (tid == 0 && ok) {
            const unsigned long long target = bar_base + n_bar * (unsigned long long)gridDim.x;
            uint32_t polls = 0;
            while (ld_acquire_u64(p.bar) < target) {
                if (++polls > kPollLimit) {
                    atomicExch(p.status, 202);
                    sh.abort_flag = 1;
                    break;
                }
            }
        }
        named_bar_sync(3, kDsThreads);
        if (sh.abort_flag) ok = false;
    };
    // the wait that follows projection `ph`
    auto wait_after = [&](int prev_ph) {
        const int kind = (prev_ph < 4 * p.n_layers) ? (prev_ph & 3) : PH_LM;
        // tensor parallel: the partial sums of o_proj / down_proj carry their own tags, so the next
        // phase needs no grid-wide wait at all; the arrival is still counted
        if (kTp && (kind == PH_O || kind == PH_DOWN)) ++n_bar;
        else grid_wait();
    };

    if (warp >= kDsWarps) {
        // =========================== stage finishers ===========================
        // Two warps: finisher f takes the stages with it % 2 == f (those of consumer group f) and requests the
        // stages of the same parity (a slot is refilled with the stage six ahead).  One finisher could not keep up
        // with the consumers where the stages are already in the ring (QKV, o_proj after the attention): 0.8 us per
        // stage against 0.5, and the backlog delayed the end of those phases by 2 us.
        const int fin = warp - kDsWarps;
        const uint64_t policy = policy_evict_first();
        DsCursor cur;
        cur.ph = -1;
        cur.rg = cur.rg_end = 0;
        cur.it = 0;
        cur.w = cur.w2 = nullptr;
        cur.row_bytes = 0;
        cur.n = cur.R = 0;
        if (lane == 0) {
            if (fin == 1) skip_stage<kTp>(p, layer_s, emb, cur, n_gemv);
            for (int k = 0; k < kDsSlots / kDsFinishers; ++k) {
                issue_next_stage<kTp>(p, layer_s, emb, cur, n_gemv, ring, sh.full_bar, policy);
                skip_stage<kTp>(p, layer_s, emb, cur, n_gemv);
            }
        }
        float best_val = -INFINITY;
        int best_idx = 0x7fffffff;
        uint32_t it = 0;
        // profiling aid: the finisher's own stamps go to slots 4..6 of the phase's trace row
        auto fstamp = [&](int ph, int which) {
            if (p.trace && lane == 0 && fin == 0) {
                const int tph = ph + (ph + 3) / 4;  // attention phases are interleaved after each QKV
                p.trace[((size_t)blockIdx.x * (5 * p.n_layers + 2) + tph) * 8 + which] = globaltimer_ns();
            }
        };
        for (int ph = 0; ph < n_gemv; ++ph) {
            const GemvDesc g = gemv_desc<kTp>(p, layer_s, ph, emb);
            if (ph > 0) wait_after(ph - 1);
            fstamp(ph, 4);
            int gb, ge;
            cta_range((g.n + g.R - 1) / g.R, gb, ge);
            const unsigned mask = (1u << g.nr) - 1u;
            // Residual rows of this CTA: one batch of L2 loads per phase, not one round trip per stage.
            const int res_rows = (g.res && !(kTp && g.scatter >= 0)) ? min((ge - gb) * g.R, g.n - gb * g.R) : 0;
            const bool res_cached = res_rows <= 128;
            if (res_cached) {
                for (int i = lane; i < res_rows; i += 32) sh.res_s[fin][i] = __half2float(__ldcg(&g.res[gb * g.R + i]));
                __syncwarp();
            }
            for (int rg = gb; rg < ge; ++rg, ++it) {
                if ((int)(it % kDsFinishers) != fin) continue;
                const int s = it % kDsSlots;
                const int row0 = rg * g.R;
                const int rows = min(g.R, g.n - row0);
                float res = 0.0f;
                if (g.res && lane < rows)
                    res = res_cached ? sh.res_s[fin][row0 - gb * g.R + lane] : __half2float(__ldcg(&g.res[row0 + lane]));
                bool got = false;
                if (ok) {
                    got = mbar_wait_warp(&sh.done_bar[s], (it / kDsSlots) & 1, p.status, 204, lane);
                    if (!got) sh.abort_flag = 1;
                }
                if (rg == gb) fstamp(ph, 5);
                if (got && lane < g.nr) {
                    const float *rp = sh.red[s][lane];
                    const float sum = ((rp[0] + rp[1]) + (rp[2] + rp[3])) + ((rp[4] + rp[5]) + (rp[6] + rp[7]));
                    if (g.kind == PH_GU) {
                        const float up = __shfl_down_sync(mask, sum, g.R);
                        if (lane < rows) g.y[row0 + lane] = __float2half_rn(silu_ref(sum) * up);
                    } else if (g.kind == PH_LM) {
                        const __half hv = __float2half_rn(sum);
                        if (lane < rows) g.y[row0 + lane] = hv;
                        float v = lane < rows ? __half2float(hv) : -INFINITY;
                        if (!(v == v)) v = -INFINITY;  // NaN never wins
                        int idx = row0 + lane;
                        for (int m = g.nr >> 1; m >= 1; m >>= 1) {
                            const float ov = __shfl_xor_sync(mask, v, m);
                            const int oi = __shfl_xor_sync(mask, idx, m);
                            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
                        }
                        idx += p.vocab_offset;  // tensor parallel: this rank holds a slice of the vocabulary
                        if (v > best_val || (v == best_val && idx < best_idx)) { best_val = v; best_idx = idx; }
                    } else if (kTp && g.scatter >= 0) {
                        // tensor parallel: this rank's partial sum goes to every rank's receive buffer
                        if (lane < rows) {
                            const size_t off = kTpRecvOff + (((size_t)(g.scatter & 1) * p.tp_size + p.tp_rank) * p.d + row0 + lane) * 8;
                            const unsigned int tag = tag_base + (unsigned int)g.scatter + 1u;
                            for (int r = 0; r < p.tp_size; ++r)
                                asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p.peer[r] + off),
                                             "r"(__float_as_uint(sum)), "r"(tag)
                                             : "memory");
                        }
                    } else if (g.kind == PH_O || g.kind == PH_DOWN) {
                        if (lane < rows) {
                            const float o = __half2float(__float2half_rn(sum));
                            const __half out = __float2half_rn(o + res);
                            g.y[row0 + lane] = out;
                            if (g.hidden_row) g.hidden_row[row0 + lane] = out;
                        }
                    } else {  // PH_QKV: RoPE on q and k rows, then q buffer / cache row `pos`
                        const int row = row0 + lane;
                        const float v = __half2float(__float2half_rn(sum));
                        const float other = __shfl_xor_sync(mask, v, 1);
                        if (lane < rows && pos >= 0 && pos < p.max_pos) {
                            if (row < n_q + n_kv) {
                                const int local = row < n_q ? row : row - n_q;
                                const float2 cs = sh.rope_cs[(local >> 1) % (p.hd >> 1)];
                                const float outv = (row & 1) ? __fmaf_rn(cs.y, other, __fmul_rn(cs.x, v))
                                                             : __fmaf_rn(cs.x, v, -__fmul_rn(cs.y, other));
                                const __half hv = __float2half_rn(outv);
                                if (row < n_q) p.q[row] = hv;
                                else g.k_cache[(size_t)pos * n_kv + local] = hv;
                            } else {
                                g.v_cache[(size_t)pos * n_kv + (row - n_q - n_kv)] = __float2half_rn(sum);
                            }
                        }
                    }
                }
                __syncwarp();
                // slot s is free (all 8 warps have read it) and its partials are consumed: refill with the stage six
                // ahead, and walk the cursor past the other finisher's stage
                if (lane == 0 && got) {
                    issue_next_stage<kTp>(p, layer_s, emb, cur, n_gemv, ring, sh.full_bar, policy);
                    skip_stage<kTp>(p, layer_s, emb, cur, n_gemv);
                }
            }
            // Stores into the peers' memory are posted over NVLink: the warp that issued them waits for
            // them itself, a fence by another thread after a CTA barrier does not cover them.
            fstamp(ph, 6);
            if (g.kind == PH_LM) {  // this CTA's best logit travels with the phase's arrival
                if (fin == 1 && lane == 0) {
                    sh.fin_best_val = best_val;
                    sh.fin_best_idx = best_idx;
                }
                named_bar_sync(4, 32 * kDsFinishers);
                if (fin == 0 && lane == 0) {
                    const float ov = sh.fin_best_val;
                    const int oi = sh.fin_best_idx;
                    if (ov > best_val || (ov == best_val && oi < best_idx)) { best_val = ov; best_idx = oi; }
                    p.amax_val[blockIdx.x] = best_val;
                    p.amax_idx[blockIdx.x] = best_idx;
                }
            }
            grid_arrive();
            if (g.kind == PH_QKV) {  // the consumers' attention phase: keep in step with its barriers
                grid_wait();
                grid_arrive();
            }
        }
        wait_after(n_gemv - 1);
        return;
    }

    // =============================== consumers ===============================
    const int grp = warp / kDsGWarps;   // consumer group of this warp
    const int gwarp = warp % kDsGWarps;  // warp index inside the group
    const int gtid = tid % kDsGThreads;  // thread index inside the group
    // RoPE angles of this position (inference.cu:673-678), once per CTA.
    if (tid < p.hd / 2) {
        const float freq = 1.0f / powf(p.rope_theta, 2.0f * (float)tid / (float)p.hd);
        const float angle = (float)pos * freq;
        sh.rope_cs[tid] = make_float2(cosf(angle), sinf(angle));
    }
    if (p.hidden && blockIdx.x == 0)
        for (int i = tid; i < p.d; i += kDsConsumers) p.hidden[i] = emb[i];

    const int G = p.nq / p.nkv;
    // profiling aid: thread 0 of every CTA stamps the global timer four times per phase
    const int trace_row = (p.trace && tid == 0) ? (int)blockIdx.x : -1;
    auto stamp = [&](int phase, int which) {
        if (trace_row >= 0) p.trace[((size_t)trace_row * (5 * p.n_layers + 2) + phase) * 8 + which] = globaltimer_ns();
    };
    int tphase = 0;
    uint32_t it = 0;

    for (int ph = 0; ph < n_gemv; ++ph) {
        const GemvDesc g = gemv_desc<kTp>(p, layer_s, ph, emb);
        const int nchunks = g.k >> 3;
        const size_t row_bytes = (size_t)g.k * 2;
        bool have[kDsJ];
#pragma unroll
        for (int j = 0; j < kDsJ; ++j) have[j] = (gtid + kDsGThreads * j) < nchunks;
        stamp(tphase, 0);
        if (g.gamma && grp == 0) {  // the gain vector does not depend on the previous phase: bring it to L2 now
#pragma unroll
            for (int j = 0; j < kDsJ / 2; ++j)
                if (have[j])
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint4 *>(g.gamma) + gtid + kDsGThreads * j));
        }
        if (ph > 0) wait_after(ph - 1);  // the phase that produced x has finished everywhere
        stamp(tphase, 1);

        // Both groups hold the whole input row in registers (packed FP16): thread t of a group owns
        // the 16-byte chunks t, t + 256, ...
        constexpr int kNormJ = kDsJ / 2;  // normalised inputs have k = d_model <= 8192
        uint4 xh[kDsJ];
        uint4 gv[kNormJ];
        if (!kTp || g.reduce < 0) {
#pragma unroll
            for (int j = 0; j < kDsJ; ++j)
                xh[j] = have[j] ? __ldcg(reinterpret_cast<const uint4 *>(g.x) + gtid + kDsGThreads * j) : make_uint4(0, 0, 0, 0);
        } else {
            // Tensor parallel: the input row is the all-reduced projection plus the previous residual
            // row, x = half(float(half(sum over ranks of partials)) + float(x_old)): the reference's
            // rounding points (inference.cu:445, :385-387) with the sum taken in rank order.
            // (1) The owner CTA of a 16-byte chunk (chunk % gridDim.x) forms it: four threads of group 0
            //     per chunk, two elements each, poll the tp_size tagged partial sums of their elements.
            // (2) It stores the chunk into the residual buffer and publishes it, tagged, in the local row.
            // (3) Every thread of every CTA polls its own chunks of the local row.
            const unsigned char *recv = p.peer[p.tp_rank] + kTpRecvOff + (size_t)(g.reduce & 1) * p.tp_size * p.d * 8;
            unsigned char *row = p.peer[p.tp_rank] + tp_row_off(p.tp_size, p.d) + (size_t)(g.reduce & 1) * p.d * 4;
            const unsigned int tag = tag_base + (unsigned int)g.reduce + 1u;
            if (grp == 0) {
                const int c = (int)blockIdx.x + (int)gridDim.x * (gtid >> 2);
                if (c < (p.d >> 3)) {
                    const int e0 = c * 8 + (gtid & 3) * 2;
                    // The loads of four ranks' pairs go out together and are repeated together until their tags are
                    // there: one round trip to L2 per four ranks when the data has arrived, not one per rank.
                    const unsigned char *src = recv + (size_t)e0 * 8;
                    const size_t rank_stride = (size_t)p.d * 8;
                    float a0 = 0.0f, a1 = 0.0f;
                    for (int r0 = 0; r0 < p.tp_size; r0 += 4) {
                        uint4 q[4];
                        uint32_t spins = 0;
                        for (;;) {
#pragma unroll
                            for (int r = 0; r < 4; ++r) {
                                if (r0 + r < p.tp_size)
                                    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                                 : "=r"(q[r].x), "=r"(q[r].y), "=r"(q[r].z), "=r"(q[r].w)
                                                 : "l"(src + (size_t)(r0 + r) * rank_stride)
                                                 : "memory");
                            }
                            bool all = true;
#pragma unroll
                            for (int r = 0; r < 4; ++r)
                                if (r0 + r < p.tp_size) all = all && q[r].y == tag && q[r].w == tag;
                            if (all || !ok) break;
                            if ((++spins & 63u) == 0) {  // another wait of this CTA gave up: do not start a new limit
                                if (*reinterpret_cast<volatile int *>(&sh.abort_flag)) break;
                                if (spins > p.tag_poll_limit) {
                                    atomicExch(p.status, 205);
                                    sh.abort_flag = 1;
                                    break;
                                }
                            }
                        }
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            if (r0 + r < p.tp_size) {  // in rank order: every rank forms the same bits
                                a0 += __uint_as_float(q[r].x);
                                a1 += __uint_as_float(q[r].z);
                            }
                        }
                    }
                    const float2 xo = __half22float2(*reinterpret_cast<const __half2 *>(g.x_old + e0));
                    const __half2 xn = __halves2half2(__float2half_rn(__half2float(__float2half_rn(a0)) + xo.x),
                                                      __float2half_rn(__half2float(__float2half_rn(a1)) + xo.y));
                    *reinterpret_cast<__half2 *>(g.x_new + e0) = xn;
                    if (g.hidden_row) *reinterpret_cast<__half2 *>(g.hidden_row + e0) = xn;
                    asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1, %2};" ::"l"(row + (size_t)(e0 >> 1) * 8),
                                 "r"(*reinterpret_cast<const uint32_t *>(&xn)), "r"(tag)
                                 : "memory");
                }
            }
            // Only group 0 polls (one chunk after the other); group 1 takes the row from shared memory afterwards (the
            // attention tiles, idle in this phase).  148 x 512 threads polling the row took enough of L2's bandwidth
            // to slow every round of polls: asking for two chunks at once instead of one cost 5 % of the step, and
            // leaving the polls to one group gained 4 % (430 -> 446 tok/s at two GPUs); a pause between rounds, nothing.
            uint4 *x_s = reinterpret_cast<uint4 *>(k_tile);  // d_model <= 8192 halves = 16 KB = the K and V tile
#pragma unroll
            for (int j = 0; j < kDsJ / 2; ++j) {
                xh[j] = make_uint4(0, 0, 0, 0);
                if (grp == 0 && have[j]) {
                    const unsigned char *src = row + (size_t)(gtid + kDsGThreads * j) * 32;  // 4 (FP16 pair, tag) slots
                    uint4 q0, q1;
                    uint32_t spins = 0;
                    for (;;) {
                        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(q0.x), "=r"(q0.y), "=r"(q0.z), "=r"(q0.w)
                                     : "l"(src)
                                     : "memory");
                        asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(q1.x), "=r"(q1.y), "=r"(q1.z), "=r"(q1.w)
                                     : "l"(src + 16)
                                     : "memory");
                        if ((q0.y == tag && q0.w == tag && q1.y == tag && q1.w == tag) || !ok) break;
                        if ((++spins & 63u) == 0) {
                            if (*reinterpret_cast<volatile int *>(&sh.abort_flag)) break;
                            if (spins > p.tag_poll_limit) {
                                atomicExch(p.status, 205);
                                sh.abort_flag = 1;
                                break;
                            }
                        }
                    }
                    xh[j] = make_uint4(q0.x, q0.z, q1.x, q1.z);
                    x_s[gtid + kDsGThreads * j] = xh[j];
                }
            }
            named_bar_sync(2, kDsConsumers);
            if (grp == 1) {
#pragma unroll
                for (int j = 0; j < kDsJ / 2; ++j)
                    if (have[j]) xh[j] = x_s[gtid + kDsGThreads * j];
            }
#pragma unroll
            for (int j = kDsJ / 2; j < kDsJ; ++j) xh[j] = make_uint4(0, 0, 0, 0);
        }
        if (g.gamma) {
#pragma unroll
            for (int j = 0; j < kNormJ; ++j)
                gv[j] = have[j] ? __ldg(reinterpret_cast<const uint4 *>(g.gamma) + gtid + kDsGThreads * j)
                                : make_uint4(0, 0, 0, 0);
            // Sum of squares in the reference's reduction order (inference.cu:309-344): a partial per
            // four consecutive elements, then a binary tree with offsets halving from (k/4)/2.  Chunk
            // c = t + 256 j holds partials 2c, 2c+1: offsets >= 512 stay inside a thread, 256..64 cross
            // warps (shared memory), 32..2 are shuffles, the last is inside a thread again.
            float p0[kNormJ], p1[kNormJ];
#pragma unroll
            for (int j = 0; j < kNormJ; ++j) sumsq_partials(xh[j], p0[j], p1[j]);
#pragma unroll
            for (int off = kNormJ / 2; off >= 1; off >>= 1) {
#pragma unroll
                for (int j = 0; j < off; ++j) {
                    p0[j] += p0[j + off];
                    p1[j] += p1[j + off];
                }
            }
            float *nb = sh.norm_buf[grp];
            nb[2 * gtid] = p0[0];
            nb[2 * gtid + 1] = p1[0];
            named_bar_sync(6 + grp, kDsGThreads);
            if (gwarp == 0) {
                float v[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float *b = nb + 2 * lane + e;
                    v[e] = ((b[0] + b[256]) + (b[128] + b[384])) + ((b[64] + b[320]) + (b[192] + b[448]));
                }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    v[0] += __shfl_down_sync(0xffffffffu, v[0], off);
                    v[1] += __shfl_down_sync(0xffffffffu, v[1], off);
                }
                if (lane == 0) sh.norm_rms[grp] = sqrtf((float)(p.eps + (double)((v[0] + v[1]) / (float)g.k)));
            }
            named_bar_sync(6 + grp, kDsGThreads);
            const float rms = sh.norm_rms[grp];
#pragma unroll
            for (int j = 0; j < kNormJ; ++j)
                if (have[j]) xh[j] = rmsnorm_apply8(xh[j], gv[j], rms);  // (0 * g) / rms would hit the division's slow path
        }
        stamp(tphase, 2);

        // ---- this CTA's row groups: ring stage `it` belongs to consumer group it % 2 ----
        int gb, ge;
        cta_range((g.n + g.R - 1) / g.R, gb, ge);
        const bool dual = g.w2 != nullptr;
        for (int rg = gb; rg < ge; ++rg, ++it) {
            if ((int)(it % kDsGroups) != grp) continue;
            const int s = it % kDsSlots;
            bool got = false;
            if (ok) {
                got = mbar_wait_warp(&sh.full_bar[s], (it / kDsSlots) & 1, p.status, 203, lane);
                if (!got) sh.abort_flag = 1;
            }
            const int rows = min(g.R, g.n - rg * g.R);
            const unsigned char *base = ring + (size_t)s * kDsSlotBytes;
            float tot = 0.0f;
            int my_row = 0;
            if (got) {
                switch (g.nr) {
                    case 8: tot = stage_dot<8>(base, row_bytes, rows, dual, xh, have, gtid, lane); my_row = row_of_lane<8>(lane); break;
                    case 4: tot = stage_dot<4>(base, row_bytes, rows, dual, xh, have, gtid, lane); my_row = row_of_lane<4>(lane); break;
                    case 2: tot = stage_dot<2>(base, row_bytes, rows, dual, xh, have, gtid, lane); my_row = row_of_lane<2>(lane); break;
                    default: tot = stage_dot<1>(base, row_bytes, rows, dual, xh, have, gtid, lane); my_row = 0; break;
                }
                if ((lane & ((32 / g.nr) - 1)) == 0) sh.red[s][my_row][gwarp] = tot;
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh.done_bar[s]);  // release: partials written, slot read
            }
        }
        grid_arrive();
        stamp(tphase, 3);
        ++tphase;

        if (g.kind == PH_QKV) {
            const int l = ph >> 2;
            // ------------------------------ attention ------------------------------
            stamp(tphase, 0);
            const DsLayer &L = layer_s[l];
            const int HD = p.hd;
            const int chunks = HD >> 3;
            const int len_total = pos + 1;
            const int n_tasks = p.nkv * p.n_splits;
            const float inv_den = sqrtf((float)HD);
            int tpd = kDsConsumers / (kDsTile * G);  // threads per (row, head) dot product
            tpd = tpd < 1 ? 1 : (tpd > 4 ? 4 : tpd);
            const int n_out = G * HD;
            auto load_rows = [&](int kvh, int t0, int r_begin, int r_end) {
                for (int c = tid + r_begin * chunks; c < r_end * chunks; c += kDsConsumers) {
                    const int r = c / chunks, ch = c % chunks;
                    const size_t goff = (size_t)(t0 + r) * n_kv + (size_t)kvh * HD + ch * 8;
                    cp_async16_ds(&k_tile[r * HD + ((ch ^ (r & 7)) * 8)], L.k_cache + goff);
                    cp_async16_ds(&v_tile[r * HD + ch * 8], L.v_cache + goff);
                }
            };
            // Cache rows below `pos` were written by earlier steps: the first tile of this CTA's first
            // task is requested before waiting for the other CTAs' q/k/v rows of this step.
            int pre_rows = 0;
            if ((int)blockIdx.x < n_tasks) {
                const int kvh = blockIdx.x / p.n_splits, begin = (blockIdx.x % p.n_splits) * p.split_len;
                pre_rows = max(0, min(kDsTile, min(begin + p.split_len, pos) - begin));
                load_rows(kvh, begin, 0, pre_rows);
            }
            grid_wait();
            stamp(tphase, 1);
            for (int task = blockIdx.x; task < n_tasks && ok; task += gridDim.x) {
                const int kvh = task / p.n_splits, split = task % p.n_splits;
                const int begin = split * p.split_len;
                const int end = min(begin + p.split_len, len_total);
                if (task != (int)blockIdx.x) named_bar_sync(1, kDsConsumers);  // previous task is done with shared memory
                for (int i = tid; i < n_out; i += kDsConsumers) sh.q_s[i] = __half2float(__ldcg(&p.q[(size_t)kvh * n_out + i]));
                if (tid < G) { sh.m_s[tid] = -INFINITY; sh.l_s[tid] = 0.0f; }
                float acc[2] = {0.0f, 0.0f};
                for (int t0 = begin; t0 < end; t0 += kDsTile) {
                    const int rows = min(kDsTile, end - t0);
                    const bool first = task == (int)blockIdx.x && t0 == begin;
                    if (!first) named_bar_sync(1, kDsConsumers);  // previous tile consumed
                    load_rows(kvh, t0, first ? pre_rows : 0, rows);
                    cp_async_wait_all_ds();
                    named_bar_sync(1, kDsConsumers);
                    // scores: dot = head * tile + row, split over tpd adjacent lanes
                    {
                        const int dot = tid / tpd, part = tid % tpd;
                        const int hh = dot / kDsTile, r = dot % kDsTile;
                        float sacc = 0.0f;
                        if (hh < G && r < rows) {
                            const int cpp = chunks / tpd;
                            for (int cc = 0; cc < cpp; ++cc) {
                                const int ch = part * cpp + cc;
                                const uint4 kv = *reinterpret_cast<const uint4 *>(&k_tile[r * HD + ((ch ^ (r & 7)) * 8)]);
                                const __half2 *kh = reinterpret_cast<const __half2 *>(&kv);
                                const float *qp = &sh.q_s[hh * HD + ch * 8];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 f = __half22float2(kh[e]);
                                    sacc = fmaf(qp[2 * e], f.x, sacc);
                                    sacc = fmaf(qp[2 * e + 1], f.y, sacc);
                                }
                            }
                        }
                        for (int m = tpd >> 1; m >= 1; m >>= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, m);
                        if (hh < G && part == 0) sh.p_s[hh * kDsTile + r] = (r < rows) ? __fdiv_rn(sacc, inv_den) : -INFINITY;
                    }
                    named_bar_sync(1, kDsConsumers);
                    if (warp < G) {  // online softmax bookkeeping of head `warp` (one tile row per lane)
                        static_assert(kDsTile == 32, "one score per lane");
                        const float s0 = sh.p_s[warp * kDsTile + lane];
                        const float tmax = warp_max(s0);
                        const float m_old = sh.m_s[warp];
                        const float m_new = fmaxf(m_old, tmax);
                        const float sc = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
                        const float e0 = (lane < rows) ? expf(s0 - m_new) : 0.0f;
                        sh.p_s[warp * kDsTile + lane] = e0;
                        const float ssum = warp_sum(e0);
                        __syncwarp();
                        if (lane == 0) {
                            sh.scale_s[warp] = sc;
                            sh.m_s[warp] = m_new;
                            sh.l_s[warp] = sh.l_s[warp] * sc + ssum;
                        }
                    }
                    named_bar_sync(1, kDsConsumers);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int o = tid + kDsConsumers * i;
                        if (o < n_out) {
                            const int hh = o / HD, dd = o % HD;
                            float a = acc[i] * sh.scale_s[hh];
                            const float *pp = &sh.p_s[hh * kDsTile];
                            for (int r = 0; r < rows; ++r) a = fmaf(pp[r], __half2float(v_tile[r * HD + dd]), a);
                            acc[i] = a;
                        }
                    }
                }
                named_bar_sync(1, kDsConsumers);
                const size_t pbase = ((size_t)kvh * p.n_splits + split) * G;
                if (tid < G) {
                    p.part_ml[(pbase + tid) * 2] = sh.m_s[tid];
                    p.part_ml[(pbase + tid) * 2 + 1] = sh.l_s[tid];
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int o = tid + kDsConsumers * i;
                    if (o < n_out) p.part_o[(pbase + o / HD) * HD + (o % HD)] = acc[i];
                }
                named_bar_sync(1, kDsConsumers);
                if (tid == 0) {
                    __threadfence();  // cumulative: orders the whole CTA's partials before the count
                    const int prev = atomicAdd(&p.attn_counters[kvh], 1);
                    sh.is_last = (prev == p.n_splits - 1);
                    if (sh.is_last) p.attn_counters[kvh] = 0;
                }
                named_bar_sync(1, kDsConsumers);
                if (sh.is_last) {
                    __threadfence();
                    // Merge in split order.  All loads of a step are independent, so each step costs
                    // about one L2 round trip: (1) every (split, head) max and sum, (2) the weights,
                    // (3) the partial outputs in batches of eight splits.
                    const int n_used = min(p.n_splits, (len_total + p.split_len - 1) / p.split_len);
                    const size_t gbase = (size_t)kvh * p.n_splits * G;
                    float *m_all = sh.norm_buf[0];  // idle during attention: [split][head]
                    float *l_all = sh.norm_buf[1];
                    for (int e = tid; e < n_used * G; e += kDsConsumers) {
                        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(&p.part_ml[(gbase + e) * 2]));
                        m_all[e] = ml.x;
                        l_all[e] = ml.y;
                    }
                    named_bar_sync(1, kDsConsumers);
                    float wgt_keep = 0.0f;
                    int e_keep = -1;
                    if (tid < n_used * G && tid < 512) {
                        const int hh = tid % G;
                        float M = -INFINITY;
                        for (int sidx = 0; sidx < n_used; ++sidx) M = fmaxf(M, m_all[sidx * G + hh]);
                        const float m = m_all[tid];
                        wgt_keep = (m == -INFINITY) ? 0.0f : expf(m - M);
                        e_keep = tid;
                    }
                    named_bar_sync(1, kDsConsumers);
                    if (e_keep >= 0) m_all[e_keep] = wgt_keep;  // m_all now holds the weights
                    named_bar_sync(1, kDsConsumers);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int o = tid + kDsConsumers * i;
                        if (o < n_out) {
                            const int hh = o / HD, dd = o % HD;
                            float num = 0.0f, den = 0.0f;
                            for (int s0 = 0; s0 < n_used; s0 += 8) {
                                float v[8];
#pragma unroll
                                for (int u = 0; u < 8; ++u)
                                    v[u] = (s0 + u < n_used) ? __ldcg(&p.part_o[(gbase + (size_t)(s0 + u) * G + hh) * HD + dd]) : 0.0f;
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    if (s0 + u < n_used) {
                                        const float wgt = m_all[(s0 + u) * G + hh];
                                        num = fmaf(wgt, v[u], num);
                                        den = fmaf(wgt, l_all[(s0 + u) * G + hh], den);
                                    }
                                }
                            }
                            p.attn[(size_t)kvh * n_out + o] = __float2half_rn(__fdiv_rn(num, den));
                        }
                    }
                }
            }
            stamp(tphase, 2);
            grid_arrive();
            stamp(tphase, 3);
            ++tphase;
        }
    }

    // Tensor parallel step without logits (prompt rows): nobody consumes the last all-reduce, so a fast
    // rank could start the next step and overwrite receive buffer 0 while a slow rank still reads it.
    // Waiting here for every rank's last partial sums keeps the ranks within one all-reduce of each
    // other, which is what the double buffering relies on.
    if (kTp && !p.with_logits) {
        const int last = 2 * p.n_layers - 1;
        const unsigned char *recv = p.peer[p.tp_rank] + kTpRecvOff + (size_t)(last & 1) * p.tp_size * p.d * 8;
        const unsigned int tag = tag_base + (unsigned int)last + 1u;
        for (int i = tid; i < p.tp_size * p.d / 2 && ok; i += kDsConsumers) {  // two (value, tag) pairs per load
            uint32_t spins = 0;
            for (;;) {
                uint4 q;
                asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
                             : "l"(recv + (size_t)i * 16)
                             : "memory");
                if (q.y == tag && q.w == tag) break;
                if ((++spins & 63u) == 0) {
                    if (*reinterpret_cast<volatile int *>(&sh.abort_flag)) break;
                    if (spins > p.tag_poll_limit) {
                        atomicExch(p.status, 207);
                        sh.abort_flag = 1;
                        break;
                    }
                }
            }
            if (*reinterpret_cast<volatile int *>(&sh.abort_flag)) break;
        }
    }

    // ---- step epilogue ----
    wait_after(n_gemv - 1);  // every CTA has finished its last phase (and published its best logit)
    if (blockIdx.x == 0 && warp == 0) {
        int token = -1;
        if (p.with_logits) {
            float v = -INFINITY;
            int idx = 0x7fffffff;
            for (int c = lane; c < (int)gridDim.x; c += 32) {
                const float ov = __ldcg(&p.amax_val[c]);
                const int oi = __ldcg(&p.amax_idx[c]);
                if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
            }
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, m);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, m);
                if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
            }
            if (kTp) {
                // each rank's best logit goes to every rank; then one more announcement round
                if (lane == 0) {
                    for (int r = 0; r < p.tp_size; ++r) {
                        volatile float *bv = reinterpret_cast<volatile float *>(p.peer[r] + kTpBestOff + 8 * p.tp_rank);
                        bv[0] = v;
                        reinterpret_cast<volatile int *>(bv)[1] = idx;
                    }
                    __threadfence_system();
                    const unsigned long long seq = tp_base + (++n_tp);
                    for (int r = 0; r < p.tp_size; ++r)
                        if (r != p.tp_rank)
                            *reinterpret_cast<volatile unsigned long long *>(p.peer[r] + kTpFlagsOff + 8 * p.tp_rank) = seq;
                    bool fine = ok;  // after a wait that gave up, the peers are not waited for either
                    for (int r = 0; r < p.tp_size && fine; ++r) {
                        if (r == p.tp_rank) continue;
                        const unsigned long long *f = reinterpret_cast<const unsigned long long *>(p.peer[p.tp_rank] + kTpFlagsOff + 8 * r);
                        unsigned long long fv;
                        uint32_t polls = 0;
                        do {
                            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(fv) : "l"(f) : "memory");
                            if (++polls > p.tag_poll_limit) { fine = false; break; }
                        } while (fv < seq);
                    }
                    if (!fine && ok) atomicExch(p.status, 206);
                    v = -INFINITY;
                    idx = 0x7fffffff;
                    for (int r = 0; r < p.tp_size; ++r) {
                        const volatile float *bv = reinterpret_cast<const volatile float *>(p.peer[p.tp_rank] + kTpBestOff + 8 * r);
                        const float ov = bv[0];
                        const int oi = reinterpret_cast<const volatile int *>(bv)[1];
                        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
                    }
                }
                idx = __shfl_sync(0xffffffffu, idx, 0);
            }
            token = idx == 0x7fffffff ? 0 : idx;
        }
        if (lane == 0) {
            const int np = pos + 1;
            if (p.with_logits) {
                p.next_token[0] = token;
                if (np < p.history_len) const_cast<int *>(p.history)[np] = token;
            }
            *p.pos = np;
            p.bar[1] = bar_base + n_bar * (unsigned long long)gridDim.x;
            if (kTp) {
                tp_state[0] = tp_base + n_tp;
                tp_state[1] = (unsigned long long)(tag_base + 2u * (unsigned int)p.n_layers);
            }
        }
    }
}

}  // namespace llmb

using namespace llmb;

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t llmb_decode_step_exchange_bytes(int tp_size, int d_model) {
    if (tp_size < 1 || d_model <= 0) return 0;
    return tp_exchange_bytes(tp_size, d_model);  // both parts: the whole-step kernel's and the row-batched path's
}

extern "C" size_t llmb_decode_step_scratch_bytes(int n_q_heads, int n_kv_heads, int head_dim, int max_splits) {
    if (n_q_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || max_splits <= 0) return 0;
    return 256 + align256((size_t)n_kv_heads * 4) + align256((size_t)n_q_heads * max_splits * 2 * 4) +
           align256((size_t)n_q_heads * max_splits * head_dim * 4) + align256(1024 * 4) + align256(1024 * 4);
}

extern "C" int llmb_decode_step(const LlmbDecodeStepArgs *a, llmb_stream_t stream_) {
    if (!a || !a->layers || !a->embed || !a->history || !a->pos || !a->x || !a->q || !a->attn || !a->h || !a->scratch)
        return LLMB_ERR_INVALID;
    if (a->with_logits && (!a->lm_head || !a->g_final || !a->logits || !a->next_token)) return LLMB_ERR_INVALID;
    if (a->n_layers <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads || a->n_splits <= 0 ||
        a->split_len <= 0 || (a->split_len % kDsTile) != 0 || a->n_splits > a->max_splits)
        return LLMB_ERR_INVALID;
    const int G = a->n_q_heads / a->n_kv_heads;
    if (a->n_splits * G > 512) return LLMB_ERR_INVALID;  // the merge keeps one weight per (split, head) in shared memory
    if ((a->head_dim != 64 && a->head_dim != 128) || G > 8 || G * a->head_dim > 2 * kDsConsumers) return LLMB_ERR_UNSUPPORTED;
    if (a->d_model % 8 || a->ffn % 8 || a->d_model > 8192 || a->ffn > 16384 || a->n_q_heads * a->head_dim > 16384)
        return LLMB_ERR_UNSUPPORTED;
    if ((uintptr_t)a->scratch & 255) return LLMB_ERR_INVALID;
    int dev = 0, sms = 0, coop = 0;
    LLMB_CUDA_OK(cudaGetDevice(&dev));
    LLMB_CUDA_OK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return LLMB_ERR_UNSUPPORTED;
    sms = sm_count_cached();
    if (sms > 1024) sms = 1024;

    DsParams p = {};
    p.layers = reinterpret_cast<const DsLayer *>(a->layers);
    p.embed = reinterpret_cast<const __half *>(a->embed);
    p.lm_head = reinterpret_cast<const __half *>(a->lm_head);
    p.g_final = reinterpret_cast<const __half *>(a->g_final);
    p.history = a->history;
    p.pos = a->pos;
    p.x = reinterpret_cast<__half *>(a->x);
    p.q = reinterpret_cast<__half *>(a->q);
    p.attn = reinterpret_cast<__half *>(a->attn);
    p.h = reinterpret_cast<__half *>(a->h);
    p.logits = reinterpret_cast<__half *>(a->logits);
    p.hidden = reinterpret_cast<__half *>(a->hidden);
    p.next_token = a->next_token;
    unsigned char *sc = static_cast<unsigned char *>(a->scratch);
    p.bar = reinterpret_cast<unsigned long long *>(sc);
    sc += 256;
    p.attn_counters = reinterpret_cast<int *>(sc);
    sc += align256((size_t)a->n_kv_heads * 4);
    p.part_ml = reinterpret_cast<float *>(sc);
    sc += align256((size_t)a->n_q_heads * a->max_splits * 2 * 4);
    p.part_o = reinterpret_cast<float *>(sc);
    sc += align256((size_t)a->n_q_heads * a->max_splits * a->head_dim * 4);
    p.amax_val = reinterpret_cast<float *>(sc);
    sc += align256(1024 * 4);
    p.amax_idx = reinterpret_cast<int *>(sc);
    p.status = device_status_ptr();
    if (!p.status) return LLMB_ERR_CUDA;
    p.trace = reinterpret_cast<unsigned long long *>(a->trace);
    p.eps = a->eps;
    p.rope_theta = a->rope_theta;
    p.n_layers = a->n_layers;
    p.d = a->d_model;
    p.nq = a->n_q_heads;
    p.nkv = a->n_kv_heads;
    p.hd = a->head_dim;
    p.ffn = a->ffn;
    p.vocab = a->vocab;
    p.embed_rows = a->embed_rows;
    p.max_pos = a->max_pos;
    p.n_splits = a->n_splits;
    p.split_len = a->split_len;
    p.with_logits = a->with_logits;
    p.history_len = a->history_len;
    p.tag_poll_limit = a->tag_poll_limit ? a->tag_poll_limit : kTagPollLimit;
    p.tp_rank = 0;
    p.tp_size = 1;
    p.vocab_offset = 0;
    p.x_alt = nullptr;
    if (a->tp_size > 1) {
        if (a->tp_size > 8 || a->tp_rank < 0 || a->tp_rank >= a->tp_size || !a->x_alt) return LLMB_ERR_INVALID;
        for (int r = 0; r < a->tp_size; ++r) {
            if (!a->peers[r]) return LLMB_ERR_INVALID;
            p.peer[r] = static_cast<unsigned char *>(a->peers[r]);
        }
        p.tp_rank = a->tp_rank;
        p.tp_size = a->tp_size;
        p.vocab_offset = a->vocab_offset;
        p.x_alt = reinterpret_cast<__half *>(a->x_alt);
    }

    const size_t smem = (size_t)kDsSlots * kDsSlotBytes + (size_t)2 * kDsTile * 128 * sizeof(__half) +
                        (size_t)a->n_layers * sizeof(DsLayer);
    static size_t smem_limit[kMaxDevices] = {}, set_plain[kMaxDevices] = {}, set_tp[kMaxDevices] = {};  // per device
    const int slot = current_device_slot();
    if (slot < 0) return LLMB_ERR_UNSUPPORTED;
    if (!smem_limit[slot]) {
        cudaFuncAttributes fa;
        int optin = 0;
        LLMB_CUDA_OK(cudaFuncGetAttributes(&fa, decode_step_kernel<true>));
        LLMB_CUDA_OK(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        smem_limit[slot] = (size_t)optin > fa.sharedSizeBytes ? (size_t)optin - fa.sharedSizeBytes : 1;
    }
    if (smem > smem_limit[slot]) return LLMB_ERR_UNSUPPORTED;  // too many layers for the shared-memory table
    LLMB_CUDA_OK(ensure_dynamic_smem(decode_step_kernel<false>, set_plain, smem));
    LLMB_CUDA_OK(ensure_dynamic_smem(decode_step_kernel<true>, set_tp, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(kDsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream_);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (p.tp_size > 1) LLMB_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_step_kernel<true>, p));
    else LLMB_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_step_kernel<false>, p));
    return LLMB_OK;
}
