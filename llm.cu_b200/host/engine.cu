// The per-token forward loop: the reference's src/inference/inference.cu re-built on the fused
// sm_100a kernels, behind the same entry points (init_cache, inference) plus tokens_to_cuda
// (src/tokenizer/tokenizer.cu:157-198).
//
// One decode step = 1 + 5 * n_layers + 2 kernels, captured once per KV-length bucket into a
// CUDA graph with programmatic-dependent-launch edges and replayed:
//
//   embed_rope                         x = Embed[token]; RoPE angles of this position
//   per layer:
//     gemv RMSNORM -> ROPE_KV          input_layernorm + q/k/v projections + RoPE + cache append
//     attn_decode                      softmax(q K^T / sqrt(hd)) V over cache rows 0..pos
//     gemv -> RESIDUAL                 o_proj + residual add
//     gemv RMSNORM -> SWIGLU           post_attention_layernorm + gate/up + SiLU(gate)*up
//     gemv -> RESIDUAL                 down_proj + residual add
//   gemv RMSNORM -> STORE              final norm + lm_head -> FP16 logits
//   argmax                             greedy token, position += 1, token appended to the history
//
// The token id and the position live in device memory, so the same graph serves every step and a
// run of steps needs no host round trip (inference_greedy).  The reference issues 483 launches,
// 96 16-MiB copies and 419 device synchronisations per token (inference.cu:149-193).
//
// KV cache: K and V are [n_layers][max_seq][n_kv_heads * head_dim] FP16, K stored after RoPE:
// the reference's row layout (inference.cu:761-768, :926) with a layer axis added.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "../csrc/common.cuh"
#include "../../include/llama3.h"
#include "host_internal.h"

using namespace llmb;

namespace {

__global__ void set_int_kernel(int *dst, int value) {
    pdl_launch_dependents();
    pdl_wait();
    *dst = value;
}

struct Engine {
    Llama3 *model = nullptr;
    cudaStream_t stream = nullptr;
    int d = 0, nq = 0, nkv = 0, hd = 0, ffn = 0, vocab = 0, embed_rows = 0, layers = 0, max_seq = 0;
    __half *x = nullptr, *q = nullptr, *attn = nullptr, *h = nullptr, *logits = nullptr;
    __half *kcache = nullptr, *vcache = nullptr;
    float *rope_cs = nullptr;
    int *d_pos = nullptr, *d_next = nullptr, *d_history = nullptr;
    void *attn_scratch = nullptr;
    void *sample_scratch = nullptr;  // device sampler: result code + [vocab] probabilities
    int max_splits = 0;
    // whole-step persistent kernel
    LlmbLayer *d_layers = nullptr;
    void *step_scratch = nullptr;
    size_t step_scratch_bytes = 0;
    int step_max_splits = 0;
    int sm_count = 148;
    bool use_step_kernel = true;
    // tensor parallel
    int tp_rank = 0, tp_size = 1;
    __half *x_alt = nullptr;
    void *exchange = nullptr;           // this rank's exchange block (peers write into it)
    size_t exchange_bytes = 0;
    void *peers[8] = {};                // every rank's block as mapped on this device
    bool tp_connected = false;
    unsigned long long *trace = nullptr;  // optional per-phase timestamps of the step kernel
    unsigned int tag_poll_limit = 0;  // spin limit of the step kernel's waits for tensor-parallel peers (0 = default)
    size_t trace_bytes = 0;
    int *h_next = nullptr;  // pinned: [0] next token, [1] device status word
    __half *hidden = nullptr;
    bool use_graph = true, use_pdl = true, copy_logits = true, hidden_dump = false;
    bool greedy_state = false;  // device history[consumed.size()] holds a sampled token not yet fed
    std::vector<int> consumed;  // ids whose K/V rows are in the cache
    std::map<int, cudaGraphExec_t> graphs;  // key: bucket * 2 + with_logits
    long long launches = 0;
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    // prompt phase: blocks of rows through the tensor-core projections
    bool batched_prefill = true;
    int prefill_min_rows = 16, prefill_chunk = 1024, pf_rows = 0;
    __half *pf_x = nullptr, *pf_xn = nullptr, *pf_q = nullptr, *pf_attn = nullptr, *pf_h = nullptr;
    float *pf_rope = nullptr;
    int *pf_pos = nullptr;
    void *pf_ws = nullptr;  // split-K workspace of the projections
    size_t pf_ws_bytes = 0;
    // batched decode: n_seqs independent sequences advance one token per step
    int bt_seqs = 0;
    __half *bt_kcache = nullptr, *bt_vcache = nullptr;  // [layers][n_seqs][max_seq][n_kv]
    __half *bt_logits = nullptr;                        // [n_seqs][vocab]
    int *bt_pos = nullptr, *bt_tok = nullptr, *bt_history = nullptr;  // [n_seqs], [n_seqs], [n_seqs][max_seq + 1]
    void *bt_attn_scratch = nullptr;
    int bt_max_splits = 0;
    int bt_split_len = 256;                             // cache rows per attention CTA (a power of two, 32..512)
    std::vector<int> bt_len;                            // rows in the cache per sequence (host view)
    std::map<int, cudaGraphExec_t> bt_graphs;           // key: attention bucket
    // profiling aid: per-CTA stamps of every small-M projection of a step (cache_debug_rows_trace)
    unsigned long long *rows_trace = nullptr;
    int rows_trace_call = 0;
};

inline Engine *eng(const CudaCache *c) { return c ? static_cast<Engine *>(c->priv) : nullptr; }

struct SplitPlan {
    int bucket, n_splits, split_len;
};

// Attention split geometry for a sequence of `len` cached rows.  The grid is baked into a
// captured graph, so lengths are bucketed to powers of two (>= 512).
SplitPlan plan_splits(int len) {
    int bucket = 512;
    while (bucket < len) bucket <<= 1;
    int split_len = bucket / 16;
    if (split_len > 128) split_len = 128;
    return {bucket, bucket / split_len, split_len};
}

int enqueue_step(Engine *e, bool with_logits, const SplitPlan &sp) {
    Llama3 *m = e->model;
    const Llama3Config &c = m->config;
    cudaStream_t s = e->stream;
    const int pdl = e->use_pdl ? 1 : 0;
    int rc = llmb_embed_rope(reinterpret_cast<const uint16_t *>(m->embed_tokens->d_fp16_tensor), e->d_history, e->d_pos,
                             1, e->d, e->embed_rows, e->hd, c.rope_theta, reinterpret_cast<uint16_t *>(e->x),
                             e->rope_cs, 1 /* token = history[pos] */, pdl, s);
    if (rc) return rc;
    if (e->hidden_dump)
        LLMB_CUDA_OK(cudaMemcpyAsync(e->hidden, e->x, (size_t)e->d * 2, cudaMemcpyDeviceToDevice, s));
    const int n_q = e->nq * e->hd, n_kv = e->nkv * e->hd;
    for (int l = 0; l < e->layers; ++l) {
        const Llama3Layer *L = m->layers[l];
        __half *kl = e->kcache + (size_t)l * e->max_seq * n_kv;
        __half *vl = e->vcache + (size_t)l * e->max_seq * n_kv;
        LlmbGemvArgs a = {};
        a.use_pdl = pdl;
        // input_layernorm + QKV + RoPE + cache append
        a.w = reinterpret_cast<const uint16_t *>(L->self_attn_q_proj->d_fp16_tensor);
        a.x = reinterpret_cast<const uint16_t *>(e->x);
        a.y = reinterpret_cast<uint16_t *>(e->q);
        a.n = n_q + 2 * n_kv;
        a.k = e->d;
        a.prologue = LLMB_PRO_RMSNORM;
        a.gamma = reinterpret_cast<const uint16_t *>(L->input_layernorm->d_fp16_tensor);
        a.eps = c.eps;
        a.epilogue = LLMB_EPI_ROPE_KV;
        a.n_q = n_q;
        a.n_kv = n_kv;
        a.head_dim = e->hd;
        a.rope_cs = e->rope_cs;
        a.k_cache = reinterpret_cast<uint16_t *>(kl);
        a.v_cache = reinterpret_cast<uint16_t *>(vl);
        a.pos = e->d_pos;
        a.max_pos = e->max_seq;
        if ((rc = llmb_gemv_f16(&a, s))) return rc;
        if ((rc = llmb_attn_decode(reinterpret_cast<const uint16_t *>(e->q), reinterpret_cast<const uint16_t *>(kl),
                                   reinterpret_cast<const uint16_t *>(vl), e->d_pos, e->nq, e->nkv, e->hd, sp.n_splits,
                                   sp.split_len, reinterpret_cast<uint16_t *>(e->attn), e->attn_scratch, pdl, s)))
            return rc;
        // o_proj + residual
        LlmbGemvArgs o = {};
        o.use_pdl = pdl;
        o.w = reinterpret_cast<const uint16_t *>(L->self_attn_o_proj->d_fp16_tensor);
        o.x = reinterpret_cast<const uint16_t *>(e->attn);
        o.y = reinterpret_cast<uint16_t *>(e->x);
        o.n = e->d;
        o.k = n_q;
        o.epilogue = LLMB_EPI_RESIDUAL;
        if ((rc = llmb_gemv_f16(&o, s))) return rc;
        // post_attention_layernorm + gate/up + SwiGLU
        LlmbGemvArgs f = {};
        f.use_pdl = pdl;
        f.w = reinterpret_cast<const uint16_t *>(L->mlp_gate_proj->d_fp16_tensor);
        f.w2 = reinterpret_cast<const uint16_t *>(L->mlp_up_proj->d_fp16_tensor);
        f.x = reinterpret_cast<const uint16_t *>(e->x);
        f.y = reinterpret_cast<uint16_t *>(e->h);
        f.n = e->ffn;
        f.k = e->d;
        f.prologue = LLMB_PRO_RMSNORM;
        f.gamma = reinterpret_cast<const uint16_t *>(L->post_attention_layernorm->d_fp16_tensor);
        f.eps = c.eps;
        f.epilogue = LLMB_EPI_SWIGLU;
        if ((rc = llmb_gemv_f16(&f, s))) return rc;
        // down_proj + residual
        LlmbGemvArgs dn = {};
        dn.use_pdl = pdl;
        dn.w = reinterpret_cast<const uint16_t *>(L->mlp_down_proj->d_fp16_tensor);
        dn.x = reinterpret_cast<const uint16_t *>(e->h);
        dn.y = reinterpret_cast<uint16_t *>(e->x);
        dn.n = e->d;
        dn.k = e->ffn;
        dn.epilogue = LLMB_EPI_RESIDUAL;
        if ((rc = llmb_gemv_f16(&dn, s))) return rc;
        if (e->hidden_dump)
            LLMB_CUDA_OK(cudaMemcpyAsync(e->hidden + (size_t)(l + 1) * e->d, e->x, (size_t)e->d * 2,
                                         cudaMemcpyDeviceToDevice, s));
    }
    if (with_logits) {
        LlmbGemvArgs lm = {};
        lm.use_pdl = pdl;
        lm.w = reinterpret_cast<const uint16_t *>(m->lm_head->d_fp16_tensor);
        lm.x = reinterpret_cast<const uint16_t *>(e->x);
        lm.y = reinterpret_cast<uint16_t *>(e->logits);
        lm.n = e->vocab;
        lm.k = e->d;
        lm.prologue = LLMB_PRO_RMSNORM;
        lm.gamma = reinterpret_cast<const uint16_t *>(m->norm->d_fp16_tensor);
        lm.eps = c.eps;
        lm.epilogue = LLMB_EPI_STORE;
        if ((rc = llmb_gemv_f16(&lm, s))) return rc;
        if ((rc = llmb_argmax_f16(reinterpret_cast<const uint16_t *>(e->logits), e->vocab, e->d_next, e->d_pos,
                                  e->d_history, e->max_seq + 1, pdl, s)))
            return rc;
    } else {
        if ((rc = llmb_advance_pos(e->d_pos, pdl, s))) return rc;
    }
    return LLMB_OK;
}

int kernels_per_step(const Engine *e, bool with_logits) {
    if (e->use_step_kernel) return 1;
    return 1 + 5 * e->layers + (with_logits ? 2 : 1);
}

// The whole step as one persistent kernel.  Attention splits: 32-row tiles, doubled until the
// task count fits about two waves of CTAs.
int launch_step_kernel(Engine *e, bool with_logits, int len) {
    const Llama3Config &c = e->model->config;
    int split_len = 32;
    const int G = e->nq / e->nkv;
    while (e->nkv * ((len + split_len - 1) / split_len) > 2 * e->sm_count || ((len + split_len - 1) / split_len) * G > 512)
        split_len *= 2;
    LlmbDecodeStepArgs a = {};
    a.layers = e->d_layers;
    a.n_layers = e->layers;
    a.d_model = e->d;
    a.n_q_heads = e->nq;
    a.n_kv_heads = e->nkv;
    a.head_dim = e->hd;
    a.ffn = e->ffn;
    a.vocab = e->vocab;
    a.embed_rows = e->embed_rows;
    a.max_pos = e->max_seq;
    a.rope_theta = c.rope_theta;
    a.eps = c.eps;
    a.embed = reinterpret_cast<const uint16_t *>(e->model->embed_tokens->d_fp16_tensor);
    a.lm_head = reinterpret_cast<const uint16_t *>(e->model->lm_head->d_fp16_tensor);
    a.g_final = reinterpret_cast<const uint16_t *>(e->model->norm->d_fp16_tensor);
    a.history = e->d_history;
    a.history_len = e->max_seq + 1;  // d_history has max_seq + 1 entries: the token sampled at the last row still fits
    a.pos = e->d_pos;
    a.x = reinterpret_cast<uint16_t *>(e->x);
    a.q = reinterpret_cast<uint16_t *>(e->q);
    a.attn = reinterpret_cast<uint16_t *>(e->attn);
    a.h = reinterpret_cast<uint16_t *>(e->h);
    a.logits = reinterpret_cast<uint16_t *>(e->logits);
    a.next_token = e->d_next;
    a.scratch = e->step_scratch;
    a.max_splits = e->step_max_splits;
    a.split_len = split_len;
    a.n_splits = (len + split_len - 1) / split_len;
    a.with_logits = with_logits ? 1 : 0;
    a.hidden = e->hidden_dump ? reinterpret_cast<uint16_t *>(e->hidden) : nullptr;
    a.trace = reinterpret_cast<uint64_t *>(e->trace);
    a.tag_poll_limit = e->tag_poll_limit;
    if (e->tp_size > 1) {
        if (!e->tp_connected) {
            set_last_error("tensor parallel cache: call cache_tp_connect() on every rank first");
            return LLMB_ERR_INVALID;
        }
        a.tp_rank = e->tp_rank;
        a.tp_size = e->tp_size;
        a.vocab_offset = e->tp_rank * e->vocab;
        a.x_alt = reinterpret_cast<uint16_t *>(e->x_alt);
        for (int r = 0; r < e->tp_size; ++r) a.peers[r] = e->peers[r];
    }
    return llmb_decode_step(&a, e->stream);
}

// Runs one step for the token at history[pos]; `len` = pos + 1 is known on the host.
int run_step(Engine *e, bool with_logits, int len) {
    const SplitPlan sp = plan_splits(len);
    e->launches += kernels_per_step(e, with_logits);
    if (e->use_step_kernel) return launch_step_kernel(e, with_logits, len);
    if (!e->use_graph || e->hidden_dump) return enqueue_step(e, with_logits, sp);
    const int key = sp.bucket * 2 + (with_logits ? 1 : 0);
    auto it = e->graphs.find(key);
    if (it == e->graphs.end()) {
        cudaGraph_t graph = nullptr;
        LLMB_CUDA_OK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        int rc = enqueue_step(e, with_logits, sp);
        cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
        if (rc) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        LLMB_CUDA_OK(ce);
        cudaGraphExec_t exec = nullptr;
        ce = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        LLMB_CUDA_OK(ce);
        it = e->graphs.emplace(key, exec).first;
    }
    LLMB_CUDA_OK(cudaGraphLaunch(it->second, e->stream));
    return LLMB_OK;
}

int set_device_int(Engine *e, int *dst, int value) {
    LLMB_CUDA_OK(launch_pdl(set_int_kernel, dim3(1), dim3(1), 0, e->stream, false, dst, value));
    return LLMB_OK;
}

// The row paths need tile-aligned projection shapes (this rank's shares under tensor parallelism).
bool rows_shapes_ok(const Engine *e) {
    const int n_q = e->nq * e->hd, n_kv = e->nkv * e->hd;
    return !e->hidden_dump && (e->hd == 64 || e->hd == 128) && (n_q + 2 * n_kv) % 128 == 0 && e->d % 128 == 0 &&
           e->ffn % 128 == 0 && n_q % 64 == 0 && n_kv % 32 == 0 && e->vocab % 8 == 0;
}

// Blocks of up to 1024 rows: all of the model on this GPU.
bool prefill_supported(const Engine *e) { return e->tp_size == 1 && rows_shapes_ok(e); }

// Tensor parallel: blocks of up to 32 rows through the weight-streaming projections with the all-reduce
// fused as peer stores (gemm_smallm.cu LLMB_EPI_TP_SCATTER + tp_rows.cu).
bool tp_rows_supported(const Engine *e) { return e->tp_size > 1 && e->tp_connected && rows_shapes_ok(e); }

void free_prefill_buffers(Engine *e) {
    cudaFree(e->pf_x); cudaFree(e->pf_xn); cudaFree(e->pf_q); cudaFree(e->pf_attn); cudaFree(e->pf_h);
    cudaFree(e->pf_rope); cudaFree(e->pf_pos); cudaFree(e->pf_ws);
    e->pf_ws = nullptr;
    e->pf_ws_bytes = 0;
    e->pf_x = e->pf_xn = e->pf_q = e->pf_attn = e->pf_h = nullptr;
    e->pf_rope = nullptr;
    e->pf_pos = nullptr;
    e->pf_rows = 0;
}

int ensure_prefill_buffers(Engine *e, int rows) {
    if (rows <= e->pf_rows) return LLMB_OK;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    free_prefill_buffers(e);
    const size_t n_q = (size_t)e->nq * e->hd;
    LLMB_CUDA_OK(cudaMalloc(&e->pf_x, (size_t)rows * e->d * 2));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_xn, (size_t)rows * e->d * 2));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_q, (size_t)rows * n_q * 2));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_attn, (size_t)rows * n_q * 2));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_h, (size_t)rows * e->ffn * 2));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_rope, (size_t)rows * e->hd * sizeof(float)));
    LLMB_CUDA_OK(cudaMalloc(&e->pf_pos, (size_t)rows * sizeof(int)));
    e->pf_ws_bytes = 4096 + (size_t)e->sm_count * 131072;
    LLMB_CUDA_OK(cudaMalloc(&e->pf_ws, e->pf_ws_bytes));
    LLMB_CUDA_OK(cudaMemsetAsync(e->pf_ws, 0, 4096, e->stream));
    e->pf_rows = rows;
    return LLMB_OK;
}

// Appends the K/V rows of history positions [from, to) to the cache, a block of rows at a time:
// the reference's layer loop (inference.cu:157-186) with every projection a tensor-core GEMM over
// the block.  No logits: the caller runs the last prompt token through the decode step.
// `ids` = the sequence's token ids on the device (position 0 first); kbase/vbase = layer 0 of the sequence's
// cache; layer_stride = elements between consecutive layers of that cache.
int prefill_rows(Engine *e, int from, int to, const int *ids, __half *kbase, __half *vbase, size_t layer_stride) {
    Llama3 *m = e->model;
    const Llama3Config &c = m->config;
    cudaStream_t s = e->stream;
    const int n_q = e->nq * e->hd, n_kv = e->nkv * e->hd;
    int rc = ensure_prefill_buffers(e, std::min(to - from, e->prefill_chunk));
    if (rc) return rc;
    auto u16 = [](const void *p) { return reinterpret_cast<const uint16_t *>(p); };
    auto u16w = [](void *p) { return reinterpret_cast<uint16_t *>(p); };
    for (int p0 = from; p0 < to; p0 += e->prefill_chunk) {
        const int rows = std::min(e->prefill_chunk, to - p0);
        if ((rc = llmb_iota_i32(e->pf_pos, p0, rows, s))) return rc;
        if ((rc = llmb_embed_rope(u16(m->embed_tokens->d_fp16_tensor), ids + p0, e->pf_pos, rows, e->d,
                                  e->embed_rows, e->hd, c.rope_theta, u16w(e->pf_x), e->pf_rope, 0, 0, s)))
            return rc;
        for (int l = 0; l < e->layers; ++l) {
            const Llama3Layer *L = m->layers[l];
            __half *kl = kbase + (size_t)l * layer_stride;
            __half *vl = vbase + (size_t)l * layer_stride;
            if ((rc = llmb_rmsnorm_rows(u16(e->pf_x), u16(L->input_layernorm->d_fp16_tensor), u16w(e->pf_xn), rows, e->d,
                                        c.eps, s)))
                return rc;
            LlmbGemmArgs g = {};
            g.a = u16(e->pf_xn);
            g.b = u16(L->self_attn_q_proj->d_fp16_tensor);  // q, k, v rows are one contiguous buffer
            g.c = u16w(e->pf_q);
            g.m = rows; g.n = n_q + 2 * n_kv; g.k = e->d;
            g.epilogue = LLMB_EPI_ROPE_KV;
            g.n_q = n_q; g.n_kv = n_kv; g.head_dim = e->hd;
            g.rope_cs = e->pf_rope;
            g.k_cache = u16w(kl); g.v_cache = u16w(vl);
            g.pos0 = p0; g.max_pos = e->max_seq;
            g.workspace = e->pf_ws; g.workspace_bytes = e->pf_ws_bytes;
            if ((rc = llmb_gemm_f16(&g, s))) return rc;
            if ((rc = llmb_attn_prefill(u16(e->pf_q), u16(kl), u16(vl), rows, p0, e->nq, e->nkv, e->hd, u16w(e->pf_attn), s)))
                return rc;
            LlmbGemmArgs o = {};
            o.a = u16(e->pf_attn);
            o.b = u16(L->self_attn_o_proj->d_fp16_tensor);
            o.c = u16w(e->pf_x);
            o.m = rows; o.n = e->d; o.k = n_q;
            o.epilogue = LLMB_EPI_RESIDUAL;
            o.workspace = e->pf_ws; o.workspace_bytes = e->pf_ws_bytes;
            if ((rc = llmb_gemm_f16(&o, s))) return rc;
            if ((rc = llmb_rmsnorm_rows(u16(e->pf_x), u16(L->post_attention_layernorm->d_fp16_tensor), u16w(e->pf_xn), rows,
                                        e->d, c.eps, s)))
                return rc;
            LlmbGemmArgs f = {};
            f.a = u16(e->pf_xn);
            f.b = u16(L->mlp_gate_proj->d_fp16_tensor);
            f.b2 = u16(L->mlp_up_proj->d_fp16_tensor);
            f.c = u16w(e->pf_h);
            f.m = rows; f.n = e->ffn; f.k = e->d;
            f.epilogue = LLMB_EPI_SWIGLU;
            f.workspace = e->pf_ws; f.workspace_bytes = e->pf_ws_bytes;
            if ((rc = llmb_gemm_f16(&f, s))) return rc;
            LlmbGemmArgs dn = {};
            dn.a = u16(e->pf_h);
            dn.b = u16(L->mlp_down_proj->d_fp16_tensor);
            dn.c = u16w(e->pf_x);
            dn.m = rows; dn.n = e->d; dn.k = e->ffn;
            dn.epilogue = LLMB_EPI_RESIDUAL;
            dn.workspace = e->pf_ws; dn.workspace_bytes = e->pf_ws_bytes;
            if ((rc = llmb_gemm_f16(&dn, s))) return rc;
        }
        e->launches += 2 + 7 * e->layers;
    }
    return LLMB_OK;
}

constexpr int kRowsTraceCtas = 1024;  // trace slots per projection (the grid of a small-M projection is smaller)

// One projection of the small-row paths; fills the fields every call shares.
LlmbGemmArgs small_gemm(Engine *e, const void *a, const void *b, void *c, int m, int n, int k, int epilogue) {
    LlmbGemmArgs g = {};
    g.a = reinterpret_cast<const uint16_t *>(a);
    g.b = reinterpret_cast<const uint16_t *>(b);
    g.c = reinterpret_cast<uint16_t *>(c);
    g.m = m; g.n = n; g.k = k;
    g.epilogue = epilogue;
    g.workspace = e->pf_ws; g.workspace_bytes = e->pf_ws_bytes;
    g.use_pdl = 1;
    if (e->rows_trace) g.trace = reinterpret_cast<uint64_t *>(e->rows_trace + (size_t)(e->rows_trace_call++) * kRowsTraceCtas * 8);
    if (epilogue == LLMB_EPI_TP_SCATTER) {
        g.tp_rank = e->tp_rank; g.tp_size = e->tp_size;
        for (int r = 0; r < e->tp_size; ++r) g.tp_peers[r] = e->peers[r];
    }
    return g;
}

// o_proj / down_proj of `m` rows and what follows it: single GPU = residual epilogue, then the RMSNorm of the
// new rows if `gamma`; tensor parallel = partial sums scattered to every rank, then the gather kernel (sum in
// rank order + residual + RMSNorm).  `xi` counts the exchanges of the step.
int row_parallel_projection(Engine *e, const void *a, const void *w, int m, int k, const void *gamma, int &xi) {
    const Llama3Config &c = e->model->config;
    auto u16 = [](const void *p) { return reinterpret_cast<const uint16_t *>(p); };
    int rc;
    if (e->tp_size > 1) {
        LlmbGemmArgs g = small_gemm(e, a, w, nullptr, m, e->d, k, LLMB_EPI_TP_SCATTER);
        g.tp_index = xi;
        if ((rc = llmb_gemm_f16(&g, e->stream))) return rc;
        rc = llmb_tp_gather_rows(e->exchange, e->tp_size, xi, reinterpret_cast<uint16_t *>(e->pf_x), u16(gamma),
                                 reinterpret_cast<uint16_t *>(e->pf_xn), m, e->d, c.eps, e->tag_poll_limit, 1, e->stream);
        ++xi;
        return rc;
    }
    LlmbGemmArgs g = small_gemm(e, a, w, e->pf_x, m, e->d, k, LLMB_EPI_RESIDUAL);
    if ((rc = llmb_gemm_f16(&g, e->stream))) return rc;
    if (gamma) rc = llmb_rmsnorm_rows(u16(e->pf_x), u16(gamma), reinterpret_cast<uint16_t *>(e->pf_xn), m, e->d, c.eps, e->stream);
    return rc;
}

// Tensor parallel prompt phase: history positions [from, to) in blocks of up to 32 rows.  Every block streams
// this rank's weight shards once (the same kernels as the batched decode step) and attends causally over the
// rank's KV heads; no logits.
int prefill_rows_tp(Engine *e, int from, int to, const int *ids, __half *kbase, __half *vbase, size_t layer_stride) {
    Llama3 *m = e->model;
    const Llama3Config &c = m->config;
    cudaStream_t s = e->stream;
    const int n_q = e->nq * e->hd, n_kv = e->nkv * e->hd;
    int rc = ensure_prefill_buffers(e, 32);
    if (rc) return rc;
    auto u16 = [](const void *p) { return reinterpret_cast<const uint16_t *>(p); };
    auto u16w = [](void *p) { return reinterpret_cast<uint16_t *>(p); };
    for (int p0 = from; p0 < to; p0 += 32) {
        const int rows = std::min(32, to - p0);
        if ((rc = llmb_iota_i32(e->pf_pos, p0, rows, s))) return rc;
        if ((rc = llmb_embed_rope(u16(m->embed_tokens->d_fp16_tensor), ids + p0, e->pf_pos, rows, e->d, e->embed_rows, e->hd,
                                  c.rope_theta, u16w(e->pf_x), e->pf_rope, 0, 0, s)))
            return rc;
        if ((rc = llmb_rmsnorm_rows(u16(e->pf_x), u16(m->layers[0]->input_layernorm->d_fp16_tensor), u16w(e->pf_xn), rows, e->d,
                                    c.eps, s)))
            return rc;
        int xi = 0;
        for (int l = 0; l < e->layers; ++l) {
            const Llama3Layer *L = m->layers[l];
            __half *kl = kbase + (size_t)l * layer_stride;
            __half *vl = vbase + (size_t)l * layer_stride;
            LlmbGemmArgs g = small_gemm(e, e->pf_xn, L->self_attn_q_proj->d_fp16_tensor, e->pf_q, rows, n_q + 2 * n_kv, e->d,
                                        LLMB_EPI_ROPE_KV);
            g.n_q = n_q; g.n_kv = n_kv; g.head_dim = e->hd;
            g.rope_cs = e->pf_rope;
            g.k_cache = u16w(kl); g.v_cache = u16w(vl);
            g.pos0 = p0; g.max_pos = e->max_seq;
            if ((rc = llmb_gemm_f16(&g, s))) return rc;
            if ((rc = llmb_attn_prefill(u16(e->pf_q), u16(kl), u16(vl), rows, p0, e->nq, e->nkv, e->hd, u16w(e->pf_attn), s)))
                return rc;
            if ((rc = row_parallel_projection(e, e->pf_attn, L->self_attn_o_proj->d_fp16_tensor, rows, n_q,
                                              L->post_attention_layernorm->d_fp16_tensor, xi)))
                return rc;
            LlmbGemmArgs f = small_gemm(e, e->pf_xn, L->mlp_gate_proj->d_fp16_tensor, e->pf_h, rows, e->ffn, e->d, LLMB_EPI_SWIGLU);
            f.b2 = u16(L->mlp_up_proj->d_fp16_tensor);
            if ((rc = llmb_gemm_f16(&f, s))) return rc;
            const void *next_gamma = l + 1 < e->layers ? m->layers[l + 1]->input_layernorm->d_fp16_tensor : nullptr;
            if ((rc = row_parallel_projection(e, e->pf_h, L->mlp_down_proj->d_fp16_tensor, rows, e->ffn, next_gamma, xi))) return rc;
        }
        if ((rc = llmb_tp_advance(e->exchange, e->tp_size, e->d, xi, 1, s))) return rc;
        e->launches += 4 + 7 * e->layers;
    }
    return LLMB_OK;
}

// Feeds ids[from..to) (history rows from..to-1), logits only for the last one.
int feed_tokens(Engine *e, const int *ids, int from, int to) {
    if (to <= from) return LLMB_ERR_INVALID;
    if (to > e->max_seq) {
        set_last_error("inference: sequence longer than the KV cache (config.max_seq)");
        return LLMB_ERR_INVALID;
    }
    // pageable source: the runtime stages it before returning, so `ids` may change afterwards
    LLMB_CUDA_OK(cudaMemcpyAsync(e->d_history + from, ids + from, sizeof(int) * (size_t)(to - from),
                                 cudaMemcpyHostToDevice, e->stream));
    int rc, first = from;
    // all but the last token as blocks of rows; the last one through the decode step, for its logits
    if (e->batched_prefill && to - 1 - from >= e->prefill_min_rows && prefill_supported(e)) {
        if ((rc = prefill_rows(e, from, to - 1, e->d_history, e->kcache, e->vcache, (size_t)e->max_seq * e->nkv * e->hd))) return rc;
        first = to - 1;
    } else if (e->batched_prefill && to - 1 - from >= e->prefill_min_rows && tp_rows_supported(e)) {
        if ((rc = prefill_rows_tp(e, from, to - 1, e->d_history, e->kcache, e->vcache, (size_t)e->max_seq * e->nkv * e->hd))) return rc;
        first = to - 1;
    }
    if ((rc = set_device_int(e, e->d_pos, first))) return rc;
    for (int p = first; p < to; ++p)
        if ((rc = run_step(e, p == to - 1, p + 1))) return rc;
    return LLMB_OK;
}

// Has any bounded device-side wait given up?  The status word is copied to pinned memory on the
// engine's stream before a synchronisation the caller makes anyway (queue_status_read), and looked
// at after it (status_result): no extra round trip.  The word stays set (the kernels then skip their
// waits) until the caller reads it with llmb_device_status().
int queue_status_read(Engine *e) {
    int *p = device_status_ptr();
    if (!p) return LLMB_ERR_CUDA;
    LLMB_CUDA_OK(cudaMemcpyAsync(e->h_next + 1, p, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    return LLMB_OK;
}

int status_result(Engine *e) {
    const int st = e->h_next[1];
    if (st != 0) {
        char msg[160];
        snprintf(msg, sizeof msg, "a bounded device-side wait gave up (status %d)%s", st,
                 st >= 205 && st <= 207 ? ": a tensor-parallel peer did not deliver its partial sums in time" : "");
        set_last_error(msg);
        return LLMB_ERR_TIMEOUT;
    }
    return LLMB_OK;
}

void destroy_engine(Engine *e) {
    if (!e) return;
    for (auto &kv : e->graphs) cudaGraphExecDestroy(kv.second);
    cudaFree(e->x); cudaFree(e->q); cudaFree(e->attn); cudaFree(e->h);
    cudaFree(e->rope_cs); cudaFree(e->d_pos); cudaFree(e->d_next); cudaFree(e->d_history);
    cudaFree(e->attn_scratch); cudaFree(e->hidden); cudaFree(e->d_layers); cudaFree(e->step_scratch);
    cudaFree(e->sample_scratch);
    for (int r = 0; r < e->tp_size; ++r)
        if (e->tp_connected && r != e->tp_rank && e->peers[r]) cudaIpcCloseMemHandle(e->peers[r]);
    cudaFree(e->exchange); cudaFree(e->x_alt); cudaFree(e->trace);
    free_prefill_buffers(e);
    for (auto &kv : e->bt_graphs) cudaGraphExecDestroy(kv.second);
    cudaFree(e->bt_kcache); cudaFree(e->bt_vcache); cudaFree(e->bt_logits); cudaFree(e->bt_pos); cudaFree(e->bt_tok);
    cudaFree(e->bt_history); cudaFree(e->bt_attn_scratch); cudaFree(e->rows_trace);
    if (e->h_next) cudaFreeHost(e->h_next);
    for (auto &ev : e->ev)
        if (ev) cudaEventDestroy(ev);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

Tensor *make_view_tensor(int rows, int cols, __half *data) {
    Tensor *t = static_cast<Tensor *>(calloc(1, sizeof(Tensor)));
    if (!t) return nullptr;
    t->ndim = static_cast<int *>(malloc(sizeof(int)));
    t->mem_len = static_cast<int *>(malloc(sizeof(int)));
    t->shape = static_cast<int *>(malloc(2 * sizeof(int)));
    if (!t->ndim || !t->mem_len || !t->shape) return t;
    *t->ndim = 2;
    t->shape[0] = rows;
    t->shape[1] = cols;
    long long n = (long long)rows * cols;
    *t->mem_len = n > 0x7fffffffLL ? 0x7fffffff : (int)n;
    t->d_fp16_tensor = data;
    t->loaded = 1;
    return t;
}

}  // namespace

extern "C" CudaCache *llama3_init_cache(Llama3 *m, int *status_out) {
    auto fail = [&](int code, const char *msg) -> CudaCache * {
        if (msg) set_last_error(msg);
        if (status_out) *status_out = code;
        return nullptr;
    };
    if (!m || !m->config_ready) return fail(LLMB_ERR_INVALID, "init_cache: call to_cuda first");
    const Llama3Config &c = m->config;
    if (!device_status_ptr()) return fail(LLMB_ERR_CUDA, "init_cache: could not allocate the device status word");
    Engine *e = new Engine();
    e->model = m;
    e->tp_rank = m->tp_rank;
    e->tp_size = m->tp_size;
    e->d = c.d_model;
    e->nq = c.n_q_heads / m->tp_size;    // this rank's shares (model.cu: shard_of)
    e->nkv = c.n_kv_heads / m->tp_size;
    e->hd = c.head_dim;
    e->ffn = c.ffn / m->tp_size;
    e->vocab = c.vocab / m->tp_size;
    e->embed_rows = m->embed_tokens->shape[0];
    e->layers = m->n_layers;
    e->max_seq = c.max_seq;
    const size_t n_q = (size_t)e->nq * e->hd, n_kv = (size_t)e->nkv * e->hd;
    const size_t kv_elems = (size_t)e->layers * e->max_seq * n_kv;
    e->max_splits = plan_splits(e->max_seq).n_splits;
    const size_t scratch = llmb_attn_decode_scratch_bytes(e->nq, e->nkv, e->hd, e->max_splits);
    cudaError_t ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking);
    auto alloc = [&](void **p, size_t bytes) {
        if (ce == cudaSuccess) ce = cudaMalloc(p, bytes);
        if (ce == cudaSuccess) ce = cudaMemset(*p, 0, bytes);
    };
    alloc(reinterpret_cast<void **>(&e->x), (size_t)e->d * 2);
    alloc(reinterpret_cast<void **>(&e->q), n_q * 2);
    alloc(reinterpret_cast<void **>(&e->attn), n_q * 2);
    alloc(reinterpret_cast<void **>(&e->h), (size_t)e->ffn * 2);
    alloc(reinterpret_cast<void **>(&e->logits), (size_t)e->vocab * 2);
    alloc(reinterpret_cast<void **>(&e->kcache), kv_elems * 2);
    alloc(reinterpret_cast<void **>(&e->vcache), kv_elems * 2);
    alloc(reinterpret_cast<void **>(&e->rope_cs), (size_t)e->hd * 4);
    alloc(reinterpret_cast<void **>(&e->d_pos), 256);
    alloc(reinterpret_cast<void **>(&e->d_next), 256);
    alloc(reinterpret_cast<void **>(&e->d_history), sizeof(int) * ((size_t)e->max_seq + 1));
    alloc(&e->attn_scratch, scratch);
    e->sm_count = sm_count_cached();
    e->step_max_splits = (e->max_seq + 31) / 32;
    e->step_scratch_bytes = llmb_decode_step_scratch_bytes(e->nq, e->nkv, e->hd, e->step_max_splits);
    alloc(&e->step_scratch, e->step_scratch_bytes);
    alloc(reinterpret_cast<void **>(&e->d_layers), sizeof(LlmbLayer) * (size_t)e->layers);
    if (e->tp_size > 1) {
        e->exchange_bytes = llmb_decode_step_exchange_bytes(e->tp_size, e->d);
        alloc(&e->exchange, e->exchange_bytes);  // plain cudaMalloc: exportable with cudaIpcGetMemHandle
        alloc(reinterpret_cast<void **>(&e->x_alt), (size_t)e->d * 2);
        e->peers[e->tp_rank] = e->exchange;
    }
    if (ce == cudaSuccess) {
        std::vector<LlmbLayer> hl((size_t)e->layers);
        for (int l = 0; l < e->layers; ++l) {
            const Llama3Layer *L = m->layers[l];
            hl[l].wqkv = reinterpret_cast<const uint16_t *>(L->self_attn_q_proj->d_fp16_tensor);
            hl[l].wo = reinterpret_cast<const uint16_t *>(L->self_attn_o_proj->d_fp16_tensor);
            hl[l].wgate = reinterpret_cast<const uint16_t *>(L->mlp_gate_proj->d_fp16_tensor);
            hl[l].wup = reinterpret_cast<const uint16_t *>(L->mlp_up_proj->d_fp16_tensor);
            hl[l].wdown = reinterpret_cast<const uint16_t *>(L->mlp_down_proj->d_fp16_tensor);
            hl[l].g_in = reinterpret_cast<const uint16_t *>(L->input_layernorm->d_fp16_tensor);
            hl[l].g_post = reinterpret_cast<const uint16_t *>(L->post_attention_layernorm->d_fp16_tensor);
            hl[l].k_cache = reinterpret_cast<uint16_t *>(e->kcache + (size_t)l * e->max_seq * n_kv);
            hl[l].v_cache = reinterpret_cast<uint16_t *>(e->vcache + (size_t)l * e->max_seq * n_kv);
        }
        ce = cudaMemcpy(e->d_layers, hl.data(), sizeof(LlmbLayer) * hl.size(), cudaMemcpyHostToDevice);
    }
    {   // the persistent kernel needs a cooperative launch and shapes inside its limits
        int dev = 0, coop = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
        const int G = e->nq / e->nkv;
        e->use_step_kernel = coop && G <= 8 && e->d <= 8192 && e->ffn <= 16384 && n_q <= 16384;
        if (e->tp_size > 1 && !e->use_step_kernel && ce == cudaSuccess) {
            destroy_engine(e);
            return fail(LLMB_ERR_UNSUPPORTED, "init_cache: tensor parallelism needs the whole-step kernel (cooperative launch)");
        }
    }
    if (ce == cudaSuccess) ce = cudaMallocHost(reinterpret_cast<void **>(&e->h_next), 256);
    for (auto &ev : e->ev)
        if (ce == cudaSuccess) ce = cudaEventCreate(&ev);
    CudaCache *cache = static_cast<CudaCache *>(calloc(1, sizeof(CudaCache)));
    llmb_half *h_logits = nullptr;
    if (ce == cudaSuccess) ce = cudaMallocHost(reinterpret_cast<void **>(&h_logits), (size_t)e->vocab * 2);
    if (ce != cudaSuccess || !cache) {
        int code = ce != cudaSuccess ? cuda_fail(ce, __FILE__, __LINE__) : LLMB_ERR_NOMEM;
        cudaFree(e->logits); cudaFree(e->kcache); cudaFree(e->vcache);
        if (h_logits) cudaFreeHost(h_logits);
        destroy_engine(e);
        free(cache);
        return fail(code, nullptr);
    }
    // The buffers were cleared on the legacy stream; the engine's stream does not wait for that one,
    // and with tensor parallelism a peer may write into the exchange block as soon as it is connected.
    cudaDeviceSynchronize();
    cache->priv = e;
    cache->PN_X = nullptr;
    cache->Q = make_view_tensor(1, (int)n_q, e->q);
    cache->K = make_view_tensor(e->layers * e->max_seq, (int)n_kv, e->kcache);
    cache->V = make_view_tensor(e->layers * e->max_seq, (int)n_kv, e->vcache);
    cache->d_attention_score_cache = nullptr;
    cache->d_feedforward_cache_upgate = e->h;
    cache->d_token_probdist = e->logits;
    cache->h_token_probdist = h_logits;
    cache->f_token_probdist = static_cast<float *>(malloc(sizeof(float) * (size_t)e->vocab));
    if (status_out) *status_out = LLMB_OK;
    return cache;
}

extern "C" CudaCache *init_cache(Llama3 *m) {
    int rc = 0;
    CudaCache *c = llama3_init_cache(m, &rc);
    if (!c) {
        printf("Error: init_cache failed (%d): %s\n", rc, llmb_last_error());
        exit(EXIT_FAILURE);  // CHECK_CUDA_ERROR in the reference exits (inference.cu:13-21)
    }
    return c;
}

extern "C" void free_cache(CudaCache *cache) {
    if (!cache) return;
    Engine *e = eng(cache);
    if (e) {
        cudaStreamSynchronize(e->stream);
        cudaFree(e->logits);
        cudaFree(e->kcache);
        cudaFree(e->vcache);
        destroy_engine(e);
    }
    auto free_view = [](Tensor *t) {
        if (!t) return;
        free(t->ndim); free(t->mem_len); free(t->shape); free(t);
    };
    free_view(cache->Q);
    free_view(cache->K);
    free_view(cache->V);
    if (cache->h_token_probdist) cudaFreeHost(cache->h_token_probdist);
    free(cache->f_token_probdist);
    free(cache);
}

extern "C" int cache_reset(CudaCache *cache) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    e->consumed.clear();
    e->greedy_state = false;
    // also brings the step kernel's arrival counter back to a known state
    LLMB_CUDA_OK(cudaMemsetAsync(e->step_scratch, 0, e->step_scratch_bytes, e->stream));
    LLMB_CUDA_OK(cudaMemsetAsync(e->attn_scratch, 0, 256, e->stream));
    // split-K arrival counters of the prompt-phase projections: a launch that wound down early leaves them set
    if (e->pf_ws) LLMB_CUDA_OK(cudaMemsetAsync(e->pf_ws, 0, 4096, e->stream));
    return LLMB_OK;
}

extern "C" int cache_set_tp_poll_limit(CudaCache *cache, unsigned int tag_poll_limit) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    e->tag_poll_limit = tag_poll_limit;
    return LLMB_OK;
}

extern "C" int cache_use_step_kernel(CudaCache *cache, int enable) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    if (!enable && e->tp_size > 1) {
        set_last_error("tensor parallel decode runs in the whole-step kernel only");
        return LLMB_ERR_UNSUPPORTED;
    }
    e->use_step_kernel = enable != 0;
    return LLMB_OK;
}

// Tensor parallel set-up, one process per GPU: every rank exports its exchange block as a CUDA IPC
// handle (64 bytes), the caller gathers the handles of all ranks in rank order (any transport:
// torch.distributed, MPI, a file) and hands the table to cache_tp_connect, which maps the peers'
// blocks into this process.
extern "C" int cache_tp_handle(CudaCache *cache, void *handle_out) {
    Engine *e = eng(cache);
    if (!e || !handle_out || e->tp_size < 2) return LLMB_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    LLMB_CUDA_OK(cudaIpcGetMemHandle(&h, e->exchange));
    memcpy(handle_out, &h, sizeof h);
    return LLMB_OK;
}

extern "C" int cache_tp_connect(CudaCache *cache, const void *handles) {
    Engine *e = eng(cache);
    if (!e || !handles || e->tp_size < 2) return LLMB_ERR_INVALID;
    if (e->tp_connected) return LLMB_OK;
    for (int r = 0; r < e->tp_size; ++r) {
        if (r == e->tp_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const unsigned char *>(handles) + (size_t)r * sizeof h, sizeof h);
        void *ptr = nullptr;
        LLMB_CUDA_OK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        e->peers[r] = ptr;
    }
    e->tp_connected = true;
    return LLMB_OK;
}

extern "C" int cache_set_options(CudaCache *cache, int use_graph, int use_pdl, int copy_logits) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    if (use_graph >= 0) e->use_graph = use_graph != 0;
    if (use_pdl >= 0 && (use_pdl != 0) != e->use_pdl) {
        e->use_pdl = use_pdl != 0;
        for (auto &kv : e->graphs) cudaGraphExecDestroy(kv.second);
        e->graphs.clear();
    }
    if (copy_logits >= 0) e->copy_logits = copy_logits != 0;
    return LLMB_OK;
}

extern "C" int cache_enable_hidden_dump(CudaCache *cache, int enable) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    if (enable && !e->hidden) LLMB_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&e->hidden), (size_t)(e->layers + 1) * e->d * 2));
    e->hidden_dump = enable != 0;
    return LLMB_OK;
}

extern "C" int cache_read_hidden(CudaCache *cache, uint16_t *h_out) {
    Engine *e = eng(cache);
    if (!e || !e->hidden || !h_out) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    LLMB_CUDA_OK(cudaMemcpy(h_out, e->hidden, (size_t)(e->layers + 1) * e->d * 2, cudaMemcpyDeviceToHost));
    return LLMB_OK;
}

// Profiling aid: per-phase timestamps of every CTA of the step kernel (last step wins); read them
// back with cache_debug_read(cache, 6, ...): [SM count][5 * n_layers + 2][8] uint64 nanoseconds.
extern "C" int cache_debug_trace(CudaCache *cache, int enable) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    if (enable && !e->trace) {
        e->trace_bytes = (size_t)e->sm_count * (5 * e->layers + 2) * 8 * sizeof(unsigned long long);
        LLMB_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&e->trace), e->trace_bytes));
        LLMB_CUDA_OK(cudaMemset(e->trace, 0, e->trace_bytes));
        LLMB_CUDA_OK(cudaDeviceSynchronize());
    } else if (!enable && e->trace) {
        LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
        cudaFree(e->trace);
        e->trace = nullptr;
    }
    return LLMB_OK;
}

// White-box access for tests: copies one of the engine's device buffers to the host.
// which: 0 = x, 1 = x_alt, 2 = q, 3 = attention output, 4 = h, 5 = this rank's exchange block,
// 6 = the step kernel's trace.
extern "C" int cache_debug_read(CudaCache *cache, int which, void *out, size_t bytes) {
    Engine *e = eng(cache);
    if (!e || !out) return LLMB_ERR_INVALID;
    const void *src = which == 0 ? (void *)e->x : which == 1 ? (void *)e->x_alt : which == 2 ? (void *)e->q
                    : which == 3 ? (void *)e->attn : which == 4 ? (void *)e->h : which == 5 ? e->exchange
                    : which == 6 ? (void *)e->trace : nullptr;
    if (!src) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    LLMB_CUDA_OK(cudaMemcpy(out, src, bytes, cudaMemcpyDeviceToHost));
    return LLMB_OK;
}

extern "C" int cache_set_prefill(CudaCache *cache, int enable, int min_rows) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    e->batched_prefill = enable != 0;
    if (min_rows > 0) e->prefill_min_rows = min_rows;
    return LLMB_OK;
}

extern "C" int cache_sample_next_token(CudaCache *cache, float temperature, int top_k, float top_p, uint64_t seed,
                                       uint64_t draw) {
    Engine *e = eng(cache);
    if (!e || !cache->h_token_probdist) return -LLMB_ERR_INVALID;
    if (!e->copy_logits || e->consumed.empty()) {
        set_last_error("cache_sample_next_token: no logits on the host (run inference() with copy_logits on first)");
        return -LLMB_ERR_INVALID;
    }
    if (e->tp_size > 1) {
        set_last_error("cache_sample_next_token: a tensor-parallel rank holds a slice of the logits only");
        return -LLMB_ERR_UNSUPPORTED;
    }
    int32_t token = -1;
    const int rc = llmb_sample_logits_host(reinterpret_cast<const uint16_t *>(cache->h_token_probdist), e->vocab, temperature,
                                           top_k, top_p, llmb_sampler_uniform(seed, draw), &token);
    return rc ? -rc : token;
}

// The same chain on the device (llmb_sample_logits): the logits never leave the GPU, only the 4-byte token
// comes back, and it is also written over the greedy token in the device history, so that
// inference_continue() goes on from the sampled token.  Falls back to nothing: a step the device kernel
// cannot take (status UNSUPPORTED) is reported to the caller, who can use cache_sample_next_token().
extern "C" int cache_sample_next_token_device(CudaCache *cache, float temperature, int top_k, float top_p, uint64_t seed,
                                              uint64_t draw) {
    Engine *e = eng(cache);
    if (!e) return -LLMB_ERR_INVALID;
    if (e->consumed.empty()) {
        set_last_error("cache_sample_next_token_device: no decode step has produced logits yet");
        return -LLMB_ERR_INVALID;
    }
    if (e->tp_size > 1) {
        set_last_error("cache_sample_next_token_device: a tensor-parallel rank holds a slice of the logits only");
        return -LLMB_ERR_UNSUPPORTED;
    }
    if (!e->sample_scratch) {
        cudaError_t ce = cudaMalloc(&e->sample_scratch, llmb_sample_scratch_bytes(e->vocab));
        if (ce != cudaSuccess) return -cuda_fail(ce, __FILE__, __LINE__);
    }
    int rc = llmb_sample_logits(reinterpret_cast<const uint16_t *>(e->logits), e->vocab, temperature, top_k, top_p, seed, draw,
                                e->sample_scratch, e->d_next, e->d_pos, e->d_history, e->max_seq + 1, 0, e->stream);
    if (rc) return -rc;
    cudaError_t ce = cudaMemcpyAsync(e->h_next, e->d_next, sizeof(int), cudaMemcpyDeviceToHost, e->stream);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(e->h_next + 2, e->sample_scratch, sizeof(int), cudaMemcpyDeviceToHost, e->stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    if (ce != cudaSuccess) return -cuda_fail(ce, __FILE__, __LINE__);
    if (e->h_next[2] != 0) {
        set_last_error(e->h_next[2] == 1 ? "device sampler: exp(logit / temperature) overflowed FP32; raise the temperature"
                                         : "device sampler: the top-p prefix runs past 1024 entries; use cache_sample_next_token");
        return -LLMB_ERR_UNSUPPORTED;
    }
    return e->h_next[0];
}

extern "C" long long cache_kernel_launches(const CudaCache *cache) {
    const Engine *e = eng(cache);
    return e ? e->launches : -1;
}

// tokenizer.cu:157-198: allocates the caller-owned activation tensor X [2048][embed_size] (zeroed)
// and the device token array.  The fused engine keeps its residual stream in its own buffer, so X
// only exists for callers that free it with _free_tensor as src/main.cu:124 does.
extern "C" int *tokens_to_cuda(int *tokens, int embed_size, Tensor *X) {
    (void)tokens;
    if (!X || embed_size <= 0) return nullptr;
    memset(X, 0, sizeof(Tensor));
    X->ndim = static_cast<int *>(malloc(sizeof(int)));
    X->mem_len = static_cast<int *>(malloc(sizeof(int)));
    X->shape = static_cast<int *>(malloc(sizeof(int) * 2));
    if (!X->ndim || !X->mem_len || !X->shape) return nullptr;
    *X->ndim = 2;
    *X->mem_len = embed_size * 2048;
    X->shape[0] = 2048;
    X->shape[1] = embed_size;
    void *p = nullptr;
    if (cudaMalloc(&p, sizeof(__half) * (size_t)*X->mem_len) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(__half) * (size_t)*X->mem_len);
    X->d_fp16_tensor = static_cast<llmb_half *>(p);
    X->loaded = 1;
    int *d_tokens = nullptr;
    if (cudaMalloc(reinterpret_cast<void **>(&d_tokens), sizeof(int) * (2048 + 1)) != cudaSuccess) return nullptr;
    return d_tokens;
}

extern "C" int inference(Llama3 *m, Tensor *X, int *d_tokens, int *h_tokens, CudaCache *cache) {
    (void)X;
    Engine *e = eng(cache);
    if (!m || !e || !h_tokens || e->model != m) {
        set_last_error("inference: null or mismatched model/cache");
        return -LLMB_ERR_INVALID;
    }
    const int count = h_tokens[0] - 1;  // tokenizer.cu:152
    if (count < 1 || count > e->max_seq) {
        set_last_error("inference: token count outside [1, max_seq]");
        return -LLMB_ERR_INVALID;
    }
    const int *ids = h_tokens + 1;
    // Reuse the cached prefix if the caller only appended (src/main.cu:121-122); else start over.
    int keep = (int)e->consumed.size();
    if (keep >= count) keep = 0;
    for (int i = 0; i < keep; ++i)
        if (e->consumed[i] != ids[i]) { keep = 0; break; }
    int rc = feed_tokens(e, ids, keep, count);
    if (rc) return -rc;
    // The reference copies the whole token array to the device on every call (inference.cu:150).
    if (d_tokens && count + 1 <= 2049)
        cudaMemcpyAsync(d_tokens, h_tokens, sizeof(int) * (size_t)(count + 1), cudaMemcpyHostToDevice, e->stream);
    if (e->copy_logits)
        cudaMemcpyAsync(cache->h_token_probdist, e->logits, (size_t)e->vocab * 2, cudaMemcpyDeviceToHost, e->stream);
    cudaMemcpyAsync(e->h_next, e->d_next, sizeof(int), cudaMemcpyDeviceToHost, e->stream);
    if ((rc = queue_status_read(e))) return -rc;
    cudaError_t ce = cudaStreamSynchronize(e->stream);
    if (ce != cudaSuccess) return -cuda_fail(ce, __FILE__, __LINE__);
    if ((rc = status_result(e))) return -rc;
    e->consumed.assign(ids, ids + count);
    e->greedy_state = true;  // the argmax kernel appended the sampled token to the device history
    return e->h_next[0];
}

extern "C" int inference_greedy(Llama3 *m, CudaCache *cache, const int *prompt, int n_prompt, int n_new, int *out_tokens,
                                float *prefill_ms, float *decode_ms) {
    Engine *e = eng(cache);
    if (!m || !e || e->model != m || !prompt || n_prompt < 1 || n_new < 1 || !out_tokens) return LLMB_ERR_INVALID;
    if (n_prompt + n_new > e->max_seq) {
        set_last_error("inference_greedy: prompt + new tokens exceed config.max_seq");
        return LLMB_ERR_INVALID;
    }
    e->consumed.clear();
    LLMB_CUDA_OK(cudaEventRecord(e->ev[0], e->stream));
    int rc = feed_tokens(e, prompt, 0, n_prompt);  // yields generated token 1 at history[n_prompt]
    if (rc) return rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[1], e->stream));
    for (int i = 1; i < n_new; ++i)
        if ((rc = run_step(e, true, n_prompt + i))) return rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[2], e->stream));
    LLMB_CUDA_OK(cudaMemcpyAsync(out_tokens, e->d_history + n_prompt, sizeof(int) * (size_t)n_new,
                                 cudaMemcpyDeviceToHost, e->stream));
    if ((rc = queue_status_read(e))) return rc;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    if ((rc = status_result(e))) return rc;
    if (prefill_ms) LLMB_CUDA_OK(cudaEventElapsedTime(prefill_ms, e->ev[0], e->ev[1]));
    if (decode_ms) LLMB_CUDA_OK(cudaEventElapsedTime(decode_ms, e->ev[1], e->ev[2]));
    // the cache now holds prompt + all but the last generated token
    e->consumed.assign(prompt, prompt + n_prompt);
    for (int i = 0; i + 1 < n_new; ++i) e->consumed.push_back(out_tokens[i]);
    e->greedy_state = true;
    return LLMB_OK;
}

extern "C" int inference_continue(Llama3 *m, CudaCache *cache, int n_steps, int *out_tokens, float *ms) {
    Engine *e = eng(cache);
    if (!m || !e || e->model != m || n_steps < 1 || !out_tokens) return LLMB_ERR_INVALID;
    if (!e->greedy_state || e->consumed.empty()) {
        set_last_error("inference_continue: no greedy run to continue");
        return LLMB_ERR_INVALID;
    }
    const int P = (int)e->consumed.size();  // rows in the cache; history[P] is the next input
    if (P + n_steps > e->max_seq) {
        set_last_error("inference_continue: would run past config.max_seq");
        return LLMB_ERR_INVALID;
    }
    int rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[0], e->stream));
    for (int i = 0; i < n_steps; ++i)
        if ((rc = run_step(e, true, P + i + 1))) return rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[1], e->stream));
    std::vector<int> fed((size_t)n_steps);
    LLMB_CUDA_OK(cudaMemcpyAsync(fed.data(), e->d_history + P, sizeof(int) * (size_t)n_steps, cudaMemcpyDeviceToHost,
                                 e->stream));
    LLMB_CUDA_OK(cudaMemcpyAsync(out_tokens, e->d_history + P + 1, sizeof(int) * (size_t)n_steps,
                                 cudaMemcpyDeviceToHost, e->stream));
    if ((rc = queue_status_read(e))) return rc;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    if ((rc = status_result(e))) return rc;
    if (ms) LLMB_CUDA_OK(cudaEventElapsedTime(ms, e->ev[0], e->ev[1]));
    e->consumed.insert(e->consumed.end(), fed.begin(), fed.end());
    return LLMB_OK;
}

// ---------------------------------------------------------------------------------------------
// Batched decode: n_seqs independent sequences, one new token each per step.  The reference's
// projections are written for m rows (kernel_standard_tiled_gemm over all rows, inference.cu:393-449,
// launched at :561-598 and :950-979); here the m = n_seqs rows of a step go through the tensor-core
// projections (llmb_gemm_f16), every weight byte is streamed once per step, and each sequence attends
// over its own cache: K, V [n_layers][n_seqs][max_seq][n_kv].  One step = 2 + 7 * n_layers + 3 kernels,
// captured once per attention bucket into a CUDA graph.
// ---------------------------------------------------------------------------------------------
namespace {

SplitPlan plan_batch_splits(int len, int split_len) {
    int bucket = 512;
    while (bucket < len) bucket <<= 1;
    return {bucket, bucket / split_len, split_len};
}

int enqueue_batch_step(Engine *e, const SplitPlan &sp) {
    e->rows_trace_call = 0;
    Llama3 *m = e->model;
    const Llama3Config &c = m->config;
    cudaStream_t s = e->stream;
    const int B = e->bt_seqs;
    const int n_q = e->nq * e->hd, n_kv = e->nkv * e->hd;
    const bool tp = e->tp_size > 1;
    auto u16 = [](const void *p) { return reinterpret_cast<const uint16_t *>(p); };
    auto u16w = [](void *p) { return reinterpret_cast<uint16_t *>(p); };
    int rc;
    if ((rc = llmb_embed_rope(u16(m->embed_tokens->d_fp16_tensor), e->bt_tok, e->bt_pos, B, e->d, e->embed_rows, e->hd,
                              c.rope_theta, u16w(e->pf_x), e->pf_rope, 0, 1, s)))
        return rc;
    if ((rc = llmb_rmsnorm_rows(u16(e->pf_x), u16(m->layers[0]->input_layernorm->d_fp16_tensor), u16w(e->pf_xn), B, e->d, c.eps, s)))
        return rc;
    const size_t layer_stride = (size_t)B * e->max_seq * n_kv;
    int xi = 0;  // tensor parallel: exchanges of this step so far
    for (int l = 0; l < e->layers; ++l) {
        const Llama3Layer *L = m->layers[l];
        __half *kl = e->bt_kcache + (size_t)l * layer_stride;
        __half *vl = e->bt_vcache + (size_t)l * layer_stride;
        LlmbGemmArgs g = small_gemm(e, e->pf_xn, L->self_attn_q_proj->d_fp16_tensor, e->pf_q, B, n_q + 2 * n_kv, e->d, LLMB_EPI_ROPE_KV);
        g.n_q = n_q; g.n_kv = n_kv; g.head_dim = e->hd;
        g.rope_cs = e->pf_rope;
        g.k_cache = u16w(kl); g.v_cache = u16w(vl);
        g.row_pos = e->bt_pos; g.seq_stride = e->max_seq; g.max_pos = e->max_seq;
        if ((rc = llmb_gemm_f16(&g, s))) return rc;
        if ((rc = llmb_attn_decode_batch(u16(e->pf_q), u16(kl), u16(vl), e->bt_pos, B, (size_t)e->max_seq, e->nq, e->nkv, e->hd,
                                         sp.n_splits, sp.split_len, u16w(e->pf_attn), e->bt_attn_scratch, 1, s)))
            return rc;
        if ((rc = row_parallel_projection(e, e->pf_attn, L->self_attn_o_proj->d_fp16_tensor, B, n_q,
                                          L->post_attention_layernorm->d_fp16_tensor, xi)))
            return rc;
        LlmbGemmArgs f = small_gemm(e, e->pf_xn, L->mlp_gate_proj->d_fp16_tensor, e->pf_h, B, e->ffn, e->d, LLMB_EPI_SWIGLU);
        f.b2 = u16(L->mlp_up_proj->d_fp16_tensor);
        if ((rc = llmb_gemm_f16(&f, s))) return rc;
        const void *next_gamma = l + 1 < e->layers ? m->layers[l + 1]->input_layernorm->d_fp16_tensor : m->norm->d_fp16_tensor;
        if ((rc = row_parallel_projection(e, e->pf_h, L->mlp_down_proj->d_fp16_tensor, B, e->ffn, next_gamma, xi))) return rc;
    }
    LlmbGemmArgs lm = small_gemm(e, e->pf_xn, m->lm_head->d_fp16_tensor, e->bt_logits, B, e->vocab, e->d, LLMB_EPI_STORE);
    if ((rc = llmb_gemm_f16(&lm, s))) return rc;
    // greedy token of every sequence -> next step's input; positions advance; history keeps what was sampled
    if (tp) {
        if ((rc = llmb_tp_argmax_rows(e->peers, e->tp_rank, e->tp_size, e->d, xi, u16(e->bt_logits), e->vocab, e->tp_rank * e->vocab, B,
                                      e->bt_tok, e->bt_pos, e->bt_history, e->max_seq + 1, e->tag_poll_limit, 1, s)))
            return rc;
        return llmb_tp_advance(e->exchange, e->tp_size, e->d, xi + 1, 1, s);
    }
    return llmb_argmax_rows_f16(u16(e->bt_logits), e->vocab, B, e->bt_tok, e->bt_pos, e->bt_history, e->max_seq + 1, 1, s);
}

// One batched step for sequences whose longest has `len` rows after it.
int run_batch_step(Engine *e, int len) {
    const SplitPlan sp = plan_batch_splits(len, e->bt_split_len);
    e->launches += 2 + 7 * e->layers + 2 + (e->tp_size > 1 ? 1 : 0);
    if (!e->use_graph) return enqueue_batch_step(e, sp);
    auto it = e->bt_graphs.find(sp.bucket);
    if (it == e->bt_graphs.end()) {
        cudaGraph_t graph = nullptr;
        LLMB_CUDA_OK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeRelaxed));
        int rc = enqueue_batch_step(e, sp);
        cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
        if (rc) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        LLMB_CUDA_OK(ce);
        cudaGraphExec_t exec = nullptr;
        ce = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        LLMB_CUDA_OK(ce);
        it = e->bt_graphs.emplace(sp.bucket, exec).first;
    }
    LLMB_CUDA_OK(cudaGraphLaunch(it->second, e->stream));
    return LLMB_OK;
}

bool batch_supported(const Engine *e) { return prefill_supported(e) || tp_rows_supported(e); }

}  // namespace

extern "C" int cache_batch_init(CudaCache *cache, int n_seqs) {
    Engine *e = eng(cache);
    if (!e || n_seqs < 1 || n_seqs > 128) return LLMB_ERR_INVALID;
    if (!batch_supported(e)) {
        set_last_error("cache_batch_init: batched decode needs head_dim 64 or 128, projection widths (this rank's q+k+v, d_model, "
                       "ffn) that are multiples of 128 and, under tensor parallelism, cache_tp_connect() first");
        return LLMB_ERR_UNSUPPORTED;
    }
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    for (auto &kv : e->bt_graphs) cudaGraphExecDestroy(kv.second);
    e->bt_graphs.clear();
    cudaFree(e->bt_kcache); cudaFree(e->bt_vcache); cudaFree(e->bt_logits); cudaFree(e->bt_pos); cudaFree(e->bt_tok);
    cudaFree(e->bt_history); cudaFree(e->bt_attn_scratch);
    e->bt_kcache = e->bt_vcache = e->bt_logits = nullptr;
    e->bt_pos = e->bt_tok = e->bt_history = nullptr;
    e->bt_attn_scratch = nullptr;
    e->bt_seqs = 0;
    const size_t n_kv = (size_t)e->nkv * e->hd;
    const size_t kv_bytes = (size_t)e->layers * n_seqs * e->max_seq * n_kv * 2;
    e->bt_max_splits = plan_batch_splits(e->max_seq, 32).n_splits;  // sized for the shortest split the engine may be set to
    const size_t scratch = llmb_attn_decode_batch_scratch_bytes(n_seqs, e->nq, e->nkv, e->hd, e->bt_max_splits);
    cudaError_t ce = cudaSuccess;
    auto alloc = [&](void **p, size_t bytes) {
        if (ce == cudaSuccess) ce = cudaMalloc(p, bytes);
        if (ce == cudaSuccess) ce = cudaMemsetAsync(*p, 0, bytes, e->stream);
    };
    alloc(reinterpret_cast<void **>(&e->bt_kcache), kv_bytes);
    alloc(reinterpret_cast<void **>(&e->bt_vcache), kv_bytes);
    alloc(reinterpret_cast<void **>(&e->bt_logits), (size_t)n_seqs * e->vocab * 2);
    alloc(reinterpret_cast<void **>(&e->bt_pos), sizeof(int) * (size_t)n_seqs);
    alloc(reinterpret_cast<void **>(&e->bt_tok), sizeof(int) * (size_t)n_seqs);
    alloc(reinterpret_cast<void **>(&e->bt_history), sizeof(int) * (size_t)n_seqs * (e->max_seq + 1));
    alloc(&e->bt_attn_scratch, scratch);
    if (ce != cudaSuccess) return cuda_fail(ce, __FILE__, __LINE__);
    int rc = ensure_prefill_buffers(e, std::max(n_seqs, e->prefill_chunk));
    if (rc) return rc;
    e->bt_seqs = n_seqs;
    e->bt_len.assign((size_t)n_seqs, 0);
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    return LLMB_OK;
}

// Profiling aid: the small-M projections of the following batched steps record per-CTA stamps (see
// LlmbGemmArgs.trace); projection number j of a step (5 per layer, then lm_head) writes at
// [j][1024 CTAs][8].  out (host, optional) receives the buffer of (5 * n_layers + 1) * 1024 * 8 uint64.
// enable = 1 allocates and arms (captured steps are dropped and captured again), 0 reads back and disarms.
extern "C" int cache_debug_rows_trace(CudaCache *cache, int enable, uint64_t *out) {
    Engine *e = eng(cache);
    if (!e) return LLMB_ERR_INVALID;
    const size_t bytes = (size_t)(5 * e->layers + 1) * kRowsTraceCtas * 8 * sizeof(unsigned long long);
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    for (auto &kv : e->bt_graphs) cudaGraphExecDestroy(kv.second);
    e->bt_graphs.clear();
    if (enable) {
        if (!e->rows_trace) LLMB_CUDA_OK(cudaMalloc(reinterpret_cast<void **>(&e->rows_trace), bytes));
        LLMB_CUDA_OK(cudaMemset(e->rows_trace, 0, bytes));
    } else if (e->rows_trace) {
        if (out) LLMB_CUDA_OK(cudaMemcpy(out, e->rows_trace, bytes, cudaMemcpyDeviceToHost));
        cudaFree(e->rows_trace);
        e->rows_trace = nullptr;
    }
    return LLMB_OK;
}

extern "C" int cache_batch_set_split_len(CudaCache *cache, int split_len) {
    Engine *e = eng(cache);
    if (!e || split_len < 32 || split_len > 512 || (split_len & (split_len - 1))) return LLMB_ERR_INVALID;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    for (auto &kv : e->bt_graphs) cudaGraphExecDestroy(kv.second);  // the split geometry is baked into the captured steps
    e->bt_graphs.clear();
    e->bt_split_len = split_len;
    return LLMB_OK;
}

// tokens: [n_seqs][n_tokens] host ids.  All but the last token of every sequence go through the block
// path into that sequence's cache; the last one is left as the input of the next cache_batch_step().
extern "C" int cache_batch_prefill(CudaCache *cache, const int *tokens, int n_tokens) {
    Engine *e = eng(cache);
    if (!e || !tokens || e->bt_seqs < 1 || n_tokens < 1) return LLMB_ERR_INVALID;
    if (n_tokens > e->max_seq) {
        set_last_error("cache_batch_prefill: prompt longer than config.max_seq");
        return LLMB_ERR_INVALID;
    }
    const int B = e->bt_seqs;
    const size_t n_kv = (size_t)e->nkv * e->hd;
    std::vector<int> last((size_t)B), pos((size_t)B, n_tokens - 1);
    int rc;
    for (int b = 0; b < B; ++b) {
        int *hist = e->bt_history + (size_t)b * (e->max_seq + 1);
        LLMB_CUDA_OK(cudaMemcpyAsync(hist, tokens + (size_t)b * n_tokens, sizeof(int) * (size_t)n_tokens, cudaMemcpyHostToDevice,
                                     e->stream));
        if (n_tokens > 1) {
            __half *kb = e->bt_kcache + (size_t)b * e->max_seq * n_kv, *vb = e->bt_vcache + (size_t)b * e->max_seq * n_kv;
            rc = e->tp_size > 1 ? prefill_rows_tp(e, 0, n_tokens - 1, hist, kb, vb, (size_t)B * e->max_seq * n_kv)
                                : prefill_rows(e, 0, n_tokens - 1, hist, kb, vb, (size_t)B * e->max_seq * n_kv);
            if (rc) return rc;
        }
        last[(size_t)b] = tokens[(size_t)b * n_tokens + n_tokens - 1];
    }
    LLMB_CUDA_OK(cudaMemcpyAsync(e->bt_tok, last.data(), sizeof(int) * (size_t)B, cudaMemcpyHostToDevice, e->stream));
    LLMB_CUDA_OK(cudaMemcpyAsync(e->bt_pos, pos.data(), sizeof(int) * (size_t)B, cudaMemcpyHostToDevice, e->stream));
    if ((rc = queue_status_read(e))) return rc;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));  // `last` and `pos` are stack-lifetime host buffers
    if ((rc = status_result(e))) return rc;
    e->bt_len.assign((size_t)B, n_tokens - 1);
    return LLMB_OK;
}

// One batched step.  tokens (optional, [n_seqs]): the input token of every sequence (teacher forcing); NULL
// feeds what the previous step sampled (or the last prompt token after cache_batch_prefill).  h_logits
// (optional, [n_seqs][vocab] FP16 bits) and next_tokens (optional, [n_seqs]) are copied back when given.
extern "C" int cache_batch_step(CudaCache *cache, const int *tokens, uint16_t *h_logits, int *next_tokens) {
    Engine *e = eng(cache);
    if (!e || e->bt_seqs < 1) return LLMB_ERR_INVALID;
    const int B = e->bt_seqs;
    const int len = e->bt_len[0] + 1;
    if (len > e->max_seq) {
        set_last_error("cache_batch_step: would run past config.max_seq");
        return LLMB_ERR_INVALID;
    }
    if (tokens) LLMB_CUDA_OK(cudaMemcpyAsync(e->bt_tok, tokens, sizeof(int) * (size_t)B, cudaMemcpyHostToDevice, e->stream));
    int rc = run_batch_step(e, len);
    if (rc) return rc;
    if (h_logits)
        LLMB_CUDA_OK(cudaMemcpyAsync(h_logits, e->bt_logits, (size_t)B * e->vocab * 2, cudaMemcpyDeviceToHost, e->stream));
    if (next_tokens)
        LLMB_CUDA_OK(cudaMemcpyAsync(next_tokens, e->bt_tok, sizeof(int) * (size_t)B, cudaMemcpyDeviceToHost, e->stream));
    if ((rc = queue_status_read(e))) return rc;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    if ((rc = status_result(e))) return rc;
    for (int &l : e->bt_len) l += 1;
    return LLMB_OK;
}

// n_steps greedy steps with the sampled tokens fed back on the device; out_tokens [n_seqs][n_steps].
extern "C" int cache_batch_greedy(CudaCache *cache, int n_steps, int *out_tokens, float *ms) {
    Engine *e = eng(cache);
    if (!e || e->bt_seqs < 1 || n_steps < 1 || !out_tokens) return LLMB_ERR_INVALID;
    const int B = e->bt_seqs, start = e->bt_len[0];
    if (start + n_steps > e->max_seq) {
        set_last_error("cache_batch_greedy: would run past config.max_seq");
        return LLMB_ERR_INVALID;
    }
    int rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[0], e->stream));
    for (int i = 0; i < n_steps; ++i)
        if ((rc = run_batch_step(e, start + i + 1))) return rc;
    LLMB_CUDA_OK(cudaEventRecord(e->ev[1], e->stream));
    // the token sampled by the step at position p sits at history[p + 1]
    LLMB_CUDA_OK(cudaMemcpy2DAsync(out_tokens, sizeof(int) * (size_t)n_steps, e->bt_history + start + 1,
                                   sizeof(int) * (size_t)(e->max_seq + 1), sizeof(int) * (size_t)n_steps, (size_t)B,
                                   cudaMemcpyDeviceToHost, e->stream));
    if ((rc = queue_status_read(e))) return rc;
    LLMB_CUDA_OK(cudaStreamSynchronize(e->stream));
    if ((rc = status_result(e))) return rc;
    if (ms) LLMB_CUDA_OK(cudaEventElapsedTime(ms, e->ev[0], e->ev[1]));
    for (int &l : e->bt_len) l += n_steps;
    return LLMB_OK;
}
