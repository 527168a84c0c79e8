// Model container and load-time upload: the reference's src/llama3/llama3.cu re-implemented.
//
//   init_llama3 / free_llama3 / _free_tensor   llama3.cu:9-154
//   to_cuda                                    llama3.cu:156-238 (H2D + BF16->FP16 per tensor)
//
// Device layout chosen for the decode kernels (not the reference's one-allocation-per-tensor):
//   * q_proj, k_proj, v_proj of a layer live back to back in ONE buffer [(n_q + 2 n_kv)][d], so
//     the fused QKV projection streams a single contiguous span; the three Tensor structs keep
//     valid row-major views into it (k and v are marked device_is_view);
//   * every other tensor has its own 256-byte-aligned allocation;
//   * to_cuda streams: this rank's window of every tensor is read straight from its shard file (pread)
//     into one of two pinned staging buffers in chunks of rows, copied to the device with
//     cudaMemcpyAsync and converted BF16 -> FP16 on the same stream, while the host already reads the
//     next chunk into the other buffer.  The host holds two staging buffers, never the model (the
//     reference reads every tensor whole into host memory at load, safetensor.cu:140-155, and
//     cudaMallocs and frees a device staging buffer per tensor, llama3.cu:203, :234).
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../csrc/common.cuh"
#include "../../include/llama3.h"
#include "../../include/llm_b200_synth.h"
#include "host_internal.h"

using namespace llmb;

static Tensor *new_tensor() { return static_cast<Tensor *>(calloc(1, sizeof(Tensor))); }

ModelPriv *llmb::model_priv(Llama3 *m) {
    if (!m) return nullptr;
    if (!m->priv) m->priv = new (std::nothrow) ModelPriv();
    return static_cast<ModelPriv *>(m->priv);
}

extern "C" int llama3_set_streaming(Llama3 *m, int enable) {
    ModelPriv *pv = model_priv(m);
    if (!pv) return LLMB_ERR_INVALID;
    pv->streaming = enable != 0;
    return LLMB_OK;
}

extern "C" int llama3_upload_stats(Llama3 *m, double *seconds, unsigned long long *bytes_read,
                                   unsigned long long *bytes_uploaded, unsigned long long *host_staging_bytes) {
    ModelPriv *pv = model_priv(m);
    if (!pv) return LLMB_ERR_INVALID;
    if (seconds) *seconds = pv->upload_seconds;
    if (bytes_read) *bytes_read = pv->bytes_read;
    if (bytes_uploaded) *bytes_uploaded = pv->bytes_uploaded;
    if (host_staging_bytes) *host_staging_bytes = pv->staging_bytes;
    return LLMB_OK;
}

extern "C" Llama3 *init_llama3(int n_layers) {
    if (n_layers <= 0) return nullptr;
    Llama3 *m = static_cast<Llama3 *>(calloc(1, sizeof(Llama3)));
    if (!m) return nullptr;
    m->n_layers = n_layers;
    m->embed_tokens = new_tensor();
    m->norm = new_tensor();
    m->lm_head = new_tensor();
    m->layers = static_cast<Llama3Layer **>(calloc((size_t)n_layers, sizeof(Llama3Layer *)));
    bool ok = m->embed_tokens && m->norm && m->lm_head && m->layers;
    for (int i = 0; ok && i < n_layers; ++i) {
        Llama3Layer *l = static_cast<Llama3Layer *>(calloc(1, sizeof(Llama3Layer)));
        if (!l) { ok = false; break; }
        l->layernum = i;
        l->input_layernorm = new_tensor();
        l->mlp_down_proj = new_tensor();
        l->mlp_gate_proj = new_tensor();
        l->mlp_up_proj = new_tensor();
        l->post_attention_layernorm = new_tensor();
        l->self_attn_k_proj = new_tensor();
        l->self_attn_o_proj = new_tensor();
        l->self_attn_q_proj = new_tensor();
        l->self_attn_v_proj = new_tensor();
        m->layers[i] = l;
        ok = l->input_layernorm && l->mlp_down_proj && l->mlp_gate_proj && l->mlp_up_proj &&
             l->post_attention_layernorm && l->self_attn_k_proj && l->self_attn_o_proj && l->self_attn_q_proj &&
             l->self_attn_v_proj;
    }
    if (!ok) {
        free_llama3(m);
        return nullptr;
    }
    // Defaults are the reference's literals; to_cuda fills the shape-derived fields.
    m->config.head_dim = 128;
    m->config.max_seq = 2048;
    m->config.rope_theta = 500000.0f;
    m->config.eps = 1e-5;
    m->tp_rank = 0;
    m->tp_size = 1;
    return m;
}

extern "C" void _free_tensor(Tensor *t) {
    if (!t) return;
    if (t->d_ndim) cudaFree(t->d_ndim);
    if (t->d_mem_len) cudaFree(t->d_mem_len);
    if (t->d_shape) cudaFree(t->d_shape);
    if (t->d_bf16_tensor) cudaFree(t->d_bf16_tensor);
    if (t->d_fp16_tensor && !t->device_is_view) cudaFree(t->d_fp16_tensor);
    free(t->ndim);
    free(t->mem_len);
    free(t->shape);
    free(t->bf16_tensor);
    free(t);
}

void llmb::for_each_tensor(Llama3 *m, const std::function<void(Tensor *, int, int)> &fn) {
    fn(m->embed_tokens, -1, LLMB_SID_EMBED);
    fn(m->lm_head, -1, LLMB_SID_LM_HEAD);
    fn(m->norm, -1, LLMB_SID_NORM);
    for (int i = 0; i < m->n_layers; ++i) {
        Llama3Layer *l = m->layers[i];
        if (!l) continue;
        fn(l->input_layernorm, i, LLMB_SLOT_INPUT_LAYERNORM);
        fn(l->mlp_down_proj, i, LLMB_SLOT_DOWN);
        fn(l->mlp_gate_proj, i, LLMB_SLOT_GATE);
        fn(l->mlp_up_proj, i, LLMB_SLOT_UP);
        fn(l->post_attention_layernorm, i, LLMB_SLOT_POST_LAYERNORM);
        fn(l->self_attn_k_proj, i, LLMB_SLOT_K);
        fn(l->self_attn_o_proj, i, LLMB_SLOT_O);
        fn(l->self_attn_q_proj, i, LLMB_SLOT_Q);
        fn(l->self_attn_v_proj, i, LLMB_SLOT_V);
    }
}

extern "C" void free_llama3(Llama3 *m) {
    if (!m) return;
    if (m->embed_tokens) _free_tensor(m->embed_tokens);
    if (m->norm) _free_tensor(m->norm);
    if (m->lm_head) _free_tensor(m->lm_head);
    if (m->layers) {
        for (int i = 0; i < m->n_layers; ++i) {
            Llama3Layer *l = m->layers[i];
            if (!l) continue;
            // q owns the fused QKV buffer; k and v are views and must go first or last alike.
            _free_tensor(l->input_layernorm);
            _free_tensor(l->mlp_down_proj);
            _free_tensor(l->mlp_gate_proj);
            _free_tensor(l->mlp_up_proj);
            _free_tensor(l->post_attention_layernorm);
            _free_tensor(l->self_attn_k_proj);
            _free_tensor(l->self_attn_o_proj);
            _free_tensor(l->self_attn_q_proj);
            _free_tensor(l->self_attn_v_proj);
            free(l);
        }
        free(m->layers);
    }
    delete static_cast<ModelPriv *>(m->priv);
    free(m);
}

extern "C" int llama3_set_config(Llama3 *m, const Llama3Config *c) {
    if (!m || !c) return LLMB_ERR_INVALID;
    if (c->d_model > 0) m->config.d_model = c->d_model;
    if (c->n_q_heads > 0) m->config.n_q_heads = c->n_q_heads;
    if (c->n_kv_heads > 0) m->config.n_kv_heads = c->n_kv_heads;
    if (c->head_dim > 0) m->config.head_dim = c->head_dim;
    if (c->ffn > 0) m->config.ffn = c->ffn;
    if (c->vocab > 0) m->config.vocab = c->vocab;
    if (c->max_seq > 0) m->config.max_seq = c->max_seq;
    if (c->rope_theta > 0.0f) m->config.rope_theta = c->rope_theta;
    if (c->eps > 0.0) m->config.eps = c->eps;
    return LLMB_OK;
}

extern "C" int llama3_set_tp(Llama3 *m, int tp_rank, int tp_size) {
    if (!m || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return LLMB_ERR_INVALID;
    if (tp_size > 8) {
        set_last_error("llama3_set_tp: at most 8 tensor-parallel ranks (one NVSwitch domain)");
        return LLMB_ERR_UNSUPPORTED;
    }
    if (m->config_ready) {
        set_last_error("llama3_set_tp: call before to_cuda / llama3_synth_weights");
        return LLMB_ERR_INVALID;
    }
    m->tp_rank = tp_rank;
    m->tp_size = tp_size;
    return LLMB_OK;
}

static int set_shape(Tensor *t, int d0, int d1) {
    free(t->ndim);
    free(t->mem_len);
    free(t->shape);
    int nd = d1 > 0 ? 2 : 1;
    t->ndim = static_cast<int *>(malloc(sizeof(int)));
    t->mem_len = static_cast<int *>(malloc(sizeof(int)));
    t->shape = static_cast<int *>(malloc(sizeof(int) * 2));
    if (!t->ndim || !t->mem_len || !t->shape) return LLMB_ERR_NOMEM;
    *t->ndim = nd;
    t->shape[0] = d0;
    t->shape[1] = d1 > 0 ? d1 : 1;
    long long n = (long long)d0 * (d1 > 0 ? d1 : 1);
    if (n > 0x7fffffffLL) return LLMB_ERR_INVALID;
    *t->mem_len = (int)n;
    return LLMB_OK;
}

// Shape checks + config derivation shared by the file and the synthetic path.
static int derive_config(Llama3 *m) {
    Llama3Config &c = m->config;
    char msg[256];
    bool missing = false;
    for_each_tensor(m, [&](Tensor *t, int, int) {
        if (!t || !t->loaded || !t->shape || !t->ndim) missing = true;
    });
    if (missing) {
        set_last_error("to_cuda: at least one tensor of the model was never loaded");
        return LLMB_ERR_INVALID;
    }
    if (*m->embed_tokens->ndim != 2 || *m->lm_head->ndim != 2) {
        set_last_error("to_cuda: embed_tokens and lm_head must be 2-D");
        return LLMB_ERR_INVALID;
    }
    c.d_model = m->embed_tokens->shape[1];
    c.vocab = m->lm_head->shape[0];
    const Llama3Layer *l0 = m->layers[0];
    c.ffn = l0->mlp_gate_proj->shape[0];
    const int q_rows = l0->self_attn_q_proj->shape[0], kv_rows = l0->self_attn_k_proj->shape[0];
    if (c.head_dim <= 0 || q_rows % c.head_dim || kv_rows % c.head_dim) {
        snprintf(msg, sizeof msg, "to_cuda: q rows %d / kv rows %d are not multiples of head_dim %d", q_rows, kv_rows,
                 c.head_dim);
        set_last_error(msg);
        return LLMB_ERR_INVALID;
    }
    c.n_q_heads = q_rows / c.head_dim;
    c.n_kv_heads = kv_rows / c.head_dim;
    if (c.n_kv_heads <= 0 || c.n_q_heads % c.n_kv_heads) {
        set_last_error("to_cuda: query heads are not a multiple of KV heads");
        return LLMB_ERR_INVALID;
    }
    auto is = [](const Tensor *t, int d0, int d1) {
        return d1 > 0 ? (*t->ndim == 2 && t->shape[0] == d0 && t->shape[1] == d1) : (*t->ndim == 1 && t->shape[0] == d0);
    };
    bool ok = is(m->lm_head, c.vocab, c.d_model) && is(m->norm, c.d_model, 0) && m->embed_tokens->shape[0] > 0;
    for (int i = 0; ok && i < m->n_layers; ++i) {
        const Llama3Layer *l = m->layers[i];
        ok = is(l->input_layernorm, c.d_model, 0) && is(l->post_attention_layernorm, c.d_model, 0) &&
             is(l->self_attn_q_proj, q_rows, c.d_model) && is(l->self_attn_k_proj, kv_rows, c.d_model) &&
             is(l->self_attn_v_proj, kv_rows, c.d_model) && is(l->self_attn_o_proj, c.d_model, q_rows) &&
             is(l->mlp_gate_proj, c.ffn, c.d_model) && is(l->mlp_up_proj, c.ffn, c.d_model) &&
             is(l->mlp_down_proj, c.d_model, c.ffn);
    }
    if (!ok) {
        set_last_error("to_cuda: tensor shapes are inconsistent with a LLaMA3 decoder");
        return LLMB_ERR_INVALID;
    }
    if (c.d_model % 8 || c.ffn % 8 || (c.head_dim != 64 && c.head_dim != 128)) {
        set_last_error("to_cuda: d_model and ffn must be multiples of 8 and head_dim 64 or 128");
        return LLMB_ERR_UNSUPPORTED;
    }
    m->config_ready = 1;
    return LLMB_OK;
}

// The window of a tensor that tensor-parallel rank `rank` of `size` keeps: q/k/v, gate/up and
// lm_head by output rows, o_proj and down_proj by input columns, the rest whole.
struct Shard {
    int row0, rows, col0, cols, full_cols;
    size_t elems() const { return (size_t)rows * cols; }
};

static Shard shard_of(const Tensor *t, int layer, int slot, int rank, int size) {
    Shard s;
    s.full_cols = *t->ndim == 2 ? t->shape[1] : 1;
    s.row0 = 0; s.rows = t->shape[0]; s.col0 = 0; s.cols = s.full_cols;
    if (size == 1) return s;
    const bool by_rows = (layer < 0 && slot == LLMB_SID_LM_HEAD) ||
                         (layer >= 0 && (slot == LLMB_SLOT_Q || slot == LLMB_SLOT_K || slot == LLMB_SLOT_V ||
                                         slot == LLMB_SLOT_GATE || slot == LLMB_SLOT_UP));
    const bool by_cols = layer >= 0 && (slot == LLMB_SLOT_O || slot == LLMB_SLOT_DOWN);
    if (by_rows) { s.rows = t->shape[0] / size; s.row0 = rank * s.rows; }
    if (by_cols) { s.cols = s.full_cols / size; s.col0 = rank * s.cols; }
    return s;
}

// Host-only view of the sharding plan (tests, loaders that slice at read time): the window of the
// tensor in (layer, slot) that this model's rank keeps, as {row0, rows, col0, cols, full_cols}.
// layer = -1 with slot LLMB_SID_EMBED / LLMB_SID_LM_HEAD / LLMB_SID_NORM names the global tensors.
extern "C" int llama3_tensor_shard(Llama3 *m, int layer, int slot, int out[5]) {
    if (!m || !out) return LLMB_ERR_INVALID;
    Tensor *found = nullptr;
    for_each_tensor(m, [&](Tensor *t, int l, int s) {
        if (l == layer && s == slot) found = t;
    });
    if (!found || !found->loaded || !found->shape) return LLMB_ERR_INVALID;
    const Shard sh = shard_of(found, layer, slot, m->tp_rank, m->tp_size);
    out[0] = sh.row0; out[1] = sh.rows; out[2] = sh.col0; out[3] = sh.cols; out[4] = sh.full_cols;
    return LLMB_OK;
}

static int check_tp(const Llama3 *m) {
    const Llama3Config &c = m->config;
    const int k = m->tp_size;
    if (k == 1) return LLMB_OK;
    if (c.n_q_heads % k || c.n_kv_heads % k || c.ffn % (8 * k) || c.vocab % k) {
        set_last_error("tensor parallel size must divide the query heads, the KV heads, ffn / 8 and the vocabulary");
        return LLMB_ERR_INVALID;
    }
    return LLMB_OK;
}

// Destination of each tensor on the device; allocates own buffers and the fused QKV buffer.
static int place_tensors(Llama3 *m) {
    const Llama3Config &c = m->config;
    const int rank = m->tp_rank, size = m->tp_size;
    int cur_layer = -1, cur_slot = 0;
    auto own = [&](Tensor *t) -> int {
        void *p = nullptr;
        LLMB_CUDA_OK(cudaMalloc(&p, shard_of(t, cur_layer, cur_slot, rank, size).elems() * 2));
        t->d_fp16_tensor = static_cast<llmb_half *>(p);
        t->device_is_view = 0;
        return LLMB_OK;
    };
    int rc;
    auto own_as = [&](Tensor *t, int layer, int slot) {
        cur_layer = layer;
        cur_slot = slot;
        return own(t);
    };
    if ((rc = own_as(m->embed_tokens, -1, LLMB_SID_EMBED)) || (rc = own_as(m->lm_head, -1, LLMB_SID_LM_HEAD)) ||
        (rc = own_as(m->norm, -1, LLMB_SID_NORM)))
        return rc;
    const size_t q_elems = (size_t)c.n_q_heads / size * c.head_dim * c.d_model;
    const size_t kv_elems = (size_t)c.n_kv_heads / size * c.head_dim * c.d_model;
    for (int i = 0; i < m->n_layers; ++i) {
        Llama3Layer *l = m->layers[i];
        if ((rc = own_as(l->input_layernorm, i, LLMB_SLOT_INPUT_LAYERNORM)) ||
            (rc = own_as(l->post_attention_layernorm, i, LLMB_SLOT_POST_LAYERNORM)) ||
            (rc = own_as(l->self_attn_o_proj, i, LLMB_SLOT_O)) || (rc = own_as(l->mlp_gate_proj, i, LLMB_SLOT_GATE)) ||
            (rc = own_as(l->mlp_up_proj, i, LLMB_SLOT_UP)) || (rc = own_as(l->mlp_down_proj, i, LLMB_SLOT_DOWN)))
            return rc;
        void *qkv = nullptr;
        LLMB_CUDA_OK(cudaMalloc(&qkv, (q_elems + 2 * kv_elems) * 2));
        llmb_half *base = static_cast<llmb_half *>(qkv);
        l->self_attn_q_proj->d_fp16_tensor = base;
        l->self_attn_q_proj->device_is_view = 0;  // owner of the fused buffer
        l->self_attn_k_proj->d_fp16_tensor = base + q_elems;
        l->self_attn_k_proj->device_is_view = 1;
        l->self_attn_v_proj->d_fp16_tensor = base + q_elems + kv_elems;
        l->self_attn_v_proj->device_is_view = 1;
    }
    return LLMB_OK;
}

// After the upload a Tensor describes what is on the device: the shard's shape.
static void set_local_shape(Tensor *t, const Shard &s) {
    t->shape[0] = s.rows;
    if (*t->ndim == 2) t->shape[1] = s.cols;
    *t->mem_len = (int)s.elems();
}

namespace {

// Two pinned host buffers and two device buffers that take turns: while chunk i is on its way to the device
// (and being converted there), the host fills the other buffer with chunk i + 1.
struct UploadPipe {
    static constexpr size_t kChunkBytes = (size_t)32 << 20;
    void *pinned[2] = {nullptr, nullptr};
    void *dev[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaStream_t stream = nullptr;
    size_t capacity = 0;
    int turn = 0;
    std::vector<int> fds;

    int open(size_t max_row_bytes, bool need_dev) {
        capacity = std::max(kChunkBytes, max_row_bytes);
        LLMB_CUDA_OK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            LLMB_CUDA_OK(cudaMallocHost(&pinned[i], capacity));
            if (need_dev) LLMB_CUDA_OK(cudaMalloc(&dev[i], capacity));
            LLMB_CUDA_OK(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        return LLMB_OK;
    }
    ~UploadPipe() {
        if (stream) cudaStreamSynchronize(stream);
        for (int i = 0; i < 2; ++i) {
            if (pinned[i]) cudaFreeHost(pinned[i]);
            if (dev[i]) cudaFree(dev[i]);
            if (done[i]) cudaEventDestroy(done[i]);
        }
        if (stream) cudaStreamDestroy(stream);
        for (int fd : fds)
            if (fd >= 0) close(fd);
    }
};

bool pread_all(int fd, void *dst, size_t bytes, unsigned long long offset) {
    unsigned char *p = static_cast<unsigned char *>(dst);
    while (bytes > 0) {
        const ssize_t got = pread(fd, p, bytes, (off_t)offset);
        if (got <= 0) return false;
        p += got;
        bytes -= (size_t)got;
        offset += (unsigned long long)got;
    }
    return true;
}

}  // namespace

extern "C" int llama3_to_cuda(Llama3 *m) {
    if (!m) return LLMB_ERR_INVALID;
    int rc = derive_config(m);
    if (rc) return rc;
    if ((rc = check_tp(m))) return rc;
    if ((rc = place_tensors(m))) return rc;
    ModelPriv *pv = model_priv(m);
    if (!pv) return LLMB_ERR_NOMEM;
    const auto t_start = std::chrono::steady_clock::now();
    const int rank = m->tp_rank, size = m->tp_size;
    size_t max_row_bytes = 0;
    bool any_bf16 = false;
    for_each_tensor(m, [&](Tensor *t, int layer, int slot) {
        max_row_bytes = std::max(max_row_bytes, (size_t)shard_of(t, layer, slot, rank, size).cols * 2);
        any_bf16 = any_bf16 || t->file_dtype != 1;
    });
    UploadPipe pipe;
    if ((rc = pipe.open(max_row_bytes, any_bf16))) return rc;
    pipe.fds.assign(pv->files.size(), -1);
    pv->bytes_read = pv->bytes_uploaded = 0;
    pv->staging_bytes = 2ull * pipe.capacity;
    int status = LLMB_OK;
    for_each_tensor(m, [&](Tensor *t, int layer, int slot) {
        if (status) return;
        const auto src_it = pv->sources.find(t);
        const bool from_file = !t->bf16_tensor && src_it != pv->sources.end();
        if (!t->bf16_tensor && !from_file) {
            set_last_error("to_cuda: tensor payload missing (neither in host memory nor in a loaded shard)");
            status = LLMB_ERR_INVALID;
            return;
        }
        int fd = -1;
        if (from_file) {
            const int fi = src_it->second.file;
            if (pipe.fds[(size_t)fi] < 0) pipe.fds[(size_t)fi] = ::open(pv->files[(size_t)fi].c_str(), O_RDONLY);
            fd = pipe.fds[(size_t)fi];
            if (fd < 0) {
                set_last_error(("to_cuda: cannot reopen " + pv->files[(size_t)fi]).c_str());
                status = LLMB_ERR_IO;
                return;
            }
        }
        const Shard sh = shard_of(t, layer, slot, rank, size);
        const size_t row_bytes = (size_t)sh.cols * 2, full_row_bytes = (size_t)sh.full_cols * 2;
        const int chunk_rows = (int)std::max<size_t>(1, pipe.capacity / row_bytes);
        uint16_t *dst = reinterpret_cast<uint16_t *>(t->d_fp16_tensor);
        for (int r0 = 0; r0 < sh.rows && !status; r0 += chunk_rows) {
            const int nr = std::min(chunk_rows, sh.rows - r0);
            const size_t bytes = (size_t)nr * row_bytes;
            const int b = pipe.turn & 1;
            cudaError_t e = cudaEventSynchronize(pipe.done[b]);  // the copy that last used this buffer has left the host
            unsigned char *stage = static_cast<unsigned char *>(pipe.pinned[b]);
            // this rank's window: rows [row0 + r0, + nr), columns [col0, col0 + cols)
            const size_t first = ((size_t)(sh.row0 + r0) * sh.full_cols + sh.col0) * 2;
            bool ok = true;
            if (from_file) {
                if (sh.cols == sh.full_cols) {
                    ok = pread_all(fd, stage, bytes, src_it->second.offset + first);
                } else {
                    for (int i = 0; i < nr && ok; ++i)
                        ok = pread_all(fd, stage + (size_t)i * row_bytes, row_bytes, src_it->second.offset + first + (size_t)i * full_row_bytes);
                }
                pv->bytes_read += bytes;
            } else {
                const unsigned char *base = reinterpret_cast<const unsigned char *>(t->bf16_tensor) + first;
                for (int i = 0; i < nr; ++i) memcpy(stage + (size_t)i * row_bytes, base + (size_t)i * full_row_bytes, row_bytes);
            }
            if (!ok) {
                set_last_error("to_cuda: short read from a shard file (changed or truncated since it was loaded?)");
                status = LLMB_ERR_IO;
                break;
            }
            uint16_t *out = dst + (size_t)r0 * sh.cols;
            if (t->file_dtype == 1) {  // F16 files pass through
                if (e == cudaSuccess) e = cudaMemcpyAsync(out, stage, bytes, cudaMemcpyHostToDevice, pipe.stream);
            } else {                   // BF16: convert on the device (llama3.cu:240-254)
                if (e == cudaSuccess) e = cudaMemcpyAsync(pipe.dev[b], stage, bytes, cudaMemcpyHostToDevice, pipe.stream);
                if (e == cudaSuccess) {
                    const int r = llmb_bf16_to_fp16(static_cast<const uint16_t *>(pipe.dev[b]), out, bytes / 2, pipe.stream);
                    if (r) status = r;
                }
            }
            if (e == cudaSuccess) e = cudaEventRecord(pipe.done[b], pipe.stream);
            if (e != cudaSuccess && !status) status = cuda_fail(e, __FILE__, __LINE__);
            pv->bytes_uploaded += bytes;
            ++pipe.turn;
        }
        free(t->bf16_tensor);  // llama3.cu:211
        t->bf16_tensor = nullptr;
        set_local_shape(t, sh);
    });
    cudaError_t e = cudaStreamSynchronize(pipe.stream);
    if (e != cudaSuccess && !status) status = cuda_fail(e, __FILE__, __LINE__);
    pv->upload_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t_start).count();
    return status;
}

extern "C" void to_cuda(Llama3 *m) {
    int rc = llama3_to_cuda(m);
    if (rc) {
        printf("Error: to_cuda failed (%d): %s\n", rc, llmb_last_error());
        exit(1);
    }
}

extern "C" int llama3_synth_weights(Llama3 *m, const Llama3Config *cfg, uint64_t seed, int bf16) {
    if (!m || !cfg) return LLMB_ERR_INVALID;
    if (cfg->d_model <= 0 || cfg->n_q_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->head_dim <= 0 || cfg->ffn <= 0 ||
        cfg->vocab <= 0)
        return LLMB_ERR_INVALID;
    int rc = llama3_set_config(m, cfg);
    if (rc) return rc;
    const Llama3Config &c = m->config;
    const int q_rows = c.n_q_heads * c.head_dim, kv_rows = c.n_kv_heads * c.head_dim;
    auto shape = [&](Tensor *t, int d0, int d1) {
        int r = set_shape(t, d0, d1);
        t->loaded = 1;
        t->file_dtype = bf16 ? 0 : 1;
        return r;
    };
    rc = shape(m->embed_tokens, c.vocab, c.d_model) | shape(m->lm_head, c.vocab, c.d_model) | shape(m->norm, c.d_model, 0);
    for (int i = 0; i < m->n_layers; ++i) {
        Llama3Layer *l = m->layers[i];
        rc |= shape(l->input_layernorm, c.d_model, 0) | shape(l->post_attention_layernorm, c.d_model, 0) |
              shape(l->self_attn_q_proj, q_rows, c.d_model) | shape(l->self_attn_k_proj, kv_rows, c.d_model) |
              shape(l->self_attn_v_proj, kv_rows, c.d_model) | shape(l->self_attn_o_proj, c.d_model, q_rows) |
              shape(l->mlp_gate_proj, c.ffn, c.d_model) | shape(l->mlp_up_proj, c.ffn, c.d_model) |
              shape(l->mlp_down_proj, c.d_model, c.ffn);
    }
    if (rc) return LLMB_ERR_INVALID;
    if ((rc = derive_config(m))) return rc;
    if ((rc = check_tp(m))) return rc;
    if ((rc = place_tensors(m))) return rc;
    const int rank = m->tp_rank, size = m->tp_size;
    size_t max_elems = 0;
    for_each_tensor(m, [&](Tensor *t, int layer, int slot) {
        const size_t n = shard_of(t, layer, slot, rank, size).elems();
        if (n > max_elems) max_elems = n;
    });
    void *staging = nullptr;
    if (bf16) LLMB_CUDA_OK(cudaMalloc(&staging, max_elems * 2));
    int status = LLMB_OK;
    for_each_tensor(m, [&](Tensor *t, int layer, int slot) {
        if (status) return;
        const Shard sh = shard_of(t, layer, slot, rank, size);
        const uint64_t n = sh.elems();
        const bool is_norm = (layer < 0 && slot == LLMB_SID_NORM) ||
                             (layer >= 0 && (slot == LLMB_SLOT_INPUT_LAYERNORM || slot == LLMB_SLOT_POST_LAYERNORM));
        const uint64_t sid = layer < 0 ? (uint64_t)slot : LLMB_LAYER_SID(layer, slot);
        uint16_t *dst = reinterpret_cast<uint16_t *>(t->d_fp16_tensor);
        // element (r, c) of the shard is element (row0 + r) * full_cols + col0 + c of the whole tensor
        const uint64_t first = (uint64_t)sh.row0 * sh.full_cols + sh.col0;
        int r;
        if (is_norm) {
            r = llmb_fill_u16(dst, 0x3C00, n, nullptr);  // gain 1.0
        } else if (bf16) {
            r = llmb_synth_2d(static_cast<uint16_t *>(staging), seed, sid, 0.02f, 1, first, sh.full_cols, sh.rows, sh.cols,
                              nullptr);
            if (!r) r = llmb_bf16_to_fp16(static_cast<const uint16_t *>(staging), dst, n, nullptr);
        } else {
            r = llmb_synth_2d(dst, seed, sid, 0.02f, 0, first, sh.full_cols, sh.rows, sh.cols, nullptr);
        }
        if (r) status = r;
        set_local_shape(t, sh);
    });
    cudaError_t e = cudaDeviceSynchronize();
    if (staging) cudaFree(staging);
    if (!status && e != cudaSuccess) status = cuda_fail(e, __FILE__, __LINE__);
    return status;
}
