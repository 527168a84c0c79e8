/*
 * Host surface of the engine: the reference's own model/cache structs and entry points
 * (abhisheknair10/LLM.cu src/llama3/llama3.cuh, src/safetensor/safetensor.cuh,
 * src/inference/inference.cuh, src/tokenizer/tokenizer.cuh), re-implemented on top of the
 * sm_100a kernels of llm_b200.h.  A driver written against the reference (src/main.cu:61-126)
 * compiles against this header and links libllm_b200.so instead of the reference's objects.
 *
 * Differences a caller can see:
 *  - dimensions are no longer literals: they are derived from the tensor shapes at to_cuda()
 *    and can be completed with llama3_set_config() (head_dim, rope_theta, eps, max_seq);
 *  - inference() keeps a per-layer KV cache, so a call costs one token, not the whole
 *    sequence (the reference recomputes every row each call, inference.cu:153-188);
 *  - inference() returns the greedy argmax computed on the device (the reference samples with
 *    temperature/top-p on the host, inference.cu:1030-1039); the FP16 logits are still left in
 *    Cache->h_token_probdist / d_token_probdist (inference.cu:1021-1025);
 *  - every entry point has an int-status twin (llama3_*): the reference-named void functions
 *    print and exit(1) as the reference does, the twins return an LLMB_ERR_* code.
 * All functions have C linkage.
 */
#ifndef LLM_B200_LLAMA3_H
#define LLM_B200_LLAMA3_H

#include <stdint.h>

#include "llm_b200.h"

#if defined(__CUDACC__) || defined(LLMB_HAVE_CUDA_FP16)
#include <cuda_fp16.h>
typedef __half llmb_half;
#else
typedef uint16_t llmb_half;
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* llama3.cuh:10-23.  The first ten fields are the reference's, in its order. */
typedef struct {
    /* host */
    int *ndim;
    int *mem_len;
    int *shape;
    uint16_t *bf16_tensor; /* payload as read from the file; freed by to_cuda */
    /* device */
    int *d_ndim;
    int *d_mem_len;
    int *d_shape;
    uint16_t *d_bf16_tensor;
    llmb_half *d_fp16_tensor;
    /* additions */
    int file_dtype;     /* 0 = BF16 (converted at load), 1 = F16 (passed through) */
    int device_is_view; /* d_fp16_tensor points into a fused buffer owned by another tensor */
    int loaded;
} Tensor;

/* llama3.cuh:28-39 */
typedef struct {
    int layernum;
    Tensor *input_layernorm;
    Tensor *mlp_down_proj;
    Tensor *mlp_gate_proj;
    Tensor *mlp_up_proj;
    Tensor *post_attention_layernorm;
    Tensor *self_attn_k_proj;
    Tensor *self_attn_o_proj;
    Tensor *self_attn_q_proj;
    Tensor *self_attn_v_proj;
} Llama3Layer;

/* The reference has no config struct: every dimension is a literal in inference.cu. */
typedef struct {
    int d_model;    /* 4096  (inference.cu:212) */
    int n_q_heads;  /* 32    (inference.cu:700) */
    int n_kv_heads; /* 8     (inference.cu:752: group of 4) */
    int head_dim;   /* 128   (inference.cu:673, 710) */
    int ffn;        /* 14336 */
    int vocab;      /* 128256 (inference.cu:24) */
    int max_seq;    /* 2048  (inference.cu:122-124): KV-cache rows per layer */
    float rope_theta; /* 500000 (inference.cu:673) */
    double eps;       /* 1e-5, a double literal in the reference (inference.cu:351) */
} Llama3Config;

/* llama3.cuh:44-50 plus the additions after n_layers. */
typedef struct {
    Tensor *embed_tokens;
    Tensor *lm_head;
    Tensor *norm;
    Llama3Layer **layers;
    int n_layers;
    /* additions */
    Llama3Config config;
    int config_ready; /* set by to_cuda once shapes are known */
    int tp_rank, tp_size;
    void *priv; /* fused device buffers */
} Llama3;

/* inference.cuh:19-34.  Same field names; K and V now hold the per-layer KV cache
 * ([n_layers * max_seq][n_kv_heads * head_dim], K stored post-RoPE) instead of one layer's
 * scratch, and the N x N score buffer is never allocated. */
typedef struct {
    Tensor *PN_X; /* unused by the fused kernels (residual add happens in the epilogues); kept NULL */
    Tensor *Q;    /* [1][n_q_heads * head_dim] query row of the current token */
    Tensor *K;
    Tensor *V;
    float *d_attention_score_cache;          /* always NULL */
    llmb_half *d_feedforward_cache_upgate;   /* [ffn] SwiGLU output of the current token */
    llmb_half *d_token_probdist;             /* [vocab] FP16 logits on the device */
    llmb_half *h_token_probdist;             /* [vocab] FP16 logits on the host (pinned) */
    float *f_token_probdist;                 /* [vocab] host scratch, kept for callers that sample */
    /* additions */
    void *priv;
} CudaCache;

/* ---- reference-named entry points ------------------------------------------------------- */
Llama3 *init_llama3(int n_layers);                                      /* llama3.cuh:58 */
void free_llama3(Llama3 *llama3);                                       /* llama3.cuh:68 */
void _free_tensor(Tensor *tensor);                                      /* llama3.cuh:77 */
void load_safetensor_weights(Llama3 *llama3_model, const char *filename); /* safetensor.cuh:26 */
void to_cuda(Llama3 *llama3);                                           /* llama3.cuh:86 */
CudaCache *init_cache(Llama3 *llama3_model);                            /* inference.cuh:447 */
int *tokens_to_cuda(int *tokens, int embed_size, Tensor *token_tensor); /* tokenizer.cuh:66 */
/* inference.cuh:71.  h_tokens[0] = count + 1, ids in h_tokens[1..count] (tokenizer.cu:143-152).
 * Processes the tokens not yet in the KV cache (all of them on the first call, one per call
 * afterwards), returns the greedy next token id, or a negative LLMB_ERR_* code.  X and
 * d_tokens are the buffers tokens_to_cuda() returned. */
int inference(Llama3 *llama3_model, Tensor *X, int *d_tokens, int *h_tokens, CudaCache *Cache);

/* ---- status-returning twins and additions ----------------------------------------------- */
int llama3_set_config(Llama3 *m, const Llama3Config *cfg); /* fields <= 0 keep their default */
int llama3_set_tp(Llama3 *m, int tp_rank, int tp_size);
int llama3_load_safetensors(Llama3 *m, const char *filename);
/* Loading streams by default: load_safetensor_weights() parses the header and records where each payload
 * lies; to_cuda() then reads this rank's window of every tensor straight from the file into two pinned
 * staging buffers (32 MB each) and overlaps the read of one chunk with the upload and BF16 -> FP16
 * conversion of the previous one, so the host never holds the model.  enable = 0 restores the reference's
 * behaviour (safetensor.cu:140-155): every payload is read into Tensor::bf16_tensor at load and kept
 * until to_cuda().  Call before loading. */
int llama3_set_streaming(Llama3 *m, int enable);
/* Figures of the last to_cuda(): wall seconds, bytes read from the shard files, bytes copied to the
 * device, and the pinned host memory it used.  Any pointer may be NULL. */
int llama3_upload_stats(Llama3 *m, double *seconds, unsigned long long *bytes_read, unsigned long long *bytes_uploaded,
                        unsigned long long *host_staging_bytes);
/* The window {row0, rows, col0, cols, full_cols} of a loaded tensor that this model's
 * tensor-parallel rank keeps: q/k/v, gate/up and lm_head split by rows, o_proj and down_proj by
 * columns, everything else whole.  layer = -1, slot 1/2/3 = embed_tokens/lm_head/norm; otherwise
 * slot is the position of the tensor in Llama3Layer (0 = input_layernorm ... 8 = v_proj). */
int llama3_tensor_shard(Llama3 *m, int layer, int slot, int out[5]);
int llama3_to_cuda(Llama3 *m);
/* Random-init model written directly in device memory with the seeded generator of
 * llm_b200_synth.h (std 0.02, norm gains 1.0), BF16 then converted by the load-time kernel
 * (bf16 != 0) or FP16 drawn directly (bf16 == 0).  cfg must be complete. */
int llama3_synth_weights(Llama3 *m, const Llama3Config *cfg, uint64_t seed, int bf16);
CudaCache *llama3_init_cache(Llama3 *m, int *status_out);
void free_cache(CudaCache *cache);
/* Forget the cached sequence (next inference() call starts a new one). */
int cache_reset(CudaCache *cache);
/* Switches: use_graph (capture each decode step into a CUDA graph, default 1), use_pdl
 * (programmatic dependent launch between kernels, default 1), copy_logits (device->host copy
 * of the logits on every call, default 1). Negative value = leave unchanged. */
int cache_set_options(CudaCache *cache, int use_graph, int use_pdl, int copy_logits);
/* Chooses between the two decode paths: 1 (default where the device allows a cooperative launch)
 * = one persistent kernel per token (llmb_decode_step); 0 = one kernel per fused operation,
 * captured into a CUDA graph (llmb_gemv_f16, llmb_attn_decode, ...). */
int cache_use_step_kernel(CudaCache *cache, int enable);
/* Spin limit of the step kernel's waits for tensor-parallel peers (0 = default, about a second): a rank
 * whose peer does not deliver within it gives up with LLMB_ERR_TIMEOUT instead of waiting on. */
int cache_set_tp_poll_limit(CudaCache *cache, unsigned int tag_poll_limit);
/* Tensor parallel decode, one process per GPU (llama3_set_tp before loading): each rank exports a
 * 64-byte CUDA IPC handle of its exchange block with cache_tp_handle(); the caller gathers all
 * ranks' handles in rank order (torch.distributed, MPI, ...) and passes the tp_size * 64 bytes to
 * cache_tp_connect().  Every rank then calls inference()/inference_greedy() with the same tokens.
 * Cache->d_token_probdist / h_token_probdist hold this rank's slice of the vocabulary
 * (rows [rank * vocab / tp_size, (rank + 1) * vocab / tp_size)).
 * The ranks wait for one another inside the step kernel with a bounded spin of a few seconds; a
 * rank that enters a step much later than its peers makes them give up (llmb_device_status 205),
 * so keep the ranks in lock-step on the host (a barrier after any long rank-local work). */
int cache_tp_handle(CudaCache *cache, void *handle_out /* 64 bytes */);
int cache_tp_connect(CudaCache *cache, const void *handles /* tp_size * 64 bytes */);
/* When enabled, every decode step also copies the residual stream after the embedding and
 * after each layer into an [n_layers + 1][d_model] FP16 device buffer (disables the graph). */
int cache_enable_hidden_dump(CudaCache *cache, int enable);
int cache_read_hidden(CudaCache *cache, uint16_t *h_out /* [n_layers+1][d_model] */);
/* Device-resident greedy generation: prefill `n_prompt` ids, then generate `n_new` tokens with
 * the sampled token fed back on the device (no host round trip per token).
 * out_tokens[n_new]; prefill_ms / decode_ms (optional) are CUDA-event times. */
int inference_greedy(Llama3 *m, CudaCache *cache, const int *prompt, int n_prompt, int n_new, int *out_tokens,
                     float *prefill_ms, float *decode_ms);
/* Continues a greedy run for n_steps more tokens from the state inference_greedy() (or a previous
 * inference_continue) left: the last sampled token is fed back on the device.  out_tokens[n_steps];
 * ms (optional) is the CUDA-event time of the n_steps steps. */
int inference_continue(Llama3 *m, CudaCache *cache, int n_steps, int *out_tokens, float *ms);
/* Test aid: copies an internal device buffer to the host (0 = residual row x, 1 = second residual
 * buffer, 2 = q, 3 = attention output, 4 = SwiGLU output h, 5 = this rank's exchange block). */
int cache_debug_read(CudaCache *cache, int which, void *out, size_t bytes);
/* Profiling aid: makes the step kernel record per-phase timestamps of every CTA; read with
 * cache_debug_read(cache, 6, ...) as [SM count][5 * n_layers + 2][8] uint64 nanoseconds
 * (consumers: entered, dependency met, input ready, done; finisher: started, first stage, last
 * stage, fenced). */
int cache_debug_trace(CudaCache *cache, int enable);
/* Prompt phase.  By default a run of >= 16 new prompt tokens goes through the block path: all but
 * the last token as blocks of up to 1024 rows (tensor-core projections, block attention), the last
 * one through the decode step for its logits.  enable = 0 feeds every prompt token through the
 * decode step instead; min_rows > 0 changes the threshold.  The block path needs the whole model
 * on this GPU (tp_size 1) and projection widths that are multiples of 128; otherwise the decode
 * step is used.  The reference runs its layer loop over all rows on every call
 * (inference.cu:157-186). */
int cache_set_prefill(CudaCache *cache, int enable, int min_rows);
/* Samples the next token from the logits the last inference() call left in
 * Cache->h_token_probdist, the way the reference's inference() does on the host
 * (sample_next_token, inference.cu:1030-1039; its constants are temperature 0.7, top-k 50,
 * top-p 0.9).  `draw` numbers the call (one uniform per call from `seed`).  Returns the token, or a
 * negative status.  The caller appends the token to its array and calls inference() again, as
 * src/main.cu:121-122 does; the engine then feeds just that token. */
int cache_sample_next_token(CudaCache *cache, float temperature, int top_k, float top_p, uint64_t seed, uint64_t draw);
/* The same sampling done by one kernel on the device logits (llmb_sample_logits): nothing but the 4-byte
 * token crosses to the host, so inference() can run with copy_logits off.  The token also replaces the
 * greedy one in the device history (inference_continue() then continues from it).  Returns the token, or a
 * negative status: -LLMB_ERR_UNSUPPORTED when top_k (after clamping to the vocabulary) exceeds 1024 or the
 * top-p prefix runs past 1024 entries; cache_sample_next_token() takes such a step. */
int cache_sample_next_token_device(CudaCache *cache, float temperature, int top_k, float top_p, uint64_t seed, uint64_t draw);
/* Batched decode: n_seqs independent sequences that advance one token per step, the m = n_seqs rows of a
 * step going through the tensor-core projections so that every weight byte is streamed once per step
 * (the reference's projections are m-row GEMMs too: inference.cu:393-449).  Each sequence has its own
 * KV cache of config.max_seq rows: K, V [n_layers][n_seqs][max_seq][n_kv].  Needs tp_size 1.
 *   cache_batch_init     allocates the batch state (n_seqs <= 128); the single-sequence state is untouched
 *   cache_batch_prefill  tokens [n_seqs][n_tokens]: all but the last token of every sequence go into its
 *                        cache as blocks of rows; the last one becomes the input of the next step
 *   cache_batch_step     one step; tokens (optional [n_seqs]) replaces the inputs (teacher forcing), else the
 *                        tokens sampled by the previous step are fed; h_logits (optional [n_seqs][vocab] FP16
 *                        bits) and next_tokens (optional [n_seqs]) receive the step's results
 *   cache_batch_greedy   n_steps steps with the greedy tokens fed back on the device, no host round trip;
 *                        out_tokens [n_seqs][n_steps], ms = CUDA-event time of the steps */
int cache_batch_init(CudaCache *cache, int n_seqs);
/* Cache rows per attention CTA of the batched step (a power of two, 32..512; default 256). */
int cache_batch_set_split_len(CudaCache *cache, int split_len);
int cache_batch_prefill(CudaCache *cache, const int *tokens, int n_tokens);
int cache_batch_step(CudaCache *cache, const int *tokens, uint16_t *h_logits, int *next_tokens);
int cache_batch_greedy(CudaCache *cache, int n_steps, int *out_tokens, float *ms);
/* Profiling aid for the batched step: enable = 1 arms per-CTA nanosecond stamps of its small-M projections
 * (LlmbGemmArgs.trace; projection j of a step, 5 per layer then lm_head, at [j][1024][8] uint64); enable = 0
 * copies the (5 * n_layers + 1) * 1024 * 8 uint64 to out (optional) and disarms. */
int cache_debug_rows_trace(CudaCache *cache, int enable, uint64_t *out);
/* Number of kernels launched (or replayed through graphs) by this cache's stream so far. */
long long cache_kernel_launches(const CudaCache *cache);

#ifdef __cplusplus
}
#endif
#endif /* LLM_B200_LLAMA3_H */
