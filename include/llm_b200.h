/*
 * llm_b200: C-ABI of the sm_100a kernels behind the LLaMA3 per-token forward loop.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream and returns an int status (0 = ok).  No entry point
 * allocates device memory unless its comment says so.  FP16 and BF16 data travel as
 * uint16_t bit patterns so that the header needs no CUDA include.
 *
 * Each declaration cites the part of the reference engine (abhisheknair10/LLM.cu, paths
 * relative to its root) that it replaces.
 */
#ifndef LLM_B200_H
#define LLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *llmb_stream_t; /* a cudaStream_t */

enum {
    LLMB_OK = 0,
    LLMB_ERR_INVALID = 1,     /* bad argument (null pointer, unsupported shape, misalignment) */
    LLMB_ERR_CUDA = 2,        /* a CUDA runtime call failed; see llmb_last_error() */
    LLMB_ERR_TIMEOUT = 3,     /* a bounded device-side wait ran out (llmb_device_status) */
    LLMB_ERR_UNSUPPORTED = 4, /* valid request that this build has no kernel for */
    LLMB_ERR_IO = 5,          /* file missing, truncated or malformed */
    LLMB_ERR_NOMEM = 6
};

/* Text of the most recent failure on the calling thread ("" if none). */
const char *llmb_last_error(void);

/* Reads and clears the per-device status word kernels set when a bounded wait gives up.
 * Synchronises the device. */
int llmb_device_status(int *status_out);

/* Library build identification: "sm_100a" and the kernels compiled in. */
const char *llmb_build_info(void);

/* ------------------------------------------------------------------------------------ */
/* Load-time conversion.  Replaces _kernel_bf16_to_fp16 (src/llama3/llama3.cu:240-254):  */
/* fp16 = RN(fp32(bf16 << 16)).  128-bit loads and stores; n elements.                   */
/* ------------------------------------------------------------------------------------ */
int llmb_bf16_to_fp16(const uint16_t *d_bf16, uint16_t *d_fp16, size_t n, llmb_stream_t stream);

/* Seeded synthetic BF16/FP16 weights written directly in device memory
 * (include/llm_b200_synth.h defines the stream).  Benchmark and test support: the reference
 * ships no weights (model_weights/README.md). */
int llmb_synth_bf16(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n,
                    llmb_stream_t stream);
int llmb_synth_fp16(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, uint64_t first, uint64_t n,
                    llmb_stream_t stream);
/* A rows x cols window of a stream: out[r][c] = element first + r * row_stride + c, so that a
 * tensor-parallel shard of a seeded tensor has the same bits as that slice of the whole tensor. */
int llmb_synth_2d(uint16_t *d_out, uint64_t seed, uint64_t sid, float std, int bf16, uint64_t first, uint64_t row_stride,
                  uint64_t rows, uint64_t cols, llmb_stream_t stream);
int llmb_fill_u16(uint16_t *d_out, uint16_t value, uint64_t n, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Step prologue.  Replaces tokens_to_embeddings / kernel_tokens_to_embeddings           */
/* (src/inference/inference.cu:196-223) for the rows processed in this call, and          */
/* precomputes the RoPE angles kernel_rope_scaling (inference.cu:640-695) would derive     */
/* per element: cs[row][i] = (cosf, sinf)(pos * theta^(-2i/head_dim)), FP32.               */
/*   tokens   : device int32 ids: row r uses tokens[r], or tokens[pos[r]] when              */
/*              tokens_by_pos != 0 (tokens is then the sequence history, so a captured      */
/*              step can be replayed while only pos advances)                              */
/*   pos      : device int32 position of each row                                         */
/*   x        : out, [n_rows][d_model] FP16                                               */
/*   rope_cs  : out, [n_rows][head_dim/2][2] FP32                                         */
/* ------------------------------------------------------------------------------------ */
int llmb_embed_rope(const uint16_t *d_embed, const int32_t *d_tokens, const int32_t *d_pos, int n_rows, int d_model,
                    int vocab, int head_dim, float rope_theta, uint16_t *d_x, float *d_rope_cs,
                    int tokens_by_pos, int use_pdl, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Batch-1 projections: y = W x with W [n][k] FP16 row-major (as the checkpoint stores it) */
/* and FP32 accumulation.  One bandwidth-bound kernel replaces kernel_standard_tiled_gemm  */
/* at m = 1 (inference.cu:393-449) together with the element-wise kernels around it:       */
/*                                                                                         */
/*  prologue LLMB_PRO_RMSNORM  kernel_compute_rms_norm (inference.cu:293-363): x is the    */
/*                             residual stream and is normalised on the fly,               */
/*                             half((x*g)/sqrtf(eps + sum(x^2)/k)), same FP32 summation    */
/*                             tree as the reference when k/4 is a power of two            */
/*  epilogue LLMB_EPI_STORE    y[n] = half(acc)                         (inference.cu:445) */
/*           LLMB_EPI_RESIDUAL y[n] = half(float(half(acc)) + float(y[n]))                 */
/*                             = GEMM + kernel_add_norm (inference.cu:377-390), in place   */
/*           LLMB_EPI_ROPE_KV  rows [0,n_q) -> RoPE -> q; rows [n_q,n_q+n_kv) -> RoPE ->   */
/*                             K cache row `pos`; rest -> V cache row `pos`                 */
/*                             = compute_qkv_tensors + rope_scaling (inference.cu:561-695)  */
/*           LLMB_EPI_SWIGLU   y[n] = half(SiLU(acc_gate) * acc_up), w = gate, w2 = up      */
/*                             = kernel_standard_tiled_gemm_ffn_swiglu (inference.cu:455)   */
/* ------------------------------------------------------------------------------------ */
enum { LLMB_PRO_NONE = 0, LLMB_PRO_RMSNORM = 1 };
enum { LLMB_EPI_STORE = 0, LLMB_EPI_RESIDUAL = 1, LLMB_EPI_ROPE_KV = 2, LLMB_EPI_SWIGLU = 3, LLMB_EPI_TP_SCATTER = 4 };

typedef struct {
    const uint16_t *w;     /* [n][k] FP16 */
    const uint16_t *w2;    /* SWIGLU only: up projection [n][k] */
    const uint16_t *x;     /* [k] FP16 input row */
    uint16_t *y;           /* output row (meaning depends on the epilogue), n or n_q elements */
    int n;                 /* output rows of w (for ROPE_KV: n_q + 2 * n_kv) */
    int k;                 /* multiple of 8, at most 16384 */
    int prologue;
    const uint16_t *gamma; /* RMSNORM: [k] FP16 gain */
    double eps;            /* RMSNORM: added in double as the reference does (1e-5) */
    int epilogue;
    /* ROPE_KV */
    int n_q;               /* query rows (n_q_heads * head_dim) */
    int n_kv;              /* key rows = value rows (n_kv_heads * head_dim) */
    int head_dim;
    const float *rope_cs;  /* [head_dim/2][2] (cos, sin) of this row's position */
    uint16_t *k_cache;     /* this layer's and sequence's K rows: [max_pos][n_kv] FP16 */
    uint16_t *v_cache;
    const int32_t *pos;    /* device: row index to write in the cache */
    int max_pos;
    int use_pdl;           /* launch with programmatic stream serialization */
} LlmbGemvArgs;

int llmb_gemv_f16(const LlmbGemvArgs *args, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Decode attention over the KV cache for one new token per sequence.  Replaces           */
/* compute_attention and its three kernels (inference.cu:698-947) for the last row:        */
/* scores (q.k)/sqrtf(head_dim) in FP32 from FP16, softmax in FP32, P.V in FP32, FP16 out; */
/* the N x N score matrix is never materialised.  The KV sequence is split across CTAs;    */
/* partial (max, sum, out) triples go through `scratch` and the last CTA of each KV head   */
/* merges them.                                                                            */
/*   q        : [n_q_heads][head_dim] FP16 (post-RoPE)                                     */
/*   k_cache  : [max_pos][n_kv_heads][head_dim] FP16 (post-RoPE), positions 0..pos valid   */
/*   out      : [n_q_heads][head_dim] FP16                                                 */
/*   scratch  : llmb_attn_decode_scratch_bytes() bytes, 256-byte aligned; the first         */
/*              n_kv_heads int32 counters must be zero before the first call (the kernel    */
/*              leaves them zero)                                                          */
/* ------------------------------------------------------------------------------------ */
size_t llmb_attn_decode_scratch_bytes(int n_q_heads, int n_kv_heads, int head_dim, int n_splits);
int llmb_attn_decode(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, const int32_t *d_pos,
                     int n_q_heads, int n_kv_heads, int head_dim, int n_splits, int split_len, uint16_t *d_out,
                     void *d_scratch, int use_pdl, llmb_stream_t stream);

/* Batched decode: one new token for each of n_seqs sequences in one launch.  With 2..256 sequences */
/* the launch is one wave of CTAs that share the 64-row tiles of all (sequence, KV head) pairs      */
/* evenly, whatever the mix of lengths (read from pos on the device, so a captured launch stays      */
/* valid as the sequences grow); a pair is cut into at most n_splits + 1 pieces of at least         */
/* split_len rows, merged in piece order by the last CTA of the pair to finish.                      */
/*   q, out   : [n_seqs][n_q_heads * head_dim];  pos : device [n_seqs], position of each new token  */
/*   k_cache  : [n_seqs][seq_stride_rows][n_kv_heads * head_dim] (this layer), likewise v_cache      */
/*   n_splits * split_len must cover the longest sequence; scratch as below, counters zero.          */
/* Replaces compute_attention (inference.cu:698-947) for the last row of each sequence.               */
size_t llmb_attn_decode_batch_scratch_bytes(int n_seqs, int n_q_heads, int n_kv_heads, int head_dim, int n_splits);
int llmb_attn_decode_batch(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                           const int32_t *d_pos, int n_seqs, size_t seq_stride_rows, int n_q_heads, int n_kv_heads,
                           int head_dim, int n_splits, int split_len, uint16_t *d_out, void *d_scratch, int use_pdl,
                           llmb_stream_t stream);

/* Profiling aid: the following launches of the decode attention record per-CTA nanosecond stamps (entry,    */
/* previous kernel complete, first tile landed, tiles done, partial published, merge done - of the CTA's last  */
/* piece) and the SM cycles its thread 0 spent waiting for tiles and using them, into d_trace: 8 uint64 per    */
/* CTA, CTA index = (seq * n_kv_heads + kv_head) * n_splits + split for one sequence, the CTA's number in the  */
/* one-wave grid for several (room for 8 x max(that, resident CTAs) entries).  NULL (default) = off.           */
int llmb_attn_decode_trace(void *d_trace);

/* The same attention for callers that may not allocate device memory (a host whose own pool  */
/* owns the device, a loop that cannot afford an allocation's synchronisation, a plug-in that  */
/* only ever sees its input and output buffers): no workspace argument, the partial results     */
/* live in a fixed 2,130,176-byte array inside the library.  No counterpart in the reference,   */
/* which allocates every buffer with cudaMalloc in init_cache (inference.cu:101-145).           */
/* Limits: n_q_heads * n_splits <= 4096, head_dim <= 128, n_kv_heads <= 64; larger requests     */
/* return LLMB_ERR_UNSUPPORTED.  The first call on each device resolves the array's address and  */
/* should be made before any stream capture begins; if the library's device code is not yet     */
/* resident on that device, that first call is also what makes the CUDA runtime load it (array   */
/* and kernels), so make it at start-up.  Calls on one device share the array: calls that may    */
/* run concurrently on the GPU race.  Calls no cudaMalloc, cudaFree or allocating routine.       */
int llmb_attn_decode_static(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache,
                            const int32_t *d_pos, int n_q_heads, int n_kv_heads, int head_dim, int n_splits,
                            int split_len, uint16_t *d_out, int use_pdl, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Greedy sampling on the device: index of the first maximum of n FP16 logits (NaN never   */
/* wins).  Replaces the host sampler sample_next_token (inference.cu:1030-1161) for greedy */
/* decoding.  Also advances the step state so a captured step can be replayed without the   */
/* host: token_out[0] = argmax; if pos_inout != NULL, (*pos_inout)++;                       */
/* if history != NULL, history[*pos_inout (after increment)] = argmax.                     */
/* ------------------------------------------------------------------------------------ */
int llmb_argmax_f16(const uint16_t *d_logits, int n, int32_t *d_token_out, int32_t *d_pos_inout,
                    int32_t *d_history, int history_len, int use_pdl, llmb_stream_t stream);

/* The same for `rows` rows of logits ([rows][n], n a multiple of 8), one CTA per row:                 */
/* token_out[r] = argmax of row r; pos_inout[r]++ (if not NULL); history[r * history_len + pos] = it.   */
int llmb_argmax_rows_f16(const uint16_t *d_logits, int n, int rows, int32_t *d_token_out, int32_t *d_pos_inout,
                         int32_t *d_history, int history_len, int use_pdl, llmb_stream_t stream);

/* position += 1 without sampling (prompt rows whose logits nobody reads). */
int llmb_advance_pos(int32_t *d_pos, int use_pdl, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Prompt phase: M rows at once.                                                          */
/*                                                                                        */
/* llmb_gemm_f16: C[m][n] = A[m][k] . B[n][k]^T on the tensor cores (tcgen05.mma, FP32      */
/* accumulators in tensor memory, operands staged by TMA).  Replaces                        */
/* kernel_standard_tiled_gemm (inference.cu:393-449) and, with LLMB_EPI_SWIGLU,             */
/* kernel_standard_tiled_gemm_ffn_swiglu (inference.cu:455-519) for m > 1 rows.  Epilogues, */
/* with the reference's FP16 rounding points:                                               */
/*   LLMB_EPI_STORE     c = half(acc)                                                        */
/*   LLMB_EPI_RESIDUAL  c = half(float(half(acc)) + float(c))          (inference.cu:377-390) */
/*   LLMB_EPI_ROPE_KV   n = n_q + 2 n_kv: RoPE on q and k with rope_cs[row], q -> c [m][n_q], */
/*                      k, v -> cache row pos0 + row                     (inference.cu:640-695) */
/*   LLMB_EPI_SWIGLU    c = half(SiLU(A.b^T) * (A.b2^T)), accumulators not rounded  (:515)     */
/* n must be a multiple of 128, k of 64; a, b, c 16-byte aligned; m is free (rows past m are   */
/* zero-filled on load and never stored).  With m <= 32 (and tile_n 0) the launch is a weight  */
/* stream: the weight tile is the 128-row MMA operand, the m rows the 32-column one, K is split */
/* until two CTAs per SM stream weights (the slices of a tile are one thread-block cluster and   */
/* add their partial sums through distributed shared memory: no workspace), bound by HBM like   */
/* llmb_gemv_f16.                                                                                */
/* ------------------------------------------------------------------------------------ */
typedef struct {
    const uint16_t *a;     /* [m][k] FP16 activations */
    const uint16_t *b;     /* [n][k] FP16 weights */
    const uint16_t *b2;    /* SWIGLU: the up projection [n][k] */
    uint16_t *c;           /* [m][n]; ROPE_KV: [m][n_q] */
    int m, n, k;
    int epilogue;
    int n_q, n_kv, head_dim;
    const float *rope_cs;  /* [m][head_dim/2][2] from llmb_embed_rope */
    uint16_t *k_cache;     /* [max_pos][n_kv] of this layer */
    uint16_t *v_cache;
    int pos0;              /* cache row of A's row 0 */
    int max_pos;
    int tile_n;            /* output columns per CTA: 0 = the widest of 128/64/32 that fills the SMs */
    void *workspace;       /* m > 32 only. Optional, 16-byte aligned, its first 4096 bytes zero before the first use (the */
    size_t workspace_bytes;/* kernel leaves them zero): lets a launch with few output tiles split K across     */
                           /* CTAs; partial sums are added in slice order.  One launch at a time per workspace; */
                           /* 4096 + SMs * 131072 bytes always suffice.                                        */
    const int32_t *row_pos;/* ROPE_KV, batched decode (one new row per sequence): device [m] cache position of   */
    int seq_stride;        /* each row; row r then goes to cache row r * seq_stride + row_pos[r] (sequence r of a */
                           /* [n_seqs][seq_stride][n_kv] cache), and pos0 is ignored.  NULL = rows pos0, pos0+1.. */
    int use_pdl;           /* m <= 32 only: launch with programmatic stream serialization; the kernel then starts  */
                           /* its weight stream while the previous kernel of the stream is still finishing and     */
                           /* waits for it (griddepcontrol.wait) before it reads a or writes anything              */
    /* LLMB_EPI_TP_SCATTER (m <= 32 only): tensor parallel, row-parallel projection (o_proj, down_proj: this rank  */
    /* holds a slice of K).  The FP32 partial sums are not stored in c: every element goes, as an 8-byte           */
    /* (value, tag) pair, straight into every rank's exchange block over NVLink (peer stores), where                */
    /* llmb_tp_gather_rows adds the ranks' partials.  tp_peers[r] = rank r's block as mapped on this device;         */
    /* tp_index = number of this exchange within the step (selects one of two receive buffers and the tag).         */
    void *tp_peers[8];
    int tp_rank, tp_size, tp_index;
    uint64_t *trace;       /* optional profiling aid (m <= 32 only): device [CTAs][8] nanosecond stamps per CTA (entry,  */
                           /* set up, previous kernel complete, first stage landed, last MMA issued, accumulators        */
                           /* complete, partials published, epilogue done); CTA index = slice * tiles + tile.  NULL in   */
                           /* production.                                                                                */
} LlmbGemmArgs;

int llmb_gemm_f16(const LlmbGemmArgs *args, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Tensor parallel, rows at once (m <= 32): the other half of the all-reduce that                */
/* LLMB_EPI_TP_SCATTER starts, fused with the residual add and the next RMSNorm.  One CTA per     */
/* row: polls (bounded) the tp_size tagged partial sums of every element in this rank's exchange  */
/* block, adds them in rank order (every rank gets the same bits),                                 */
/*   x[r][c] = half(float(half(sum)) + float(x[r][c]))     (inference.cu:445, :377-390)            */
/* and, if gamma != NULL, xn = RMSNorm(x) * gamma with the reference's reduction order              */
/* (inference.cu:293-363).  exchange = this rank's block of llmb_decode_step_exchange_bytes() bytes. */
/* llmb_tp_argmax_rows: the greedy token of every row from the ranks' vocabulary slices: local      */
/* first maximum, exchanged through tagged slots, every rank picks the same winner; pos and        */
/* history advance as in llmb_argmax_rows_f16.  llmb_tp_advance ends a step: the exchange counter   */
/* moves on by n_exchanges (2 * n_layers, + 1 if llmb_tp_argmax_rows ran).                          */
/* Replaces the NCCL all-reduce a tensor-parallel port of the reference would place after o_proj    */
/* and down_proj.                                                                                  */
/* ------------------------------------------------------------------------------------ */
int llmb_tp_gather_rows(void *d_exchange, int tp_size, int tp_index, uint16_t *d_x, const uint16_t *d_gamma, uint16_t *d_xn,
                        int m, int d, double eps, uint32_t poll_limit, int use_pdl, llmb_stream_t stream);
int llmb_tp_argmax_rows(void *const *d_peers, int tp_rank, int tp_size, int d_model, int tp_index, const uint16_t *d_logits,
                        int n_local, int vocab_offset, int rows, int32_t *d_token_out, int32_t *d_pos_inout,
                        int32_t *d_history, int history_len, uint32_t poll_limit, int use_pdl, llmb_stream_t stream);
int llmb_tp_advance(void *d_exchange, int tp_size, int d_model, int n_exchanges, int use_pdl, llmb_stream_t stream);

/* RMSNorm of m rows of d FP16 values: y = half(x * gamma / rms(x)), the reduction order and  */
/* rounding of kernel_compute_rms_norm / kernel_compute_norm_tensor (inference.cu:272-375).    */
int llmb_rmsnorm_rows(const uint16_t *d_x, const uint16_t *d_gamma, uint16_t *d_y, int m, int d, double eps,
                      llmb_stream_t stream);

/* Causal attention of m new rows (positions pos0 .. pos0 + m - 1, whose K/V rows are already   */
/* in the cache) over cache rows 0 .. pos0 + row.  Replaces compute_attention                    */
/* (inference.cu:698-947) for a block of rows; same arithmetic as llmb_attn_decode.              */
/*   q, out : [m][n_q_heads * head_dim] FP16;  head_dim 64 or 128                                */
int llmb_attn_prefill(const uint16_t *d_q, const uint16_t *d_k_cache, const uint16_t *d_v_cache, int m, int pos0,
                      int n_q_heads, int n_kv_heads, int head_dim, uint16_t *d_out, llmb_stream_t stream);

/* d_out[i] = first + i: the positions of a block of prompt rows for llmb_embed_rope. */
int llmb_iota_i32(int32_t *d_out, int first, int n, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* Host-side temperature / top-k / top-p sampling over the FP16 logits of a step: the        */
/* arithmetic of sample_next_token (inference.cu:1030-1161), which the reference runs on the  */
/* host after every step:                                                                     */
/*   t_i = expf(float(logit_i) / temperature); p_i = t_i / sum(t) (FP32, index order);        */
/*   order by p descending (ties: lower index first; the reference's qsort leaves ties         */
/*   unspecified); the first top_k entries are renormalised to sum 1 (the reference's top-k    */
/*   pass, whose own pick it discards); then the shortest prefix whose running sum reaches     */
/*   top_p is renormalised and the first entry whose running sum exceeds u is returned         */
/*   (entry 0 if none does).                                                                  */
/* Only the first top_k entries are ever ordered unless the prefix runs past them.             */
/* u in [0, 1) replaces the reference's unseeded rand() / RAND_MAX; llmb_sampler_uniform        */
/* gives a reproducible one from (seed, draw).  temperature > 0, 1 <= top_k, 0 < top_p <= 1.    */
/* Like the reference, no maximum is subtracted before expf: a logit / temperature above ~88   */
/* overflows, which is reported as LLMB_ERR_UNSUPPORTED instead of returning a token.           */
/* Pure host code: no device is touched.                                                      */
/* ------------------------------------------------------------------------------------ */
int llmb_sample_logits_host(const uint16_t *h_logits_fp16, int vocab, float temperature, int top_k, float top_p,
                            float u, int32_t *token_out);
float llmb_sampler_uniform(uint64_t seed, uint64_t draw);

/* The same chain on the device, over the FP16 logits a decode step left in device memory: one      */
/* kernel, no copy of the logits to the host.  u = llmb_sampler_uniform(seed, draw).  The sum of the */
/* t_i is a tree over threads and expf is CUDA's, so probabilities can differ from the host code's  */
/* by a few FP32 ulps; the token differs only if u lies that close to a boundary.  Orders at most    */
/* 1024 entries: top_k (after clamping to vocab) above that returns LLMB_ERR_UNSUPPORTED.            */
/*   scratch   : llmb_sample_scratch_bytes(vocab) bytes, 256-byte aligned; its first int32 is the     */
/*               result code of the last call: 0 ok, 1 expf overflow, 2 the top-p prefix ran past    */
/*               1024 entries (token_out is -1 in both cases: use the host sampler for that step)    */
/*   token_out : the sampled id; if pos and history are given, history[*pos] = id as well (the       */
/*               position the decode step has already advanced to: the next step then feeds it)     */
size_t llmb_sample_scratch_bytes(int vocab);
int llmb_sample_logits(const uint16_t *d_logits, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
                       uint64_t draw, void *d_scratch, int32_t *d_token_out, int32_t *d_pos, int32_t *d_history,
                       int history_len, int use_pdl, llmb_stream_t stream);

/* ------------------------------------------------------------------------------------ */
/* One whole decode step as a single persistent kernel: every phase of the reference's     */
/* inference() loop body (inference.cu:149-193) for one new row -- embedding row, per layer */
/* RMSNorm + QKV + RoPE + cache append, attention over the cache, o_proj + residual,        */
/* RMSNorm + SwiGLU FFN + residual, then final norm, lm_head and greedy argmax -- with the  */
/* weights of all projections streamed through one shared-memory ring across the phase      */
/* boundaries.  One CTA per SM, cooperative launch.  Same arithmetic and rounding points as  */
/* llmb_gemv_f16 / llmb_attn_decode.                                                        */
/*   history[pos] is the input token; with_logits != 0: logits[vocab], next_token[0] and     */
/*   history[pos + 1] are written; pos is advanced by one.                                   */
/*   scratch: llmb_decode_step_scratch_bytes() bytes, 256-byte aligned, zeroed once before   */
/*   the first launch and whenever llmb_device_status() reports a non-zero status.           */
/*   split_len must be a multiple of 32; n_splits * split_len >= pos + 1.                    */
/* ------------------------------------------------------------------------------------ */
typedef struct {
    const uint16_t *wqkv;   /* [(n_q + 2 n_kv)][d_model]: q, k, v rows back to back */
    const uint16_t *wo;     /* [d_model][n_q] */
    const uint16_t *wgate;  /* [ffn][d_model] */
    const uint16_t *wup;    /* [ffn][d_model] */
    const uint16_t *wdown;  /* [d_model][ffn] */
    const uint16_t *g_in;   /* input_layernorm gain [d_model] */
    const uint16_t *g_post; /* post_attention_layernorm gain [d_model] */
    uint16_t *k_cache;      /* [max_pos][n_kv] */
    uint16_t *v_cache;
} LlmbLayer;

typedef struct {
    const LlmbLayer *layers; /* device array [n_layers] */
    int n_layers, d_model, n_q_heads, n_kv_heads, head_dim, ffn, vocab, embed_rows, max_pos;
    float rope_theta;
    double eps;
    const uint16_t *embed, *lm_head, *g_final;
    const int32_t *history; /* device: token ids by position; history[pos + 1] is written */
    int history_len;
    int32_t *pos;           /* device: rows already in the cache = position of this token */
    uint16_t *x, *q, *attn, *h, *logits; /* [d_model], [n_q], [n_q], [ffn], [vocab] */
    int32_t *next_token;
    void *scratch;
    int max_splits;         /* the value scratch was sized for */
    int n_splits, split_len;
    int with_logits;
    uint16_t *hidden;       /* optional [n_layers + 1][d_model]: residual stream after each layer */
    /* Tensor parallel (tp_size > 1): n_q_heads, n_kv_heads, ffn and vocab above are this rank's
     * shares (q/k/v, gate/up, lm_head split by rows; o_proj, down_proj by columns; KV cache by KV
     * head).  After o_proj and down_proj each rank stores its FP32 partial sums straight into every
     * rank's exchange block over NVLink, the ranks synchronise through flags in those blocks, and
     * every rank forms x = half(half(sum of partials) + x_old) itself: the all-reduce is part of
     * the kernel.  peers[r] = device address, valid on this GPU, of rank r's exchange block of
     * llmb_decode_step_exchange_bytes() bytes (zeroed once; own block at peers[tp_rank]).
     * logits then hold this rank's vocabulary slice; next_token is the same on every rank. */
    int tp_rank, tp_size, vocab_offset;
    uint16_t *x_alt;        /* [d_model] second residual buffer */
    void *peers[8];
    uint64_t *trace;        /* optional profiling aid, device [SM count][5 * n_layers + 2][8] nanosecond
                               stamps, one row per CTA; per phase: consumers entered, dependency met, input
                               ready, done; finisher started, first stage, last stage, fenced.  NULL in
                               production. */
    uint32_t tag_poll_limit; /* tensor parallel: spins a wait for peer data may take before the kernel gives
                                up with status 205-207; 0 = 2^20 (about a second) */
} LlmbDecodeStepArgs;

size_t llmb_decode_step_scratch_bytes(int n_q_heads, int n_kv_heads, int head_dim, int max_splits);
size_t llmb_decode_step_exchange_bytes(int tp_size, int d_model);
int llmb_decode_step(const LlmbDecodeStepArgs *args, llmb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LLM_B200_H */
