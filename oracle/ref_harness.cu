/*
 * TEST INFRASTRUCTURE ONLY.  Non-interactive driver for the UNMODIFIED reference engine
 * (abhisheknair10/LLM.cu).  It replaces only the reference's src/main.cu (an interactive chat
 * loop that needs the gated tokenizer.json) and calls the reference's own public functions in
 * the order main.cu:61-123 does: init_llama3 -> load_safetensor_weights (one call per shard) ->
 * to_cuda -> init_cache -> tokens_to_cuda -> inference() per generated token.
 *
 * Teacher forcing: after each call the next token appended to the array is the one given in
 * the token file, not the sampled one (the reference samples with temperature/top-p on the
 * host, inference.cu:1030-1039).  The FP16 logits the reference leaves in
 * Cache->h_token_probdist (inference.cu:1021-1025) are written out per step.
 *
 * usage: ref_harness <n_layers> <tokens.i32> <n_prompt> <n_steps> <logits_out.f16|-> <shard>...
 *   tokens.i32 : little-endian int32 ids, at least n_prompt + n_steps - 1 of them
 *   output     : n_steps rows of 128256 FP16 logits; one JSON line with per-step seconds on stdout
 */
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <cuda_runtime.h>

#include "inference/inference.cuh"
#include "llama3/llama3.cuh"
#include "safetensor/safetensor.cuh"
#include "tokenizer/tokenizer.cuh"

static const int kVocab = 128256;  /* inference.cu:24 */
static const int kMaxTokens = 2048; /* main.cu:119, tokenizer.cu:107 */

int main(int argc, char **argv) {
    if (argc < 7) {
        fprintf(stderr, "usage: %s n_layers tokens.i32 n_prompt n_steps logits_out|- shard...\n", argv[0]);
        return 2;
    }
    int n_layers = atoi(argv[1]);
    const char *tok_path = argv[2];
    int n_prompt = atoi(argv[3]);
    int n_steps = atoi(argv[4]);
    const char *out_path = argv[5];
    if (n_prompt < 1 || n_steps < 1 || n_prompt + n_steps > kMaxTokens) {
        fprintf(stderr, "n_prompt + n_steps must be in [2, %d]\n", kMaxTokens);
        return 2;
    }

    std::vector<int> ids((size_t)n_prompt + n_steps);
    FILE *tf = fopen(tok_path, "rb");
    if (!tf) { perror(tok_path); return 2; }
    size_t got = fread(ids.data(), sizeof(int), ids.size(), tf);
    fclose(tf);
    if ((int)got < n_prompt + n_steps - 1) {
        fprintf(stderr, "token file too short: %zu ids\n", got);
        return 2;
    }

    auto t0 = std::chrono::steady_clock::now();
    Llama3 *model = init_llama3(n_layers);
    for (int i = 6; i < argc; ++i) load_safetensor_weights(model, argv[i]);
    to_cuda(model);
    CudaCache *cache = init_cache(model);
    cudaDeviceSynchronize();
    double load_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();

    /* Token array convention (tokenizer.cu:143,152): [0] = count + 1, ids in [1..count]. */
    int *tokens = (int *)malloc(sizeof(int) * (kMaxTokens + 1));
    for (int i = 0; i < n_prompt; ++i) tokens[1 + i] = ids[i];
    tokens[0] = n_prompt + 1;

    Tensor *X = (Tensor *)malloc(sizeof(Tensor));
    int *d_tokens = tokens_to_cuda(tokens, 4096, X);

    FILE *of = nullptr;
    if (strcmp(out_path, "-") != 0) {
        of = fopen(out_path, "wb");
        if (!of) { perror(out_path); return 2; }
    }

    std::vector<double> secs;
    std::vector<int> sampled;
    for (int s = 0; s < n_steps; ++s) {
        auto a = std::chrono::steady_clock::now();
        int next = inference(model, X, d_tokens, tokens, cache);
        cudaDeviceSynchronize();
        secs.push_back(std::chrono::duration<double>(std::chrono::steady_clock::now() - a).count());
        sampled.push_back(next);
        if (of) fwrite(cache->h_token_probdist, sizeof(__half), kVocab, of);
        cudaError_t err = cudaGetLastError();
        if (err != cudaSuccess) {
            fprintf(stderr, "CUDA error after step %d: %s\n", s, cudaGetErrorString(err));
            return 3;
        }
        if (s + 1 < n_steps) {
            tokens[tokens[0]] = ids[n_prompt + s]; /* main.cu:121-122, teacher-forced */
            tokens[0] = tokens[0] + 1;
        }
    }
    if (of) fclose(of);

    printf("{\"n_layers\": %d, \"n_prompt\": %d, \"n_steps\": %d, \"load_s\": %.3f, \"step_s\": [", n_layers,
           n_prompt, n_steps, load_s);
    for (size_t i = 0; i < secs.size(); ++i) printf("%s%.6f", i ? ", " : "", secs[i]);
    printf("], \"sampled\": [");
    for (size_t i = 0; i < sampled.size(); ++i) printf("%s%d", i ? ", " : "", sampled[i]);
    printf("]}\n");
    return 0;
}
