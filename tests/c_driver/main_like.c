/*
 * A driver in the shape of the reference's src/main.cu:61-126, written in plain C against
 * include/llama3.h and linked to libllm_b200.so: init_llama3 -> load_safetensor_weights (one call
 * per shard) -> to_cuda -> init_cache -> tokens_to_cuda -> inference() per generated token with the
 * returned token appended to the array (main.cu:121-122) -> free.  The tokenizer and the chat loop
 * of main.cu are left out; the prompt ids come from the command line.
 *
 * usage: main_like <n_layers> <head_dim> <max_seq> <n_new> <id,id,...> <shard>...
 * prints the generated ids, one per line.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "llama3.h"

int main(int argc, char **argv) {
    if (argc < 7) {
        fprintf(stderr, "usage: %s n_layers head_dim max_seq n_new id,id,... shard...\n", argv[0]);
        return 2;
    }
    int n_layers = atoi(argv[1]);
    int n_new = atoi(argv[4]);

    Llama3 *llama3_model = init_llama3(n_layers);
    Llama3Config partial;
    memset(&partial, 0, sizeof partial); /* fields <= 0 keep their defaults (the reference's literals) */
    partial.head_dim = atoi(argv[2]);
    partial.max_seq = atoi(argv[3]);
    if (llama3_set_config(llama3_model, &partial) != LLMB_OK) return 3;
    for (int i = 6; i < argc; ++i) load_safetensor_weights(llama3_model, argv[i]);
    to_cuda(llama3_model);
    CudaCache *Cache = init_cache(llama3_model);

    /* token array convention of tokenizer.cu:143-152: [0] = count + 1, ids in [1..count] */
    int *tokens = (int *)malloc(sizeof(int) * 2049);
    int count = 0;
    for (char *tok = strtok(argv[5], ","); tok && count < 2047; tok = strtok(NULL, ",")) tokens[++count] = atoi(tok);
    tokens[0] = count + 1;

    Tensor *X = (Tensor *)malloc(sizeof(Tensor));
    int *d_tokens = tokens_to_cuda(tokens, llama3_model->embed_tokens->shape[1], X);
    if (!d_tokens) return 4;

    for (int s = 0; s < n_new; ++s) {
        int next = inference(llama3_model, X, d_tokens, tokens, Cache);
        if (next < 0) {
            fprintf(stderr, "inference failed (%d): %s\n", -next, llmb_last_error());
            return 5;
        }
        printf("%d\n", next);
        tokens[tokens[0]] = next; /* main.cu:121-122 */
        tokens[0] = tokens[0] + 1;
    }
    /* the struct layout is the reference's: a driver may read the logits where the reference leaves them */
    if (!Cache->h_token_probdist || !Cache->d_token_probdist) return 6;

    free_cache(Cache);
    _free_tensor(X);
    free_llama3(llama3_model);
    free(tokens);
    return 0;
}
