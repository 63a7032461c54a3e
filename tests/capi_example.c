/* A C program over the library's C interface: opens a model folder, generates greedily for two prompts through a
 * sink, then drives the step function by hand. Prints token ids; the test compares them with the Python entry
 * point's. Usage: capi_example MODEL_DIR */
#include <stdio.h>
#include <stdlib.h>

#include "engine.h"

struct collect {
    int32_t tokens[2][16];
    int n[2];
};

static void on_token(void *ctx, int32_t request, int32_t token, int32_t last) {
    struct collect *c = (struct collect *)ctx;
    (void)last;
    if (request < 2 && c->n[request] < 16) c->tokens[request][c->n[request]++] = token;
}

int main(int argc, char **argv) {
    char err[LM_ERROR_BYTES];
    if (argc != 2) return 2;
    lm *bad = lm_open("/nowhere/at/all", NULL, err);
    if (bad || !err[0]) { fprintf(stderr, "a missing folder was opened\n"); return 1; }
    lm_options options = {"float32", 128, 4, 0, "fast", NULL};
    lm *model = lm_open(argv[1], &options, err);            /* after a failure the next call works */
    if (!model) { fprintf(stderr, "lm_open: %s\n", err); return 1; }
    lm_info info;
    lm_get_info(model, &info);
    printf("vocab %d context %d layers %d\n", info.vocab_size, info.context, info.layers);

    const int32_t p0[] = {5, 17, 3, 99, 42}, p1[] = {7, 7, 1};
    lm_request requests[2] = {{p0, 5}, {p1, 3}};
    lm_generation generation = {6, 0.0f, 0, 0.0f, 0, NULL, 0};      /* greedy, 6 tokens, no stop ids */
    struct collect got = {{{0}}, {0, 0}};
    lm_sink sink = {&got, on_token, NULL};
    if (lm_generate(model, requests, 2, &generation, &sink) != LM_OK) { fprintf(stderr, "lm_generate: %s\n", lm_last_error()); return 1; }
    for (int r = 0; r < 2; ++r) {
        printf("generated %d:", r);
        for (int i = 0; i < got.n[r]; ++i) printf(" %d", got.tokens[r][i]);
        printf("\n");
    }

    /* the step function: the first prompt whole, then its argmax token by hand */
    int slot = lm_slot_alloc(model);
    if (slot < 0) { fprintf(stderr, "lm_slot_alloc: %s\n", lm_last_error()); return 1; }
    float *logits = (float *)malloc(sizeof(float) * (size_t)info.vocab_size);
    int32_t slots[1] = {slot}, counts[1] = {5};
    uint8_t want[1] = {1};
    if (lm_step(model, slots, counts, 1, p0, want, logits) != LM_OK) { fprintf(stderr, "lm_step: %s\n", lm_last_error()); return 1; }
    int best = 0;
    for (int v = 1; v < info.vocab_size; ++v) if (logits[v] > logits[best]) best = v;
    printf("step argmax %d length %d\n", best, lm_slot_length(model, slot));
    int32_t bad_token[1] = {info.vocab_size};
    counts[0] = 1;
    if (lm_step(model, slots, counts, 1, bad_token, want, logits) != LM_ERR_ARGUMENT) { fprintf(stderr, "a token outside the vocabulary was taken\n"); return 1; }
    printf("refused: %s\n", lm_last_error());
    if (lm_slot_free(model, slot) != LM_OK || lm_slot_free(model, slot) == LM_OK) { fprintf(stderr, "slot_free\n"); return 1; }
    free(logits);
    lm_close(model);
    return 0;
}
