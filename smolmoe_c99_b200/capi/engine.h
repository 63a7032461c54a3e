/* The C interface of the library: open a model folder, generate for a batch of requests through a token
 * sink, or drive the step function yourself -- slots, tokens in, logits out.
 *
 * Its shape follows the reference's C interface for front ends (src/desktop.h:35-72: an opaque handle, an options
 * struct, a sink of callbacks, NULL with a message when opening fails; src/engine_sink.h:9-23: the sink and its
 * stop poll; src/util.h:28-56: a status per call and a last-error message, after which the next call still works).
 *
 * There is ONE engine behind it: the functions call the library's Python engine (smolmoe_c99_b200.engine) inside
 * this process, through an interpreter that lm_open starts if the program has none (a Python program that loads
 * this library uses its own). The engine's parts are Python classes found by name in registries, which is what
 * lets a new mixer or feed-forward be added without touching the library; a second engine in C++ beside it would
 * be exactly the second forward pass, cache and loader this library does not have. What runs on the GPU is the same
 * CUDA kernels either way.
 *
 * Threads: calls on one handle must not overlap. Token ids are int32. Functions that return int return 0 for
 * success and a negative status otherwise, with a message in lm_last_error() (per thread). */
#ifndef SMOLMOE_B200_ENGINE_H
#define SMOLMOE_B200_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LM_ERROR_BYTES 512

enum {
    LM_OK = 0,
    LM_ERR_ARGUMENT = -1, /* a value the library refuses: the message names it (src/util.h: SM_ERR_RANGE and the like) */
    LM_ERR_RUNTIME = -2,  /* the engine failed: CUDA, a kernel's refusal, out of memory */
    LM_ERR_PYTHON = -3    /* the interpreter or the package could not be started */
};

typedef struct lm lm;

typedef struct lm_options {
    const char *dtype;    /* "bfloat16" (NULL: the same) or "float32", the true 32-bit path */
    int32_t context;      /* positions a sequence may hold; 0: min(the model's limit, 2048) (src/main.c:746-747) */
    int32_t batch;        /* most sequences that start together; 0: 8 */
    int32_t step_tokens;  /* most tokens one step brings; 0: no limit (the reference's --batch, src/main.c:106) */
    const char *kernels;  /* "fast" (NULL: the same) or "plain" */
    const char *package_root; /* folder that holds the smolmoe_c99_b200 package; NULL: found from this library's own path */
} lm_options;

/* Where generated tokens go (src/engine_sink.h). Pointers are valid during the call only. */
typedef struct lm_sink {
    void *ctx;
    /* every token as it is chosen; last != 0 on a request's final token (a stop token, or the limit) */
    void (*token)(void *ctx, int32_t request, int32_t token, int32_t last);
    /* polled once per step; nonzero ends the generation there. NULL: never stopped */
    int (*stop)(void *ctx);
} lm_sink;

typedef struct lm_request {
    const int32_t *tokens; /* the prompt */
    int32_t n;
} lm_request;

typedef struct lm_generation {
    int32_t tokens;        /* most new tokens per request (the reference's --tokens; 0: 64) */
    float temperature;     /* 0: greedy */
    int32_t top_k;         /* 0: all; the reference's default is 40 */
    float top_p;           /* in (0, 1]; 0: 0.95 */
    uint32_t seed;         /* nonzero; 0: 1 */
    const int32_t *stop_ids; /* NULL with n_stop_ids < 0: the configuration's end-of-sequence ids */
    int32_t n_stop_ids;
} lm_generation;

typedef struct lm_info {
    int32_t vocab_size, context, batch, layers;
    int64_t weight_bytes, cache_bytes;
    /* of the last lm_generate (src/main.c:347-382) */
    int32_t prompt_tokens, generated_tokens;
    double prefill_seconds, decode_seconds;
} lm_info;

/* Opens the folder (config.json + model.safetensors). NULL with a message in err when it cannot. */
lm *lm_open(const char *folder, const lm_options *options, char err[LM_ERROR_BYTES]);
/* The same for random weights of the configuration in config_json (a file), with a seed. */
lm *lm_open_random(const char *config_json, uint32_t seed, const lm_options *options, char err[LM_ERROR_BYTES]);
void lm_close(lm *model);
void lm_get_info(lm *model, lm_info *out);

/* Generates for n requests: batches of `batch` that start together, every token to the sink as it is chosen. */
int lm_generate(lm *model, const lm_request *requests, int32_t n, const lm_generation *generation, const lm_sink *sink);

/* The step function (Engine.step): slot_alloc gives a sequence of length 0, or a negative status when none is free. */
int lm_slot_alloc(lm *model);
int lm_slot_free(lm *model, int32_t slot);
int lm_slot_length(lm *model, int32_t slot);
/* Sequence i brings counts[i] >= 1 tokens (all of them one after another in `tokens`) onto its current length;
 * want[i] != 0 asks for the logits after its last token. logits receives vocab_size floats per wanted sequence,
 * in order (may be NULL when nothing is wanted). */
int lm_step(lm *model, const int32_t *slots, const int32_t *counts, int32_t n_sequences, const int32_t *tokens,
            const uint8_t *want, float *logits);

const char *lm_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
