/* mynah_slm_b200: the C interface of the engine.
 *
 * From a model folder (config.json + model.safetensors) or a configuration and a seed to logits and generated
 * token ids on one B200, for callers that are not Python. Every function that can fail returns a code (0 = ok)
 * and, when the caller gives a buffer, leaves a message there; the library never prints and never exits
 * (the reference's rule for its public header, mynah-slm include/mynah_slm.h:4-8). The reference's header has
 * load / free / accessors (include/mynah_slm.h:38-47); its step and its generation loop are internal
 * (src/arch_qwen3.h:52-62 mynah_slm_state_init / mynah_slm_forward, src/generate.h:16-52 mynah_slm_generate) and are
 * mirrored here for a batch of sequences.
 *
 * How it is built: the engine's composition layer (parts, schedule, graphs, generation loop) is Python, its
 * kernels and its cache books are native. This library hosts a Python interpreter (or joins the one of the
 * calling process), loads the package and forwards every call to the same step function, generation loop and
 * sampler that the Python entry point and the command line use; there is no second forward pass. The
 * interpreter is found through MYNAH_PYTHON (else the one the library was built with) and the package through
 * MYNAH_SLM_B200_ROOT (else the checkout the library was built in). Calls may come from any thread; they are
 * serialised.
 */
#ifndef MYNAH_SLM_B200_H
#define MYNAH_SLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

enum mynah_status {
    MYNAH_OK = 0,
    MYNAH_ERR_ARGUMENT = 1,     /* a bad argument: unknown slot, token outside the vocabulary, wanted place out of range ... */
    MYNAH_ERR_CONFIG = 2,       /* config.json: a missing or ill-typed key, an unknown architecture */
    MYNAH_ERR_WEIGHTS = 3,      /* the checkpoint does not fit the model (the message lists every tensor) */
    MYNAH_ERR_CACHE_FULL = 4,   /* no page or no slot left */
    MYNAH_ERR_DEVICE = 5,       /* no sm_100 device, the kernel library is missing, a kernel reported a fault */
    MYNAH_ERR_INTERNAL = 6,     /* the interpreter or the package could not be started, or anything else */
    MYNAH_STOPPED = 7           /* mynah_generate: the callback asked to stop (results hold what was made) */
};

typedef struct mynah_engine mynah_engine;

/* ---- load / free / accessors (include/mynah_slm.h:38-47) */
/* dtype: "bfloat16" or "float32" (true 32-bit). max_tokens sizes the cache: the most tokens that live sequences
 * hold at any time, each sequence's count rounded up to a multiple of mynah_page_size(). max_seqs <= 0: as many
 * slots as pages. */
int mynah_engine_create(const char* model_folder, const char* dtype, int max_tokens, int max_seqs,
                        mynah_engine** out, char* err, size_t errlen);
/* The same model with random weights made on the device from config_json (a file's path) and a seed: no
 * checkpoint is read or written. */
int mynah_engine_create_random(const char* config_json, uint64_t seed, const char* dtype, int max_tokens, int max_seqs,
                               mynah_engine** out, char* err, size_t errlen);
void mynah_engine_free(mynah_engine*);
int mynah_engine_vocab_size(const mynah_engine*);
int mynah_engine_max_positions(const mynah_engine*);
int mynah_engine_hidden_size(const mynah_engine*);
int mynah_engine_n_layers(const mynah_engine*);
int mynah_engine_free_tokens(const mynah_engine*);        /* tokens the free pages can still hold */
int mynah_engine_eos_ids(const mynah_engine*, int32_t* ids, int capacity);    /* returns how many the model has */
int mynah_page_size(void);

/* ---- sequences: a slot per live sequence (src/arch_qwen3.h:52 state_init has one state with one counter) */
int mynah_slot_open(mynah_engine*, int* slot, char* err, size_t errlen);
int mynah_slot_close(mynah_engine*, int slot, char* err, size_t errlen);      /* gives its pages back */
int mynah_slot_length(const mynah_engine*, int slot);                         /* positions in the cache, -1: not open */

/* ---- the step function (src/arch_qwen3.h:60-62 forward(state, token, logits): one token of one sequence)
 * n sequences that either all bring the next piece of their prompts or all go on by one token. tokens holds the
 * new tokens of all sequences one after another (n_new[i] of sequence i); want holds, likewise, n_want[i] places
 * among sequence i's new tokens whose logits are asked for. logits_out (host memory, float32) receives
 * [sum of n_want, vocab] rows in the order of the sequences and of their places. */
int mynah_step(mynah_engine*, int n, const int* slots, const int* n_new, const int32_t* tokens,
               const int* n_want, const int* want, float* logits_out, char* err, size_t errlen);

/* ---- sampling (src/sampler.h:13-26: the same fields with the same meanings) */
typedef struct {
    float temp;                /* <= 0: greedy, first maximum, no other filter */
    uint32_t top_k;            /* 0 = off */
    float top_p;               /* 1.0 = off */
    float min_p;               /* 0.0 = off */
    float repeat_penalty;      /* 1.0 = off */
    float freq_penalty;
    float presence_penalty;
    uint32_t penalty_window;
    uint64_t seed;
} mynah_sampler_params;
void mynah_sampler_defaults(mynah_sampler_params*);     /* temp 0.6, top-k 20, top-p 0.95 (src/sampler.c:27-36) */

/* One token from each of n_rows rows of logits [n_rows, vocab] (host, float32; not modified) with the device's
 * sampler: temperature, top-k, min-p, top-p, then the draw from rng[i], the splitmix64 state of row i, which is
 * advanced (NULL: greedy needs none). Penalties look at a sequence's accepted tokens and are applied by
 * mynah_generate only. */
int mynah_sample(mynah_engine*, const float* logits, int n_rows, const mynah_sampler_params*, uint64_t* rng,
                 int32_t* tokens_out, char* err, size_t errlen);

/* ---- generation (src/generate.h:16-52) */
typedef struct {
    const int32_t* tokens;     /* the prompt */
    int n_tokens;
    int max_new;
} mynah_request;

enum mynah_finish { MYNAH_FINISH_STOP = 0, MYNAH_FINISH_LENGTH = 1, MYNAH_FINISH_CONTEXT = 2, MYNAH_FINISH_CALLBACK = 3 };

typedef struct {
    int32_t* tokens;           /* caller's buffer of at least the request's max_new entries */
    int n_tokens;              /* out: tokens written (a stop token is not among them) */
    int produced;              /* out: tokens sampled, the stop token included */
    int finish;                /* out: enum mynah_finish */
} mynah_result;

typedef struct {
    double load_s, prefill_s, decode_s, ttft_s;      /* src/timing.h:15-28 */
    int n_prompt, n_gen;
} mynah_timing;

/* Called for every emitted token, in step order; non-zero ends that request (src/generate.h:16). */
typedef int (*mynah_token_cb)(void* ctx, int request, int32_t token);

/* Generates for every request: as many per batch as max_batch and the cache allow, the prompts of a batch in one
 * step, then one token per live sequence per step; a stop token ends a sequence before it is emitted; requests
 * that end give their slot and pages back at once; batches follow one another until all requests are done.
 * stop_ids NULL with n_stop < 0: the model's own stop set; n_stop == 0: none. cb and timing may be NULL. */
int mynah_generate(mynah_engine*, const mynah_request* requests, int n_requests, const mynah_sampler_params*,
                   const int32_t* stop_ids, int n_stop, int max_batch, mynah_token_cb cb, void* cb_ctx,
                   mynah_result* results, mynah_timing* timing, char* err, size_t errlen);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif

#endif
