/* A C program over include/mynah_slm_b200.h, compiled and run by tests/test_gpu_capi.py.
 *
 *   capi_program replay   <model> <dtype> <max_tokens> <script.bin> <out dir>
 *   capi_program generate <model> <dtype> <max_tokens> <prompts.bin> <max_new> <temp> <seed> <stop id or -1>
 *   capi_program errors   <model>
 *
 * <model>: a model folder, or "random:<config.json>:<seed>". All files hold little-endian int32 numbers.
 * script.bin: n_steps, then per step: step id, n_entries, per entry (request id, n_tokens, tokens..., n_want,
 * places...), n_end, request ids that end. replay maps request ids to slots, calls mynah_step and writes
 * <out dir>/<step id>.f32 for every step in which something is wanted (the replay program bin/trace_run in C).
 * prompts.bin: n_prompts, then per prompt n_tokens, tokens.... Everything this program has to say goes to
 * stdout; the library itself must stay silent. */
#include <inttypes.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "mynah_slm_b200.h"

static char err[4096];

static int32_t* read_ints(const char* path, long* n) {
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    fseek(f, 0, SEEK_END);
    const long bytes = ftell(f);
    fseek(f, 0, SEEK_SET);
    int32_t* a = (int32_t*)malloc((size_t)bytes + 4);
    *n = (long)fread(a, 4, (size_t)bytes / 4, f);
    fclose(f);
    return a;
}

static int open_model(const char* model, const char* dtype, int max_tokens, mynah_engine** e) {
    if (strncmp(model, "random:", 7) == 0) {
        char path[2048];
        snprintf(path, sizeof path, "%s", model + 7);
        char* colon = strrchr(path, ':');
        uint64_t seed = 0;
        if (colon) {
            seed = strtoull(colon + 1, NULL, 10);
            *colon = '\0';
        }
        return mynah_engine_create_random(path, seed, dtype, max_tokens, 0, e, err, sizeof err);
    }
    return mynah_engine_create(model, dtype, max_tokens, 0, e, err, sizeof err);
}

#define MAX_REQ 256

static int replay(int argc, char** argv) {
    if (argc != 7) return 2;
    mynah_engine* e = NULL;
    int rc = open_model(argv[2], argv[3], atoi(argv[4]), &e);
    if (rc) { printf("error %d: %s\n", rc, err); return 1; }
    const int V = mynah_engine_vocab_size(e);
    printf("vocab %d layers %d hidden %d positions %d page %d free %d\n", V, mynah_engine_n_layers(e), mynah_engine_hidden_size(e),
           mynah_engine_max_positions(e), mynah_page_size(), mynah_engine_free_tokens(e));
    long n = 0;
    int32_t* s = read_ints(argv[5], &n);
    if (!s) { printf("error: cannot read %s\n", argv[5]); return 1; }
    int slot_of[MAX_REQ];
    for (int i = 0; i < MAX_REQ; i++) slot_of[i] = -1;
    long p = 0;
    const int n_steps = s[p++];
    for (int st = 0; st < n_steps; st++) {
        const int step_id = s[p++], n_entries = s[p++];
        int slots[MAX_REQ], n_new[MAX_REQ], n_want[MAX_REQ];
        int32_t* tokens = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n + 1));
        int* want = (int*)malloc(sizeof(int) * (size_t)(n + 1));
        int nt = 0, nw = 0;
        for (int i = 0; i < n_entries; i++) {
            const int req = s[p++];
            if (slot_of[req] < 0) {
                rc = mynah_slot_open(e, &slot_of[req], err, sizeof err);
                if (rc) { printf("error %d: %s\n", rc, err); return 1; }
            }
            slots[i] = slot_of[req];
            n_new[i] = s[p++];
            for (int j = 0; j < n_new[i]; j++) tokens[nt++] = s[p++];
            n_want[i] = s[p++];
            for (int j = 0; j < n_want[i]; j++) want[nw++] = s[p++];
        }
        float* logits = (float*)malloc(sizeof(float) * (size_t)(nw > 0 ? nw : 1) * (size_t)V);
        rc = mynah_step(e, n_entries, slots, n_new, tokens, n_want, want, logits, err, sizeof err);
        if (rc) { printf("error %d: %s\n", rc, err); return 1; }
        if (nw > 0) {
            char path[2048];
            snprintf(path, sizeof path, "%s/%d.f32", argv[6], step_id);
            FILE* f = fopen(path, "wb");
            fwrite(logits, sizeof(float), (size_t)nw * (size_t)V, f);
            fclose(f);
            /* greedy through the sampler entry point: the first maximum of every row */
            int32_t* picked = (int32_t*)malloc(sizeof(int32_t) * (size_t)nw);
            mynah_sampler_params sp;
            mynah_sampler_defaults(&sp);
            sp.temp = 0.0f;
            rc = mynah_sample(e, logits, nw, &sp, NULL, picked, err, sizeof err);
            if (rc) { printf("error %d: %s\n", rc, err); return 1; }
            for (int r = 0; r < nw; r++) {
                int best = 0;
                for (int v = 1; v < V; v++) if (logits[(size_t)r * V + v] > logits[(size_t)r * V + best]) best = v;
                if (best != picked[r]) { printf("error: mynah_sample picked %d, the maximum is at %d\n", picked[r], best); return 1; }
            }
            free(picked);
        }
        const int n_end = s[p++];
        for (int i = 0; i < n_end; i++) {
            const int req = s[p++];
            rc = mynah_slot_close(e, slot_of[req], err, sizeof err);
            if (rc) { printf("error %d: %s\n", rc, err); return 1; }
            slot_of[req] = -1;
        }
        printf("done %d\n", step_id);
        fflush(stdout);
        free(tokens); free(want); free(logits);
    }
    printf("free %d\n", mynah_engine_free_tokens(e));
    mynah_engine_free(e);
    return 0;
}

struct seen { int calls; int stop_after; };

static int on_token(void* ctx, int request, int32_t token) {
    struct seen* s = (struct seen*)ctx;
    (void)token;
    s->calls++;
    return (s->stop_after > 0 && request == 0 && s->calls >= s->stop_after) ? 1 : 0;
}

static int generate(int argc, char** argv) {
    if (argc != 10) return 2;
    mynah_engine* e = NULL;
    int rc = open_model(argv[2], argv[3], atoi(argv[4]), &e);
    if (rc) { printf("error %d: %s\n", rc, err); return 1; }
    long n = 0;
    int32_t* s = read_ints(argv[5], &n);
    if (!s) { printf("error: cannot read %s\n", argv[5]); return 1; }
    const int max_new = atoi(argv[6]);
    long p = 0;
    const int n_req = s[p++];
    mynah_request* reqs = (mynah_request*)calloc((size_t)n_req, sizeof *reqs);
    mynah_result* res = (mynah_result*)calloc((size_t)n_req, sizeof *res);
    for (int i = 0; i < n_req; i++) {
        reqs[i].n_tokens = s[p++];
        reqs[i].tokens = &s[p];
        p += reqs[i].n_tokens;
        reqs[i].max_new = max_new;
        res[i].tokens = (int32_t*)calloc((size_t)max_new, sizeof(int32_t));
    }
    mynah_sampler_params sp;
    mynah_sampler_defaults(&sp);
    sp.temp = (float)atof(argv[7]);
    sp.top_k = 0;
    sp.top_p = 1.0f;
    sp.seed = strtoull(argv[8], NULL, 10);
    int32_t stop = atoi(argv[9]);
    struct seen seen = {0, 0};
    mynah_timing tm;
    rc = mynah_generate(e, reqs, n_req, &sp, stop >= 0 ? &stop : NULL, stop >= 0 ? 1 : 0, 64, on_token, &seen, res, &tm, err, sizeof err);
    if (rc) { printf("error %d: %s\n", rc, err); return 1; }
    int emitted = 0;
    for (int i = 0; i < n_req; i++) {
        printf("request %d finish %d produced %d tokens", i, res[i].finish, res[i].produced);
        for (int j = 0; j < res[i].n_tokens; j++) printf(" %d", res[i].tokens[j]);
        printf("\n");
        emitted += res[i].n_tokens;
    }
    printf("callback calls %d emitted %d prompt %d generated %d decode_s_positive %d\n", seen.calls, emitted, tm.n_prompt, tm.n_gen,
           tm.decode_s > 0.0 || tm.n_gen == n_req);
    /* again, and the callback ends request 0 after its third token */
    struct seen early = {0, 3};
    for (int i = 0; i < n_req; i++) reqs[i].max_new = max_new;
    rc = mynah_generate(e, reqs, 1, &sp, NULL, 0, 64, on_token, &early, res, NULL, err, sizeof err);
    printf("stopped rc %d finish %d n %d\n", rc, res[0].finish, res[0].n_tokens);
    mynah_engine_free(e);
    return 0;
}

static int errors(int argc, char** argv) {
    if (argc != 3) return 2;
    mynah_engine* e = NULL;
    int rc = mynah_engine_create("/nonexistent/folder", "bfloat16", 256, 0, &e, err, sizeof err);
    printf("missing folder: rc %d engine %s message: %s\n", rc, e ? "set" : "null", err);
    rc = mynah_engine_create(argv[2], "float16", 256, 0, &e, err, sizeof err);
    printf("bad dtype: rc %d message: %s\n", rc, err);
    rc = open_model(argv[2], "float32", 128, &e);
    if (rc) { printf("error %d: %s\n", rc, err); return 1; }
    int slot = -1;
    mynah_slot_open(e, &slot, err, sizeof err);
    int n_new = 1, n_want = 1, want = 0;
    int32_t tok = 1 << 30;
    float* logits = (float*)malloc(sizeof(float) * (size_t)mynah_engine_vocab_size(e));
    rc = mynah_step(e, 1, &slot, &n_new, &tok, &n_want, &want, logits, err, sizeof err);
    printf("token out of range: rc %d message: %s\n", rc, err);
    int other = 77;
    tok = 1;
    rc = mynah_step(e, 1, &other, &n_new, &tok, &n_want, &want, logits, err, sizeof err);
    printf("unknown slot: rc %d message: %s\n", rc, err);
    int32_t many[200];
    for (int i = 0; i < 200; i++) many[i] = 1;
    n_new = 200;
    n_want = 0;
    rc = mynah_step(e, 1, &slot, &n_new, many, &n_want, &want, logits, err, sizeof err);
    printf("cache full: rc %d message: %s\n", rc, err);
    rc = mynah_step(e, 1, &slot, &n_new, many, &n_want, &want, logits, NULL, 0);         /* no buffer: the code alone */
    printf("no buffer: rc %d length %d\n", rc, mynah_slot_length(e, slot));
    rc = mynah_slot_close(e, 5, err, sizeof err);
    printf("close unknown: rc %d message: %s\n", rc, err);
    mynah_engine_free(e);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 2 && strcmp(argv[1], "replay") == 0) return replay(argc, argv);
    if (argc >= 2 && strcmp(argv[1], "generate") == 0) return generate(argc, argv);
    if (argc >= 2 && strcmp(argv[1], "errors") == 0) return errors(argc, argv);
    printf("usage: capi_program replay|generate|errors ...\n");
    return 2;
}
