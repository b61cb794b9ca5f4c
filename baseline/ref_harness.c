/* Times the reference engine (mynah-org/mynah-slm, unmodified, built from its own sources) on the benchmark's
 * workload: n sequences one after another (the reference runs one sequence at a time, token by token), each a
 * prompt of prompt_len tokens and then warmup + steps greedy decode steps; decode time is summed over the
 * sequences. Calls only the reference's own functions: mynah_slm_load, mynah_slm_state_init / _reset,
 * mynah_slm_forward (src/arch_qwen3.h:52-62), the loop of src/generate.c:25-48 without its text side.
 *
 *   ref_harness <model.gguf> <n_seqs> <prompt_len> <warmup> <steps> <threads> <probe_tokens> <budget_seconds>
 *
 * It first times probe_tokens prompt tokens; if the whole run would take longer than budget_seconds it prints
 * "too_slow <tokens per second>" and stops. Otherwise it prints "ok <decode tokens> <decode seconds> <prompt
 * tokens> <prompt seconds>". */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "arch_qwen3.h"
#include "mynah_slm.h"
#include "model.h"
#include "threads.h"

static double now(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static uint32_t next_id(uint64_t* s, uint32_t vocab) {          /* uniform random token ids, seeded */
    *s = *s * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)((*s >> 33) % vocab);
}

static uint32_t argmax(const float* v, uint32_t n) {
    uint32_t best = 0;
    for (uint32_t i = 1; i < n; i++) if (v[i] > v[best]) best = i;
    return best;
}

int main(int argc, char** argv) {
    if (argc != 9) {
        printf("usage: ref_harness <model.gguf> <n_seqs> <prompt_len> <warmup> <steps> <threads> <probe_tokens> <budget_seconds>\n");
        return 2;
    }
    const int n_seqs = atoi(argv[2]), prompt_len = atoi(argv[3]), warmup = atoi(argv[4]), steps = atoi(argv[5]);
    const int threads = atoi(argv[6]);
    int probe = atoi(argv[7]);
    if (probe > prompt_len + warmup + steps) probe = prompt_len + warmup + steps;      /* the state holds no more */
    const double budget = atof(argv[8]);
    char err[512];
    mynah_slm_model_t* m = mynah_slm_load(argv[1], err, sizeof err);
    if (!m) { printf("error load: %s\n", err); return 1; }
    if (threads > 0) mynah_slm_threads_init(threads);
    const uint32_t vocab = mynah_slm_vocab_size(m);
    mynah_slm_state st;
    if (mynah_slm_state_init(&st, m, (uint32_t)(prompt_len + warmup + steps + 8), err, sizeof err) != 0) {
        printf("error state: %s\n", err);
        return 1;
    }
    uint64_t seed = 2;
    /* how fast is a prompt token? (the cache is short here, so this flatters the reference) */
    double t0 = now();
    for (int i = 0; i < probe; i++) if (mynah_slm_forward(&st, next_id(&seed, vocab), NULL) != 0) { printf("error forward\n"); return 1; }
    const double per_token = (now() - t0) / (probe > 0 ? probe : 1);
    const double projected = per_token * ((double)n_seqs * (prompt_len + warmup + steps));
    if (probe > 0 && projected > budget) {
        printf("too_slow %.2f %.0f\n", 1.0 / per_token, projected);
        return 0;
    }
    double decode_s = 0.0, prompt_s = 0.0;
    for (int s = 0; s < n_seqs; s++) {
        mynah_slm_state_reset(&st);
        t0 = now();
        for (int i = 0; i + 1 < prompt_len; i++) if (mynah_slm_forward(&st, next_id(&seed, vocab), NULL) != 0) { printf("error forward\n"); return 1; }
        uint32_t next = next_id(&seed, vocab);
        prompt_s += now() - t0;
        for (int i = 0; i < warmup; i++) {
            if (mynah_slm_forward(&st, next, st.logits) != 0) { printf("error forward\n"); return 1; }
            next = argmax(st.logits, vocab);
        }
        t0 = now();
        for (int i = 0; i < steps; i++) {
            if (mynah_slm_forward(&st, next, st.logits) != 0) { printf("error forward\n"); return 1; }
            next = argmax(st.logits, vocab);
        }
        decode_s += now() - t0;
    }
    printf("ok %d %.6f %d %.6f\n", n_seqs * steps, decode_s, n_seqs * (prompt_len - 1), prompt_s);
    mynah_slm_state_free(&st);
    mynah_slm_free(m);
    return 0;
}
