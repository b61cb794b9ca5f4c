/* Host-side runtime of mynah_slm_b200: the cache's books (pages, slots, what each live sequence holds in
 * every storage group) and the packing of a step's batch description. Plain C interface; nothing here touches
 * a device. Functions that can fail return -1 (or NULL) and leave a message for mynah_host_last_error(); the
 * library never prints.
 *
 * The reference keeps one sequence with one counter (mynah-slm src/arch_qwen3.h:25, n_past) and has no such
 * interface (include/mynah_slm.h:38-47 exposes load/free/accessors only).
 */
#ifndef MYNAH_SLM_B200_HOST_H
#define MYNAH_SLM_B200_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Positions a page of the cache holds. Defined here and nowhere else: the kernels include this header and
 * Python asks mynah_page_tokens(). */
#define MYNAH_PAGE_TOKENS 64
int mynah_page_tokens(void);

const char* mynah_host_last_error(void);

/* out[i] = (float)(mean + std * normal(seed, tensor_key, i)), i < n, stored as float32 (dtype 0) or bfloat16
 * (dtype 1): the random-weights mode on the host. The numbers are those of mynah_random_normal.h, which the
 * device's mynah_randn_fill evaluates too. */
int mynah_randn_fill_host(void* out, int dtype, long long n, unsigned long long seed, unsigned long long tensor_key,
                          double mean, double std);

/* ---- a pool of pages 0..n-1: freed pages are the next handed out; every page knows its owner */
typedef struct mynah_pool mynah_pool;
mynah_pool* mynah_pool_create(int n_pages);
void mynah_pool_destroy(mynah_pool*);
int mynah_pool_take(mynah_pool*, int n, int owner, int32_t* pages_out);          /* all n or none */
int mynah_pool_give_back(mynah_pool*, const int32_t* pages, int n, int owner);
int mynah_pool_owner(const mynah_pool*, int page);                               /* -1: free, -2: no such page */
int mynah_pool_n_free(const mynah_pool*);
int mynah_pool_n_pages(const mynah_pool*);

/* ---- sequence slots */
typedef struct mynah_slots mynah_slots;
mynah_slots* mynah_slots_create(int n_slots);
void mynah_slots_destroy(mynah_slots*);
int mynah_slots_take(mynah_slots*);
int mynah_slots_give_back(mynah_slots*, int slot);
int mynah_slots_in_use(const mynah_slots*, int slot);
int mynah_slots_n_free(const mynah_slots*);
int mynah_slots_n_slots(const mynah_slots*);

/* ---- what the live sequences hold. windows[g]: 0 keeps every position, W keeps the last W */
typedef struct mynah_books mynah_books;
mynah_books* mynah_books_create(int n_groups, const int32_t* windows, int n_pages, int max_seqs);
void mynah_books_destroy(mynah_books*);
int mynah_books_open(mynah_books*);                                              /* a slot */
int mynah_books_close(mynah_books*, int slot);
int mynah_books_length(const mynah_books*, int slot);                            /* -1: not open */
int mynah_books_pages_needed(const mynah_books*, int slot, int n_new);
int mynah_books_reserve(mynah_books*, int slot, int n_new);                      /* pages for n_new more positions, in every group or in none */
int mynah_books_commit(mynah_books*, int slot, int n_new);                       /* the positions are written; windowed groups give pages back */
int mynah_books_held(const mynah_books*, int slot, int group, int32_t* pages_out, int cap, int32_t* base_out);   /* count */
int mynah_books_live_slots(const mynah_books*, int32_t* out, int cap);           /* count, ascending */
const mynah_pool* mynah_books_pool(const mynah_books*, int group);
const mynah_slots* mynah_books_slots(const mynah_books*);

/* ---- one step's batch description, packed into one int32 buffer (the layout of engine/context.py).
 * off[] holds the offsets of tokens, tok_seq, tok_pos, cu_q, kv_len, slots, want, then indptr, base, ids for each
 * group; T, B, W and ids_cap[g] are the capacities (padding is written up to them). Entry i brings n_tok[i]
 * tokens (consecutive in tokens[]) for slot slot[i] and wants n_want[i] of their places (consecutive in want[],
 * relative to the entry's first token). Returns the longest entry, the number of wanted rows through *n_rows. */
int mynah_step_fill(const mynah_books*, int32_t* buf, const int32_t* off, int T, int B, int W, const int32_t* ids_cap,
                    int n_entries, const int32_t* slot, const int32_t* n_tok, const int32_t* tokens,
                    const int32_t* n_want, const int32_t* want, int32_t* n_rows);

/* ---- one decoded token for each of n live sequences, in one call: checks (slots open and distinct, token ids below
 * `vocab`, lengths below `max_positions`), a page for the new position in every group, and the step's description
 * as mynah_step_fill writes it (no wanted rows: a decode graph returns every row). Returns the longest sequence
 * after the step. mynah_books_commit_many advances the sequences once the step has been launched. */
int mynah_decode_prepare(mynah_books*, int n, const int32_t* slot, const int32_t* token, int vocab, int max_positions,
                         int32_t* buf, const int32_t* off, int T, int B, int W, const int32_t* ids_cap);
int mynah_books_commit_many(mynah_books*, int n, const int32_t* slot, int n_new);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif
