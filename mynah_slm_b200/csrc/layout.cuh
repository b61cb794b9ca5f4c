// Layout of the paged key/value cache and of a step's batch description, as
// the kernels see them.
//
// Storage of one cache entry (one run of a layer): K and V are each
// [n_pages][kv_heads][PAGE_TOKENS][head_dim]. A sequence holds a list of
// pages; logical page p of sequence b (positions [p*64, p*64+64)) is
// page_ids[page_indptr[b] + p - page_base[b]]. page_base is 0 for a group
// that keeps all keys; a windowed group gives back the pages that have left
// the window and page_base counts them.
#pragma once

#include "common.cuh"
#include "../include/mynah_slm_b200_host.h"      // MYNAH_PAGE_TOKENS: the one definition of a page's size

constexpr int PAGE_TOKENS = MYNAH_PAGE_TOKENS;

// Bits of the status word that kernels set instead of touching memory they
// were not given. The host reads the word when it fetches a step's results.
enum MynahStatus : int {
    MYNAH_ST_PAGE_RANGE = 1,      // a position maps to no page of its sequence
    MYNAH_ST_POS_RANGE = 2,       // a position lies outside the rotation table
    MYNAH_ST_TOKEN_RANGE = 4,     // a token id lies outside the vocabulary
    MYNAH_ST_SPLIT_RANGE = 8,     // a decode launch has fewer page splits than a sequence has visible pages
    MYNAH_ST_TIMEOUT = 16,        // a bounded wait inside a kernel ran out
};

struct PageTable {
    const int* indptr;    // [B+1]
    const int* ids;       // [indptr[B]]
    const int* base;      // [B] first logical page that is still held
    int n_pages;          // pages in the pool (bound of every id)
};

// Index of the physical page that holds position `pos` of sequence b, or -1.
__device__ __forceinline__ int page_of(const PageTable& pt, int b, int pos) {
    const int lp = pos / PAGE_TOKENS - pt.base[b];
    const int lo = pt.indptr[b], hi = pt.indptr[b + 1];
    if (lp < 0 || lo + lp >= hi) return -1;
    const int id = pt.ids[lo + lp];
    return (id >= 0 && id < pt.n_pages) ? id : -1;
}
