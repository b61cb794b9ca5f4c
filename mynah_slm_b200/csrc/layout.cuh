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

// The query tiles of a step's sequences are numbered one after another, sequence by sequence, a sequence's last
// (longest) tile first. Finds tile number `flat`: its sequence and its tile within the sequence; false when the step
// has fewer tiles (a grid is sized for the most tiles that the step's rows can make: rows / tile_rows + sequences,
// since a captured step knows its rows but not how they divide). Warp 0 takes a prefix sum over the sequences' tile
// counts, 32 sequences at a time; every thread of the CTA must call this (it synchronises the CTA).
__device__ __forceinline__ bool find_query_tile(const int* __restrict__ cu_q, int B, int tile_rows, int flat, int& b, int& tile) {
    __shared__ int found_s[2];
    if (B == 1) {                                                    // one sequence: nothing to look for
        const int tiles = (cu_q[1] - cu_q[0] + tile_rows - 1) / tile_rows;
        b = 0;
        tile = tiles - 1 - flat;
        return flat < tiles;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        int found_b = -1, found_t = 0, base = 0;
        for (int b0 = 0; b0 < B && found_b < 0; b0 += 32) {
            const int bb = b0 + lane;
            const int tiles = bb < B ? (cu_q[bb + 1] - cu_q[bb] + tile_rows - 1) / tile_rows : 0;
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int excl = incl - tiles;
            const unsigned hit = __ballot_sync(0xffffffffu, tiles > 0 && flat >= base + excl && flat < base + incl);
            if (hit != 0u) {
                const int src = __ffs(hit) - 1;
                found_b = b0 + src;
                found_t = __shfl_sync(0xffffffffu, tiles, src) - 1 - (flat - base - __shfl_sync(0xffffffffu, excl, src));
            }
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            found_s[0] = found_b;
            found_s[1] = found_t;
        }
    }
    __syncthreads();
    b = found_s[0];
    tile = found_s[1];
    return b >= 0;
}

// Index of the physical page that holds position `pos` of sequence b, or -1.
__device__ __forceinline__ int page_of(const PageTable& pt, int b, int pos) {
    const int lp = pos / PAGE_TOKENS - pt.base[b];
    const int lo = pt.indptr[b], hi = pt.indptr[b + 1];
    if (lp < 0 || lo + lp >= hi) return -1;
    const int id = pt.ids[lo + lp];
    return (id >= 0 && id < pt.n_pages) ? id : -1;
}
