// Decode attention on tensor cores, for bfloat16 and head sizes 64 and 128.
//
// Same contract as the general split kernel of attn_decode.cu: one CTA per
// (page, kv head, sequence) writes the partial result of the sequence's s-th
// visible page (unnormalised output, running maximum, sum) to scratch, and the
// combine step merges a sequence's pages in page order. The difference is how
// a page is processed: its K and V tiles (64 keys x head_dim, contiguous in
// the paged cache) are copied to shared memory with 16-byte asynchronous
// copies into a swizzled layout; the scores of all query heads of the group
// (up to 16) against the 64 keys are one small matrix product on the tensor
// cores (mma.sync m16n8k16, bf16 in, fp32 out), the softmax of the page is
// fp32, and probabilities times V is a second product with the probabilities
// rounded to bf16. Keys outside the visible range are never copied: their
// rows are zero-filled, so stale contents of a page cannot reach a product.
//
// score = dot * (1/sqrtf(head_dim)), maximum subtracted
// (mynah-slm src/kernels.c:228-250, :207-220).
#include "layout.cuh"
#include "head_prep.cuh"
#include "tcgen05.cuh"

#include <stdlib.h>

namespace {

constexpr int KEYS = PAGE_TOKENS;     // 64 keys per CTA
constexpr int WARPS = 4;
constexpr int MAX_G = 16;             // query heads per kv head that one MMA tile holds
constexpr int MERGE_MAX_BYTES = KEYS * 64 * 2;   // the merge's weights: (heads per group) * (pages) floats; the smaller K tile holds them

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;     // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct TcArgs {
    int H, KV, ldq;
    int window, S;
    float scale;
};

// Byte offset of 16-byte chunk c of row r in a tile whose rows hold CH chunks:
// the low three bits of the chunk index are xor-ed with the row, so the eight
// rows of an 8x8 matrix fall into eight different bank groups.
template <int CH> __device__ __forceinline__ int swz(int r, int c) { return (r * CH + (c ^ (r & 7))) * 16; }

// Where 16-byte chunk c of row r of a [64 keys x HD] tile lies in shared memory.
// TileSwz: as the 16-byte asynchronous copies of this file lay it out (rows of HD / 8 chunks).
// TileTma: as a TMA copy with the 128-byte swizzle leaves it: halves of 64 columns one after the other, rows of 128 bytes.
template <int HD> struct TileSwz {
    static __device__ __forceinline__ int off(int r, int c) { return swz<HD / 8>(r, c); }
};
template <int HD> struct TileTma {
    static __device__ __forceinline__ int off(int r, int c) { return (c >> 3) * (KEYS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4); }
};
// Who works on a page together: the whole CTA, or the four consumer warps of the streaming kernel (its fifth warp
// feeds them and must not be waited for).
struct SyncCta {
    static __device__ __forceinline__ void sync() { __syncthreads(); }
};
struct SyncConsumers {
    static __device__ __forceinline__ void sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
};

// One visible page of one (sequence, kv head): what a CTA of the one-shot kernel, or one turn of the persistent
// kernel's loop, works on.
struct PageJob {
    int s, g, b;                      // index among the sequence's visible pages, kv head, sequence
    int page;                         // physical page
    int k_first, k_last;              // rows of the tile in use
    size_t row0;                      // partial of head g*G+i: row0 + i*S
    bool empty;                       // nothing of this page is visible
};

template <int HD>
__device__ __forceinline__ PageJob page_job(int s, int g, int b, const int* __restrict__ kv_len, const PageTable& pt,
                                            const TcArgs& a, int* __restrict__ status, bool reporter) {
    PageJob j;
    j.s = s; j.g = g; j.b = b; j.page = -1; j.k_first = 0; j.k_last = -1;
    const int G = a.H / a.KV;
    const int hi = kv_len[b];
    const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
    int key_begin = 0, key_end = 0;
    if (hi > 0) {
        const int pg0 = lo / PAGE_TOKENS, pg1 = (hi - 1) / PAGE_TOKENS + 1;
        if (pg1 - pg0 > a.S && reporter && s == 0) atomicOr(status, MYNAH_ST_SPLIT_RANGE);
        const int mp = pg0 + s;
        if (mp < pg1) {
            key_begin = max(lo, mp * PAGE_TOKENS);
            key_end = min(hi, (mp + 1) * PAGE_TOKENS);
            j.page = page_of(pt, b, mp * PAGE_TOKENS);
            if (j.page < 0) {
                if (reporter) atomicOr(status, MYNAH_ST_PAGE_RANGE);
                key_end = key_begin;
            }
        }
    }
    j.row0 = ((size_t)b * a.H + (size_t)g * G) * a.S + s;
    j.empty = key_begin >= key_end;
    if (!j.empty) {
        j.k_first = key_begin % PAGE_TOKENS;
        j.k_last = (key_end - 1) % PAGE_TOKENS;
    }
    return j;
}

__device__ __forceinline__ void write_empty_partial(const PageJob& j, const TcArgs& a, float* __restrict__ part_ml) {
    const int G = a.H / a.KV;
    for (int i = threadIdx.x; i < G; i += blockDim.x) {
        part_ml[(j.row0 + (size_t)i * a.S) * 2] = -INFINITY;
        part_ml[(j.row0 + (size_t)i * a.S) * 2 + 1] = 0.f;
    }
}

// The page's K tile, then its V tile, each as its own copy group. Rows that are not visible are zero-filled.
template <int HD>
__device__ __forceinline__ void issue_page_copies(const PageJob& j, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                                  const TcArgs& a, uint32_t k_base, uint32_t v_base) {
    constexpr int CH = HD / 8;
    const bf16* k_src = k_cache + ((size_t)j.page * a.KV + j.g) * PAGE_TOKENS * HD;
    const bf16* v_src = v_cache + ((size_t)j.page * a.KV + j.g) * PAGE_TOKENS * HD;
    for (int i = threadIdx.x; i < KEYS * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(k_base + swz<CH>(r, c), k_src + (size_t)r * HD + c * 8, r >= j.k_first && r <= j.k_last);
    }
    cp_async_commit();
    for (int i = threadIdx.x; i < KEYS * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(v_base + swz<CH>(r, c), v_src + (size_t)r * HD + c * 8, r >= j.k_first && r <= j.k_last);
    }
    cp_async_commit();
}

// Q as the A operand: rows = query heads of the group (zero beyond G), straight from global memory.
template <int HD>
__device__ __forceinline__ void load_q_fragments(const PageJob& j, const bf16* __restrict__ q, const TcArgs& a, uint32_t (&qa)[HD / 16][4]) {
    const int G = a.H / a.KV;
    const int lane = threadIdx.x & 31;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    const bf16* q0 = q + (size_t)j.b * a.ldq + (size_t)(j.g * G) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
        const int col = ks * 16 + c0;
        qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col) : 0u;
        qa[ks][1] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col) : 0u;
        qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col + 8) : 0u;
        qa[ks][3] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col + 8) : 0u;
    }
}

// The page's partial result. Where the K and V fragments come from is the caller's business: k_frag(ks, kb) gives
// the B fragments of this warp's 16 keys for dims [16 ks, 16 ks + 16), v_frag(ks, nt, vb) those of keys
// [16 ks, 16 ks + 16) for this warp's n-tiles nt and nt + 1; before_k() and before_v() run before the first use of
// each (waits and barriers, if the fragments still lie in shared memory). The arithmetic, and so every bit of the
// result, is the same whoever provides them.
template <int HD, class SYNC, class KFRAG, class VFRAG, class BEFORE_K, class BEFORE_V>
__device__ __forceinline__ void compute_page_core(const PageJob& job, const uint32_t (&qa)[HD / 16][4], const TcArgs& a,
                                                  KFRAG k_frag, VFRAG v_frag, BEFORE_K before_k, BEFORE_V before_v,
                                                  bf16* p_s, float (*red_m)[MAX_G], float (*red_l)[MAX_G],
                                                  float* __restrict__ part_o, float* __restrict__ part_ml) {
    constexpr int KSTEPS = HD / 16, NT = HD / 32;
    const int G = a.H / a.KV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k_first = job.k_first, k_last = job.k_last;
    const size_t row0 = job.row0;

    before_k();

    // ---- scores: warp w takes keys [16w, 16w+16): two n-tiles of 8 keys
    float sc[2][4] = {};
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
        uint32_t kb[4];
        k_frag(ks, kb);
        mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
        mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
    }
    // C layout: sc[t][0..1] -> head lane/4, keys 16w + 8t + (lane%4)*2 + {0,1}; sc[t][2..3] -> head lane/4 + 8
    const int hrow = lane >> 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int key = warp * 16 + t * 8 + (lane & 3) * 2 + (e & 1);
            const bool vis = key >= k_first && key <= k_last;
            sc[t][e] = vis ? sc[t][e] * a.scale : -INFINITY;
            mx[e >> 1] = fmaxf(mx[e >> 1], sc[t][e]);
        }
#pragma unroll
    for (int j = 0; j < 2; j++) {
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 1));
        mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 2));
    }
    if ((lane & 3) == 0) {
        red_m[warp][hrow] = mx[0];
        red_m[warp][hrow + 8] = mx[1];
    }
    SYNC::sync();
    float m[2], l[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int h = hrow + 8 * j;
        m[j] = fmaxf(fmaxf(red_m[0][h], red_m[1][h]), fmaxf(red_m[2][h], red_m[3][h]));   // finite: a visible key exists
    }
    // probabilities: fp32 for the sum, rounded to bf16 for the second product
#pragma unroll
    for (int t = 0; t < 2; t++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float p0 = expf(sc[t][2 * j] - m[j]), p1 = expf(sc[t][2 * j + 1] - m[j]);   // exp(-inf) = 0
            l[j] += p0 + p1;
            const int h = hrow + 8 * j, key = warp * 16 + t * 8 + (lane & 3) * 2;
            const __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
            // p_s rows hold 64 keys = 8 chunks; same swizzle as the tiles
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<unsigned char*>(p_s) + swz<8>(h, key >> 3) + (key & 7) * 2) = pp;
        }
    }
#pragma unroll
    for (int j = 0; j < 2; j++) {
        l[j] += __shfl_xor_sync(0xffffffffu, l[j], 1);
        l[j] += __shfl_xor_sync(0xffffffffu, l[j], 2);
    }
    if ((lane & 3) == 0) {
        red_l[warp][hrow] = l[0];
        red_l[warp][hrow + 8] = l[1];
    }
    before_v();                                       // (a barrier: the probabilities and the sums are in shared memory)

    // ---- output: warp w takes dims [w*HD/4, (w+1)*HD/4): HD/32 n-tiles of 8, four k-steps of 16 keys
    float oc[NT][4] = {};
    {
        const uint32_t p_base = smem_u32(p_s);
        const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ks++) {
            uint32_t pa[4];
            // A operand (P, row-major [head][key]): matrices 0: heads 0-7, keys k0..+7; 1: heads 8-15, same keys;
            // 2: heads 0-7, keys +8; 3: heads 8-15, keys +8
            ldmatrix_x4(pa, p_base + swz<8>((mat & 1) * 8 + rr, ks * 2 + (mat >> 1)));
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t vb[4];
                v_frag(ks, nt, vb);
                mma_bf16(oc[nt], pa, vb[0], vb[1]);
                mma_bf16(oc[nt + 1], pa, vb[2], vb[3]);
            }
        }
    }
    // ---- write the partial: rows of heads < G
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int h = hrow + 8 * j;
        if (h < G) {
            float* o = part_o + (row0 + (size_t)h * a.S) * HD;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int d = warp * (HD / 4) + nt * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(o + d) = make_float2(oc[nt][2 * j], oc[nt][2 * j + 1]);
            }
        }
    }
    if (tid < G) {
        const float ls = (red_l[0][tid] + red_l[1][tid]) + (red_l[2][tid] + red_l[3][tid]);
        const float mm = fmaxf(fmaxf(red_m[0][tid], red_m[1][tid]), fmaxf(red_m[2][tid], red_m[3][tid]));
        part_ml[(row0 + (size_t)tid * a.S) * 2] = mm;
        part_ml[(row0 + (size_t)tid * a.S) * 2 + 1] = ls;
    }
}

// The fragments of a page's tiles in shared memory, as compute_page_core wants them.
// K (non-transposed load): matrices 0: keys 0-7 of the warp's 16, dims k0..k0+7; 1: keys 0-7, dims +8; 2: keys 8-15,
// dims k0; 3: keys 8-15, dims +8. V [key][dim] (transposed load): matrices 0: keys k0..+7, dims n0..+7; 1: keys +8,
// same dims; 2: keys k0..+7, dims n0+8; 3: keys +8, dims n0+8.
template <int HD, class TILE>
__device__ __forceinline__ void load_k_frag(uint32_t k_base, int ks, uint32_t (&kb)[4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mat = lane >> 3, rr = lane & 7;
    ldmatrix_x4(kb, k_base + TILE::off(warp * 16 + (mat >> 1) * 8 + rr, ks * 2 + (mat & 1)));
}
template <int HD, class TILE>
__device__ __forceinline__ void load_v_frag(uint32_t v_base, int ks, int nt, uint32_t (&vb)[4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mat = lane >> 3, rr = lane & 7;
    ldmatrix_x4_trans(vb, v_base + TILE::off(ks * 16 + (mat & 1) * 8 + rr, warp * (HD / 32) + nt + (mat >> 1)));
}

// From the tiles in shared memory. PENDING_K / PENDING_V: copy groups that may still be in flight when the K tile,
// then the V tile, are needed (those of later pages). Ends with the CTA in step.
template <int HD, int PENDING_K, int PENDING_V>
__device__ __forceinline__ void compute_page(const PageJob& job, const uint32_t (&qa)[HD / 16][4], const TcArgs& a,
                                             uint32_t k_base, uint32_t v_base, bf16* p_s, float (*red_m)[MAX_G], float (*red_l)[MAX_G],
                                             float* __restrict__ part_o, float* __restrict__ part_ml) {
    compute_page_core<HD, SyncCta>(
        job, qa, a,
        [&](int ks, uint32_t (&kb)[4]) { load_k_frag<HD, TileSwz<HD>>(k_base, ks, kb); },
        [&](int ks, int nt, uint32_t (&vb)[4]) { load_v_frag<HD, TileSwz<HD>>(v_base, ks, nt, vb); },
        [&]() { cp_async_wait<PENDING_K>(); __syncthreads(); },       // K has landed (V may still be in flight)
        [&]() { cp_async_wait<PENDING_V>(); __syncthreads(); },       // V has landed
        p_s, red_m, red_l, part_o, part_ml);
}

// One CTA a page; six CTAs an SM cover one another's waits. (Persistent CTAs that prefetch their next page were
// built and measured slower: 5.7 against 3.9 ms a step at batch 64; three CTAs an SM, and each turn of the loop
// pays the chain of dependent reads that finds its next page.)
template <int HD> __device__ __forceinline__ void merge_pages(const float* __restrict__, const float* __restrict__, bf16* __restrict__,
                                                              size_t, int, int, int, float*, float*, float*);

// MERGE: the CTA that finishes a (sequence, kv head) last also merges its pages (a count per pair, zero before the
// first launch and left zero by every launch), which saves the merge's launch; without it the merge is a launch
// of its own with a CTA per head.
template <int HD, bool MERGE>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                      const int* __restrict__ kv_len, PageTable pt, TcArgs a,
                      float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ status,
                      unsigned* __restrict__ counters, bf16* __restrict__ out, int ldo) {
    __shared__ __align__(128) unsigned char k_s[KEYS * HD * 2];     // reused by the merge for the pages' weights
    __shared__ __align__(128) unsigned char v_s[KEYS * HD * 2];     // reused by the merge for its series
    __shared__ __align__(16) bf16 p_s[MAX_G * KEYS];  // probabilities [head][key], rows of 8 chunks, swizzled
    __shared__ float red_m[WARPS][MAX_G], red_l[WARPS][MAX_G];
    __shared__ int last_flag;
    griddep_launch();
    griddep_wait();
    const PageJob job = page_job<HD>(blockIdx.x, blockIdx.y, blockIdx.z, kv_len, pt, a, status, threadIdx.x == 0);
    if (job.empty) {
        write_empty_partial(job, a, part_ml);
        if (!MERGE) return;
    } else {
        issue_page_copies<HD>(job, k_cache, v_cache, a, smem_u32(k_s), smem_u32(v_s));
        uint32_t qa[HD / 16][4];
        load_q_fragments<HD>(job, q, a, qa);
        compute_page<HD, 1, 0>(job, qa, a, smem_u32(k_s), smem_u32(v_s), p_s, red_m, red_l, part_o, part_ml);
    }
    if (MERGE) {
        const int b = job.b, g = job.g, G = a.H / a.KV;
        __syncthreads();                              // the CTA's partial is written ...
        if (threadIdx.x == 0) {
            unsigned old;                             // ... and released with the count (the fence is cumulative)
            asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;\n" : "=r"(old) : "l"(counters + (size_t)b * a.KV + g) : "memory");
            last_flag = old == gridDim.x - 1;
            if (last_flag) counters[(size_t)b * a.KV + g] = 0;
        }
        __syncthreads();
        if (!last_flag) return;
        const int hi = kv_len[b];
        const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
        const int n_vis = hi > 0 ? min(a.S, (hi - 1) / PAGE_TOKENS + 1 - lo / PAGE_TOKENS) : 0;
        merge_pages<HD>(part_o, part_ml, out + (size_t)b * ldo + (size_t)g * G * HD, ((size_t)b * a.H + (size_t)g * G) * a.S,
                        G, a.S, n_vis, reinterpret_cast<float*>(k_s), reinterpret_cast<float*>(v_s), red_m[0]);
    }
}

// Merge of the pages of one (sequence, kv head) by a CTA of WARPS warps: the G heads of the group, n_vis pages.
// A warp computes a head's weights exp(m_s - max) and the sum of the weighted sums; the output rows are added
// up in NS interleaved series (series k takes pages k, k + NS, ...) that are then added in order. The order
// depends on the number of pages alone, so a sequence gets the same bits in every batch and from either
// kernel that calls this. `w_s`: G * S floats, `acc_s`: NS * HD floats, `inv_s`: MAX_G floats, all shared.
template <int HD>
__device__ __forceinline__ void merge_pages(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            bf16* __restrict__ out_row, size_t r0g, int G, int S, int n_vis,
                                            float* w_s, float* acc_s, float* inv_s) {
    // (G may also be 1 with r0g and out_row pointing at one head: a head's arithmetic does not involve the others.)
    constexpr int LPR = HD / 4, NS = WARPS * 32 / LPR;
    constexpr int AHEAD = 8;                          // output rows a thread fetches before it has their weights
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ld4 = tid % LPR, slot = tid / LPR;
    // the first head's output rows are on their way while the weights are worked out
    float4 o_first[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; k++) {
        const int s2 = slot + k * NS;
        o_first[k] = s2 < n_vis ? __ldcg(reinterpret_cast<const float4*>(part_o + (r0g + s2) * HD) + ld4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int i = warp; i < G; i += WARPS) {
        const size_t r0h = r0g + (size_t)i * S;
        // a lane keeps the pages' (maximum, sum) pairs it has read: up to 4 of them (128 pages), else it reads again
        float2 ml_r[4];
        float mmax = -INFINITY;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int s2 = lane + 32 * k;
            ml_r[k] = s2 < n_vis ? __ldcg(reinterpret_cast<const float2*>(part_ml + (r0h + s2) * 2)) : make_float2(-INFINITY, 0.f);
            mmax = fmaxf(mmax, ml_r[k].x);
        }
        for (int s2 = lane + 128; s2 < n_vis; s2 += 32) mmax = fmaxf(mmax, __ldcg(part_ml + (r0h + s2) * 2));
        mmax = warp_max(mmax);
        float ls = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int s2 = lane + 32 * k;
            if (s2 < n_vis) {
                const float w = ml_r[k].x == -INFINITY ? 0.f : expf(ml_r[k].x - mmax);
                w_s[i * S + s2] = w;
                ls = fmaf(ml_r[k].y, w, ls);
            }
        }
        for (int s2 = lane + 128; s2 < n_vis; s2 += 32) {
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (r0h + s2) * 2));
            const float w = ml.x == -INFINITY ? 0.f : expf(ml.x - mmax);
            w_s[i * S + s2] = w;
            ls = fmaf(ml.y, w, ls);
        }
        ls = warp_sum(ls);
        if (lane == 0) inv_s[i] = ls > 0.f ? 1.0f / ls : 0.f;
    }
    __syncthreads();
    for (int i = 0; i < G; i++) {
        const size_t r0h = r0g + (size_t)i * S;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        auto add = [&](const float4& o, float w) {
            if (w != 0.f) {                           // a page without visible keys wrote no output row
                acc.x = fmaf(o.x, w, acc.x); acc.y = fmaf(o.y, w, acc.y);
                acc.z = fmaf(o.z, w, acc.z); acc.w = fmaf(o.w, w, acc.w);
            }
        };
        int s2 = slot;
        if (i == 0) {
#pragma unroll
            for (int k = 0; k < AHEAD; k++, s2 += NS)
                if (s2 < n_vis) add(o_first[k], w_s[s2]);
        }
#pragma unroll 8
        for (; s2 < n_vis; s2 += NS)
            add(__ldcg(reinterpret_cast<const float4*>(part_o + (r0h + s2) * HD) + ld4), w_s[i * S + s2]);
        reinterpret_cast<float4*>(acc_s + slot * HD)[ld4] = acc;
        __syncthreads();
        for (int d = tid; d < HD; d += WARPS * 32) {
            float os = 0.f;
#pragma unroll
            for (int k = 0; k < NS; k++) os += acc_s[k * HD + d];
            out_row[(size_t)i * HD + d] = __float2bfloat16_rn(os * inv_s[i]);
        }
        __syncthreads();
    }
}

// The merge as a launch of its own: one CTA per (head, sequence).
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                         const int* __restrict__ kv_len, int window, int H, int S, int ldo) {
    constexpr int NS = WARPS * 32 / (HD / 4);
    extern __shared__ float w_s[];
    __shared__ __align__(16) float acc_s[NS * HD];
    __shared__ float inv_s[MAX_G];
    const int h = blockIdx.x, b = blockIdx.y;
    griddep_wait();
    griddep_launch_small();
    const int hi = kv_len[b];
    const int lo = window > 0 ? max(0, hi - window) : 0;
    const int n_vis = hi > 0 ? min(S, (hi - 1) / PAGE_TOKENS + 1 - lo / PAGE_TOKENS) : 0;
    merge_pages<HD>(part_o, part_ml, out + (size_t)b * ldo + (size_t)h * HD, ((size_t)b * H + h) * S, 1, S, n_vis, w_s, acc_s, inv_s);
}

// ---------------------------------------------------------------------------------------------------------
// The whole attention of a decode step in one launch: what qk_norm_rope_store, the page kernel above and the
// combine kernel do one after the other. A CTA takes one visible page of one (sequence, kv head):
//   - it norms and rotates the group's query heads itself (fp32, rounded to bf16 as the separate pass stores them);
//   - the CTA whose page holds the new position norms and rotates the new k, copies the new v, writes both to
//     the cache and puts them into its tiles directly (the row is left out of the asynchronous copy, so the
//     cache is never read where this launch writes it);
//   - it writes its partial result, and the CTA that finishes a (sequence, kv head) last merges the pages in
//     page order. The order of the merge does not depend on which CTA does it.
// The counters are zero before the first launch and are left zero by every launch.
struct FusedArgs {
    int H, KV, ldq, ldo;
    int window, S;
    int n_pos, write_kv;
    float scale, qk_eps;
};

template <int HD, bool MERGE>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_fused_kernel(const bf16* __restrict__ qkv, VecRef q_gain, VecRef k_gain,
                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ tok_pos, const int* __restrict__ kv_len, PageTable pt,
                         bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, FusedArgs a,
                         float* __restrict__ part_o, float* __restrict__ part_ml, unsigned* __restrict__ counters,
                         bf16* __restrict__ out, int* __restrict__ status) {
    constexpr int CH = HD / 8, KSTEPS = HD / 16;
    constexpr int QLD = HD + 8;                       // padded row of the query tile: no bank conflicts on its loads
    __shared__ __align__(128) unsigned char k_s[KEYS * HD * 2];     // reused by the merge for the pages' weights
    __shared__ __align__(128) unsigned char v_s[KEYS * HD * 2];     // reused by the merge for its series
    __shared__ __align__(16) bf16 q_s[MAX_G * QLD];   // the queries; once they are in registers, the probabilities
    __shared__ float red_m[WARPS][MAX_G], red_l[WARPS][MAX_G];
    __shared__ int last_flag;
    bf16* p_s = q_s;
    static_assert(MAX_G * QLD >= MAX_G * KEYS, "the probabilities must fit where the queries were");

    const int s = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int G = a.H / a.KV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    griddep_launch();
    griddep_wait();
    const int hi = kv_len[b];
    const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
    const int pos = hi > 0 ? tok_pos[b] : 0;
    int key_begin = 0, key_end = 0, page = -1, n_vis = 0, mp = 0;
    if (hi > 0) {
        const int pg0 = lo / PAGE_TOKENS, pg1 = (hi - 1) / PAGE_TOKENS + 1;
        n_vis = min(pg1 - pg0, a.S);
        if (pg1 - pg0 > a.S && tid == 0 && s == 0) atomicOr(status, MYNAH_ST_SPLIT_RANGE);
        mp = pg0 + s;
        if (mp < pg1) {
            key_begin = max(lo, mp * PAGE_TOKENS);
            key_end = min(hi, (mp + 1) * PAGE_TOKENS);
            page = page_of(pt, b, mp * PAGE_TOKENS);
            if (page < 0) {
                if (tid == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
                key_end = key_begin;
            }
            if (cos_t != nullptr && (pos < 0 || pos >= a.n_pos)) {
                if (tid == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
                key_end = key_begin;
            }
        }
    }
    const size_t row0 = ((size_t)b * a.H + (size_t)g * G) * a.S + s;
    if (key_begin >= key_end) {
        for (int i = tid; i < G; i += blockDim.x) {
            part_ml[(row0 + (size_t)i * a.S) * 2] = -INFINITY;
            part_ml[(row0 + (size_t)i * a.S) * 2 + 1] = 0.f;
        }
    } else {
        const int k_first = key_begin % PAGE_TOKENS, k_last = (key_end - 1) % PAGE_TOKENS;
        const int r_new = (a.write_kv && pos >= mp * PAGE_TOKENS && pos < (mp + 1) * PAGE_TOKENS) ? pos % PAGE_TOKENS : -1;
        const size_t tile = ((size_t)page * a.KV + g) * PAGE_TOKENS * HD;
        const uint32_t k_base = smem_u32(k_s), v_base = smem_u32(v_s);
        for (int i = tid; i < KEYS * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            if (r != r_new) cp_async_16(k_base + swz<CH>(r, c), k_cache + tile + (size_t)r * HD + c * 8, r >= k_first && r <= k_last);
        }
        cp_async_commit();
        for (int i = tid; i < KEYS * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            if (r != r_new) cp_async_16(v_base + swz<CH>(r, c), v_cache + tile + (size_t)r * HD + c * 8, r >= k_first && r <= k_last);
        }
        cp_async_commit();

        // ---- the group's queries: norm, rotation, to shared memory as bf16; rows beyond G are zero.
        // Heads lie side by side in a warp (head_prep.cuh), as in the rope/store pass, whose bits these are.
        constexpr int LPH = HeadLanes<HD>::LPH, HPW = HeadLanes<HD>::HPW;
        const int sub = lane / LPH, li = lane % LPH;
        const bool rotate = cos_t != nullptr, has_gain = q_gain.p != nullptr;
        float rc[8], rs[8], qgv[8], kgv[8];
        if (rotate) load_rotation<HD>(cos_t, sin_t, pos, lane, rc, rs);
        if (has_gain) {
            load_gain8(q_gain, li * 8, qgv);
            load_gain8(k_gain, li * 8, kgv);
        }
        const bf16* qrow = qkv + (size_t)b * a.ldq;
        for (int hbase = warp * HPW; hbase < MAX_G; hbase += WARPS * HPW) {      // uniform over the warp
            const int h = hbase + sub;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (h < G) load8<bf16>(qrow + (size_t)(g * G + h) * HD + li * 8, v);
            head_norm_rotate<HD>(v, has_gain, qgv, a.qk_eps, rotate, rc, rs, lane);
            if (h >= G) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = 0.f;
            }
            if (h < MAX_G) store8<bf16>(q_s + h * QLD + li * 8, v);
        }
        // ---- the new position's k and v, by the CTA that has its page: to the cache and into the tiles
        if (r_new >= 0 && warp == WARPS - 1) {
            float kv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (sub == 0) load8<bf16>(qrow + (size_t)(a.H + g) * HD + li * 8, kv);
            head_norm_rotate<HD>(kv, has_gain, kgv, a.qk_eps, rotate, rc, rs, lane);    // the whole warp; one lane group holds the head
            if (sub == 0) {
                const uint4 vraw = *reinterpret_cast<const uint4*>(qrow + (size_t)(a.H + a.KV + g) * HD + li * 8);
                uint4 ko;
                __nv_bfloat162* kh = reinterpret_cast<__nv_bfloat162*>(&ko);
#pragma unroll
                for (int j = 0; j < 4; j++) kh[j] = __floats2bfloat162_rn(kv[2 * j], kv[2 * j + 1]);
                *reinterpret_cast<uint4*>(k_cache + tile + (size_t)r_new * HD + li * 8) = ko;
                *reinterpret_cast<uint4*>(v_cache + tile + (size_t)r_new * HD + li * 8) = vraw;
                *reinterpret_cast<uint4*>(k_s + swz<CH>(r_new, li)) = ko;       // a lane's eight elements are one 16-byte chunk
                *reinterpret_cast<uint4*>(v_s + swz<CH>(r_new, li)) = vraw;
            }
        }
        cp_async_wait<1>();                           // K has landed (V may still be in flight)
        __syncthreads();

        uint32_t qa[KSTEPS][4];
        {
            const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                const int col = ks * 16 + c0;
                qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_s + r0 * QLD + col);
                qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_s + (r0 + 8) * QLD + col);
                qa[ks][2] = *reinterpret_cast<const uint32_t*>(q_s + r0 * QLD + col + 8);
                qa[ks][3] = *reinterpret_cast<const uint32_t*>(q_s + (r0 + 8) * QLD + col + 8);
            }
        }
        // the page's partial result: the same code as the pages' kernel (the probabilities go where the queries were)
        PageJob job;
        job.s = s; job.g = g; job.b = b; job.page = page;
        job.k_first = k_first; job.k_last = k_last; job.row0 = row0; job.empty = false;
        const TcArgs ta{a.H, a.KV, a.ldq, a.window, a.S, a.scale};
        compute_page<HD, 1, 0>(job, qa, ta, k_base, v_base, p_s, red_m, red_l, part_o, part_ml);
    }

    if (!MERGE) return;                               // the merge is a launch of its own (a CTA a head)
    // ---- the CTA that finishes this (sequence, kv head) last merges the pages
    __syncthreads();                                  // the CTA's partial is written ...
    if (tid == 0) {
        unsigned old;                                 // ... and released with the count (the fence is cumulative)
        asm volatile("atom.add.acq_rel.gpu.u32 %0, [%1], 1;\n" : "=r"(old) : "l"(counters + (size_t)b * a.KV + g) : "memory");
        last_flag = old == gridDim.x - 1;
        if (last_flag) counters[(size_t)b * a.KV + g] = 0;
    }
    __syncthreads();
    if (!last_flag) return;
    merge_pages<HD>(part_o, part_ml, out + (size_t)b * a.ldo + (size_t)g * G * HD, ((size_t)b * a.H + (size_t)g * G) * a.S,
                    G, a.S, n_vis, reinterpret_cast<float*>(k_s), reinterpret_cast<float*>(v_s), red_m[0]);
}


// ---------------------------------------------------------------------------------------------------------
// The pages' kernel as a stream: persistent CTAs, fed by TMA.
//
// The same partial results as attn_decode_tc_kernel, page by page and bit for bit (the same compute_page on the
// same numbers), so the same merge follows. What differs is who fetches: a fifth warp walks the CTA's share of the
// step's pages (every sequence's visible pages times the kv heads, dealt out round-robin) ahead of the four
// warps that compute, looks each page up and has the TMA unit copy its K and V tiles (two boxes of 64 x 64 each for
// a head size of 128) and the group's query heads into the next free stage of a ring; an mbarrier per stage
// counts the bytes in. The computing warps never wait for a table lookup, and the memory system always has the
// next pages' requests while a page is worked on: that is what the one-page CTAs get from six CTAs an SM
// covering one another, without their launch, drain and tail. Keys outside the visible range arrive with the page
// (a copy is a whole tile): their scores are masked as before, and their rows of V are zeroed in shared memory
// before the second product, so that stale contents of a page cannot reach it.
struct StreamJob {
    int b, g, k_first, k_last, empty, partial;
    unsigned long long row0;
};

constexpr int STREAM_THREADS = (WARPS + 1) * 32;
constexpr int STREAM_MAX_SEQS = 1024;             // sequences whose page counts a CTA keeps in shared memory

template <int HD>
__host__ __device__ constexpr int stream_q_stride(int G) { return ((G * HD * 2 + 127) / 128) * 128; }

template <int HD, int STAGES>
__global__ void __launch_bounds__(STREAM_THREADS)
attn_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const bf16* __restrict__ q, const int* __restrict__ kv_len, PageTable pt, TcArgs a, int B,
                          float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ status) {
    using namespace tc5;
    constexpr int TILE = KEYS * HD * 2;
    constexpr int CH = HD / 8;
    const int G = a.H / a.KV;
    const int q_stride = stream_q_stride<HD>(G);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* tiles = smem;                                   // [STAGES][K tile, V tile]
    unsigned char* q_area = tiles + STAGES * 2 * TILE;             // [STAGES][q_stride]
    bf16* p_s = reinterpret_cast<bf16*>(q_area + STAGES * q_stride);
    float (*red_m)[MAX_G] = reinterpret_cast<float (*)[MAX_G]>(p_s + MAX_G * KEYS);
    float (*red_l)[MAX_G] = red_m + WARPS;
    StreamJob* jobs = reinterpret_cast<StreamJob*>(red_l + WARPS);
    uint64_t* bars = reinterpret_cast<uint64_t*>(jobs + STAGES);   // full[STAGES], empty[STAGES]
    int* cum = reinterpret_cast<int*>(bars + 2 * STAGES);          // cum[b]: visible pages of the sequences before b
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(smem_u32(&bars[i]), 1);
            mbar_init(smem_u32(&bars[STAGES + i]), WARPS);        // every computing warp gives a stage back itself
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    griddep_launch();
    griddep_wait();
    for (int b = tid; b < B; b += STREAM_THREADS) {
        const int hi = kv_len[b];
        const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
        int n = 0;
        if (hi > 0) {
            n = (hi - 1) / PAGE_TOKENS + 1 - lo / PAGE_TOKENS;
            if (n > a.S) {
                if (blockIdx.x == 0) atomicOr(status, MYNAH_ST_SPLIT_RANGE);
                n = a.S;
            }
        }
        cum[b + 1] = n;
    }
    __syncthreads();
    if (tid == 0) {
        cum[0] = 0;
        for (int b = 0; b < B; b++) cum[b + 1] += cum[b];
    }
    __syncthreads();
    const long long n_items = (long long)cum[B] * a.KV;             // kv head fastest: neighbours in memory go to neighbouring CTAs

    if (warp == WARPS) {
        // ---- the feeder
        if (lane == 0) {
            int b = 0;
            long long it = 0;
            for (long long item = blockIdx.x; item < n_items; item += gridDim.x, it++) {
                const int st = (int)(it % STAGES);
                const uint32_t parity = (uint32_t)((it / STAGES) & 1);
                if (!mbar_wait(smem_u32(&bars[STAGES + st]), parity ^ 1u)) {
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    break;
                }
                const int g = (int)(item % a.KV);
                const int pg = (int)(item / a.KV);
                while (pg >= cum[b + 1]) b++;
                const PageJob j = page_job<HD>(pg - cum[b], g, b, kv_len, pt, a, status, true);
                StreamJob sj;
                sj.b = b; sj.g = g; sj.k_first = j.k_first; sj.k_last = j.k_last; sj.empty = j.empty ? 1 : 0;
                sj.partial = (j.k_first > 0 || j.k_last < KEYS - 1) ? 1 : 0;
                sj.row0 = (unsigned long long)j.row0;
                jobs[st] = sj;
                const uint32_t full = smem_u32(&bars[st]);
                if (j.empty) {
                    mbar_arrive(full);
                    continue;
                }
                const uint32_t k_dst = smem_u32(tiles + (size_t)st * 2 * TILE), v_dst = k_dst + TILE;
                const uint32_t q_dst = smem_u32(q_area + (size_t)st * q_stride);
                const uint32_t q_bytes = (uint32_t)(G * HD * 2);
                mbar_expect_tx(full, 2 * TILE + q_bytes);
                const int y = (j.page * a.KV + g) * PAGE_TOKENS;
#pragma unroll
                for (int h = 0; h < HD / 64; h++) {
                    tma_load_2d(k_dst + h * (KEYS * 128), &map_k, h * 64, y, full);
                    tma_load_2d(v_dst + h * (KEYS * 128), &map_v, h * 64, y, full);
                }
                const bf16* q_src = q + (size_t)b * a.ldq + (size_t)(g * G) * HD;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(q_dst), "l"(q_src), "r"(q_bytes), "r"(full) : "memory");
            }
        }
        return;
    }

    // ---- the four warps that compute
    long long it = 0;
    for (long long item = blockIdx.x; item < n_items; item += gridDim.x, it++) {
        const int st = (int)(it % STAGES);
        const uint32_t parity = (uint32_t)((it / STAGES) & 1);
        if (!mbar_wait(smem_u32(&bars[st]), parity)) {
            if (tid == 0) atomicOr(status, MYNAH_ST_TIMEOUT);
            break;
        }
        const StreamJob sj = jobs[st];
        bool released = false;
        PageJob job;
        job.s = 0; job.g = sj.g; job.b = sj.b; job.page = 0;
        job.k_first = sj.k_first; job.k_last = sj.k_last; job.row0 = (size_t)sj.row0; job.empty = sj.empty != 0;
        if (job.empty) {
            for (int i = tid; i < G; i += WARPS * 32) {
                part_ml[(job.row0 + (size_t)i * a.S) * 2] = -INFINITY;
                part_ml[(job.row0 + (size_t)i * a.S) * 2 + 1] = 0.f;
            }
        } else {
            unsigned char* k_t = tiles + (size_t)st * 2 * TILE;
            unsigned char* v_t = k_t + TILE;
            if (sj.partial) {
                for (int i = tid; i < KEYS * CH; i += WARPS * 32) {
                    const int r = i / CH, c = i % CH;
                    if (r < job.k_first || r > job.k_last)
                        *reinterpret_cast<uint4*>(v_t + TileTma<HD>::off(r, c)) = make_uint4(0, 0, 0, 0);
                }
            }
            // Q as the A operand, from the stage (rows beyond the group are zero)
            uint32_t qa[HD / 16][4];
            {
                const bf16* q0 = reinterpret_cast<const bf16*>(q_area + (size_t)st * q_stride);
                const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    const int col = ks * 16 + c0;
                    qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col) : 0u;
                    qa[ks][1] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col) : 0u;
                    qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col + 8) : 0u;
                    qa[ks][3] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col + 8) : 0u;
                }
            }
            if (sj.partial) SyncConsumers::sync();                 // the zeroed rows of V are in place
            // this warp's fragments of both tiles into registers, and the stage goes back to the feeder at once: a
            // stage that is being computed on is a stage without a copy in flight
            uint32_t kf[HD / 16][4], vf[KEYS / 16][HD / 64][4];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ks++) load_k_frag<HD, TileTma<HD>>(smem_u32(k_t), ks, kf[ks]);
#pragma unroll
            for (int ks = 0; ks < KEYS / 16; ks++)
#pragma unroll
                for (int nt = 0; nt < HD / 32; nt += 2) load_v_frag<HD, TileTma<HD>>(smem_u32(v_t), ks, nt, vf[ks][nt / 2]);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[STAGES + st]));
            released = true;
            compute_page_core<HD, SyncConsumers>(
                job, qa, a,
                [&](int ks, uint32_t (&kb)[4]) { kb[0] = kf[ks][0]; kb[1] = kf[ks][1]; kb[2] = kf[ks][2]; kb[3] = kf[ks][3]; },
                [&](int ks, int nt, uint32_t (&vb)[4]) { vb[0] = vf[ks][nt / 2][0]; vb[1] = vf[ks][nt / 2][1]; vb[2] = vf[ks][nt / 2][2]; vb[3] = vf[ks][nt / 2][3]; },
                []() {}, []() { SyncConsumers::sync(); },
                p_s, red_m, red_l, part_o, part_ml);
        }
        if (!released && lane == 0) mbar_arrive(smem_u32(&bars[STAGES + st]));
        SyncConsumers::sync();                                     // the page's scratch (probabilities, sums) is free again
    }
}

template <int HD>
size_t stream_smem_bytes(int G, int stages, int B) {
    return 1024 + (size_t)stages * 2 * KEYS * HD * 2 + (size_t)stages * stream_q_stride<HD>(G) + MAX_G * KEYS * 2 +
           2 * WARPS * MAX_G * sizeof(float) + (size_t)stages * sizeof(StreamJob) + 2 * (size_t)stages * 8 + (size_t)(B + 1) * sizeof(int) + 16;
}

// 0: never, 1: where it pays (the default), 2: wherever it can run. MYNAH_ATTN_STREAM sets it at start,
// mynah_attn_decode_stream_mode() later (tests compare the two routes).
int g_stream_mode = -1;
int stream_mode() {
    if (g_stream_mode < 0) {
        const char* e = getenv("MYNAH_ATTN_STREAM");
        g_stream_mode = e != nullptr && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 1;
    }
    return g_stream_mode;
}
int stream_stages() {
    static const int n = [] {
        const char* e = getenv("MYNAH_ATTN_STREAM_STAGES");
        return e != nullptr && e[0] == '3' ? 3 : 2;
    }();
    return n;
}

template <int HD, int STAGES>
int launch_stream(const void* q, const void* k_cache, const void* v_cache, const int* kv_len, const PageTable& pt, const TcArgs& a,
                  int B, int n_pages, float* part_o, float* part_ml, int* status, cudaStream_t stream) {
    auto kern = attn_decode_stream_kernel<HD, STAGES>;
    const int G = a.H / a.KV;
    const size_t smem = stream_smem_bytes<HD>(G, STAGES, B);
    static size_t allowed = 0;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("attn_decode_tc (stream): %s", cudaGetErrorString(e));
        allowed = smem;
    }
    CUtensorMap mk, mv;
    if (tc5::make_map(&mk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)n_pages * a.KV * PAGE_TOKENS, HD, HD, PAGE_TOKENS, 64)) return -1;
    if (tc5::make_map(&mv, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)n_pages * a.KV * PAGE_TOKENS, HD, HD, PAGE_TOKENS, 64)) return -1;
    const int per_sm = (int)((227 * 1024) / (smem + 1024));
    const long long items = (long long)B * a.KV * a.S;
    const long long want = (long long)mynah_sm_count() * (per_sm < 1 ? 1 : per_sm);
    const unsigned grid = (unsigned)(items < want ? items : want);
    mynah_launch(kern, dim3(grid), dim3(STREAM_THREADS), smem, stream, mk, mv, (const bf16*)q, kv_len, pt, a, B, part_o, part_ml, status);
    return mynah_check_launch("attn_decode_tc (stream)");
}

}  // namespace

// Chooses between the one-page CTAs and the streaming kernel for the pages of a decode step: 0 never the stream,
// 1 where it pays, 2 wherever it can run. Returns the mode that was set before.
MYNAH_API int mynah_attn_decode_stream_mode(int mode) {
    const int before = stream_mode();
    if (mode >= 0 && mode <= 2) g_stream_mode = mode;
    return before;
}

// Whether the tensor-core kernel takes these sizes (bfloat16 only).
MYNAH_API int mynah_attn_decode_tc_supported(int H, int KV, int HD) {
    return (HD == 64 || HD == 128) && KV > 0 && H % KV == 0 && H / KV <= MAX_G;
}

// Same arguments and scratch layout as mynah_attn_decode; bfloat16 only. `counters`: B * KV words that are zero
// before the first call (every call leaves them zero), or null: with them the pages' kernel also merges, by the
// CTA that finishes a (sequence, kv head) last; without them the merge is a second launch. The result is the same.
MYNAH_API int mynah_attn_decode_tc(
    const void* q, void* out, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, float* scratch, unsigned* counters, int* status, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(mynah_attn_decode_tc_supported(H, KV, HD), "attn_decode_tc: H=%d KV=%d head_dim=%d is not taken by this kernel", H, KV, HD);
    MYNAH_REQUIRE(ldq % 8 == 0, "attn_decode_tc: query row stride %d must be a multiple of 8", ldq);
    MYNAH_REQUIRE(n_splits >= 1 && n_splits <= 65535 && B <= 65535 && KV <= 65535, "attn_decode_tc: launch too large");
    MYNAH_REQUIRE(scratch != nullptr, "attn_decode_tc: no scratch memory given");
    const TcArgs a{H, KV, ldq, window, n_splits, 1.0f / sqrtf((float)HD)};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)B * H * n_splits * HD;
    const dim3 grid(n_splits, KV, B);
    if (counters != nullptr) {
        MYNAH_REQUIRE((size_t)(H / KV) * n_splits * sizeof(float) <= MERGE_MAX_BYTES,
                      "attn_decode_tc: %d pages a sequence exceed what the merge holds", n_splits);
        if (HD == 128)
            mynah_launch(attn_decode_tc_kernel<128, true>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         kv_len, pt, a, part_o, part_ml, status, counters, (bf16*)out, ldo);
        else
            mynah_launch(attn_decode_tc_kernel<64, true>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         kv_len, pt, a, part_o, part_ml, status, counters, (bf16*)out, ldo);
        return mynah_check_launch("attn_decode_tc (merging)");
    }
    // The pages as a stream through persistent CTAs once there are many waves of one-page CTAs (six an SM); the
    // partial results are the same bits either way. Measured at the 0.6B shape: 64 sequences of 2,060 positions
    // 3.69 -> 3.63 ms a step, of 3,900 positions 6.03 -> 5.73; 16 sequences of 2,060 positions 1.74 -> 1.76 (so not there).
    const long long n_ctas = (long long)n_splits * KV * B;
    const bool as_stream = stream_mode() != 0 && B <= STREAM_MAX_SEQS && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 &&
                           ((uintptr_t)v_cache & 15) == 0 && (stream_mode() == 2 || n_ctas >= (long long)mynah_sm_count() * 6 * 16);
    if (as_stream) {
        int rc;
        if (HD == 128)
            rc = stream_stages() == 3 ? launch_stream<128, 3>(q, k_cache, v_cache, kv_len, pt, a, B, n_pages, part_o, part_ml, status, stream)
                                      : launch_stream<128, 2>(q, k_cache, v_cache, kv_len, pt, a, B, n_pages, part_o, part_ml, status, stream);
        else
            rc = stream_stages() == 3 ? launch_stream<64, 3>(q, k_cache, v_cache, kv_len, pt, a, B, n_pages, part_o, part_ml, status, stream)
                                      : launch_stream<64, 2>(q, k_cache, v_cache, kv_len, pt, a, B, n_pages, part_o, part_ml, status, stream);
        if (rc) return rc;
    } else {
        if (HD == 128)
            mynah_launch(attn_decode_tc_kernel<128, false>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         kv_len, pt, a, part_o, part_ml, status, (unsigned*)nullptr, (bf16*)nullptr, 0);
        else
            mynah_launch(attn_decode_tc_kernel<64, false>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         kv_len, pt, a, part_o, part_ml, status, (unsigned*)nullptr, (bf16*)nullptr, 0);
        if (mynah_check_launch("attn_decode_tc")) return -1;
    }
    const size_t dyn = (size_t)n_splits * sizeof(float);
    MYNAH_REQUIRE(dyn <= MERGE_MAX_BYTES, "attn_decode_tc: %d pages a sequence exceed what the merge holds", n_splits);
    if (HD == 128)
        mynah_launch(attn_decode_merge_kernel<128>, dim3(H, B), dim3(WARPS * 32), dyn, stream, part_o, part_ml, (bf16*)out, kv_len, window, H, n_splits, ldo);
    else
        mynah_launch(attn_decode_merge_kernel<64>, dim3(H, B), dim3(WARPS * 32), dyn, stream, part_o, part_ml, (bf16*)out, kv_len, window, H, n_splits, ldo);
    return mynah_check_launch("attn_decode_merge");
}

// The fused decode attention: q, k, v rows [B, (H + 2 KV) * HD] as the projection left them (with write_kv = 0
// only the q columns are read and the cache is taken as complete); gains may be null (no per-head norm), the
// tables may be null (no rotation; else the whole head is rotated). `counters`: B * KV words, zero before the
// first call. Scratch as mynah_attn_decode.
MYNAH_API int mynah_attn_decode_fused(
    const void* qkv, void* out, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* q_gain, const void* k_gain, int gain_dtype, float qk_eps,
    const float* cos_t, const float* sin_t, int n_pos, const int* tok_pos,
    void* k_cache, void* v_cache, int write_kv, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, float* scratch, unsigned* counters, int* status, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(mynah_attn_decode_tc_supported(H, KV, HD), "attn_decode_fused: H=%d KV=%d head_dim=%d is not taken by this kernel", H, KV, HD);
    MYNAH_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0, "attn_decode_fused: row strides %d, %d must be multiples of 8", ldq, ldo);
    MYNAH_REQUIRE(n_splits >= 1 && n_splits <= 65535 && B <= 65535 && KV <= 65535, "attn_decode_fused: launch too large");
    MYNAH_REQUIRE(scratch != nullptr, "attn_decode_fused: no scratch memory given");
    MYNAH_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "attn_decode_fused: the two rotation tables go together");
    MYNAH_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "attn_decode_fused: the two gains go together");
    MYNAH_REQUIRE((size_t)(H / KV) * n_splits * sizeof(float) <= MERGE_MAX_BYTES,
                  "attn_decode_fused: %d pages a sequence exceed what the merge holds", n_splits);
    const size_t dyn = 0;
    const FusedArgs a{H, KV, ldq, ldo, window, n_splits, n_pos, write_kv, 1.0f / sqrtf((float)HD), qk_eps};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)B * H * n_splits * HD;
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    const dim3 grid(n_splits, KV, B);
    if (counters == nullptr) {
        // without counters: the pages' CTAs do not merge; the merge follows as a launch of its own (the same bits)
        if (HD == 128)
            mynah_launch(attn_decode_fused_kernel<128, false>, grid, dim3(WARPS * 32), dyn, stream, (const bf16*)qkv, qg, kg, cos_t, sin_t, tok_pos,
                         kv_len, pt, (bf16*)k_cache, (bf16*)v_cache, a, part_o, part_ml, counters, (bf16*)out, status);
        else
            mynah_launch(attn_decode_fused_kernel<64, false>, grid, dim3(WARPS * 32), dyn, stream, (const bf16*)qkv, qg, kg, cos_t, sin_t, tok_pos,
                         kv_len, pt, (bf16*)k_cache, (bf16*)v_cache, a, part_o, part_ml, counters, (bf16*)out, status);
        if (mynah_check_launch("attn_decode_fused (pages)")) return -1;
        const size_t dyn_m = (size_t)n_splits * sizeof(float);
        if (HD == 128)
            mynah_launch(attn_decode_merge_kernel<128>, dim3(H, B), dim3(WARPS * 32), dyn_m, stream, part_o, part_ml, (bf16*)out, kv_len, window, H, n_splits, ldo);
        else
            mynah_launch(attn_decode_merge_kernel<64>, dim3(H, B), dim3(WARPS * 32), dyn_m, stream, part_o, part_ml, (bf16*)out, kv_len, window, H, n_splits, ldo);
        return mynah_check_launch("attn_decode_merge");
    }
    if (HD == 128)
        mynah_launch(attn_decode_fused_kernel<128, true>, grid, dim3(WARPS * 32), dyn, stream, (const bf16*)qkv, qg, kg, cos_t, sin_t, tok_pos,
                     kv_len, pt, (bf16*)k_cache, (bf16*)v_cache, a, part_o, part_ml, counters, (bf16*)out, status);
    else
        mynah_launch(attn_decode_fused_kernel<64, true>, grid, dim3(WARPS * 32), dyn, stream, (const bf16*)qkv, qg, kg, cos_t, sin_t, tok_pos,
                     kv_len, pt, (bf16*)k_cache, (bf16*)v_cache, a, part_o, part_ml, counters, (bf16*)out, status);
    return mynah_check_launch("attn_decode_fused");
}
