// Prompt attention on the fifth-generation tensor cores, for bfloat16 and head sizes 64 and 128.
//
// Same contract as attn_prefill_generic: a ragged batch of prompts (or of pieces of prompts that continue what
// the cache holds), causal, optionally windowed, grouped-query, K and V read from the paged cache, which already
// holds this step's keys and values. One CTA takes 128 consecutive queries of one (sequence, head) and walks
// over the visible keys in tiles of 128 (two pages):
//
//   warp 0     one lane brings Q once and then each tile's K and V pages into shared memory with TMA
//              (cp.async.bulk.tensor, 128-byte swizzle); a page is one box per 64 columns of the head;
//   warp 1     one lane issues tcgen05.mma: S = Q.K^T (both operands K-major in shared memory) into tensor
//              memory, and O += P.V with P read from tensor memory and V from shared memory as an MN-major
//              operand (V is stored [key][dim], which is what the product needs as its B matrix);
//   warps 2-9  the softmax: two threads share a query row (one lane of tensor memory), one for each half of a
//              tile's keys. A thread reads its 64 scores, the two exchange their maxima through shared memory,
//              rescale their halves of the row of O in tensor memory if the reference maximum moved,
//              exponentiate (fp32, base 2 with the scale folded in), add up, and write the probabilities back
//              as bf16 over the scores they came from.
//
// Hand-over is by mbarriers: TMA completes transactions on q_full / k_full / v_full; tcgen05.commit arrives on
// s_full (scores ready, K tile free) and o_done (O updated, V tile free); the softmax warps arrive on p_full.
// K, V and the scores have two buffers each: the scores of tile j+1 are computed and its K and V loaded while the
// softmax works on tile j. A thread keeps its 64 scores in registers. The maximum that the sums are
// scaled by follows the row's true maximum lazily (only when it grows by more than 2^8), so O is rarely rescaled.
//
// Keys that a row must not see (later positions, positions before its window, the unused tail of the last
// page) are masked by selecting -inf for their scores, so whatever the tile holds there cannot reach a result;
// the rows of V beyond the sequence's end are zeroed in shared memory before the second product, because a
// probability of zero times a stale NaN would still be NaN.
//
// score = dot * (1/sqrtf(head_dim)), maximum subtracted (mynah-slm src/kernels.c:228-250, :207-220).
// Every wait is bounded (2 s); a wait that runs out sets MYNAH_ST_TIMEOUT, and the CTA drains its copies, frees
// its tensor memory and returns.
#include "tcgen05.cuh"

#include <stdlib.h>

namespace {

using namespace tc5;

constexpr int BQ = 128;               // queries per CTA (the lanes of tensor memory)
constexpr int BKV = 128;              // keys per tile
constexpr int THREADS = 320;          // warp 0 TMA, warp 1 MMA, warps 2-9 softmax
constexpr int HALF_BYTES = 128 * 128; // 128 rows of 128 bytes: one 64-column half of a tile

struct PfArgs {
    int B, H, KV, ldo;
    int window;
    float scale_log2;                 // (1 / sqrt(head_dim)) * log2(e)
};

// With -DMYNAH_ATTN_STAMPS the CTA of head 0 that walks the most key tiles writes its SM's cycle counter at fixed
// points of every role's loop (a diagnostic build; mynah_attn_prefill_stamps copies the table out).
#ifdef MYNAH_ATTN_STAMPS
constexpr int STAMP_TILES = 32, STAMP_POINTS = 8;
__device__ long long g_stamps[10][STAMP_TILES][STAMP_POINTS];
constexpr int SPAN_CTAS = 1 << 16;
__device__ long long g_spans[SPAN_CTAS][2];                          // every CTA's entry and exit on the global timer (ns)
#define STAMP(j, p)                                                                                  \
    do {                                                                                             \
        if (stamp_on && lane == 0 && (j) < STAMP_TILES) g_stamps[warp][(j)][(p)] = clock64();       \
    } while (0)
#else
#define STAMP(j, p) do { } while (0)
#endif

// K-major operand, 128-byte swizzle, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand, 128-byte swizzle: a row of 128 bytes holds 64 consecutive MN elements of one k; groups of
// 8 k 1024 bytes apart (stride offset), the next 64 MN elements `lbo` bytes further on (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
    return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulator, bf16 operands, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t idesc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// A wait that all lanes of a warp agree on, so that the warp-wide instructions after it keep all their lanes.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two fp32 operations an instruction (each half is the plain round-to-nearest operation), and the maximum of
// three: the softmax warps are bound by the number of instructions they issue.
__device__ __forceinline__ void fma2(float& x0, float& x1, float a0, float a1, float b, float c) {
    asm("{ .reg .b64 ra, rb, rc, rd;\n\t mov.b64 ra, {%2, %3};\n\t mov.b64 rb, {%4, %4};\n\t mov.b64 rc, {%5, %5};\n\t"
        " fma.rn.f32x2 rd, ra, rb, rc;\n\t mov.b64 {%0, %1}, rd; }"
        : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& x0, float& x1, float a0, float a1) {
    asm("{ .reg .b64 ra, rb;\n\t mov.b64 ra, {%0, %1};\n\t mov.b64 rb, {%2, %3};\n\t add.rn.f32x2 ra, ra, rb;\n\t mov.b64 {%0, %1}, ra; }"
        : "+f"(x0), "+f"(x1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// NS: stages of K, V and the scores. 2: a CTA an SM, the next tile's scores and operands under this tile's softmax.
// 1: half the shared and tensor memory, so that two CTAs share an SM and one's softmax runs under the other's products.
template <int HD, int NS>
__global__ void __launch_bounds__(THREADS, NS == 1 ? 2 : 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ cu_q,
                            const int* __restrict__ kv_len, PageTable pt, PfArgs a, bf16* __restrict__ out,
                            int* __restrict__ status) {
    constexpr int HALVES = HD / 64;
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;            // Q, K and V tiles: 128 rows x HD
    constexpr int PAGE_BYTES = PAGE_TOKENS * 128;              // one page in one half: 64 rows of 128 bytes
    constexpr int TMEM_COLS = NS == 2 ? 512 : 256;             // NS score buffers of 128 columns, the output behind them
    constexpr int O_COL = NS * 128;
    auto stage_of = [](int j) { return NS == 2 ? (j & 1) : 0; };
    auto use_of = [](int j) { return (uint32_t)(NS == 2 ? ((j >> 1) & 1) : (j & 1)); };   // parity of tile j's use of its stage
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = smem;
    unsigned char* k_s = q_s + TILE_BYTES;                     // NS stages
    unsigned char* v_s = k_s + NS * TILE_BYTES;                // NS stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + NS * TILE_BYTES);
    const uint32_t q_full = smem_u32(bars), k_full = smem_u32(bars + 1), v_full = smem_u32(bars + 3);   // [2] each, 8 bytes apart
    const uint32_t s_full = smem_u32(bars + 5), v_free = smem_u32(bars + 7);
    const uint32_t p_full = smem_u32(bars + 9), o_done = smem_u32(bars + 11), x_full = smem_u32(bars + 12);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    float* xch = reinterpret_cast<float*>(bars + 16);          // [2 buffers][2 groups][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.y numbers the step's query tiles (find_query_tile); numbers beyond them leave at once.
    int b, qt;
    if (!find_query_tile(cu_q, a.B, BQ, blockIdx.y, b, qt)) return;    // the whole CTA: nothing is set up yet
    const int h = blockIdx.x;
    const int q_begin = cu_q[b], n_q = cu_q[b + 1] - q_begin;
    const int q0 = qt * BQ;
    const int kvl = kv_len[b], past = kvl - n_q;
    const int rows_valid = min(BQ, n_q - q0);
    const int kt_hi = (past + q0 + rows_valid - 1) / BKV;      // tile of the last key that the last row sees
    const int kt_lo = a.window > 0 ? max(0, past + q0 - a.window + 1) / BKV : 0;
    const int n_tiles = kt_hi - kt_lo + 1;
    const int lo_min = a.window > 0 ? max(0, past + q0 - a.window + 1) : 0;    // the first key that any row of the tile sees
    const int kvh = h / (a.H / a.KV);
#ifdef MYNAH_ATTN_STAMPS
    const bool stamp_on = blockIdx.x == 0 && blockIdx.y == 0;
    const unsigned span_id = blockIdx.x + gridDim.x * blockIdx.y;
    if (threadIdx.x == 0 && span_id < SPAN_CTAS) g_spans[span_id][0] = (long long)now_ns();
#endif

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(k_full + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1);
            mbar_init(v_free + 8 * i, 1);
            mbar_init(p_full + 8 * i, 8);                      // one arrival per softmax warp
            mbar_init(x_full + 8 * i, 8);
        }
        mbar_init(o_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched behind another kernel with programmatic dependent launch, everything above ran while that kernel was
    // finishing (it read only the step's description, which no kernel writes); the queries and the cache are not
    // touched before this returns. A no-op for an ordinary launch.
    griddep_wait();

    // Tile j uses stage j & 1 of K, V and the scores; its barriers are in their (j >> 1)-th use.
    if (warp == 0) {
        if (lane == 0) {                                       // ---- TMA producer
            mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
            for (int hf = 0; hf < HALVES; hf++)
                tma_load_2d(smem_u32(q_s + hf * HALF_BYTES), &map_q, h * HD + hf * 64, q_begin + q0, q_full);
            int k_issued = 0, v_issued = 0;
            for (int j = 0; j < n_tiles; j++) {
                const int st = stage_of(j);
                const uint32_t prev_use = use_of(j) ^ 1;       // parity of the stage's use before this one
                const int key0 = (kt_lo + j) * BKV;
                // A page is brought only if it holds a key that some row of the tile sees: the first page of the
                // first tile may lie wholly before the window (a cache that keeps a window has given it back),
                // the second page of the last tile beyond the sequence's end.
                const bool need0 = key0 + PAGE_TOKENS > lo_min, need1 = key0 + PAGE_TOKENS < kvl;
                const int p0 = need0 ? page_of(pt, b, key0) : -1;
                const int p1 = need1 ? page_of(pt, b, key0 + PAGE_TOKENS) : -1;
                if ((need0 && p0 < 0) || (need1 && p1 < 0) || (!need0 && !need1)) {
                    atomicOr(status, MYNAH_ST_PAGE_RANGE);
                    break;
                }
                const uint32_t bytes = ((p0 >= 0 ? 1 : 0) + (p1 >= 0 ? 1 : 0)) * HALVES * PAGE_BYTES;
                if (j >= NS && !mbar_wait(s_full + 8 * st, prev_use)) {     // the scores of tile j-NS are done: its K is free
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    break;
                }
                unsigned char* kd = k_s + st * TILE_BYTES;
                mbar_expect_tx(k_full + 8 * st, bytes);
#pragma unroll
                for (int hf = 0; hf < HALVES; hf++) {
                    if (p0 >= 0) tma_load_2d(smem_u32(kd + hf * HALF_BYTES), &map_k, hf * 64, (p0 * a.KV + kvh) * PAGE_TOKENS, k_full + 8 * st);
                    if (p1 >= 0) tma_load_2d(smem_u32(kd + hf * HALF_BYTES + PAGE_BYTES), &map_k, hf * 64, (p1 * a.KV + kvh) * PAGE_TOKENS, k_full + 8 * st);
                }
                k_issued = j + 1;
                if (j >= NS && !mbar_wait(v_free + 8 * st, prev_use)) {     // the second product of tile j-NS is done: its V is free
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    break;
                }
                unsigned char* vd = v_s + st * TILE_BYTES;
                mbar_expect_tx(v_full + 8 * st, bytes);
#pragma unroll
                for (int hf = 0; hf < HALVES; hf++) {
                    if (p0 >= 0) tma_load_2d(smem_u32(vd + hf * HALF_BYTES), &map_v, hf * 64, (p0 * a.KV + kvh) * PAGE_TOKENS, v_full + 8 * st);
                    if (p1 >= 0) tma_load_2d(smem_u32(vd + hf * HALF_BYTES + PAGE_BYTES), &map_v, hf * 64, (p1 * a.KV + kvh) * PAGE_TOKENS, v_full + 8 * st);
                }
                v_issued = j + 1;
            }
            griddep_launch_late();                             // all of this CTA's tiles have been asked for
            // whatever was started still lands in this CTA's shared memory: wait for it before leaving (bounded)
            mbar_wait(q_full, 0);
            for (int j = max(0, k_issued - NS); j < k_issued; j++) mbar_wait(k_full + 8 * stage_of(j), use_of(j));
            for (int j = max(0, v_issued - NS); j < v_issued; j++) mbar_wait(v_full + 8 * stage_of(j), use_of(j));
        }
    } else if (warp == 1) {
        if (lane == 0) {                                       // ---- MMA issuer
            constexpr uint32_t idesc_s = idesc(BKV, false), idesc_o = idesc(HD, true);
            const uint32_t t_o = tmem_base + O_COL;
            const uint32_t q_addr = smem_u32(q_s), k_addr = smem_u32(k_s), v_addr = smem_u32(v_s);
            auto scores = [&](int j) {                         // S[stage of j] = Q . K_j^T
                const int st = stage_of(j);
#pragma unroll
                for (int k = 0; k < HD / 16; k++) {
                    const uint32_t off = (k / 4) * HALF_BYTES + (k % 4) * 32;
                    tc_mma(tmem_base + st * BKV, desc_k_major(q_addr + off), desc_k_major(k_addr + st * TILE_BYTES + off), idesc_s, k != 0);
                }
                tc_commit(s_full + 8 * st);
            };
            bool ok = mbar_wait(q_full, 0) && mbar_wait(k_full, 0);
            if (ok) {
                tc_fence_after();
                scores(0);
            }
            for (int j = 0; j < n_tiles && ok; j++) {
                const int st = stage_of(j);
                STAMP(j, 0);
                if (NS == 2 && j + 1 < n_tiles) {              // the next tile's scores, while the softmax works on this one.
                    // Their buffer held the probabilities of tile j-1; the product that read them was issued before.
                    ok = mbar_wait(k_full + 8 * stage_of(j + 1), use_of(j + 1));
                    if (!ok) break;
                    tc_fence_after();
                    STAMP(j, 1);
                    scores(j + 1);
                }
                STAMP(j, 2);
                ok = mbar_wait(p_full + 8 * st, use_of(j)) && mbar_wait(v_full + 8 * st, use_of(j));
                if (!ok) break;
                tc_fence_after();
                STAMP(j, 3);
#pragma unroll
                for (int k = 0; k < BKV / 16; k++)             // 16 keys a step: 8 columns of packed probabilities, 16 rows of V
                    tc_mma_ts(t_o, tmem_base + st * BKV + (NS == 2 ? k * 8 : (k / 4) * 64 + (k % 4) * 8), desc_mn_major(v_addr + st * TILE_BYTES + k * 16 * 128, HALF_BYTES),
                              idesc_o, (j | k) != 0);
                tc_commit(v_free + 8 * st);
                tc_commit(o_done);
                STAMP(j, 4);
                if (NS == 1 && j + 1 < n_tiles) {              // one score buffer: the next scores overwrite these probabilities,
                    ok = mbar_wait(k_full, use_of(j + 1));     // so they are issued behind the product that reads them
                    if (!ok) break;
                    tc_fence_after();
                    scores(j + 1);
                }
            }
            if (!ok) atomicOr(status, MYNAH_ST_TIMEOUT);
        }
    } else {
        // ---- softmax: warps 2..5 take the first 64 keys of a tile, warps 6..9 the other 64; a warp reads the lane
        // quadrant (warp % 4) of tensor memory, so two threads, one in each group, share a query row.
        const int grp = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int qpos = past + q0 + row;
        const int lo_r = a.window > 0 ? max(0, qpos - a.window + 1) : 0;
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t t_o = t_row + O_COL + grp * (HD / 2);   // this thread's half of the row of O
        constexpr int HALF_KEYS = BKV / 2;
        float m_ref = -INFINITY, l = 0.f;                      // the maximum that the sums are scaled by; the sum over this thread's keys
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            const int st = stage_of(j);
            const uint32_t use = use_of(j);
            const int xst = j & 1;                             // the exchange has two buffers whatever NS is
            const uint32_t xuse = (j >> 1) & 1;
            const int key0 = (kt_lo + j) * BKV + grp * HALF_KEYS;     // this thread's first key
            const uint32_t t_s = t_row + st * BKV;
            STAMP(j, 0);
            if (!warp_wait(s_full + 8 * st, use)) { ok = false; break; }
            tc_fence_after();
            STAMP(j, 1);
            // does any row of the tile have a key, among this group's, that it must not see?
            const bool need_mask = key0 + HALF_KEYS - 1 > past + q0 || key0 + HALF_KEYS > kvl ||
                                   (a.window > 0 && key0 < past + q0 + BQ - a.window);
            const int hi = min(qpos, kvl - 1) - key0;          // the last of this thread's scores that its row sees
            const int lo = a.window > 0 ? lo_r - key0 : -(1 << 30);
            // 32 of the thread's scores (the c-th half of them), those that the row must not see set to -inf
            auto fetch32 = [&](int c, float (&v)[32]) {
                tc_ld32(t_s + grp * HALF_KEYS + c * 32, reinterpret_cast<uint32_t(&)[32]>(v));
                if (need_mask) {                               // a compare with a constant and a select per score
                    if (a.window > 0) {
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] = (c * 32 + e <= hi && c * 32 + e >= lo) ? v[e] : -INFINITY;
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] = c * 32 + e <= hi ? v[e] : -INFINITY;
                    }
                }
            };
            float s[NS == 2 ? HALF_KEYS : 1];                  // NS == 2: a thread keeps its 64 scores; NS == 1: it fetches them twice
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if constexpr (NS == 2) {
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; c++) tc_ld32_nowait(t_s + grp * HALF_KEYS + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; c++) tc_wait_ld(reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
                STAMP(j, 2);
                if (need_mask) {
                    if (a.window > 0) {
#pragma unroll
                        for (int e = 0; e < HALF_KEYS; e++) s[e] = (e <= hi && e >= lo) ? s[e] : -INFINITY;
                    } else {
#pragma unroll
                        for (int e = 0; e < HALF_KEYS; e++) s[e] = e <= hi ? s[e] : -INFINITY;
                    }
                }
#pragma unroll
                for (int e = 0; e < HALF_KEYS; e += 2) mx4[(e >> 1) & 3] = max3(mx4[(e >> 1) & 3], s[e], s[e + 1]);
            } else {
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; c++) {
                    float v[32];
                    fetch32(c, v);
#pragma unroll
                    for (int e = 0; e < 32; e += 2) mx4[(e >> 1) & 3] = max3(mx4[(e >> 1) & 3], v[e], v[e + 1]);
                }
                STAMP(j, 2);
            }
            const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the row's maximum over both groups, through shared memory (two buffers: a value is read before the
            // barrier of the next tile, and overwritten only after it)
            xch[(xst * 2 + grp) * BQ + row] = mx_own;
            __syncwarp();
            STAMP(j, 3);
            if (lane == 0) mbar_arrive(x_full + 8 * xst);
            if (!warp_wait(x_full + 8 * xst, xuse)) { ok = false; break; }
            STAMP(j, 4);
            const float m_new = fmaxf(mx_own, xch[(xst * 2 + (grp ^ 1)) * BQ + row]) * a.scale_log2;
            // The reference maximum follows the true one lazily: while the row's maximum stays within 2^8 of it
            // nothing is rescaled (the probabilities just exceed one by up to that factor, which fp32 sums and
            // bf16 products carry without loss). Both threads of a row take the same decision.
            float alpha = 1.0f;
            if (m_new > m_ref + 8.0f || (m_ref == -INFINITY && m_new != -INFINITY)) {
                alpha = ex2(m_ref - m_new);                    // 0 for the first visible key
                m_ref = m_new;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;      // a row that has seen nothing yet
            // O is touched only when some row of the warp has to be rescaled; then the product of the tile before
            // must have finished. (A wait that is skipped is not missed later: o_done can be at most one phase
            // ahead of the tile whose probabilities have not been handed over yet.)
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                if (!warp_wait(o_done, (j - 1) & 1)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 64; c++) {
                    uint32_t r[32];
                    tc_ld32(t_o + c * 32, r);
#pragma unroll
                    for (int e = 0; e < 32; e++) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
                    tc_st32(t_o + c * 32, r);
                }
                tc_wait_st();
            }
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};              // two pairs of running sums
            if constexpr (NS == 2) {
                uint32_t pk[HALF_KEYS / 2];
#pragma unroll
                for (int e = 0; e < HALF_KEYS; e += 2) {
                    float x0, x1;
                    fma2(x0, x1, s[e], s[e + 1], a.scale_log2, -m_use);
                    const float p0 = ex2(x0), p1 = ex2(x1);                       // 2^-inf = 0
                    add2(sum4[e & 2], sum4[(e & 2) + 1], p0, p1);
                    pk[e >> 1] = pack2(p0, p1);
                }
                STAMP(j, 5);
                // over the scores: both groups have theirs in registers since the exchange above
                tc_st32(t_s + grp * (HALF_KEYS / 2), pk);
            } else {
                // The scores are fetched again, 32 at a time, and a group's probabilities go over its own scores
                // (columns [64 g, 64 g + 32) of the buffer), behind the ones already fetched.
#pragma unroll
                for (int c = 0; c < HALF_KEYS / 32; c++) {
                    float v[32];
                    fetch32(c, v);
                    uint32_t pk[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 2) {
                        float x0, x1;
                        fma2(x0, x1, v[e], v[e + 1], a.scale_log2, -m_use);
                        const float p0 = ex2(x0), p1 = ex2(x1);
                        add2(sum4[e & 2], sum4[(e & 2) + 1], p0, p1);
                        pk[e >> 1] = pack2(p0, p1);
                    }
                    tc_st16(t_s + grp * HALF_KEYS + c * 16, pk);
                }
                STAMP(j, 5);
            }
            tc_wait_st();
            STAMP(j, 6);
            l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            // Rows of V that were not brought (beyond the sequence's end, or a first page wholly before the window)
            // hold whatever was there: zero them, a probability of zero times a stale NaN would still be NaN.
            const int tile_key0 = (kt_lo + j) * BKV;
            const bool past_end = tile_key0 + BKV > kvl, before_window = tile_key0 + PAGE_TOKENS <= lo_min;
            if (past_end || before_window) {
                if (!warp_wait(v_full + 8 * st, use)) { ok = false; break; }
                if ((past_end && row >= kvl - tile_key0) || (before_window && row < PAGE_TOKENS)) {
                    for (int hf = grp; hf < HALVES; hf += 2) {
                        uint4* dst = reinterpret_cast<uint4*>(v_s + st * TILE_BYTES + hf * HALF_BYTES + row * 128);
#pragma unroll
                        for (int i = 0; i < 8; i++) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                fence_async_smem();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * st);
            STAMP(j, 7);
        }
        // the row sum over both groups, through the same exchange (its barriers are in use n_tiles by now)
        if (ok) {
            const int st = n_tiles & 1;
            xch[(st * 2 + grp) * BQ + row] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(x_full + 8 * st);
            if (!warp_wait(x_full + 8 * st, (n_tiles >> 1) & 1)) ok = false;
            else l += xch[(st * 2 + (grp ^ 1)) * BQ + row];
        }
        if (ok && !warp_wait(o_done, (n_tiles - 1) & 1)) ok = false;
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* o_row = out + (size_t)(q_begin + q0 + row) * a.ldo + (size_t)h * HD + grp * (HD / 2);
#pragma unroll 1
            for (int c = 0; c < HD / 64; c++) {
                uint32_t r[32];
                tc_ld32(t_o + c * 32, r);
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        reinterpret_cast<uint4*>(o_row + c * 32)[i] =
                            make_uint4(pack2(__uint_as_float(r[8 * i]) * inv, __uint_as_float(r[8 * i + 1]) * inv),
                                       pack2(__uint_as_float(r[8 * i + 2]) * inv, __uint_as_float(r[8 * i + 3]) * inv),
                                       pack2(__uint_as_float(r[8 * i + 4]) * inv, __uint_as_float(r[8 * i + 5]) * inv),
                                       pack2(__uint_as_float(r[8 * i + 6]) * inv, __uint_as_float(r[8 * i + 7]) * inv));
                }
            }
        } else if (lane == 0) {
            atomicOr(status, MYNAH_ST_TIMEOUT);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
#ifdef MYNAH_ATTN_STAMPS
    if (threadIdx.x == 0 && span_id < SPAN_CTAS) g_spans[span_id][1] = (long long)now_ns();
#endif
}

template <int HD, int NS>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, int n_tokens, int B, int max_q_len, const int* cu_q,
           const int* kv_len, PageTable pt, PfArgs a, bf16* out, int* status, cudaStream_t stream) {
    constexpr size_t smem = (1 + 2 * NS) * (size_t)(HD / 64) * HALF_BYTES + 128 + 2 * 2 * BQ * sizeof(float) + 1024;
    auto kern = attn_prefill_tcgen05_kernel<HD, NS>;
    static bool opted = false;
    if (!opted) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("attn_prefill_tcgen05: %s", cudaGetErrorString(e));
        opted = true;
    }
    (void)max_q_len;
    const dim3 grid(a.H, ceil_div(n_tokens, BQ) + B, 1);
    if (mynah_launch(kern, grid, dim3(THREADS), smem, stream, mq, mk, mv, cu_q, kv_len, pt, a, out, status) != cudaSuccess)
        return mynah_fail("attn_prefill_tcgen05: %s", cudaGetErrorString(cudaGetLastError()));
    return mynah_check_launch("attn_prefill_tcgen05");
}

}  // namespace

#ifdef MYNAH_ATTN_STAMPS
// out: [10 warps][32 tiles][8 points] of the stamped CTA's cycle counts (host memory).
MYNAH_API int mynah_attn_prefill_stamps(long long* out) {
    return cudaMemcpyFromSymbol(out, g_stamps, sizeof(g_stamps)) == cudaSuccess ? 0 : -1;
}
// out: [65536 CTAs][entry, exit] in nanoseconds of the device's global timer (CTA number x + X * (y + Y * z)).
MYNAH_API int mynah_attn_prefill_spans(long long* out) {
    return cudaMemcpyFromSymbol(out, g_spans, sizeof(g_spans)) == cudaSuccess ? 0 : -1;
}
#endif

// 0: chosen by the number of CTAs (the default, or MYNAH_ATTN_PREFILL_STAGES), 1: one stage and two CTAs an SM, 2: two
// stages and one CTA an SM. Both forms give the same bits.
static int g_stages_mode = -1;
static int stages_mode() {
    if (g_stages_mode < 0) {
        const char* e = getenv("MYNAH_ATTN_PREFILL_STAGES");
        g_stages_mode = e != nullptr && (e[0] == '1' || e[0] == '2') ? e[0] - '0' : 0;
    }
    return g_stages_mode;
}
MYNAH_API int mynah_attn_prefill_tcgen05_stages(int mode) {
    MYNAH_REQUIRE(mode >= 0 && mode <= 2, "attn_prefill_tcgen05_stages: mode %d is none of 0, 1, 2", mode);
    g_stages_mode = mode;
    return 0;
}

MYNAH_API int mynah_attn_prefill_tcgen05_supported(int H, int KV, int HD) {
    return (HD == 64 || HD == 128) && KV > 0 && H % KV == 0;
}

// q: [n_tokens, ldq] bf16 with head h in columns [h * HD, (h + 1) * HD); out: [n_tokens, ldo]; the cache tensors
// are [n_pages, KV, 64, HD] bf16. Otherwise the arguments of mynah_attn_prefill_generic.
MYNAH_API int mynah_attn_prefill_tcgen05(
    const void* q, void* out, int n_tokens, int B, int max_q_len, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* cu_q, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int* status, cudaStream_t stream) {
    if (B == 0 || max_q_len == 0 || n_tokens == 0) return 0;
    MYNAH_REQUIRE(mynah_attn_prefill_tcgen05_supported(H, KV, HD), "attn_prefill_tcgen05: H=%d KV=%d head_dim=%d is not taken by this kernel", H, KV, HD);
    MYNAH_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                  ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0,
                  "attn_prefill_tcgen05: rows must be 16-byte aligned (strides %d, %d)", ldq, ldo);
    MYNAH_REQUIRE(ceil_div(n_tokens, BQ) + B <= 65535 && (long long)n_pages * KV * PAGE_TOKENS < (1ll << 31), "attn_prefill_tcgen05: launch too large");
    MYNAH_REQUIRE(status != nullptr, "attn_prefill_tcgen05: a status word is required");
    CUtensorMap mq, mk, mv;
    if (make_map(&mq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n_tokens, (long long)H * HD, ldq, BQ, 64)) return -1;
    if (make_map(&mk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)n_pages * KV * PAGE_TOKENS, HD, HD, PAGE_TOKENS, 64)) return -1;
    if (make_map(&mv, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (long long)n_pages * KV * PAGE_TOKENS, HD, HD, PAGE_TOKENS, 64)) return -1;
    const PfArgs a{B, H, KV, ldo, window, (1.0f / sqrtf((float)HD)) * 1.4426950408889634f};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    // Two CTAs an SM pay once there are several waves of CTAs (64 prompts of 2,048 tokens and 32 heads: 2.97 against
    // 3.34 ms; 4 prompts: 221 against 236 us); with one wave or two, the longest CTA's own chain sets the time and it
    // is longer with one stage (one prompt of 16 heads: 39.7 against 28.0 us).
    const int mode = stages_mode();
    const long long ctas = (long long)H * (ceil_div(n_tokens, BQ) + B);
    const int stages = mode != 0 ? mode : (ctas >= 8ll * mynah_sm_count() ? 1 : 2);
    if (stages == 1) {
        if (HD == 128) return launch<128, 1>(mq, mk, mv, n_tokens, B, max_q_len, cu_q, kv_len, pt, a, (bf16*)out, status, stream);
        return launch<64, 1>(mq, mk, mv, n_tokens, B, max_q_len, cu_q, kv_len, pt, a, (bf16*)out, status, stream);
    }
    if (HD == 128) return launch<128, 2>(mq, mk, mv, n_tokens, B, max_q_len, cu_q, kv_len, pt, a, (bf16*)out, status, stream);
    return launch<64, 2>(mq, mk, mv, n_tokens, B, max_q_len, cu_q, kv_len, pt, a, (bf16*)out, status, stream);
}
