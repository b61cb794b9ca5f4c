// The whole decode step of a stack of pre-norm attention + SwiGLU layers as ONE
// persistent kernel: one CTA per SM, all layers, a grid-wide barrier between
// the phases of a layer instead of a kernel boundary. For a handful of
// sequences a decode step is some 170 dependent launches of a few microseconds
// each; here it is one launch and five barriers per layer.
//
// Phases of a layer (rows = sequences of the batch, at most 16):
//   1  residual (+ pending add) -> RMSNorm -> q,k,v product            -> qkv
//   2  per (sequence, kv head, page): per-head norm and rotation of q;
//      on the page that holds the new position also of k, which is written
//      to the cache with v; scores, softmax and PV of the page on tensor
//      cores; the CTA that finishes a (sequence, kv head) last merges its
//      pages in page order                                               -> attn
//   3  o product                                                        -> delta
//   4  residual + delta -> RMSNorm -> gate/up product -> SwiGLU           -> act
//   5  down product                                                     -> delta
// and after the last layer: residual + delta -> RMSNorm -> head -> fp32 logits.
//
// The arithmetic is that of the separate kernels (rope_cache.cu,
// attn_decode_tc.cu, gemv_decode.cu): same formulas, same rounding points
// (activations bf16 between products, residual and all sums fp32), pages
// merged in page order. Formulas as in mynah-slm src/arch_qwen3.c:178-252 and
// src/kernels.c.
//
// The barrier is a counter and a generation word in global memory. Every spin
// is bounded by a wall-clock limit; a CTA that gives up sets an abort word
// that every other spin watches, so all CTAs leave the kernel.
#include "layout.cuh"

namespace {

constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int TEAM = 128;                 // threads that work on one page in phase 2
constexpr int MAX_M = 16;
constexpr int MAX_G = 16;
constexpr int MAX_GROUPS = 4;
constexpr int XPAD = 32;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct LayerDesc {
    const bf16* w_qkv;
    const bf16* w_o;
    const bf16* w_gu;
    const bf16* w_down;
    const void* norm1;
    const void* norm2;
    const void* q_gain;
    const void* k_gain;
    int norm1_dt, norm2_dt, qk_dt;
    bf16* k_cache;
    bf16* v_cache;
    const float* cos_t;
    const float* sin_t;
    int n_pos;
    int group;
    int window;
    int pad_;
};

struct StepArgs {
    int n_layers, M, D, H, KV, HD, F, V, S_max;
    float eps, qk_eps;
    const LayerDesc* layers;
    const int* tokens;
    const int* tok_pos;
    const int* kv_len;
    PageTable pt[MAX_GROUPS];
    const bf16* embed;
    const void* final_gain;
    int final_dt;
    const bf16* head;
    float* x0;
    float* x1;
    bf16* qkv;
    bf16* attn_out;
    bf16* delta;
    bf16* act;
    float* part_o;
    float* part_ml;
    unsigned* counters;
    float* logits;
    unsigned* bar_count;
    unsigned* bar_gen;
    int* abort_word;
    int* status;
    int n_groups;
    unsigned long long* trace;   // optional: CTA 0 writes a time stamp after every phase (for tuning)
    int table_offset;      // byte offset of the page table in dynamic shared memory, or -1: look pages up in global memory
};

// What the step's sequences look like, read once per launch into shared memory.
struct StepMeta {
    int kv_len[MAX_M], pos[MAX_M];
    int window[MAX_GROUPS];
    int n_vis[MAX_GROUPS][MAX_M], pg0[MAX_GROUPS][MAX_M];
    const int* pages;      // [group][row][S_max] physical page of the s-th visible page, or null
};

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
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
__device__ __forceinline__ void team_sync(int team) { asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "n"(TEAM) : "memory"); }
template <int CH> __device__ __forceinline__ int swz(int r, int c) { return (r * CH + (c ^ (r & 7))) * 16; }
__device__ __forceinline__ float sigmoid_stable(float v) {
    const float e = expf(-fabsf(v));
    return (v >= 0.f ? 1.0f : e) / (1.0f + e);
}

__device__ __forceinline__ unsigned atom_add_acq_rel(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void red_add_release(unsigned* p, unsigned v) {
    asm volatile("red.add.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// All CTAs of the grid meet here. Returns false when the step has been aborted.
__device__ bool grid_barrier(const StepArgs& a) {
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        const unsigned gen = ld_acquire(a.bar_gen);               // read before arriving
        const unsigned prev = atom_add_acq_rel(a.bar_count, 1u);
        if (prev == gridDim.x - 1) {
            *reinterpret_cast<volatile unsigned*>(a.bar_count) = 0;
            red_add_release(a.bar_gen, 1u);
        } else {
            const unsigned long long t0 = now_ns();
            for (unsigned it = 0; ld_acquire(a.bar_gen) == gen; it++) {
                if ((it & 63u) == 63u) {
                    if (*reinterpret_cast<volatile int*>(a.abort_word) != 0) { ok = 0; break; }
                    if (now_ns() - t0 > WAIT_LIMIT_NS) {
                        atomicOr(a.status, MYNAH_ST_TIMEOUT);
                        atomicExch(a.abort_word, 1);
                        ok = 0;
                        break;
                    }
                }
            }
        }
        ok_s = ok;
    }
    __syncthreads();
    return ok_s != 0;
}

// Every CTA asks for its share of a weight matrix to be brought into L2 (one request per 128-byte line).
__device__ __forceinline__ void prefetch_matrix(const void* w, size_t bytes) {
    const size_t lines = (bytes + 127) / 128;
    const size_t per = (lines + gridDim.x - 1) / gridDim.x;
    const size_t lo = (size_t)blockIdx.x * per, hi = lo + per < lines ? lo + per : lines;
    const char* base = static_cast<const char*>(w);
    for (size_t i = lo + threadIdx.x; i < hi; i += THREADS) prefetch_l2(base + i * 128);
}

// RMSNorm of M rows into shared memory as bf16. src(m, i) gives the fp32 value of the row (residual plus
// pending add, or the embedding); CTA 0 also writes it to x_out. Teams of warps share a row.
template <typename Src>
__device__ void norm_rows(bf16* xs, int ldx, int M, int D, Src src, VecRef gain, float eps, float* x_out, float* part) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int mp = 1;
    while (mp < M && mp < WARPS) mp <<= 1;
    const int wpr = WARPS / mp, sub = warp % wpr;
    for (int m0 = 0; m0 < M; m0 += mp) {
        const int m = m0 + warp / wpr;
        const bool on = m < M;
        float ss = 0.f;
        if (on)
            for (int i = sub * 32 + lane; i < D; i += wpr * 32) {
                const float v = src(m, i);
                ss += v * v;
            }
        ss = warp_sum(ss);
        __syncthreads();
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < wpr; w++) tot += part[(warp / wpr) * wpr + w];
        const float s = 1.0f / sqrtf(tot / (float)D + eps);
        if (on)
            for (int i = sub * 32 + lane; i < D; i += wpr * 32) {
                const float v = src(m, i);
                if (x_out != nullptr && blockIdx.x == 0) x_out[(size_t)m * D + i] = v;
                xs[m * ldx + i] = __float2bfloat16_rn((v * s) * gain.at(i));
            }
    }
    const int rows_x = M > 8 ? 16 : 8;
    for (int i = threadIdx.x; i < (rows_x - M) * (D / 8); i += THREADS) {
        const int m = M + i / (D / 8), c = i % (D / 8);
        *reinterpret_cast<uint4*>(xs + m * ldx + c * 8) = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
}

// bf16 rows from global memory into shared memory (rows beyond M zero).
__device__ void load_rows(bf16* xs, int ldx, const bf16* x, int M, int K) {
    const int rows_x = M > 8 ? 16 : 8;
    for (int i = threadIdx.x; i < rows_x * (K / 8); i += THREADS) {
        const int m = i / (K / 8), c = i % (K / 8);
        *reinterpret_cast<uint4*>(xs + m * ldx + c * 8) =
            m < M ? *reinterpret_cast<const uint4*>(x + (size_t)m * K + c * 8) : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
}

enum { OUT_BF16 = 0, OUT_SWIGLU = 1, OUT_F32 = 2 };

// y[M, N] = xs[M, K] . W[N, K]^T over the CTA's share of 8-row groups. The 8 warps of the CTA are
// ksplit warps on each of 8/ksplit groups at a time; ksplit is chosen so that the groups of the whole grid
// are covered in as few rounds as possible. A warp loads its k-blocks eight at a time before it multiplies;
// the warps of a group add their partial sums in warp order. For SwiGLU W holds N gate rows, then N up rows.
template <int EPI>
__device__ void gemv_phase(const bf16* __restrict__ W, int N, int K, const bf16* xs, int ldx, int M, void* out, int ldo,
                           float (*red)[32][8]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nkb = K / 32, groups = (N + 7) / 8;
    const bool two = M > 8;
    int gpc = 1;                                                     // groups per CTA and round
    while (gpc < 8 && gpc * (int)gridDim.x < groups) gpc <<= 1;
    const int ksplit = WARPS / gpc, sub = warp % ksplit, gslot = warp / ksplit;
    const int rounds = (groups + gpc * gridDim.x - 1) / (gpc * gridDim.x);
    for (int r = 0; r < rounds; r++) {
        const int item = (r * gridDim.x + blockIdx.x) * gpc + gslot;
        const bool item_ok = item < groups;
        const int n0 = item * 8, row = n0 + g;
        const bool row_ok = item_ok && row < N;
        const bf16* wg = W + (size_t)(row_ok ? row : 0) * K;
        const bf16* wu = EPI == OUT_SWIGLU ? W + (size_t)((row_ok ? row : 0) + N) * K : nullptr;
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        if (item_ok) {
            for (int j0 = sub; j0 < nkb; j0 += ksplit * 8) {
                uint4 wv[8], uv[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int kb = j0 + u * ksplit;
                    const bool ok = kb < nkb && row_ok;
                    wv[u] = ok ? __ldg(reinterpret_cast<const uint4*>(wg + kb * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
                    if (EPI == OUT_SWIGLU) uv[u] = ok ? __ldg(reinterpret_cast<const uint4*>(wu + kb * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int kb = j0 + u * ksplit;
                    if (kb < nkb) {
                        const uint4 xa = *reinterpret_cast<const uint4*>(xs + g * ldx + kb * 32 + t * 8);
                        uint4 xb = make_uint4(0, 0, 0, 0);
                        if (two) xb = *reinterpret_cast<const uint4*>(xs + (g + 8) * ldx + kb * 32 + t * 8);
                        const uint32_t a1[4] = {xa.x, xb.x, xa.y, xb.y}, a2[4] = {xa.z, xb.z, xa.w, xb.w};
                        mma_bf16(c0, a1, wv[u].x, wv[u].y);
                        mma_bf16(c0, a2, wv[u].z, wv[u].w);
                        if (EPI == OUT_SWIGLU) {
                            mma_bf16(c1, a1, uv[u].x, uv[u].y);
                            mma_bf16(c1, a2, uv[u].z, uv[u].w);
                        }
                    }
                }
            }
        }
        if (ksplit > 1) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                red[warp][lane][e] = c0[e];
                if (EPI == OUT_SWIGLU) red[warp][lane][4 + e] = c1[e];
            }
            __syncthreads();
        }
        if (sub == 0 && item_ok) {
            float s0[4], s1[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                s0[e] = c0[e];
                s1[e] = c1[e];
            }
            for (int w = 1; w < ksplit; w++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s0[e] += red[warp + w][lane][e];
                    if (EPI == OUT_SWIGLU) s1[e] += red[warp + w][lane][4 + e];
                }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int m = g + 8 * half;
                if (m >= M) continue;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int n = n0 + 2 * t + j;
                    if (n >= N) continue;
                    float v = s0[2 * half + j];
                    if (EPI == OUT_SWIGLU) {
                        const float gt = round_to<bf16>(v), up = round_to<bf16>(s1[2 * half + j]);
                        v = (gt * sigmoid_stable(gt)) * up;
                    }
                    if (EPI == OUT_F32) static_cast<float*>(out)[(size_t)m * ldo + n] = v;
                    else static_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(v);
                }
            }
        }
        if (ksplit > 1) __syncthreads();
    }
}

// Shared memory of phase 2, per team of four warps: two stages of K and V tiles.
template <int HD>
struct alignas(128) TeamSmem {
    unsigned char k[2][PAGE_TOKENS * HD * 2];
    unsigned char v[2][PAGE_TOKENS * HD * 2];
    bf16 p[MAX_G * PAGE_TOKENS];
    bf16 q[MAX_G * HD];
    float red_m[4][MAX_G], red_l[4][MAX_G];
    float w[1024];                // page weights of the merge (S_max <= 1024)
    float row_kv[2 * HD];         // the new position's k (normed, rotated) and v
    int last_flag;
};

// Per-head norm and rotation of one head held by a warp (lane owns HD/32 consecutive elements), as rope_cache.cu.
template <int HD>
__device__ __forceinline__ void head_norm_rope(float (&v)[HD / 32], VecRef gain, float eps, const float* cos_t, const float* sin_t,
                                               int pos, int lane) {
    constexpr int EPL = HD / 32;
    if (gain.p != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; j++) ss += v[j] * v[j];
        ss = warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int j = 0; j < EPL; j++) v[j] = v[j] * (sc * gain.at(lane * EPL + j));
    }
    if (cos_t != nullptr) {
        const int i0 = (lane & 15) * EPL;
        const float* c = cos_t + (size_t)pos * (HD / 2) + i0;
        const float* sn = sin_t + (size_t)pos * (HD / 2) + i0;
#pragma unroll
        for (int j = 0; j < EPL; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
            v[j] = lane < 16 ? v[j] * c[j] - other * sn[j] : v[j] * c[j] + other * sn[j];
        }
    }
}

struct PageItem {
    int b, kvh, s;          // sequence, kv head, index among the visible pages
    int page;               // physical page, -1: none
    int k_first, k_last;    // rows of the tile in use
    int r_new;              // row of the new position in this page, or -1
};

// Phase 2 for one team: its share of the (sequence, kv head, page) items, the copy of the next item's tiles
// in flight while the current one is worked on.
template <int HD>
__device__ void attention_phase(const StepArgs& a, const LayerDesc& L, const StepMeta& meta, TeamSmem<HD>& sm, int team) {
    constexpr int CH = HD / 8, KSTEPS = HD / 16, EPL = HD / 32, NT = HD / 32;
    const int tid = threadIdx.x % TEAM, warp = tid >> 5, lane = tid & 31;
    const int G = a.H / a.KV, grp = L.group;
    const float scale = 1.0f / sqrtf((float)HD);
    const int ldq = (a.H + 2 * a.KV) * HD;
    const int n_items = a.M * a.KV * a.S_max, stride = gridDim.x * 2;
    const VecRef qg{L.q_gain, L.qk_dt}, kg{L.k_gain, L.qk_dt};
    const bool pos_bad_possible = L.cos_t != nullptr;
    for (int i = tid; i < MAX_G * HD; i += TEAM) sm.q[i] = __float2bfloat16_rn(0.f);

    // the next item at or after `item` that has a visible page (uniform over the team)
    auto next_real = [&](int item, PageItem& it) -> int {
        for (; item < n_items; item += stride) {
            const int s = item % a.S_max, kvh = (item / a.S_max) % a.KV, b = item / (a.S_max * a.KV);
            const int hi = meta.kv_len[b];
            if (hi <= 0 || s >= meta.n_vis[grp][b]) continue;
            const int lo = meta.window[grp] > 0 ? max(0, hi - meta.window[grp]) : 0;
            const int mp = meta.pg0[grp][b] + s;
            const int key_begin = max(lo, mp * PAGE_TOKENS), key_end = min(hi, (mp + 1) * PAGE_TOKENS);
            it.b = b; it.kvh = kvh; it.s = s;
            it.page = meta.pages != nullptr ? meta.pages[((size_t)grp * a.M + b) * a.S_max + s] : page_of(a.pt[grp], b, mp * PAGE_TOKENS);
            const int pos = meta.pos[b];
            if (pos_bad_possible && (pos < 0 || pos >= L.n_pos)) it.page = -2;
            it.k_first = key_begin % PAGE_TOKENS;
            it.k_last = (key_end - 1) % PAGE_TOKENS;
            it.r_new = (pos >= mp * PAGE_TOKENS && pos < (mp + 1) * PAGE_TOKENS) ? pos % PAGE_TOKENS : -1;
            return item;
        }
        return n_items;
    };
    auto issue = [&](const PageItem& it, int stage) {
        if (it.page >= 0) {
            const size_t tile = ((size_t)it.page * a.KV + it.kvh) * PAGE_TOKENS * HD;
            const uint32_t k_base = smem_u32(sm.k[stage]), v_base = smem_u32(sm.v[stage]);
            for (int i = tid; i < PAGE_TOKENS * CH; i += TEAM) {
                const int r = i / CH, c = i % CH;
                const bool ok = r >= it.k_first && r <= it.k_last && r != it.r_new;
                cp_async_16(k_base + swz<CH>(r, c), L.k_cache + tile + (size_t)r * HD + c * 8, ok);
                cp_async_16(v_base + swz<CH>(r, c), L.v_cache + tile + (size_t)r * HD + c * 8, ok);
            }
        }
        cp_async_commit();
    };

    PageItem cur, nxt;
    int item = next_real(blockIdx.x * 2 + team, cur);
    int stage = 0;
    if (item < n_items) issue(cur, 0);
    while (item < n_items) {
        const int item_next = next_real(item + stride, nxt);
        cp_async_wait<0>();
        team_sync(team);                                           // cur's tiles have landed; the other stage is free
        if (item_next < n_items) issue(nxt, stage ^ 1);
        const int b = cur.b, kvh = cur.kvh;
        const size_t row0 = ((size_t)b * a.H + (size_t)kvh * G) * a.S_max + cur.s;
        const int pos = meta.pos[b];
        if (cur.page < 0) {
            if (tid == 0) atomicOr(a.status, cur.page == -2 ? MYNAH_ST_POS_RANGE : MYNAH_ST_PAGE_RANGE);
            for (int i = tid; i < G; i += TEAM) {
                a.part_ml[(row0 + (size_t)i * a.S_max) * 2] = -INFINITY;
                a.part_ml[(row0 + (size_t)i * a.S_max) * 2 + 1] = 0.f;
            }
        } else {
            const int k_first = cur.k_first, k_last = cur.k_last, r_new = cur.r_new;
            const size_t tile = ((size_t)cur.page * a.KV + kvh) * PAGE_TOKENS * HD;
            const uint32_t k_base = smem_u32(sm.k[stage]), v_base = smem_u32(sm.v[stage]);
            // q of the group's heads: norm, rotation, to shared memory as bf16 (rows beyond G stay zero)
            const bf16* qrow = a.qkv + (size_t)b * ldq;
            for (int h = warp; h < G; h += 4) {
                float v[EPL];
#pragma unroll
                for (int j = 0; j < EPL; j++) v[j] = to_f32(qrow[(size_t)(kvh * G + h) * HD + lane * EPL + j]);
                head_norm_rope<HD>(v, qg, a.qk_eps, L.cos_t, L.sin_t, pos, lane);
#pragma unroll
                for (int j = 0; j < EPL; j++) sm.q[h * HD + lane * EPL + j] = __float2bfloat16_rn(v[j]);
            }
            // the new position's k and v: computed by the team that has its page, written to the cache and to the tiles
            if (r_new >= 0 && warp == 3) {
                float kv[EPL], vv[EPL];
#pragma unroll
                for (int j = 0; j < EPL; j++) {
                    kv[j] = to_f32(qrow[(size_t)(a.H + kvh) * HD + lane * EPL + j]);
                    vv[j] = to_f32(qrow[(size_t)(a.H + a.KV + kvh) * HD + lane * EPL + j]);
                }
                head_norm_rope<HD>(kv, kg, a.qk_eps, L.cos_t, L.sin_t, pos, lane);
#pragma unroll
                for (int j = 0; j < EPL; j++) {
                    const int d = lane * EPL + j;
                    const bf16 kb16 = __float2bfloat16_rn(kv[j]), vb16 = __float2bfloat16_rn(vv[j]);
                    L.k_cache[tile + (size_t)r_new * HD + d] = kb16;
                    L.v_cache[tile + (size_t)r_new * HD + d] = vb16;
                    *reinterpret_cast<bf16*>(sm.k[stage] + swz<CH>(r_new, d / 8) + (d % 8) * 2) = kb16;
                    *reinterpret_cast<bf16*>(sm.v[stage] + swz<CH>(r_new, d / 8) + (d % 8) * 2) = vb16;
                }
            }
            team_sync(team);

            uint32_t qa[KSTEPS][4];
            {
                const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
                    const int col = ks * 16 + c0;
                    qa[ks][0] = *reinterpret_cast<const uint32_t*>(sm.q + r0 * HD + col);
                    qa[ks][1] = *reinterpret_cast<const uint32_t*>(sm.q + (r0 + 8) * HD + col);
                    qa[ks][2] = *reinterpret_cast<const uint32_t*>(sm.q + r0 * HD + col + 8);
                    qa[ks][3] = *reinterpret_cast<const uint32_t*>(sm.q + (r0 + 8) * HD + col + 8);
                }
            }
            float sc[2][4] = {};
            {
                const int mat = lane >> 3, rr = lane & 7;
                const int key = warp * 16 + (mat >> 1) * 8 + rr;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
                    uint32_t kb[4];
                    ldmatrix_x4(kb, k_base + swz<CH>(key, ks * 2 + (mat & 1)));
                    mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
                    mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
                }
            }
            const int hrow = lane >> 2;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int t2 = 0; t2 < 2; t2++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = warp * 16 + t2 * 8 + (lane & 3) * 2 + (e & 1);
                    const bool vis = key >= k_first && key <= k_last;
                    sc[t2][e] = vis ? sc[t2][e] * scale : -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sc[t2][e]);
                }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 1));
                mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 2));
            }
            if ((lane & 3) == 0) {
                sm.red_m[warp][hrow] = mx[0];
                sm.red_m[warp][hrow + 8] = mx[1];
            }
            team_sync(team);
            float m[2], l[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int h = hrow + 8 * j;
                m[j] = fmaxf(fmaxf(sm.red_m[0][h], sm.red_m[1][h]), fmaxf(sm.red_m[2][h], sm.red_m[3][h]));
            }
#pragma unroll
            for (int t2 = 0; t2 < 2; t2++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const float p0 = expf(sc[t2][2 * j] - m[j]), p1 = expf(sc[t2][2 * j + 1] - m[j]);
                    l[j] += p0 + p1;
                    const int h = hrow + 8 * j, key = warp * 16 + t2 * 8 + (lane & 3) * 2;
                    *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<unsigned char*>(sm.p) + swz<8>(h, key >> 3) + (key & 7) * 2) =
                        __floats2bfloat162_rn(p0, p1);
                }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                l[j] += __shfl_xor_sync(0xffffffffu, l[j], 1);
                l[j] += __shfl_xor_sync(0xffffffffu, l[j], 2);
            }
            if ((lane & 3) == 0) {
                sm.red_l[warp][hrow] = l[0];
                sm.red_l[warp][hrow + 8] = l[1];
            }
            team_sync(team);
            float oc[NT][4] = {};
            {
                const uint32_t p_base = smem_u32(sm.p);
                const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
                for (int ks = 0; ks < PAGE_TOKENS / 16; ks++) {
                    uint32_t pa[4];
                    ldmatrix_x4(pa, p_base + swz<8>((mat & 1) * 8 + rr, ks * 2 + (mat >> 1)));
#pragma unroll
                    for (int nt = 0; nt < NT; nt += 2) {
                        uint32_t vb[4];
                        ldmatrix_x4_trans(vb, v_base + swz<CH>(ks * 16 + (mat & 1) * 8 + rr, warp * (HD / 32) + nt + (mat >> 1)));
                        mma_bf16(oc[nt], pa, vb[0], vb[1]);
                        mma_bf16(oc[nt + 1], pa, vb[2], vb[3]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int h = hrow + 8 * j;
                if (h < G) {
                    float* o = a.part_o + (row0 + (size_t)h * a.S_max) * HD;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
                        *reinterpret_cast<float2*>(o + warp * (HD / 4) + nt * 8 + (lane & 3) * 2) = make_float2(oc[nt][2 * j], oc[nt][2 * j + 1]);
                }
            }
            if (tid < G) {
                a.part_ml[(row0 + (size_t)tid * a.S_max) * 2] =
                    fmaxf(fmaxf(sm.red_m[0][tid], sm.red_m[1][tid]), fmaxf(sm.red_m[2][tid], sm.red_m[3][tid]));
                a.part_ml[(row0 + (size_t)tid * a.S_max) * 2 + 1] = (sm.red_l[0][tid] + sm.red_l[1][tid]) + (sm.red_l[2][tid] + sm.red_l[3][tid]);
            }
        }
        // ---- the team that finishes this (sequence, kv head) last merges its pages, in page order
        const int n_vis = meta.n_vis[grp][b];
        __threadfence();
        team_sync(team);
        if (tid == 0) {
            const unsigned old = atomicAdd(a.counters + b * a.KV + kvh, 1u);
            sm.last_flag = old == (unsigned)(n_vis - 1);
            if (sm.last_flag) a.counters[b * a.KV + kvh] = 0;      // ready for the next layer
        }
        team_sync(team);
        if (sm.last_flag) {
            __threadfence();
            const int S = min(n_vis, a.S_max);
            for (int i = 0; i < G; i++) {
                const int h = kvh * G + i;
                const size_t r0h = ((size_t)b * a.H + h) * a.S_max;
                float mx = -INFINITY;
                for (int s2 = tid; s2 < S; s2 += TEAM) mx = fmaxf(mx, __ldcg(a.part_ml + (r0h + s2) * 2));
                mx = warp_max(mx);
                if (lane == 0) sm.red_m[warp][0] = mx;
                team_sync(team);
                mx = fmaxf(fmaxf(sm.red_m[0][0], sm.red_m[1][0]), fmaxf(sm.red_m[2][0], sm.red_m[3][0]));
                for (int s2 = tid; s2 < S; s2 += TEAM) {
                    const float ms = __ldcg(a.part_ml + (r0h + s2) * 2);
                    sm.w[s2] = ms == -INFINITY ? 0.f : expf(ms - mx);
                }
                team_sync(team);
                float ls = 0.f;
                for (int s2 = 0; s2 < S; s2++) ls += __ldcg(a.part_ml + (r0h + s2) * 2 + 1) * sm.w[s2];   // page order
                const float inv = ls > 0.f ? 1.0f / ls : 0.f;
                for (int d = tid; d < HD; d += TEAM) {
                    float os = 0.f;
#pragma unroll 4
                    for (int s2 = 0; s2 < S; s2++) {
                        const float w = sm.w[s2];
                        os += w != 0.f ? __ldcg(a.part_o + (r0h + s2) * HD + d) * w : 0.f;
                    }
                    a.attn_out[(size_t)b * a.H * HD + (size_t)h * HD + d] = __float2bfloat16_rn(os * inv);
                }
                team_sync(team);
            }
        }
        cur = nxt;
        item = item_next;
        stage ^= 1;
    }
    cp_async_wait<0>();
}

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
decode_step_kernel(const StepArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float red[WARPS][32][8];
    __shared__ float part[WARPS];
    __shared__ StepMeta meta;
    bf16* xs = reinterpret_cast<bf16*>(smem);
    const int M = a.M, D = a.D;
    float* x_cur = a.x0;
    float* x_nxt = a.x1;
    const int QKV_N = (a.H + 2 * a.KV) * HD;

    // ---- the step's sequences, once: lengths, positions, visible pages per storage group
    if (threadIdx.x < MAX_GROUPS) meta.window[threadIdx.x] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int l = 0; l < a.n_layers; l++) meta.window[a.layers[l].group] = a.layers[l].window;
        meta.pages = a.table_offset >= 0 ? reinterpret_cast<const int*>(smem + a.table_offset) : nullptr;
    }
    if (threadIdx.x < M) {
        meta.kv_len[threadIdx.x] = a.kv_len[threadIdx.x];
        meta.pos[threadIdx.x] = a.tok_pos[threadIdx.x];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.n_groups * M; i += THREADS) {
        const int g = i / M, b = i % M, hi = meta.kv_len[b];
        const int lo = meta.window[g] > 0 ? max(0, hi - meta.window[g]) : 0;
        const int pg0 = lo / PAGE_TOKENS, pg1 = hi > 0 ? (hi - 1) / PAGE_TOKENS + 1 : pg0;
        meta.pg0[g][b] = pg0;
        meta.n_vis[g][b] = hi > 0 ? pg1 - pg0 : 0;
        if (pg1 - pg0 > a.S_max) atomicOr(a.status, MYNAH_ST_SPLIT_RANGE);
    }
    __syncthreads();
    if (a.table_offset >= 0) {
        int* table = reinterpret_cast<int*>(smem + a.table_offset);
        for (int i = threadIdx.x; i < a.n_groups * M * a.S_max; i += THREADS) {
            const int s = i % a.S_max, b = (i / a.S_max) % M, g = i / (a.S_max * M);
            table[i] = s < meta.n_vis[g][b] ? page_of(a.pt[g], b, (meta.pg0[g][b] + s) * PAGE_TOKENS) : -1;
        }
    }
    {   // the first layer's weights on their way into L2
        const LayerDesc& L0 = a.layers[0];
        prefetch_matrix(L0.w_qkv, (size_t)QKV_N * D * 2);
        prefetch_matrix(L0.w_o, (size_t)D * a.H * HD * 2);
        prefetch_matrix(L0.w_gu, (size_t)2 * a.F * D * 2);
        prefetch_matrix(L0.w_down, (size_t)D * a.F * 2);
    }
    __syncthreads();

    int n_stamp = 0;
    auto stamp = [&]() { if (a.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && n_stamp < 64) a.trace[n_stamp++] = now_ns(); };
    stamp();
    for (int l = 0; l < a.n_layers; l++) {
        const LayerDesc& L = a.layers[l];
        // ---- phase 1: residual (+ add) -> norm -> q,k,v
        {
            const int ldx = D + XPAD;
            if (l == 0) {
                const bf16* emb = a.embed;
                const int* toks = a.tokens;
                const int V = a.V;
                auto src = [=](int m, int i) {
                    const int t = toks[m];
                    return (t >= 0 && t < V) ? to_f32(emb[(size_t)t * D + i]) : 0.f;
                };
                norm_rows(xs, ldx, M, D, src, VecRef{L.norm1, L.norm1_dt}, a.eps, x_nxt, part);
            } else {
                const float* xc = x_cur;
                const bf16* dl = a.delta;
                auto src = [=](int m, int i) { return __ldcg(xc + (size_t)m * D + i) + to_f32(dl[(size_t)m * D + i]); };
                norm_rows(xs, ldx, M, D, src, VecRef{L.norm1, L.norm1_dt}, a.eps, x_nxt, part);
            }
            float* tmp = x_cur; x_cur = x_nxt; x_nxt = tmp;
            gemv_phase<OUT_BF16>(L.w_qkv, QKV_N, D, xs, ldx, M, a.qkv, QKV_N, red);
        }
        stamp();
        // the next layer's weights (or the first part of the head) start towards L2 while this layer runs
        if (l + 1 < a.n_layers) {
            const LayerDesc& Ln = a.layers[l + 1];
            prefetch_matrix(Ln.w_qkv, (size_t)QKV_N * D * 2);
            prefetch_matrix(Ln.w_o, (size_t)D * a.H * HD * 2);
            prefetch_matrix(Ln.w_gu, (size_t)2 * a.F * D * 2);
            prefetch_matrix(Ln.w_down, (size_t)D * a.F * 2);
        } else {
            const size_t head_bytes = (size_t)a.V * D * 2;
            prefetch_matrix(a.head, head_bytes < ((size_t)64 << 20) ? head_bytes : ((size_t)64 << 20));
        }
        if (!grid_barrier(a)) return;
        stamp();
        // ---- phase 2: attention over the cache, the new position included
        attention_phase<HD>(a, L, meta, reinterpret_cast<TeamSmem<HD>*>(smem)[threadIdx.x / TEAM], threadIdx.x / TEAM);
        stamp();
        if (!grid_barrier(a)) return;
        stamp();
        // ---- phase 3: o
        {
            const int K = a.H * HD, ldx = K + XPAD;
            load_rows(xs, ldx, a.attn_out, M, K);
            gemv_phase<OUT_BF16>(L.w_o, D, K, xs, ldx, M, a.delta, D, red);
        }
        stamp();
        if (!grid_barrier(a)) return;
        stamp();
        // ---- phase 4: residual + delta -> norm -> gate/up -> SwiGLU
        {
            const int ldx = D + XPAD;
            const float* xc = x_cur;
            const bf16* dl = a.delta;
            auto src = [=](int m, int i) { return __ldcg(xc + (size_t)m * D + i) + to_f32(dl[(size_t)m * D + i]); };
            norm_rows(xs, ldx, M, D, src, VecRef{L.norm2, L.norm2_dt}, a.eps, x_nxt, part);
            float* tmp = x_cur; x_cur = x_nxt; x_nxt = tmp;
            gemv_phase<OUT_SWIGLU>(L.w_gu, a.F, D, xs, ldx, M, a.act, a.F, red);
        }
        if (!grid_barrier(a)) return;
        // ---- phase 5: down
        {
            const int K = a.F, ldx = K + XPAD;
            load_rows(xs, ldx, a.act, M, K);
            gemv_phase<OUT_BF16>(L.w_down, D, K, xs, ldx, M, a.delta, D, red);
        }
        if (!grid_barrier(a)) return;
    }
    // ---- head: residual + delta -> norm -> logits
    {
        const int ldx = D + XPAD;
        const float* xc = x_cur;
        const bf16* dl = a.delta;
        auto src = [=](int m, int i) { return __ldcg(xc + (size_t)m * D + i) + to_f32(dl[(size_t)m * D + i]); };
        norm_rows(xs, ldx, M, D, src, VecRef{a.final_gain, a.final_dt}, a.eps, nullptr, part);
        gemv_phase<OUT_F32>(a.head, a.V, D, xs, ldx, M, a.logits, a.V, red);
    }
}

constexpr size_t TABLE_MAX_BYTES = 32 * 1024;

size_t step_buffers(int M, int D, int H, int HD, int F) {
    const size_t rows = M > 8 ? 16 : 8;
    size_t xs = rows * (size_t)(D + XPAD) * 2;
    xs = xs > rows * (size_t)(H * HD + XPAD) * 2 ? xs : rows * (size_t)(H * HD + XPAD) * 2;
    xs = xs > rows * (size_t)(F + XPAD) * 2 ? xs : rows * (size_t)(F + XPAD) * 2;
    const size_t att = 2 * (HD == 128 ? sizeof(TeamSmem<128>) : sizeof(TeamSmem<64>));
    return (((xs > att ? xs : att) + 127) / 128) * 128;
}

// Dynamic shared memory: the phase buffers, then (when small enough) the table of visible pages.
size_t step_smem(int M, int D, int H, int HD, int F, int n_groups, int S_max, int* table_offset) {
    const size_t buf = step_buffers(M, D, H, HD, F);
    const size_t table = (size_t)n_groups * M * S_max * 4;
    if (table <= TABLE_MAX_BYTES) {
        if (table_offset) *table_offset = (int)buf;
        return buf + table;
    }
    if (table_offset) *table_offset = -1;
    return buf;
}

}  // namespace

// Sizes this kernel takes: bfloat16, up to 16 rows, head_dim 64 or 128, widths that are multiples of 32.
MYNAH_API int mynah_decode_step_supported(int M, int D, int H, int KV, int HD, int F, int V, int S_max) {
    if (M < 1 || M > MAX_M || (HD != 64 && HD != 128) || KV < 1 || H % KV != 0 || H / KV > MAX_G) return 0;
    if (D % 32 != 0 || (H * HD) % 32 != 0 || F % 32 != 0 || V < 8 || S_max < 1 || S_max > 1024) return 0;
    return step_smem(M, D, H, HD, F, MAX_GROUPS, S_max, nullptr) <= 220 * 1024;
}

MYNAH_API int mynah_decode_step_layer_bytes(void) { return (int)sizeof(LayerDesc); }

// Fills one LayerDesc (host memory, `mynah_decode_step_layer_bytes()` bytes) from plain arguments.
MYNAH_API int mynah_decode_step_fill_layer(void* dst, const void* w_qkv, const void* w_o, const void* w_gu, const void* w_down,
                                           const void* norm1, int norm1_dt, const void* norm2, int norm2_dt,
                                           const void* q_gain, const void* k_gain, int qk_dt, void* k_cache, void* v_cache,
                                           const float* cos_t, const float* sin_t, int n_pos, int group, int window) {
    MYNAH_REQUIRE(group >= 0 && group < MAX_GROUPS, "decode_step: at most %d storage groups", MAX_GROUPS);
    LayerDesc L = {};
    L.w_qkv = (const bf16*)w_qkv; L.w_o = (const bf16*)w_o; L.w_gu = (const bf16*)w_gu; L.w_down = (const bf16*)w_down;
    L.norm1 = norm1; L.norm2 = norm2; L.q_gain = q_gain; L.k_gain = k_gain;
    L.norm1_dt = norm1_dt; L.norm2_dt = norm2_dt; L.qk_dt = qk_dt;
    L.k_cache = (bf16*)k_cache; L.v_cache = (bf16*)v_cache; L.cos_t = cos_t; L.sin_t = sin_t;
    L.n_pos = n_pos; L.group = group; L.window = window;
    *static_cast<LayerDesc*>(dst) = L;
    return 0;
}

// One decode step. `layers`: device array of n_layers LayerDesc. `ints`: the step's batch description (device):
// tokens [M], tok_pos [M], kv_len [M]. Page tables per storage group: indptr/ids/base arrays of n_groups pointers.
// Work buffers (device): x0, x1 fp32 [M, D]; qkv bf16 [M, (H+2KV)HD]; attn_out bf16 [M, H*HD]; delta bf16 [M, D];
// act bf16 [M, F]; part fp32 [M*H*S_max*(HD+2)]; counters u32 [M*KV] (zero); sync u32 [4] (zero before the first
// step); logits fp32 [M, V]. The launch is cooperative: all CTAs are resident at once.
MYNAH_API int mynah_decode_step(
    int n_layers, int M, int D, int H, int KV, int HD, int F, int V, int S_max, float eps, float qk_eps,
    const void* layers, const int* tokens, const int* tok_pos, const int* kv_len,
    int n_groups, const int* const* pt_indptr, const int* const* pt_ids, const int* const* pt_base, const int* pt_pages,
    const void* embed, const void* final_gain, int final_dt, const void* head,
    float* x0, float* x1, void* qkv, void* attn_out, void* delta, void* act, float* part, unsigned* counters,
    unsigned* sync_words, float* logits, int sm_count, int* status, unsigned long long* trace, cudaStream_t stream) {
    MYNAH_REQUIRE(mynah_decode_step_supported(M, D, H, KV, HD, F, V, S_max), "decode_step: these sizes are not taken");
    MYNAH_REQUIRE(n_groups >= 1 && n_groups <= MAX_GROUPS && n_layers >= 1, "decode_step: bad layer or group count");
    StepArgs a = {};
    a.n_layers = n_layers; a.M = M; a.D = D; a.H = H; a.KV = KV; a.HD = HD; a.F = F; a.V = V; a.S_max = S_max;
    a.eps = eps; a.qk_eps = qk_eps;
    a.layers = static_cast<const LayerDesc*>(layers);
    a.tokens = tokens; a.tok_pos = tok_pos; a.kv_len = kv_len;
    for (int g = 0; g < n_groups; g++) a.pt[g] = PageTable{pt_indptr[g], pt_ids[g], pt_base[g], pt_pages[g]};
    a.embed = (const bf16*)embed; a.final_gain = final_gain; a.final_dt = final_dt; a.head = (const bf16*)head;
    a.x0 = x0; a.x1 = x1; a.qkv = (bf16*)qkv; a.attn_out = (bf16*)attn_out; a.delta = (bf16*)delta; a.act = (bf16*)act;
    a.part_o = part; a.part_ml = part + (size_t)M * H * S_max * HD;
    a.counters = counters; a.logits = logits;
    a.bar_count = sync_words; a.bar_gen = sync_words + 1; a.abort_word = reinterpret_cast<int*>(sync_words + 2);
    a.status = status;
    a.trace = trace;
    a.n_groups = n_groups;
    const size_t smem = step_smem(M, D, H, HD, F, n_groups, S_max, &a.table_offset);
    void (*kern)(const StepArgs) = HD == 128 ? decode_step_kernel<128> : decode_step_kernel<64>;
    static size_t opted[2] = {0, 0};
    size_t& mine = opted[HD == 128 ? 1 : 0];
    if (smem > mine) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("decode_step: %s", cudaGetErrorString(e));
        mine = smem;
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem);
    if (e != cudaSuccess || per_sm < 1) return mynah_fail("decode_step: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
    void* params[] = {&a};
    e = cudaLaunchCooperativeKernel((const void*)kern, dim3(sm_count > 0 ? sm_count : 148), dim3(THREADS), params, smem, stream);
    if (e != cudaSuccess) return mynah_fail("decode_step: %s", cudaGetErrorString(e));
    return 0;
}
