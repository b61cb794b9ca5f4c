// Attention of a decode step: one query per sequence against that sequence's
// cached keys, split over the key range so that a small batch still fills
// the GPU, then combined.
//
// The unit of splitting is one page (64 positions): split s of a sequence is
// the s-th page it can see. The partial results of a sequence's pages are
// combined in page order, so a sequence's output has the same bits whatever
// else is in the batch and however large the launch was made.
//
// Split kernel: one CTA per (page, kv head [x head tile], sequence). It reads
// each K/V byte of its range once and serves all query heads of the group
// from it (GQA: query head h reads kv head h / (H/KV), mynah-slm
// src/kernels.c:256-261). A lane owns 8 consecutive dims of a key; the lanes
// of a key reduce the dot by shuffles; each key slot of a warp keeps its own
// running maximum, sum and output, merged at the end in a fixed order.
// Combine kernel: merges the splits of one (sequence, head).
//
// score = dot * (1/sqrtf(head_dim)); maximum subtracted; fp32 throughout
// (src/kernels.c:228-250, :207-220). The partial results live in scratch
// memory that the caller provides: part_o [B][H][S][HD] and part_ml
// [B][H][S][2] floats.
#include "layout.cuh"

namespace {

constexpr int WARPS = 4;

struct DecodeArgs {
    int H, KV, HD, ldq, ldo;
    int window;          // 0: all keys
    int S;               // pages a sequence may see at most (grid size and scratch stride)
    int lpk;             // lanes per key: power of two >= HD/8, <= 32
    float scale;
};

template <int GT>
struct HeadState {
    float m[GT], l[GT], acc[GT][8];
};

template <typename T, int GT>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ kv_len, PageTable pt, DecodeArgs a,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ status) {
    const int s = blockIdx.x, b = blockIdx.z;
    const int G = a.H / a.KV;
    const int tiles = (G + GT - 1) / GT;
    const int g = blockIdx.y / tiles, h0 = g * G + (blockIdx.y % tiles) * GT;   // first query head of this CTA
    const int n_heads = min(GT, g * G + G - h0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lpk = a.lpk, kpw = 32 / lpk;
    const int u = lane % lpk, slot = lane / lpk;
    const int HD = a.HD;
    const bool lane_on = u * 8 < HD;

    // key range of this split: the s-th page of the visible range
    const int hi = kv_len[b];
    int lo = 0;
    if (a.window > 0) lo = max(0, hi - a.window);
    int key_begin = 0, key_end = 0;
    if (hi > 0) {
        const int pg0 = lo / PAGE_TOKENS, pg1 = (hi - 1) / PAGE_TOKENS + 1;
        if (pg1 - pg0 > a.S) {                         // the launch is too small for this sequence: say so
            if (threadIdx.x == 0 && s == 0) atomicOr(status, MYNAH_ST_SPLIT_RANGE);
        }
        const int mp = pg0 + s;
        if (mp < pg1) {
            key_begin = max(lo, mp * PAGE_TOKENS);
            key_end = min(hi, (mp + 1) * PAGE_TOKENS);
        }
    }

    float qv[GT][8];
#pragma unroll
    for (int i = 0; i < GT; i++) {
#pragma unroll
        for (int j = 0; j < 8; j++) qv[i][j] = 0.f;
        if (i < n_heads && lane_on) load8(q + (size_t)b * a.ldq + (size_t)(h0 + i) * HD + u * 8, qv[i]);
    }

    HeadState<GT> st;
#pragma unroll
    for (int i = 0; i < GT; i++) {
        st.m[i] = -INFINITY;
        st.l[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) st.acc[i][j] = 0.f;
    }

    const int pt_lo = pt.indptr[b], pt_cnt = pt.indptr[b + 1] - pt_lo, pt_base = pt.base[b];
    bool bad_page = false;
    for (int base = key_begin + warp * kpw; base < key_end; base += WARPS * kpw) {
        const int key = base + slot;
        const bool valid = key < key_end;
        float kf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, vf[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        bool have = false;
        if (valid) {
            const int lp = key / PAGE_TOKENS - pt_base;
            int page = (lp >= 0 && lp < pt_cnt) ? pt.ids[pt_lo + lp] : -1;
            if (page >= pt.n_pages) page = -1;
            if (page < 0) {
                bad_page = true;
            } else if (lane_on) {
                const size_t off = (((size_t)page * a.KV + g) * PAGE_TOKENS + key % PAGE_TOKENS) * HD + u * 8;
                load8(k_cache + off, kf);
                load8(v_cache + off, vf);
            }
            have = page >= 0;
        }
#pragma unroll
        for (int i = 0; i < GT; i++) {
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) d = fmaf(qv[i][j], kf[j], d);
            for (int o = lpk >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (have) {
                const float sc = d * a.scale;
                const float m_new = fmaxf(st.m[i], sc);
                const float alpha = expf(st.m[i] - m_new);
                const float p = expf(sc - m_new);
                st.l[i] = st.l[i] * alpha + p;
                st.m[i] = m_new;
#pragma unroll
                for (int j = 0; j < 8; j++) st.acc[i][j] = fmaf(p, vf[j], st.acc[i][j] * alpha);
            }
        }
    }
    if (bad_page) atomicOr(status, MYNAH_ST_PAGE_RANGE);

    // merge the key slots of a warp (lanes that own the same dims), then the warps
#pragma unroll
    for (int i = 0; i < GT; i++) {
        for (int o = lpk; o < 32; o <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, st.m[i], o);
            const float l2 = __shfl_xor_sync(0xffffffffu, st.l[i], o);
            const float mn = fmaxf(st.m[i], m2);
            const float a1 = mn == -INFINITY ? 0.f : expf(st.m[i] - mn);
            const float a2 = mn == -INFINITY ? 0.f : expf(m2 - mn);
            st.l[i] = st.l[i] * a1 + l2 * a2;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float o2 = __shfl_xor_sync(0xffffffffu, st.acc[i][j], o);
                st.acc[i][j] = st.acc[i][j] * a1 + o2 * a2;
            }
            st.m[i] = mn;
        }
    }
    __shared__ float sm_m[WARPS][GT], sm_l[WARPS][GT];
    __shared__ float sm_o[WARPS][GT][256];
    if (slot == 0 && lane_on) {
#pragma unroll
        for (int i = 0; i < GT; i++) {
            if (u == 0) {
                sm_m[warp][i] = st.m[i];
                sm_l[warp][i] = st.l[i];
            }
#pragma unroll
            for (int j = 0; j < 8; j++) sm_o[warp][i][u * 8 + j] = st.acc[i][j];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_heads * HD; idx += blockDim.x) {
        const int i = idx / HD, d = idx % HD;
        float mn = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; w++) mn = fmaxf(mn, sm_m[w][i]);
        float ls = 0.f, os = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; w++) {
            const float aw = mn == -INFINITY ? 0.f : expf(sm_m[w][i] - mn);
            ls += sm_l[w][i] * aw;
            os += sm_o[w][i][d] * aw;
        }
        const size_t row = ((size_t)b * a.H + (h0 + i)) * a.S + s;
        part_o[row * HD + d] = os;
        if (d == 0) {
            part_ml[row * 2] = mn;
            part_ml[row * 2 + 1] = ls;
        }
    }
}

template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           T* __restrict__ out, const int* __restrict__ kv_len, int window,
                                           int H, int HD, int S_max, int ldo) {
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t row0 = ((size_t)b * H + h) * S_max;
    // only the pages the sequence can see have partial results
    const int hi = kv_len[b];
    const int lo = window > 0 ? max(0, hi - window) : 0;
    const int S = hi > 0 ? min(S_max, (hi - 1) / PAGE_TOKENS + 1 - lo / PAGE_TOKENS) : 0;
    float mn = -INFINITY;
    for (int s = 0; s < S; s++) mn = fmaxf(mn, part_ml[(row0 + s) * 2]);
    float ls = 0.f;
    for (int s = 0; s < S; s++) {
        const float m = part_ml[(row0 + s) * 2];
        ls += mn == -INFINITY ? 0.f : part_ml[(row0 + s) * 2 + 1] * expf(m - mn);
    }
    const float inv = ls > 0.f ? 1.0f / ls : 0.f;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float os = 0.f;
        for (int s = 0; s < S; s++) {
            const float m = part_ml[(row0 + s) * 2];
            if (m != -INFINITY) os += part_o[(row0 + s) * HD + d] * expf(m - mn);
        }
        out[(size_t)b * ldo + (size_t)h * HD + d] = from_f32<T>(os * inv);
    }
}

template <typename T>
int launch_decode(const void* q, void* out, int B, const DecodeArgs& a, const void* k_cache, const void* v_cache,
                  const int* kv_len, const PageTable& pt, float* part_o, float* part_ml, int* status,
                  cudaStream_t stream) {
    const int G = a.H / a.KV;
    const int gt = G == 1 ? 1 : (G == 2 ? 2 : 4);
    const int tiles = ceil_div(G, gt);
    const dim3 grid(a.S, a.KV * tiles, B);
    const T* qp = (const T*)q;
    const T* kp = (const T*)k_cache;
    const T* vp = (const T*)v_cache;
    if (gt == 1)
        attn_decode_split_kernel<T, 1><<<grid, WARPS * 32, 0, stream>>>(qp, kp, vp, kv_len, pt, a, part_o, part_ml, status);
    else if (gt == 2)
        attn_decode_split_kernel<T, 2><<<grid, WARPS * 32, 0, stream>>>(qp, kp, vp, kv_len, pt, a, part_o, part_ml, status);
    else
        attn_decode_split_kernel<T, 4><<<grid, WARPS * 32, 0, stream>>>(qp, kp, vp, kv_len, pt, a, part_o, part_ml, status);
    if (mynah_check_launch("attn_decode_split")) return -1;
    const int threads = a.HD >= 128 ? 128 : (a.HD >= 64 ? 64 : 32);
    attn_decode_combine_kernel<T><<<dim3(a.H, B), threads, 0, stream>>>(part_o, part_ml, (T*)out, kv_len, a.window, a.H, a.HD, a.S, a.ldo);
    return mynah_check_launch("attn_decode_combine");
}

}  // namespace

// Floats of scratch that a decode step of these sizes needs:
// part_o [B][H][S][HD] followed by part_ml [B][H][S][2].
MYNAH_API long long mynah_attn_decode_scratch_floats(int B, int H, int HD, int n_splits) {
    return (long long)B * H * n_splits * (HD + 2);
}

// q: [B, ldq], one row per sequence; out: [B, ldo]. head_dim must be a
// multiple of 8 (16-byte rows) and at most 256.
MYNAH_API int mynah_attn_decode(
    const void* q, void* out, int dtype, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, float* scratch, int* status, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && KV > 0 && HD > 0 && H % KV == 0, "attn_decode: bad sizes B=%d H=%d KV=%d HD=%d", B, H, KV, HD);
    MYNAH_REQUIRE(HD % 8 == 0 && HD <= 256, "attn_decode: head_dim %d must be a multiple of 8 and at most 256", HD);
    MYNAH_REQUIRE(ldq % 8 == 0, "attn_decode: query row stride %d must be a multiple of 8", ldq);
    MYNAH_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attn_decode: bad split count %d", n_splits);
    MYNAH_REQUIRE(B <= 65535, "attn_decode: batch %d exceeds one launch", B);
    MYNAH_REQUIRE(scratch != nullptr, "attn_decode: no scratch memory given");
    int lpk = 1;
    while (lpk * 8 < HD) lpk <<= 1;
    const DecodeArgs a{H, KV, HD, ldq, ldo, window, n_splits, lpk, 1.0f / sqrtf((float)HD)};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)B * H * n_splits * HD;
    if (dtype == MYNAH_F32)
        return launch_decode<float>(q, out, B, a, k_cache, v_cache, kv_len, pt, part_o, part_ml, status, stream);
    if (dtype == MYNAH_BF16)
        return launch_decode<bf16>(q, out, B, a, k_cache, v_cache, kv_len, pt, part_o, part_ml, status, stream);
    return mynah_fail("attn_decode: unsupported dtype %d", dtype);
}

// ---------------------------------------------------------------------------
// The same decode attention for callers that must not allocate: the partial
// results go to a fixed array of this library instead of caller-provided
// scratch. See no_alloc.h for who needs this and for the rules of use.
#include "no_alloc.h"

#include <mutex>

namespace {

static __device__ __align__(256) float g_no_alloc_scratch[MYNAH_NO_ALLOC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
std::mutex g_no_alloc_mutex;
float* g_no_alloc_ptr[MAX_DEVICES] = {};

// Device address of the array on the current device. In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, looked up once per device.
int no_alloc_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return mynah_fail("attn_decode_no_alloc: no current device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return mynah_fail("attn_decode_no_alloc: device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_no_alloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return mynah_fail("attn_decode_no_alloc: cannot find the scratch array on device %d: %s", dev,
                              cudaGetErrorString(e));
        g_no_alloc_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_no_alloc_ptr[dev];
    return 0;
}

}  // namespace

MYNAH_API int mynah_attn_decode_no_alloc(
    const void* q, void* out, int dtype, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, int* status, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && HD > 0 && n_splits >= 1, "attn_decode_no_alloc: bad sizes B=%d H=%d HD=%d splits=%d", B, H, HD, n_splits);
    const long long need = mynah_attn_decode_scratch_floats(B, H, HD, n_splits);
    MYNAH_REQUIRE(need <= (long long)MYNAH_NO_ALLOC_SCRATCH_FLOATS,
                  "attn_decode_no_alloc: B=%d H=%d head_dim=%d splits=%d need %lld floats of scratch, the built-in "
                  "array holds %d; use mynah_attn_decode with scratch of your own",
                  B, H, HD, n_splits, need, MYNAH_NO_ALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (no_alloc_scratch(&scratch) != 0) return -1;
    return mynah_attn_decode(q, out, dtype, B, H, KV, HD, ldq, ldo, k_cache, v_cache, kv_len, page_indptr, page_ids,
                             page_base, n_pages, window, n_splits, scratch, status, stream);
}
