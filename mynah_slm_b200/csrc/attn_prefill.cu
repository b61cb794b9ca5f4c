// Causal grouped-query attention of a ragged batch over the paged cache:
// every query of the step reads the keys of its own sequence at positions
// <= its own (and > its own - window, when the layer has a window), wherever
// they were written: in this step or in earlier ones.
//
// This is the general kernel: any head_dim up to 256, any number of heads and
// groups, both precisions, any mix of query lengths (one token included). It
// is the only attention of the 32-bit path's prompts, and the fallback of the
// bf16 path for head sizes the tensor-core kernel does not take.
//
// Formulas: score = dot(q, k) * (1/sqrtf(head_dim)), scale after the dot;
// softmax with the maximum subtracted; out = sum_t p_t v_t; query head h
// reads kv head h / (H/KV)  (mynah-slm src/kernels.c:228-250, :207-220).
// Scores, softmax and the output sum are fp32. Keys are taken 32 at a time at
// positions that are multiples of 32, so a query's sum runs in the same
// order whatever else is in the batch.
#include "layout.cuh"

namespace {

constexpr int QT = 16;          // queries per CTA
constexpr int KT = 32;          // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int QPW = QT / WARPS; // queries per warp
constexpr int MAXC = 8;         // head_dim <= 32 * MAXC

struct PrefillArgs {
    int B, H, KV, HD, ldq, ldo;
    int window;                 // 0: all keys
    float scale;
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
attn_prefill_generic_kernel(const TA* __restrict__ q, TA* __restrict__ out,
                            const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                            const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                            PageTable pt, PrefillArgs a, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int HD = a.HD, KS = HD + 1;                 // padded key rows: lanes read distinct banks
    float* Ks = smem;                                  // [KT][HD+1]
    float* Vs = Ks + KT * KS;                          // [KT][HD]
    float* Qs = Vs + KT * HD;                          // [QT][HD]

    int b, tile;
    if (!find_query_tile(cu_q, a.B, QT, blockIdx.x, b, tile)) return;   // blockIdx.x numbers the step's query tiles
    const int h = blockIdx.y;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int tile0 = tile * QT;
    const int n_kv = kv_len[b];
    const int past = n_kv - q_len;                     // position of the sequence's first query
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = h / (a.H / a.KV);
    const int nq = min(QT, q_len - tile0);

    for (int i = threadIdx.x; i < QT * HD; i += blockDim.x) {
        const int qi = i / HD, d = i % HD;
        Qs[i] = qi < nq ? to_f32(q[(size_t)(q0 + tile0 + qi) * a.ldq + (size_t)h * HD + d]) : 0.f;
    }

    float m[QPW], l[QPW], acc[QPW][MAXC];
#pragma unroll
    for (int i = 0; i < QPW; i++) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < MAXC; c++) acc[i][c] = 0.f;
    }

    const int p_first = past + tile0, p_last = past + tile0 + nq - 1;
    int k_lo = 0;
    if (a.window > 0) k_lo = max(0, p_first - a.window + 1);
    k_lo = (k_lo / KT) * KT;

    for (int kt = k_lo; kt <= p_last; kt += KT) {
        __syncthreads();                               // previous tile consumed; Qs written (first pass)
        const int page = page_of(pt, b, kt);
        if (page < 0) {
            if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
            return;                                    // uniform over the CTA
        }
        const size_t base = (((size_t)page * a.KV + kvh) * PAGE_TOKENS + kt % PAGE_TOKENS) * HD;
        const int n_keys = min(KT, n_kv - kt);         // rows past the sequence's end are not read
        for (int i = threadIdx.x; i < KT * HD; i += blockDim.x) {
            const int j = i / HD, d = i % HD;
            const bool ok = j < n_keys;
            Ks[j * KS + d] = ok ? to_f32(k_cache[base + i]) : 0.f;
            Vs[i] = ok ? to_f32(v_cache[base + i]) : 0.f;
        }
        __syncthreads();

#pragma unroll
        for (int i = 0; i < QPW; i++) {
            const int qi = warp * QPW + i;
            if (qi >= nq) continue;                    // uniform over the warp
            const int p = past + tile0 + qi;
            const int key = kt + lane;
            const float* qrow = Qs + qi * HD;
            const float* krow = Ks + lane * KS;
            float dot = 0.f;
            for (int d = 0; d < HD; d++) dot = fmaf(qrow[d], krow[d], dot);
            bool vis = key <= p && key < n_kv;
            if (a.window > 0) vis = vis && key > p - a.window;
            const float s = vis ? dot * a.scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            if (m_new == -INFINITY) continue;          // no visible key yet (uniform)
            const float alpha = expf(m[i] - m_new);    // exp(-inf) = 0 on the first tile
            const float pj = expf(s - m_new);
            l[i] = l[i] * alpha + warp_sum(pj);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < MAXC; c++) acc[i][c] *= alpha;
            for (int j = 0; j < KT; j++) {
                const float pb = __shfl_sync(0xffffffffu, pj, j);
#pragma unroll
                for (int c = 0; c < MAXC; c++) {
                    const int d = lane + 32 * c;
                    if (d < HD) acc[i][c] = fmaf(pb, Vs[j * HD + d], acc[i][c]);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < QPW; i++) {
        const int qi = warp * QPW + i;
        if (qi >= nq) continue;
        const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
        TA* o = out + (size_t)(q0 + tile0 + qi) * a.ldo + (size_t)h * HD;
#pragma unroll
        for (int c = 0; c < MAXC; c++) {
            const int d = lane + 32 * c;
            if (d < HD) o[d] = from_f32<TA>(acc[i][c] * inv);
        }
    }
}

}  // namespace

// q: [T, ldq] with head h at columns [h*HD, (h+1)*HD); out: [T, ldo] likewise.
MYNAH_API int mynah_attn_prefill_generic(
    const void* q, void* out, int dtype, int n_tokens, int B, int max_q_len, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* cu_q, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int* status, cudaStream_t stream) {
    if (B == 0 || max_q_len == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && KV > 0 && HD > 0 && H % KV == 0, "attn_prefill: bad sizes B=%d H=%d KV=%d HD=%d", B, H, KV, HD);
    MYNAH_REQUIRE(HD <= 32 * MAXC, "attn_prefill: head_dim %d exceeds %d", HD, 32 * MAXC);
    MYNAH_REQUIRE(H <= 65535, "attn_prefill: H=%d exceeds one launch", H);
    MYNAH_REQUIRE(window >= 0, "attn_prefill: negative window");
    const PrefillArgs a{B, H, KV, HD, ldq, ldo, window, 1.0f / sqrtf((float)HD)};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const size_t smem = sizeof(float) * ((size_t)KT * (HD + 1) + (size_t)KT * HD + (size_t)QT * HD);
    (void)max_q_len;
    MYNAH_REQUIRE(n_tokens >= 0, "attn_prefill: negative row count");
    const dim3 grid(ceil_div(n_tokens, QT) + B, H, 1);               // the most query tiles that n_tokens rows in B sequences make
    cudaError_t e = cudaSuccess;
    if (dtype == MYNAH_F32) {
        auto kern = attn_prefill_generic_kernel<float, float>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("attn_prefill: %s", cudaGetErrorString(e));
        kern<<<grid, WARPS * 32, smem, stream>>>((const float*)q, (float*)out, (const float*)k_cache,
                                                 (const float*)v_cache, cu_q, kv_len, pt, a, status);
    } else if (dtype == MYNAH_BF16) {
        auto kern = attn_prefill_generic_kernel<bf16, bf16>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("attn_prefill: %s", cudaGetErrorString(e));
        kern<<<grid, WARPS * 32, smem, stream>>>((const bf16*)q, (bf16*)out, (const bf16*)k_cache,
                                                 (const bf16*)v_cache, cu_q, kv_len, pt, a, status);
    } else {
        return mynah_fail("attn_prefill: unsupported dtype %d", dtype);
    }
    return mynah_check_launch("attn_prefill_generic");
}
