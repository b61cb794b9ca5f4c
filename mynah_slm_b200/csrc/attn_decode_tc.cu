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

namespace {

constexpr int KEYS = PAGE_TOKENS;     // 64 keys per CTA
constexpr int WARPS = 4;
constexpr int MAX_G = 16;             // query heads per kv head that one MMA tile holds

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

template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                      const int* __restrict__ kv_len, PageTable pt, TcArgs a,
                      float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ status) {
    constexpr int CH = HD / 8;                       // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    __shared__ __align__(128) unsigned char k_s[KEYS * HD * 2];
    __shared__ __align__(128) unsigned char v_s[KEYS * HD * 2];
    __shared__ __align__(16) bf16 p_s[MAX_G * KEYS];  // probabilities [head][key], rows of 8 chunks, swizzled
    __shared__ float red_m[WARPS][MAX_G], red_l[WARPS][MAX_G];

    const int s = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
    const int G = a.H / a.KV;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    griddep_launch();
    griddep_wait();
    const int hi = kv_len[b];
    const int lo = a.window > 0 ? max(0, hi - a.window) : 0;
    int key_begin = 0, key_end = 0, page = -1;
    if (hi > 0) {
        const int pg0 = lo / PAGE_TOKENS, pg1 = (hi - 1) / PAGE_TOKENS + 1;
        if (pg1 - pg0 > a.S && tid == 0 && s == 0) atomicOr(status, MYNAH_ST_SPLIT_RANGE);
        const int mp = pg0 + s;
        if (mp < pg1) {
            key_begin = max(lo, mp * PAGE_TOKENS);
            key_end = min(hi, (mp + 1) * PAGE_TOKENS);
            page = page_of(pt, b, mp * PAGE_TOKENS);
            if (page < 0) {
                if (tid == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
                key_end = key_begin;
            }
        }
    }
    const size_t row0 = ((size_t)b * a.H + (size_t)g * G) * a.S + s;     // partial of head g*G+i: row0 + i*S
    if (key_begin >= key_end) {                       // nothing of this page is visible: an empty partial
        for (int i = tid; i < G; i += blockDim.x) {
            part_ml[(row0 + (size_t)i * a.S) * 2] = -INFINITY;
            part_ml[(row0 + (size_t)i * a.S) * 2 + 1] = 0.f;
        }
        return;
    }
    const int k_first = key_begin % PAGE_TOKENS, k_last = (key_end - 1) % PAGE_TOKENS;   // rows of the tile in use

    // ---- copy K, then V, each as its own group
    const bf16* k_src = k_cache + ((size_t)page * a.KV + g) * PAGE_TOKENS * HD;
    const bf16* v_src = v_cache + ((size_t)page * a.KV + g) * PAGE_TOKENS * HD;
    const uint32_t k_base = smem_u32(k_s), v_base = smem_u32(v_s);
    for (int i = tid; i < KEYS * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(k_base + swz<CH>(r, c), k_src + (size_t)r * HD + c * 8, r >= k_first && r <= k_last);
    }
    cp_async_commit();
    for (int i = tid; i < KEYS * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(v_base + swz<CH>(r, c), v_src + (size_t)r * HD + c * 8, r >= k_first && r <= k_last);
    }
    cp_async_commit();

    // ---- Q as the A operand: rows = query heads of the group (zero beyond G), straight from global memory
    uint32_t qa[KSTEPS][4];
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
        const bf16* q0 = q + (size_t)b * a.ldq + (size_t)(g * G) * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const int col = ks * 16 + c0;
            qa[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col) : 0u;
            qa[ks][1] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col) : 0u;
            qa[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)r0 * HD + col + 8) : 0u;
            qa[ks][3] = r0 + 8 < G ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(r0 + 8) * HD + col + 8) : 0u;
        }
    }

    cp_async_wait<1>();                               // K has landed (V may still be in flight)
    __syncthreads();

    // ---- scores: warp w takes keys [16w, 16w+16): two n-tiles of 8 keys
    float sc[2][4] = {};
    {
        const int mat = lane >> 3, rr = lane & 7;     // ldmatrix: thread -> (matrix, row)
        // matrices: 0: keys 0-7, dims k0..k0+7; 1: keys 0-7, dims +8; 2: keys 8-15, dims k0; 3: keys 8-15, dims +8
        const int key = warp * 16 + (mat >> 1) * 8 + rr;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            uint32_t kb[4];
            ldmatrix_x4(kb, k_base + swz<CH>(key, ks * 2 + (mat & 1)));
            mma_bf16(sc[0], qa[ks], kb[0], kb[1]);
            mma_bf16(sc[1], qa[ks], kb[2], kb[3]);
        }
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
    __syncthreads();
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
    cp_async_wait<0>();                               // V has landed
    __syncthreads();

    // ---- output: warp w takes dims [w*HD/4, (w+1)*HD/4): HD/32 n-tiles of 8, four k-steps of 16 keys
    constexpr int NT = HD / 32;
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
                // B operand from V [key][dim] (transposed load): matrices 0: keys k0..+7, dims n0..+7; 1: keys +8, same dims;
                // 2: keys k0..+7, dims n0+8; 3: keys +8, dims n0+8
                const int key = ks * 16 + (mat & 1) * 8 + rr;
                const int chunk = warp * (HD / 32) + nt + (mat >> 1);
                ldmatrix_x4_trans(vb, v_base + swz<CH>(key, chunk));
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

// Merge of a sequence's pages, in page order: one CTA per (head, sequence).
template <typename T>
__global__ void attn_decode_combine_fast_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                T* __restrict__ out, const int* __restrict__ kv_len, int window,
                                                int H, int HD, int S_max, int ldo) {
    extern __shared__ float w_s[];                    // weights exp(m_s - M) of the pages
    __shared__ float red[32];
    __shared__ float inv_s;
    const int h = blockIdx.x, b = blockIdx.y;
    const size_t row0 = ((size_t)b * H + h) * S_max;
    griddep_wait();
    griddep_launch();
    const int hi = kv_len[b];
    const int lo = window > 0 ? max(0, hi - window) : 0;
    const int S = hi > 0 ? min(S_max, (hi - 1) / PAGE_TOKENS + 1 - lo / PAGE_TOKENS) : 0;
    float mx = -INFINITY;
    for (int s = threadIdx.x; s < S; s += blockDim.x) mx = fmaxf(mx, part_ml[(row0 + s) * 2]);
    mx = warp_max(mx);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = -INFINITY;
    for (int w = 0; w < (int)((blockDim.x + 31) >> 5); w++) mx = fmaxf(mx, red[w]);
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
        const float m = part_ml[(row0 + s) * 2];
        w_s[s] = m == -INFINITY ? 0.f : expf(m - mx);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ls = 0.f;
        for (int s = 0; s < S; s++) ls += part_ml[(row0 + s) * 2 + 1] * w_s[s];     // page order
        inv_s = ls > 0.f ? 1.0f / ls : 0.f;
    }
    __syncthreads();
    const float inv = inv_s;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float os = 0.f;
        for (int s = 0; s < S; s++) {
            const float w = w_s[s];
            if (w != 0.f) os += part_o[(row0 + s) * HD + d] * w;
        }
        out[(size_t)b * ldo + (size_t)h * HD + d] = from_f32<T>(os * inv);
    }
}

}  // namespace

// Whether the tensor-core kernel takes these sizes (bfloat16 only).
MYNAH_API int mynah_attn_decode_tc_supported(int H, int KV, int HD) {
    return (HD == 64 || HD == 128) && KV > 0 && H % KV == 0 && H / KV <= MAX_G;
}

// Same arguments and scratch layout as mynah_attn_decode; bfloat16 only.
MYNAH_API int mynah_attn_decode_tc(
    const void* q, void* out, int B, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int n_splits, float* scratch, int* status, cudaStream_t stream) {
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
    if (HD == 128)
        mynah_launch(attn_decode_tc_kernel<128>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                                                    kv_len, pt, a, part_o, part_ml, status);
    else
        mynah_launch(attn_decode_tc_kernel<64>, grid, dim3(WARPS * 32), 0, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                                                                   kv_len, pt, a, part_o, part_ml, status);
    if (mynah_check_launch("attn_decode_tc")) return -1;
    const int threads = HD >= 128 ? 128 : 64;
    mynah_launch(attn_decode_combine_fast_kernel<bf16>, dim3(H, B), dim3(threads), n_splits * sizeof(float), stream,
        part_o, part_ml, (bf16*)out, kv_len, window, H, HD, n_splits, ldo);
    return mynah_check_launch("attn_decode_combine");
}
