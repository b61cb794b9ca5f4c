// Attention of a prompt step on tensor cores: bfloat16, head sizes 64 and 128,
// a ragged batch over the paged cache, causal, optionally windowed, grouped
// query heads. Same contract as the general kernel of attn_prefill.cu.
//
// One CTA takes 64 consecutive queries of one sequence and one query head
// (four warps of 16 query rows). It walks the sequence's pages from the first
// that any of its queries can see to the one that holds its last query; a page
// is exactly one 64-key tile. K and V tiles are copied to shared memory with
// 16-byte asynchronous copies into a swizzled layout, two tiles in flight;
// rows at positions the sequence does not have yet are zero-filled instead of
// copied. Scores are one tensor-core product (mma.sync m16n8k16, bf16 in, fp32
// out), the softmax runs online in fp32 over the tiles in position order, the
// probabilities are rounded to bf16 for the product with V.
//
// score = dot * (1/sqrtf(head_dim)), maximum subtracted; query head h reads kv
// head h / (H/KV) (mynah-slm src/kernels.c:228-261, :207-220).
#include "layout.cuh"

namespace {

constexpr int QT = 64;                // queries per CTA
constexpr int KT = PAGE_TOKENS;       // keys per tile = one page
constexpr int WARPS = 4;

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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
template <int CH> __device__ __forceinline__ int swz(int r, int c) { return (r * CH + (c ^ (r & 7))) * 16; }

struct PrefillTcArgs {
    int B, H, KV, ldq, ldo;
    int window;
    float scale_log2;                 // (1/sqrt(head_dim)) * log2(e)
};

template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
attn_prefill_tc_kernel(const bf16* __restrict__ q, bf16* __restrict__ out,
                       const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                       const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                       PageTable pt, PrefillTcArgs a, int* __restrict__ status) {
    constexpr int CH = HD / 8, KSTEPS = HD / 16, NT_S = KT / 8, NT_O = HD / 8;
    constexpr int TILE_BYTES = KT * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                                  // [QT][HD]
    unsigned char* kv_s = smem + QT * HD * 2;                   // 2 stages x (K tile, V tile)

    int b, tile;
    if (!find_query_tile(cu_q, a.B, QT, blockIdx.x, b, tile)) return;   // blockIdx.x numbers the step's query tiles, a sequence's long tiles first
    const int h = blockIdx.y;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int tile0 = tile * QT;
    const int n_kv = kv_len[b];
    const int past = n_kv - q_len;
    const int nq = min(QT, q_len - tile0);
    const int kvh = h / (a.H / a.KV);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    const int p_first = past + tile0, p_last = p_first + nq - 1;
    const int k_lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int pg_first = k_lo / KT, pg_last = p_last / KT;

    // ---- Q tile -> shared memory (rows beyond the sequence are zero)
    const uint32_t q_base = smem_u32(q_s);
    for (int i = tid; i < QT * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(q_base + swz<CH>(r, c), q + (size_t)(q0 + tile0 + (r < nq ? r : 0)) * a.ldq + (size_t)h * HD + c * 8, r < nq);
    }
    cp_async_commit();

    bool bad = false;
    auto load_tile = [&](int pg, int stage) {
        const int page = page_of(pt, b, pg * KT);
        if (page < 0) bad = true;
        const size_t base = ((size_t)(page < 0 ? 0 : page) * a.KV + kvh) * KT * HD;
        const int rows = page < 0 ? 0 : min(KT, n_kv - pg * KT);           // rows the sequence has written
        const uint32_t kb = smem_u32(kv_s + stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        for (int i = tid; i < KT * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            cp_async_16(kb + swz<CH>(r, c), k_cache + base + (size_t)r * HD + c * 8, r < rows);
            cp_async_16(vb + swz<CH>(r, c), v_cache + base + (size_t)r * HD + c * 8, r < rows);
        }
        cp_async_commit();
    };
    load_tile(pg_first, 0);

    cp_async_wait<1>();                                          // Q has landed
    __syncthreads();
    uint32_t qa[KSTEPS][4];
    {
        const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++)
            ldmatrix_x4(qa[ks], q_base + swz<CH>(warp * 16 + (mat & 1) * 8 + rr, ks * 2 + (mat >> 1)));
    }

    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int pos_r[2] = {p_first + warp * 16 + g, p_first + warp * 16 + g + 8};   // positions of this thread's two rows

    for (int pg = pg_first; pg <= pg_last; pg++) {
        const int stage = (pg - pg_first) & 1;
        if (pg + 1 <= pg_last) {
            load_tile(pg + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kb = smem_u32(kv_s + stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;

        // ---- S = Q K^T for this warp's 16 rows against the 64 keys
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
                for (int j = 0; j < NT_S / 2; j++) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, kb + swz<CH>(j * 16 + (mat >> 1) * 8 + rr, ks * 2 + (mat & 1)));
                    mma_bf16(s[2 * j], qa[ks], kf[0], kf[1]);
                    mma_bf16(s[2 * j + 1], qa[ks], kf[2], kf[3]);
                }
            }
        }
        // ---- scale, mask (only tiles that touch an edge), online softmax
        const int key0 = pg * KT;
        const bool edge = key0 + KT - 1 > p_first + warp * 16 || (a.window > 0 && key0 < p_last - a.window + 1) ||
                          key0 + KT > n_kv;
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int i = 0; i < NT_S; i++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[i][e] * a.scale_log2;
                if (edge) {
                    const int key = key0 + i * 8 + t * 2 + (e & 1), p = pos_r[e >> 1];
                    bool vis = key <= p && key < n_kv;
                    if (a.window > 0) vis = vis && key > p - a.window;
                    if (!vis) v = -INFINITY;
                }
                s[i][e] = v;
                m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            m_new[j] = fmaxf(m_new[j], __shfl_xor_sync(0xffffffffu, m_new[j], 1));
            m_new[j] = fmaxf(m_new[j], __shfl_xor_sync(0xffffffffu, m_new[j], 2));
            alpha[j] = m_new[j] == -INFINITY ? 1.f : exp2f(m_run[j] - m_new[j]);     // exp2(-inf) = 0 on the first tile
            m_run[j] = m_new[j];
        }
        float l_add[2] = {0.f, 0.f};
        uint32_t pa[KT / 16][4];
#pragma unroll
        for (int i = 0; i < NT_S; i++) {
            const float mm0 = m_new[0] == -INFINITY ? 0.f : m_new[0], mm1 = m_new[1] == -INFINITY ? 0.f : m_new[1];
            const float p0 = exp2f(s[i][0] - mm0), p1 = exp2f(s[i][1] - mm0);
            const float p2 = exp2f(s[i][2] - mm1), p3 = exp2f(s[i][3] - mm1);
            l_add[0] += p0 + p1;
            l_add[1] += p2 + p3;
            // the C fragments of two neighbouring key tiles are the A fragment of one 16-key step
            pa[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
            pa[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int j = 0; j < 2; j++) l_run[j] = l_run[j] * alpha[j] + l_add[j];
#pragma unroll
        for (int i = 0; i < NT_O; i++) {
            o[i][0] *= alpha[0];
            o[i][1] *= alpha[0];
            o[i][2] *= alpha[1];
            o[i][3] *= alpha[1];
        }
        // ---- O += P V
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int ks = 0; ks < KT / 16; ks++) {
#pragma unroll
                for (int i = 0; i < NT_O / 2; i++) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vb + swz<CH>(ks * 16 + (mat & 1) * 8 + rr, i * 2 + (mat >> 1)));
                    mma_bf16(o[2 * i], pa[ks], vf[0], vf[1]);
                    mma_bf16(o[2 * i + 1], pa[ks], vf[2], vf[3]);
                }
            }
        }
        __syncthreads();                                         // the stage may be overwritten by the next load
    }
    if (bad && tid == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);

    // ---- normalise and store
#pragma unroll
    for (int j = 0; j < 2; j++) {
        float l = l_run[j];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int r = warp * 16 + g + 8 * j;
        if (r >= nq) continue;
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        bf16* orow = out + (size_t)(q0 + tile0 + r) * a.ldo + (size_t)h * HD;
#pragma unroll
        for (int i = 0; i < NT_O; i++)
            *reinterpret_cast<uint32_t*>(orow + i * 8 + t * 2) = pack_bf16(o[i][2 * j] * inv, o[i][2 * j + 1] * inv);
    }
}

template <int HD>
int launch_prefill_tc(const dim3& grid, size_t smem, cudaStream_t stream, const bf16* q, bf16* out, const bf16* k, const bf16* v,
                      const int* cu_q, const int* kv_len, const PageTable& pt, const PrefillTcArgs& a, int* status) {
    auto kern = attn_prefill_tc_kernel<HD>;
    static bool opted = false;
    if (!opted) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("attn_prefill_tc: %s", cudaGetErrorString(e));
        opted = true;
    }
    kern<<<grid, WARPS * 32, smem, stream>>>(q, out, k, v, cu_q, kv_len, pt, a, status);
    return mynah_check_launch("attn_prefill_tc");
}

}  // namespace

MYNAH_API int mynah_attn_prefill_tc_supported(int H, int KV, int HD) {
    return (HD == 64 || HD == 128) && KV > 0 && H % KV == 0;
}

// Same arguments as mynah_attn_prefill_generic; bfloat16 only.
MYNAH_API int mynah_attn_prefill_tc(
    const void* q, void* out, int n_tokens, int B, int max_q_len, int H, int KV, int HD, int ldq, int ldo,
    const void* k_cache, const void* v_cache, const int* cu_q, const int* kv_len,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    int window, int* status, cudaStream_t stream) {
    if (B == 0 || max_q_len == 0) return 0;
    MYNAH_REQUIRE(mynah_attn_prefill_tc_supported(H, KV, HD), "attn_prefill_tc: H=%d KV=%d head_dim=%d is not taken by this kernel", H, KV, HD);
    MYNAH_REQUIRE(ldq % 8 == 0 && ldo % 2 == 0, "attn_prefill_tc: row strides %d, %d are not aligned", ldq, ldo);
    MYNAH_REQUIRE(B <= 65535 && H <= 65535 && window >= 0, "attn_prefill_tc: launch too large");
    const PrefillTcArgs a{B, H, KV, ldq, ldo, window, (1.0f / sqrtf((float)HD)) * 1.4426950408889634f};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    (void)max_q_len;
    MYNAH_REQUIRE(n_tokens >= 0, "attn_prefill_tc: negative row count");
    const dim3 grid(ceil_div(n_tokens, QT) + B, H, 1);               // the most query tiles that n_tokens rows in B sequences make
    const size_t smem = (size_t)QT * HD * 2 + 4 * (size_t)KT * HD * 2;
    if (HD == 128)
        return launch_prefill_tc<128>(grid, smem, stream, (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                      cu_q, kv_len, pt, a, status);
    return launch_prefill_tc<64>(grid, smem, stream, (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                 cu_q, kv_len, pt, a, status);
}
