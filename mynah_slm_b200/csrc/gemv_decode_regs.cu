// The decode products with the weights loaded straight into registers (the form of this kernel before the ring of
// asynchronous copies in gemv_decode.cu): kept beside it for the shapes where many thin CTAs, four an SM, still
// stream better than two fat ones, and as the other side of the comparison. The arithmetic is the same.
//
// Matrix products of a decode step: y[M, N] = x[M, K] . W[N, K]^T for a
// handful of rows M (at most 16: one row per sequence of the batch), bf16
// operands, fp32 accumulation. The weights are read once, straight from global
// memory, 16 bytes per lane; the kernel is bound by that stream, so what is
// fused around it costs no extra pass over memory:
//
//   prologue  RMSNorm of the residual stream (with the pending residual add)
//             computed by every CTA into shared memory, so the normalised rows
//             are never written out; CTA 0 also writes the updated residual.
//   epilogue  plain bf16 rows | SwiGLU of a gate row and its up row | fp32 rows
//             (the output head's logits).
//
// Tensor-core mapping (mma.sync m16n8k16): the batch rows are the 16 rows of
// the A operand, eight weight rows are the 8 columns of the B operand, so one
// warp instruction covers 8 weight rows x 16 k. Each lane loads 16 contiguous
// bytes of a weight row; the k indices inside a block of 32 are permuted
// consistently for both operands (a dot product does not care about the order
// of its terms), which is what lets a lane use its 16 bytes as two B fragments
// without any shuffle. The 8 warps of a CTA split K and add their partial sums
// in warp order, so the result does not depend on timing.
//
// y = W.x with W [out, in] row-major, as in the reference
// (mynah-slm src/arch_qwen3.c:51-52); norm as src/kernels.c:118-128; SwiGLU as
// src/kernels.c:193-205.
#include "common.cuh"
#include "gemv_norm_rows.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_M = 16;
constexpr int XPAD = 32;              // elements of padding per row of x in shared memory (bank spread)

enum Epilogue : int { EPI_BF16 = 0, EPI_SWIGLU = 1, EPI_F32 = 2 };

struct GemvArgs {
    const bf16* W;
    int N, K, M;                      // N: rows of W that produce outputs (for SwiGLU: gate rows; up rows follow at +N)
    const bf16* x_bf16;               // [M, K] when there is no norm prologue
    const float* x_res;               // [M, K] residual (norm prologue)
    const bf16* delta;                // [M, K] pending add, or null
    float* x_res_out;                 // [M, K] updated residual, written by CTA 0 when delta is given
    VecRef gain;
    float eps;
    void* out;
    int ldo;
    int groups_per_cta;               // groups of 8 weight rows each CTA works through
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float stable_sigmoid_f(float v) {
    // e^-|v| never overflows; the select keeps both branches of the reference's stable form exact
    const float e = expf(-fabsf(v));
    return (v >= 0.f ? 1.0f : e) / (1.0f + e);
}

// MODE: how the input rows reach the tensor cores. ROWS_DIRECT: each lane loads its fragments straight from global
// memory (no shared memory, any K); ROWS_STAGED: the CTA copies the rows into shared memory first (a little faster
// while they are small); ROWS_NORM: the norm prologue computes them into shared memory.
enum RowsMode : int { ROWS_DIRECT = 0, ROWS_STAGED = 1, ROWS_NORM = 2 };

// U: 16-byte loads of a weight row that a lane keeps in flight (per operand); 8 for long rows, so that a warp's
// share of K is one or two round trips to memory instead of two or three.
template <int EPI, int MODE, int U>
__global__ void __launch_bounds__(THREADS)
gemv_decode_regs_kernel(GemvArgs a) {
    constexpr bool NORM = MODE == ROWS_NORM;
    constexpr bool STAGED = MODE != ROWS_DIRECT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                    // [MAX_M or 8][K + XPAD]
    __shared__ float red[WARPS][32][EPI == EPI_SWIGLU ? 8 : 4];
    const int K = a.K, M = a.M, ldx = K + XPAD;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rows_x = M > 8 ? 16 : 8;
    const int nkb = K / 32;                                          // blocks of 32 k

    // ---- the first weights of this CTA, before anything an earlier kernel wrote is touched: the
    // weights are never written, so their loads may run while the kernel before this one finishes
    uint4 wv[U], uv[EPI == EPI_SWIGLU ? U : 1];
    uint4 xa[MODE == ROWS_DIRECT ? U : 1], xb[MODE == ROWS_DIRECT ? U : 1];                                              // without the norm: the rows' fragments, straight from global memory
    auto load_rows = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < (MODE == ROWS_DIRECT ? U : 0); u++) {
            const int kb = kb0 + u * WARPS;
            const bool ok = kb < nkb;
            xa[u] = ok && g < M ? *reinterpret_cast<const uint4*>(a.x_bf16 + (size_t)g * K + kb * 32 + t * 8) : make_uint4(0, 0, 0, 0);
            xb[u] = ok && g + 8 < M ? *reinterpret_cast<const uint4*>(a.x_bf16 + (size_t)(g + 8) * K + kb * 32 + t * 8) : make_uint4(0, 0, 0, 0);
        }
    };
    auto load_weights = [&](int n0, int kb0) {
        const int row = n0 + g;
        const bool row_ok = row < a.N;
        const bf16* w_gate = a.W + (size_t)(row_ok ? row : 0) * K;
        const bf16* w_up = EPI == EPI_SWIGLU ? a.W + (size_t)((row_ok ? row : 0) + a.N) * K : nullptr;
#pragma unroll
        for (int u = 0; u < U; u++) {                                // U (2U with the up rows) x 16 bytes in flight per lane
            const int kb = kb0 + u * WARPS;
            const bool ok = kb < nkb && row_ok;
            wv[u] = ok ? __ldg(reinterpret_cast<const uint4*>(w_gate + kb * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
            if (EPI == EPI_SWIGLU)
                uv[EPI == EPI_SWIGLU ? u : 0] = ok ? __ldg(reinterpret_cast<const uint4*>(w_up + kb * 32 + t * 8)) : make_uint4(0, 0, 0, 0);
        }
    };
    const int n_first = blockIdx.x * a.groups_per_cta * 8;
    griddep_launch();
    load_weights(n_first, warp);
    griddep_wait();

    // ---- the input rows, in bf16, into shared memory
    if (NORM) {
        const NormRowsArgs nr{a.x_res, a.delta, a.x_res_out, a.gain, a.eps, M, K};
        norm_rows_to_smem<WARPS>(nr, xs, ldx, warp, lane);
    } else if (STAGED) {
        for (int i = tid; i < M * (K / 8); i += THREADS) {
            const int m = i / (K / 8), c = i % (K / 8);
            *reinterpret_cast<uint4*>(xs + m * ldx + c * 8) = *reinterpret_cast<const uint4*>(a.x_bf16 + (size_t)m * K + c * 8);
        }
    }
    if (STAGED) {
        for (int i = tid; i < (rows_x - M) * (K / 8); i += THREADS) {   // rows beyond the batch are zero
            const int m = M + i / (K / 8), c = i % (K / 8);
            *reinterpret_cast<uint4*>(xs + m * ldx + c * 8) = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
    }

    for (int gi = 0; gi < a.groups_per_cta; gi++) {
        const int n0 = (blockIdx.x * a.groups_per_cta + gi) * 8;
        if (n0 >= a.N) break;                                        // uniform over the CTA
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        for (int kb0 = warp; kb0 < nkb; kb0 += WARPS * U) {
            if (gi != 0 || kb0 != warp) load_weights(n0, kb0);       // the first batch is already here
            if (!STAGED) load_rows(kb0);                             // (from L1 after the CTA's first group of rows)
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int kb = kb0 + u * WARPS;
                if (kb < nkb) {                                      // uniform over the warp
                    uint4 xa_u, xb_u = make_uint4(0, 0, 0, 0);
                    if (STAGED) {
                        xa_u = *reinterpret_cast<const uint4*>(xs + g * ldx + kb * 32 + t * 8);
                        if (rows_x == 16) xb_u = *reinterpret_cast<const uint4*>(xs + (g + 8) * ldx + kb * 32 + t * 8);
                    } else {
                        xa_u = xa[MODE == ROWS_DIRECT ? u : 0];
                        xb_u = xb[MODE == ROWS_DIRECT ? u : 0];
                    }
                    const uint32_t a1[4] = {xa_u.x, xb_u.x, xa_u.y, xb_u.y};   // k-permuted: both operands use the same order
                    const uint32_t a2[4] = {xa_u.z, xb_u.z, xa_u.w, xb_u.w};
                    mma_bf16(c0, a1, wv[u].x, wv[u].y);
                    mma_bf16(c0, a2, wv[u].z, wv[u].w);
                    if (EPI == EPI_SWIGLU) {
                        mma_bf16(c1, a1, uv[EPI == EPI_SWIGLU ? u : 0].x, uv[EPI == EPI_SWIGLU ? u : 0].y);
                        mma_bf16(c1, a2, uv[EPI == EPI_SWIGLU ? u : 0].z, uv[EPI == EPI_SWIGLU ? u : 0].w);
                    }
                }
            }
        }
        // the weights of this CTA have been read: the kernel behind this one may start (it reads its own first
        // weights while this one adds up and stores, and waits for these stores before it touches the rows)
        if (gi == a.groups_per_cta - 1 || n0 + 8 >= a.N) griddep_launch_late();
        if (gi == a.groups_per_cta - 1 || n0 + 8 >= a.N) griddep_launch_late();
        // ---- add the warps' partial sums in warp order
#pragma unroll
        for (int e = 0; e < 4; e++) {
            red[warp][lane][e] = c0[e];
            if (EPI == EPI_SWIGLU) red[warp][lane][4 + e] = c1[e];
        }
        __syncthreads();
        if (warp == 0) {
            float s0[4], s1[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                s0[e] = red[0][lane][e];
                if (EPI == EPI_SWIGLU) s1[e] = red[0][lane][4 + e];
            }
            for (int w = 1; w < WARPS; w++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    s0[e] += red[w][lane][e];
                    if (EPI == EPI_SWIGLU) s1[e] += red[w][lane][4 + e];
                }
            }
            // C layout: s[0..1] -> batch row g, weight rows n0 + 2t + {0,1}; s[2..3] -> batch row g + 8
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int m = g + 8 * half;
                if (m >= M) continue;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int n = n0 + 2 * t + j;
                    if (n >= a.N) continue;
                    float v = s0[2 * half + j];
                    if (EPI == EPI_SWIGLU) {
                        // both rounded to the activation type first, as when gate and up are stored before the activation
                        const float gt = round_to<bf16>(v), up = round_to<bf16>(s1[2 * half + j]);
                        v = (gt * stable_sigmoid_f(gt)) * up;
                    }
                    if (EPI == EPI_F32) static_cast<float*>(a.out)[(size_t)m * a.ldo + n] = v;
                    else static_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(v);
                }
            }
        }
        __syncthreads();
    }
}

template <int EPI, int MODE, int U>
int launch_u(const GemvArgs& a, int n_ctas, size_t smem, cudaStream_t stream) {
    auto kern = gemv_decode_regs_kernel<EPI, MODE, U>;
    static int allowed = 0;                           // per instantiation: the largest size opted in to so far
    // dynamic plus the kernel's static shared memory (up to 9 KB) must stay under 48 KB unless opted in
    if (smem > 36 * 1024 && (int)smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("gemv_decode: %s", cudaGetErrorString(e));
        allowed = (int)smem;
    }
    mynah_launch(kern, dim3(n_ctas), dim3(THREADS), smem, stream, a);
    return mynah_check_launch("gemv_decode");
}

template <int EPI, int MODE>
int launch(const GemvArgs& a, int n_ctas, size_t smem, cudaStream_t stream) {
    // long rows without the up rows: eight loads a lane in flight (a warp's share of K = 2,048 is then one batch)
    if (EPI != EPI_SWIGLU && a.K >= 2048) return launch_u<EPI, MODE, 8>(a, n_ctas, smem, stream);
    return launch_u<EPI, MODE, 4>(a, n_ctas, smem, stream);
}

}  // namespace


// epilogue: 0 bf16 rows [M, N]; 1 SwiGLU: W holds N gate rows then N up rows, out is [M, N] bf16; 2 fp32 rows.
// With x_res given the norm prologue runs (delta, x_res_out optional together); otherwise x_bf16 is the input.
int mynah_gemv_decode_regs(const void* W, int N, int K, int M, const void* x_bf16,
                                const float* x_res, const void* delta, float* x_res_out,
                                const void* gain, int gain_dtype, float eps,
                                void* out, int ldo, int epilogue, int sm_count, cudaStream_t stream) {
    MYNAH_REQUIRE((x_res != nullptr) != (x_bf16 != nullptr), "gemv_decode: give either the residual or bf16 input rows");
    MYNAH_REQUIRE(x_res == nullptr || gain != nullptr, "gemv_decode: the norm prologue needs a gain");
    MYNAH_REQUIRE((delta == nullptr) == (x_res_out == nullptr), "gemv_decode: delta and the updated residual go together");
    MYNAH_REQUIRE(epilogue >= 0 && epilogue <= 2 && ldo >= N, "gemv_decode: bad epilogue or output stride");
    GemvArgs a;
    a.W = (const bf16*)W; a.N = N; a.K = K; a.M = M;
    a.x_bf16 = (const bf16*)x_bf16; a.x_res = x_res; a.delta = (const bf16*)delta; a.x_res_out = x_res_out;
    a.gain = VecRef{gain, gain_dtype}; a.eps = eps; a.out = out; a.ldo = ldo;
    const int groups = ceil_div(N, 8);
    const int target = (sm_count > 0 ? sm_count : mynah_sm_count()) * 4;          // one group of rows a CTA while that gives at most four CTAs an SM (their registers fill it)
    a.groups_per_cta = groups <= target ? 1 : ceil_div(groups, target);
    const int n_ctas = ceil_div(groups, a.groups_per_cta);
    const bool norm = x_res != nullptr;
    const size_t rows_bytes = (size_t)(M > 8 ? 16 : 8) * (K + XPAD) * 2;
    MYNAH_REQUIRE(!norm || rows_bytes <= 200 * 1024, "gemv_decode: rows of K=%d do not fit shared memory for the norm prologue", K);
    // staged while the rows need no opt-in (several CTAs fit an SM); beyond that, straight from global memory
    const int mode = norm ? ROWS_NORM : (rows_bytes <= 36 * 1024 ? ROWS_STAGED : ROWS_DIRECT);
    const size_t smem = mode == ROWS_DIRECT ? 0 : rows_bytes;
    switch (epilogue * 3 + mode) {
        case 0: return launch<EPI_BF16, ROWS_DIRECT>(a, n_ctas, smem, stream);
        case 1: return launch<EPI_BF16, ROWS_STAGED>(a, n_ctas, smem, stream);
        case 2: return launch<EPI_BF16, ROWS_NORM>(a, n_ctas, smem, stream);
        case 3: return launch<EPI_SWIGLU, ROWS_DIRECT>(a, n_ctas, smem, stream);
        case 4: return launch<EPI_SWIGLU, ROWS_STAGED>(a, n_ctas, smem, stream);
        case 5: return launch<EPI_SWIGLU, ROWS_NORM>(a, n_ctas, smem, stream);
        case 6: return launch<EPI_F32, ROWS_DIRECT>(a, n_ctas, smem, stream);
        case 7: return launch<EPI_F32, ROWS_STAGED>(a, n_ctas, smem, stream);
        default: return launch<EPI_F32, ROWS_NORM>(a, n_ctas, smem, stream);
    }
}
