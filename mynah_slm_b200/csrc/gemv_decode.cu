// Matrix products of a decode step: y[M, N] = x[M, K] . W[N, K]^T for a
// handful of rows M (at most 16: one row per sequence of the batch), bf16
// operands, fp32 accumulation. The weights are read once, 16 bytes per lane,
// by asynchronous copies into a ring of the lane's own slots in shared memory:
// a lane always has several batches of its weights in flight (a B200 needs
// well over 100 KB in flight an SM to reach its memory bandwidth, far more
// than registers hold), across the end of a group of rows and on into the
// next. The kernel is bound by that stream, so what is fused around it costs
// no extra pass over memory:
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

#include <stdlib.h>

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_M = 16;
constexpr int XPAD = 32;              // elements of padding per row of x in shared memory (bank spread)
#ifndef MYNAH_GEMV_STAGES
#define MYNAH_GEMV_STAGES 5
#endif
#ifndef MYNAH_GEMV_CTAS
#define MYNAH_GEMV_CTAS 2
#endif
constexpr int STAGES = MYNAH_GEMV_STAGES;   // batches of a lane's weights in its ring (all but one in flight while that one is multiplied)
constexpr int CTAS_PER_SM = MYNAH_GEMV_CTAS;
constexpr int COPIES = 4;             // 16-byte copies a lane and batch: four blocks of a weight row, or two of a gate and two of an up row
constexpr int RING_BYTES = THREADS * STAGES * COPIES * 16;

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

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                                    // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}

template <int EPI, int MODE>
__global__ void __launch_bounds__(THREADS, CTAS_PER_SM)
gemv_decode_kernel(GemvArgs a, int rows_bytes) {
    constexpr bool NORM = MODE == ROWS_NORM;
    constexpr bool STAGED = MODE != ROWS_DIRECT;
    constexpr int U = EPI == EPI_SWIGLU ? COPIES / 2 : COPIES;       // blocks of 32 k of a weight row in a batch
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                    // [MAX_M or 8][K + XPAD]
    // the ring: slot (stage, copy) of thread tid; consecutive threads lie side by side
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem_raw + rows_bytes) + threadIdx.x * 16;
    __shared__ float red[WARPS][32][EPI == EPI_SWIGLU ? 8 : 4];
    const int K = a.K, M = a.M, ldx = K + XPAD;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rows_x = M > 8 ? 16 : 8;
    const int nkb = K / 32;                                          // blocks of 32 k

    // ---- the CTA's work as one sequence of batches: group after group (eight weight rows each), and within a
    // group the warp's share of K in batches of U blocks
    // the groups are dealt out evenly: CTA i takes groups [i * groups / n, (i + 1) * groups / n), so CTAs differ by one group at most
    const int groups = (a.N + 7) / 8;
    const int g_first = (int)((long long)blockIdx.x * groups / gridDim.x), g_end = (int)((long long)(blockIdx.x + 1) * groups / gridDim.x);
    const int n_first = g_first * 8;
    const int nb = (nkb + WARPS * U - 1) / (WARPS * U);             // batches a group
    const int my_groups = g_end - g_first;
    const int total = my_groups * nb;
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
    // The copies of batch j (group j / nb, blocks from warp + (j % nb) * WARPS * U on) into stage j % STAGES, as one
    // group of asynchronous copies; beyond the CTA's work an empty group, so that the count of groups stays in step.
    auto issue = [&](int j) {
        if (j < total) {
            const int n0 = n_first + (j / nb) * 8, kb0 = warp + (j % nb) * WARPS * U;
            const int row = n0 + g;
            const bool row_ok = row < a.N;
            const bf16* w_gate = a.W + (size_t)(row_ok ? row : 0) * K;
            const bf16* w_up = EPI == EPI_SWIGLU ? a.W + (size_t)((row_ok ? row : 0) + a.N) * K : nullptr;
            const uint32_t stage = ring + (uint32_t)(j % STAGES) * (COPIES * THREADS * 16);
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int kb = kb0 + u * WARPS;
                const bool ok = kb < nkb && row_ok;
                cp_async_16(stage + u * (THREADS * 16), w_gate + (ok ? kb * 32 + t * 8 : 0), ok);
                if (EPI == EPI_SWIGLU) cp_async_16(stage + (U + u) * (THREADS * 16), w_up + (ok ? kb * 32 + t * 8 : 0), ok);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    // ---- the first batches of this CTA's weights, before anything an earlier kernel wrote is touched: the
    // weights are never written, so their copies may run while the kernel before this one finishes
    griddep_launch();
#pragma unroll
    for (int j = 0; j < STAGES - 1; j++) issue(j);
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

    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
    int gi = 0, bi = 0;                                              // group and batch within it of batch j
    for (int j = 0; j < total; j++) {
        issue(j + STAGES - 1);                                       // (into the stage that batch j - 1 has just left)
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1));  // batch j has landed: a lane reads only its own copies
        const int n0 = n_first + gi * 8, kb0 = warp + bi * WARPS * U;
        const unsigned char* stage = smem_raw + rows_bytes + (size_t)(j % STAGES) * (COPIES * THREADS * 16) + tid * 16;
        if (!STAGED) load_rows(kb0);                                 // (from L1 after the CTA's first group of rows)
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int kb = kb0 + u * WARPS;
            if (kb < nkb) {                                          // uniform over the warp
                const uint4 wv = *reinterpret_cast<const uint4*>(stage + u * (THREADS * 16));
                uint4 xa_u, xb_u = make_uint4(0, 0, 0, 0);
                if (STAGED) {
                    xa_u = *reinterpret_cast<const uint4*>(xs + g * ldx + kb * 32 + t * 8);
                    if (rows_x == 16) xb_u = *reinterpret_cast<const uint4*>(xs + (g + 8) * ldx + kb * 32 + t * 8);
                } else {
                    xa_u = xa[MODE == ROWS_DIRECT ? u : 0];
                    xb_u = xb[MODE == ROWS_DIRECT ? u : 0];
                }
                const uint32_t a1[4] = {xa_u.x, xb_u.x, xa_u.y, xb_u.y};       // k-permuted: both operands use the same order
                const uint32_t a2[4] = {xa_u.z, xb_u.z, xa_u.w, xb_u.w};
                mma_bf16(c0, a1, wv.x, wv.y);
                mma_bf16(c0, a2, wv.z, wv.w);
                if (EPI == EPI_SWIGLU) {
                    const uint4 uv = *reinterpret_cast<const uint4*>(stage + (U + u) * (THREADS * 16));
                    mma_bf16(c1, a1, uv.x, uv.y);
                    mma_bf16(c1, a2, uv.z, uv.w);
                }
            }
        }
        if (++bi < nb) continue;
        bi = 0;
        // ---- the end of a group. Once the last of the CTA's weights have been asked for, the kernel behind this
        // one may start (it reads its own first weights while this one adds up and stores, and waits for these
        // stores before it touches the rows)
        if (gi == my_groups - 1) griddep_launch_late();
        // add the warps' partial sums in warp order
#pragma unroll
        for (int e = 0; e < 4; e++) {
            red[warp][lane][e] = c0[e];
            if (EPI == EPI_SWIGLU) red[warp][lane][4 + e] = c1[e];
            c0[e] = 0.f;
            c1[e] = 0.f;
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
                for (int jj = 0; jj < 2; jj++) {
                    const int n = n0 + 2 * t + jj;
                    if (n >= a.N) continue;
                    float v = s0[2 * half + jj];
                    if (EPI == EPI_SWIGLU) {
                        // both rounded to the activation type first, as when gate and up are stored before the activation
                        const float gt = round_to<bf16>(v), up = round_to<bf16>(s1[2 * half + jj]);
                        v = (gt * stable_sigmoid_f(gt)) * up;
                    }
                    if (EPI == EPI_F32) static_cast<float*>(a.out)[(size_t)m * a.ldo + n] = v;
                    else static_cast<bf16*>(a.out)[(size_t)m * a.ldo + n] = __float2bfloat16_rn(v);
                }
            }
        }
        __syncthreads();
        gi++;
    }
    asm volatile("cp.async.wait_group 0;\n" ::);                     // (only empty groups are left)
}

template <int EPI, int MODE>
int launch(const GemvArgs& a, int n_ctas, size_t rows_bytes, cudaStream_t stream) {
    auto kern = gemv_decode_kernel<EPI, MODE>;
    const size_t smem = rows_bytes + RING_BYTES;
    static int allowed = 0;                           // per instantiation: the largest size opted in to so far
    if ((int)smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("gemv_decode: %s", cudaGetErrorString(e));
        allowed = (int)smem;
    }
    mynah_launch(kern, dim3(n_ctas), dim3(THREADS), smem, stream, a, (int)rows_bytes);
    return mynah_check_launch("gemv_decode");
}

// Where the ring does better than registers: measured with CUDA events on the four products of the 0.6B, 4B and
// 8B shapes at 1 to 16 rows (time through registers / time through the ring). Long rows of few outputs (0.6B o and
// down: 1.02 to 1.19), gate and up of long rows (8B: 1.22 to 1.45) and very long rows (8B down: 1.04 to 1.22) gain;
// the others lose (0.6B gate/up 0.83, 4B o 0.7, 4B down 0.6, q/k/v of 4B and 8B 0.85 to 0.9: there many thin CTAs,
// four an SM, keep more of the memory system busy than two fat ones).
// Inside a decode step of one or two rows (captured with programmatic dependent launch) the ring's four batches go
// out under the kernel before, and all four products of the 0.6B shape gain: 0.956 -> 0.890 ms a step at one row
// (0.915 with the rule below alone).
bool gemv_ring_pays(int M, int N, int K, int epilogue, int sm_count) {
    (void)sm_count;
    if (M <= 2 && (long long)N * K <= (1ll << 24)) return true;
    if (epilogue == EPI_SWIGLU) return K >= 4096;
    return (N <= 1024 && K >= 2048) || (N >= 4096 && K >= 8192);
}

}  // namespace

// Whether the kernel takes these sizes.
MYNAH_API int mynah_gemv_decode_supported(int M, int N, int K) {
    return M >= 1 && M <= MAX_M && N >= 1 && K >= 32 && K % 32 == 0;
}

// epilogue: 0 bf16 rows [M, N]; 1 SwiGLU: W holds N gate rows then N up rows, out is [M, N] bf16; 2 fp32 rows.
// With x_res given the norm prologue runs (delta, x_res_out optional together); otherwise x_bf16 is the input.
int mynah_gemv_decode_regs(const void* W, int N, int K, int M, const void* x_bf16, const float* x_res, const void* delta,
                           float* x_res_out, const void* gain, int gain_dtype, float eps, void* out, int ldo, int epilogue,
                           int sm_count, cudaStream_t stream);

// 0: the weights through registers (gemv_decode_regs.cu), 1: through the ring, 2: whichever the shape does better with.
static int g_gemv_mode = -1;
static int gemv_mode() {
    if (g_gemv_mode < 0) {
        const char* e = getenv("MYNAH_GEMV_MODE");                   // 0, 1 or 2 at start; mynah_gemv_decode_mode() later
        g_gemv_mode = e != nullptr && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 2;
    }
    return g_gemv_mode;
}
MYNAH_API int mynah_gemv_decode_mode(int mode) {
    const int before = gemv_mode();
    if (mode >= 0 && mode <= 2) g_gemv_mode = mode;
    return before;
}

MYNAH_API int mynah_gemv_decode(const void* W, int N, int K, int M, const void* x_bf16,
                                const float* x_res, const void* delta, float* x_res_out,
                                const void* gain, int gain_dtype, float eps,
                                void* out, int ldo, int epilogue, int sm_count, cudaStream_t stream) {
    MYNAH_REQUIRE(mynah_gemv_decode_supported(M, N, K), "gemv_decode: M=%d N=%d K=%d is not taken by this kernel", M, N, K);
    {
        const size_t rb = (size_t)(M > 8 ? 16 : 8) * (K + XPAD) * 2;
        const bool ring_can = x_res == nullptr || rb + RING_BYTES <= 200 * 1024;
        const bool use_ring = gemv_mode() == 1 ? ring_can : gemv_mode() == 0 ? false : ring_can && gemv_ring_pays(M, N, K, epilogue, sm_count);
        if (!use_ring)
            return mynah_gemv_decode_regs(W, N, K, M, x_bf16, x_res, delta, x_res_out, gain, gain_dtype, eps, out, ldo, epilogue, sm_count, stream);
    }
    MYNAH_REQUIRE((x_res != nullptr) != (x_bf16 != nullptr), "gemv_decode: give either the residual or bf16 input rows");
    MYNAH_REQUIRE(x_res == nullptr || gain != nullptr, "gemv_decode: the norm prologue needs a gain");
    MYNAH_REQUIRE((delta == nullptr) == (x_res_out == nullptr), "gemv_decode: delta and the updated residual go together");
    MYNAH_REQUIRE(epilogue >= 0 && epilogue <= 2 && ldo >= N, "gemv_decode: bad epilogue or output stride");
    GemvArgs a;
    a.W = (const bf16*)W; a.N = N; a.K = K; a.M = M;
    a.x_bf16 = (const bf16*)x_bf16; a.x_res = x_res; a.delta = (const bf16*)delta; a.x_res_out = x_res_out;
    a.gain = VecRef{gain, gain_dtype}; a.eps = eps; a.out = out; a.ldo = ldo;
    // Two CTAs an SM (their rings fill its shared memory), each with a run of consecutive groups of eight rows: the
    // ring carries a lane's copies across the end of a group, so few fat CTAs stream as well as many thin ones and
    // stage the input rows less often.
    const int groups = ceil_div(N, 8);
    const int target = (sm_count > 0 ? sm_count : mynah_sm_count()) * CTAS_PER_SM;
    const int n_ctas = groups < target ? groups : target;
    a.groups_per_cta = ceil_div(groups, n_ctas);
    const bool norm = x_res != nullptr;
    const size_t rows_bytes = (size_t)(M > 8 ? 16 : 8) * (K + XPAD) * 2;
    MYNAH_REQUIRE(!norm || rows_bytes + RING_BYTES <= 200 * 1024, "gemv_decode: rows of K=%d do not fit shared memory for the norm prologue", K);
    // staged while two CTAs with their rings still fit an SM; beyond that, straight from global memory
    const int mode = norm ? ROWS_NORM : (rows_bytes <= 24 * 1024 ? ROWS_STAGED : ROWS_DIRECT);
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
