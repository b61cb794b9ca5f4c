// bf16 matrix product on the fifth-generation tensor cores:
//   C[M, N] = A[M, K] . W[N, K]^T,  fp32 accumulation in tensor memory.
//
// One CTA computes a 128 x BN tile of C (BN = 128 or 256). Operand tiles of
// 64 k (128 bytes per row) are brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) through a ring of stages; one
// elected thread issues tcgen05.mma (cta_group::1, kind::f16, M = 128, N = BN,
// K = 16 per instruction) with shared-memory descriptors for both operands
// (both are K-major: activations [M, K] and weights [N, K] as stored); the
// accumulator lives in tensor memory (BN columns of 128 lanes) and is read
// back with tcgen05.ld by four epilogue warps, one per 32-lane quadrant.
// Warp roles: 0 TMA producer, 1 MMA issuer and tensor-memory owner, 2..5
// epilogue. Stage hand-over is by mbarriers: TMA completes transactions on
// `full`, tcgen05.commit arrives on `empty` when the instructions that read a
// stage have finished, and on `acc_full` when the whole tile is accumulated.
//
// Epilogues: bf16 rows; fp32 rows (logits); SwiGLU, where the B tile is 128
// gate rows followed by the matching 128 up rows of the fused gate/up matrix,
// so the activation (mynah-slm src/kernels.c:193-205) is applied to the
// accumulator and only [M, F] is ever written.
//
// Every wait on an mbarrier is bounded by a wall-clock limit; a wait that runs
// out sets a status bit, and the CTA still drains what it started, frees its
// tensor memory and returns. Rows of A or W beyond the matrix are zero-filled
// by TMA, and the epilogue stores only what lies inside C.
#include "layout.cuh"

#include <cuda.h>

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. False when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = now_ns();
    for (uint32_t it = 0;; it++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 255u) == 255u && now_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ float sigmoid_stable(float v) {
    if (v >= 0.f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}

template <int BN, int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    void* __restrict__ C, int M, int N, int K, int ldc, int up_offset, int* __restrict__ status) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE = A_BYTES + B_BYTES;
    constexpr int STAGES = BN == 256 ? 4 : 6;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), acc_full = smem_u32(bars + 2 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x, m_tile = blockIdx.y;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {                                           // ---- TMA producer
            int issued = 0;
            for (int kb = 0; kb < nk; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1) || *abort_flag) {
                    *abort_flag = 1;
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    break;
                }
                const uint32_t a_dst = smem_u32(smem + s * STAGE), b_dst = a_dst + A_BYTES;
                mbar_expect_tx(full0 + 8 * s, STAGE);
                tma_load_2d(a_dst, &map_a, kb * BK, m_tile * BM, full0 + 8 * s);
                if (EPI == EPI_SWIGLU) {                           // 128 gate rows, then their 128 up rows
                    tma_load_2d(b_dst, &map_b, kb * BK, n_tile * 128, full0 + 8 * s);
                    tma_load_2d(b_dst + 128 * BK * 2, &map_b, kb * BK, up_offset + n_tile * 128, full0 + 8 * s);
                } else {
#pragma unroll
                    for (int j = 0; j < BN / 128; j++)
                        tma_load_2d(b_dst + j * 128 * BK * 2, &map_b, kb * BK, n_tile * BN + j * 128, full0 + 8 * s);
                }
                issued = kb + 1;
            }
            if (*abort_flag) {
                // copies that were started still land in this CTA's shared memory: wait for them (bounded)
                for (int kb = max(0, issued - STAGES); kb < issued; kb++) mbar_wait(full0 + 8 * (kb % STAGES), (kb / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                           // ---- MMA issuer
            constexpr uint32_t idesc = umma_idesc(BN);
            bool ok = true;
            for (int kb = 0; kb < nk && ok; kb++) {
                const int s = kb % STAGES;
                const uint32_t ph = (kb / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, ph) || *abort_flag) {
                    *abort_flag = 1;
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * STAGE), b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    tc_mma(tmem_base, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0);
                tc_commit(empty0 + 8 * s);                         // the stage is free once these have read it
            }
            tc_commit(acc_full);                                   // arrives when everything issued above is done
        }
    } else {                                                       // ---- epilogue: warps 2..5 -> lane quadrants 2,3,0,1
        const int quad = warp & 3;
        const bool ok = mbar_wait(acc_full, 0) && !*abort_flag;
        if (!ok && lane == 0) atomicOr(status, MYNAH_ST_TIMEOUT);
        tc_fence_after();
        const int row = m_tile * BM + quad * 32 + lane;
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
        if (ok) {
            if (EPI == EPI_SWIGLU) {
                bf16* out = static_cast<bf16*>(C);
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t g[32], u[32];
                    tc_ld32(t_row + c0, g);
                    tc_ld32(t_row + 128 + c0, u);
                    if (row < M) {
                        const int col0 = n_tile * 128 + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            float o[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                // gate and up rounded to bf16 first, as when they are stored before the activation
                                const float gv = round_to<bf16>(__uint_as_float(g[j + e])), uv = round_to<bf16>(__uint_as_float(u[j + e]));
                                o[e] = (gv * sigmoid_stable(gv)) * uv;
                            }
                            if (col0 + j + 8 <= N) store8(out + (size_t)row * ldc + col0 + j, o);
                            else
                                for (int e = 0; e < 8; e++)
                                    if (col0 + j + e < N) out[(size_t)row * ldc + col0 + j + e] = __float2bfloat16_rn(o[e]);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(t_row + c0, r);
                    if (row < M) {
                        const int col0 = n_tile * BN + c0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            float o[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) o[e] = __uint_as_float(r[j + e]);
                            if (EPI == EPI_F32) {
                                float* out = static_cast<float*>(C) + (size_t)row * ldc + col0 + j;
                                if (col0 + j + 8 <= N) store8(out, o);
                                else
                                    for (int e = 0; e < 8; e++)
                                        if (col0 + j + e < N) out[e] = o[e];
                            } else {
                                bf16* out = static_cast<bf16*>(C) + (size_t)row * ldc + col0 + j;
                                if (col0 + j + 8 <= N) store8(out, o);
                                else
                                    for (int e = 0; e < 8; e++)
                                        if (col0 + j + e < N) out[e] = __float2bfloat16_rn(o[e]);
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN) : "memory");
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [rows, cols] bf16 row-major, boxes of 128 rows x 64 columns, 128-byte swizzle; out-of-range reads give zero.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return mynah_fail("gemm_tcgen05: the driver does not provide cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {BK, 128};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mynah_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

template <int BN, int EPI>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int ldc, int up_offset,
                int* status, cudaStream_t stream) {
    constexpr int STAGES = BN == 256 ? 4 : 6;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256;
    auto kern = gemm_tcgen05_kernel<BN, EPI>;
    static bool opted = false;
    if (!opted) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
        opted = true;
    }
    const int n_tiles = EPI == EPI_SWIGLU ? ceil_div(N, 128) : ceil_div(N, BN);
    const dim3 grid(n_tiles, ceil_div(M, BM));
    kern<<<grid, THREADS, smem, stream>>>(ma, mb, C, M, N, K, ldc, up_offset, status);
    return mynah_check_launch("gemm_tcgen05");
}

}  // namespace

MYNAH_API int mynah_gemm_tcgen05_supported(int M, int N, int K) {
    return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0;      // rows of 16-byte multiples for TMA
}

// epilogue 0: C bf16 [M, N]; 1: C fp32 [M, N]; 2: SwiGLU, W holds N gate rows then N up rows, C bf16 [M, N].
// A [M, K] and W [rows, K] are bf16, row-major, 16-byte aligned. `status` receives MYNAH_ST_TIMEOUT if a wait ran out.
MYNAH_API int mynah_gemm_tcgen05(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int epilogue,
                                 int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    MYNAH_REQUIRE(mynah_gemm_tcgen05_supported(M, N, K), "gemm_tcgen05: M=%d N=%d K=%d is not taken (K must be a multiple of 8)", M, N, K);
    MYNAH_REQUIRE(epilogue >= 0 && epilogue <= 2 && ldc >= N, "gemm_tcgen05: bad epilogue or output stride");
    MYNAH_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)C & 15) == 0 && ldc % 8 == 0,
                  "gemm_tcgen05: operands must be 16-byte aligned and the output stride a multiple of 8");
    MYNAH_REQUIRE(status != nullptr, "gemm_tcgen05: a status word is required");
    MYNAH_REQUIRE(ceil_div(M, BM) <= 65535, "gemm_tcgen05: %d rows exceed one launch", M);
    CUtensorMap ma, mb;
    if (make_map(&ma, A, M, K)) return -1;
    if (make_map(&mb, W, epilogue == EPI_SWIGLU ? 2LL * N : N, K)) return -1;
    if (epilogue == EPI_SWIGLU) return launch_gemm<256, EPI_SWIGLU>(ma, mb, C, M, N, K, ldc, N, status, stream);
    // narrow tiles when wide ones would leave most SMs idle
    const bool wide = (long long)ceil_div(N, 256) * ceil_div(M, BM) >= 120 || N > 4096;
    if (epilogue == EPI_F32)
        return wide ? launch_gemm<256, EPI_F32>(ma, mb, C, M, N, K, ldc, 0, status, stream)
                    : launch_gemm<128, EPI_F32>(ma, mb, C, M, N, K, ldc, 0, status, stream);
    return wide ? launch_gemm<256, EPI_BF16>(ma, mb, C, M, N, K, ldc, 0, status, stream)
                : launch_gemm<128, EPI_BF16>(ma, mb, C, M, N, K, ldc, 0, status, stream);
}
