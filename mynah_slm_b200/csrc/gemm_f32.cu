// True fp32 matrix product for the 32-bit path: C[M,N] = A[M,K] . W[N,K]^T.
//
// Plain FFMA on CUDA cores, no tensor-core mode of any kind. Each output
// element is one chain of fused multiply-adds over k = 0..K-1 in ascending
// order, so its bits depend only on its row of A and its row of W: not on M,
// not on the tile it falls in, not on what else is in the batch. That makes
// the 32-bit path bit-stable under every way of cutting the work, which is
// what lets it expose faults of the cache or the batch.
//
// Weights are [out, in] row-major and y = W.x as in the reference
// (mynah-slm src/arch_qwen3.c:51-52).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;            // tx -> columns (n), ty -> rows (m)
    float acc[TM][TN] = {};

    // each thread stages 4 elements of A and 4 of W per k-slab
    const int lr = tid / 4;            // 0..63: row inside the tile
    const int lk = (tid % 4) * 4;      // 0,4,8,12: first k inside the slab

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int k = k0 + lk + j;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + j][lr] = (am < M && k < K) ? A[(size_t)am * lda + k] : 0.f;
            Ws[lk + j][lr] = (wn < N && k < K) ? W[(size_t)wn * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

}  // namespace

MYNAH_API int mynah_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K,
                             int lda, int ldw, int ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    MYNAH_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    MYNAH_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: a leading dimension is smaller than its row");
    const int gy = ceil_div(M, BM);
    MYNAH_REQUIRE(gy <= 65535, "gemm_f32: %d rows exceed one launch (%d)", M, 65535 * BM);
    const dim3 grid(ceil_div(N, BN), gy);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
    return mynah_check_launch("gemm_f32");
}
