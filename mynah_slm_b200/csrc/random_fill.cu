// Random weights made on the device: every element is a function of (seed, tensor key, element index), so a
// model of any size starts without a file, and the same tensor can be made again anywhere, element by element.
// The arithmetic is in include/mynah_random_normal.h, shared with the host's folder writer.
#include "common.cuh"
#include "../include/mynah_random_normal.h"

template <typename T>
__global__ void randn_fill_kernel(T* __restrict__ out, long long n, unsigned long long state, double mean, double std) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = mynah_rn_value(state, (unsigned long long)i, mean, std);
        if constexpr (sizeof(T) == 4) {
            out[i] = v;
        } else {
            const unsigned short b = mynah_rn_bf16_bits(v);
            out[i] = *reinterpret_cast<const bf16*>(&b);
        }
    }
}

// out[i] = mean + std * normal(seed, tensor_key, i) for i < n, stored as float32 or bfloat16.
MYNAH_API int mynah_randn_fill(void* out, int dtype, long long n, unsigned long long seed, unsigned long long tensor_key,
                               double mean, double std, cudaStream_t stream) {
    if (n == 0) return 0;
    MYNAH_REQUIRE(n > 0 && out != nullptr, "randn_fill: bad size %lld", n);
    MYNAH_REQUIRE(dtype == MYNAH_F32 || dtype == MYNAH_BF16, "randn_fill: unsupported dtype %d", dtype);
    const unsigned long long state = mynah_rn_state(seed, tensor_key);
    const int threads = 256;
    const long long want = ceil_div_ll(n, threads);
    const int blocks = (int)(want < (long long)mynah_sm_count() * 16 ? want : (long long)mynah_sm_count() * 16);
    if (dtype == MYNAH_F32)
        randn_fill_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, state, mean, std);
    else
        randn_fill_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)out, n, state, mean, std);
    return mynah_check_launch("randn_fill");
}
