// Shared helpers of the sm_100a kernels: element types, conversions, warp and
// block reductions, and the error convention of the exported C entry points.
//
// Every exported launcher returns 0 on success. On a refused size or a failed
// launch it returns a negative code and leaves a message that
// `mynah_last_error()` hands out. Nothing here writes to stderr.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <utility>

#define MYNAH_API extern "C" __attribute__((visibility("default")))

enum MynahDtype : int { MYNAH_F32 = 0, MYNAH_BF16 = 1 };

// Sets the message that mynah_last_error() returns; always returns -1.
int mynah_fail(const char* fmt, ...);
// Checks the launch that has just been made.
int mynah_check_launch(const char* what);
// Multiprocessors of the current device (asked once per device), for launchers whose caller passes none.
int mynah_sm_count();

#define MYNAH_REQUIRE(cond, ...)                     \
    do {                                             \
        if (!(cond)) return mynah_fail(__VA_ARGS__); \
    } while (0)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// The value a tensor of type T would hold after a store and a load.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

// A gain or table of weights whose storage type is chosen at run time.
struct VecRef {
    const void* p;
    int dtype;
    __device__ __forceinline__ float at(int i) const {
        return dtype == MYNAH_F32 ? static_cast<const float*>(p)[i]
                                  : __bfloat162float(static_cast<const bf16*>(p)[i]);
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. The
// order of the additions is fixed by the thread layout, not by timing.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = lane < nw ? smem32[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// 8 consecutive elements as floats, from either storage type (16-byte aligned).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// Programmatic dependent launch: a kernel launched with the attribute may
// start while the kernel before it on the stream is still running. Until its
// griddep_wait() returns it may touch only memory no kernel writes (weights,
// lookup tables); after it, everything the earlier kernels wrote is visible.
// griddep_launch() lets the next kernel begin its own preamble. Both are
// no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#ifdef MYNAH_PDL_EARLY
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#else
__device__ __forceinline__ void griddep_launch() {}
#endif

// The same for the small kernels between the products (norms, rotation and cache write, merge): their few CTAs
// start at once, so letting the product behind them start too costs them nothing, and that product's CTAs
// fetch their first weights while these still run.
__device__ __forceinline__ void griddep_launch_small() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The same for a kernel that has issued the last of its long loads: what follows it may begin its own (one row:
// 0.969 -> 0.956 ms a decode step at the 0.6B shape; eight rows: no difference). MYNAH_PDL_NO_LATE builds without.
#ifndef MYNAH_PDL_NO_LATE
__device__ __forceinline__ void griddep_launch_late() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#else
__device__ __forceinline__ void griddep_launch_late() {}
#endif

// 1: launch the decode-path kernels with the programmatic-serialization attribute.
int mynah_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t mynah_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = mynah_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }
