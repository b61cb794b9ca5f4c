// Brings ranges of global memory into the L2 cache without any SM waiting for them.
//
// A decode step of a small batch is a chain of short kernels, each of which streams a few megabytes of weights
// that nothing before it in the chain produces. Launched on a second stream beside the chain, this kernel asks
// the memory system for the weights the chain will want next (cp.async.bulk.prefetch.L2), so that the chain's
// kernels find them in L2 instead of waiting for DRAM. It reads and writes nothing itself; a range it is given
// only has to be readable.
#include "common.cuh"

namespace {

constexpr int MAX_RANGES = 8;
constexpr unsigned CHUNK = 8192;                  // bytes one thread asks for

struct Ranges {
    const unsigned char* base[MAX_RANGES];
    unsigned long long bytes[MAX_RANGES];         // multiples of 16
    unsigned long long first_chunk[MAX_RANGES + 1];
    int n;
};

__global__ void l2_prefetch_kernel(const Ranges r) {
    const unsigned long long total = r.first_chunk[r.n];
    for (unsigned long long c = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; c < total;
         c += (unsigned long long)gridDim.x * blockDim.x) {
        int i = 0;
        while (i + 1 < r.n && c >= r.first_chunk[i + 1]) i++;
        const unsigned long long off = (c - r.first_chunk[i]) * CHUNK;
        const unsigned long long left = r.bytes[i] - off;
        const unsigned size = left < CHUNK ? (unsigned)left : CHUNK;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(r.base[i] + off), "r"(size) : "memory");
    }
}

}  // namespace

// Up to 8 ranges (addresses 16-byte aligned; sizes are rounded down to multiples of 16 bytes).
MYNAH_API int mynah_l2_prefetch(const void* const* ptrs, const unsigned long long* bytes, int n, cudaStream_t stream) {
    MYNAH_REQUIRE(n >= 0 && n <= MAX_RANGES, "l2_prefetch: %d ranges, at most %d are taken", n, MAX_RANGES);
    Ranges r;
    r.n = 0;
    r.first_chunk[0] = 0;
    for (int i = 0; i < n; i++) {
        const unsigned long long b = bytes[i] & ~15ull;
        if (ptrs[i] == nullptr || b == 0) continue;
        MYNAH_REQUIRE(((uintptr_t)ptrs[i] & 15) == 0, "l2_prefetch: range %d does not start on a 16-byte boundary", i);
        r.base[r.n] = static_cast<const unsigned char*>(ptrs[i]);
        r.bytes[r.n] = b;
        r.first_chunk[r.n + 1] = r.first_chunk[r.n] + (b + CHUNK - 1) / CHUNK;
        r.n++;
    }
    if (r.n == 0) return 0;
    const unsigned long long chunks = r.first_chunk[r.n];
    const int threads = 128;
    const long long want = (long long)((chunks + threads - 1) / threads);
    const int blocks = (int)(want < 64 ? want : 64);
    l2_prefetch_kernel<<<blocks, threads, 0, stream>>>(r);
    return mynah_check_launch("l2_prefetch");
}
