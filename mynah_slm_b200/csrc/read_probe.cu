// A plain reader: how fast this device hands 16 KB pieces of global memory, taken in shuffled order, to its SMs
// when nothing is done with them. One lane a CTA keeps `stages` bulk copies into shared memory in flight. It is
// the yardstick for the kernels that stream the cache and the weights: what a given number of bytes in flight an
// SM can reach at all (`python bench.py --only reader`).
#include "tcgen05.cuh"

namespace {

constexpr int PIECE = 16384;

__global__ void read_probe_kernel(const unsigned char* __restrict__ base, const int* __restrict__ order, int n_pieces, int stages,
                                  unsigned long long* __restrict__ sink, int* __restrict__ status) {
    using namespace tc5;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t bars[16];
    if (threadIdx.x != 0) return;
    for (int i = 0; i < stages; i++) mbar_init(smem_u32(&bars[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    int mine = 0;
    for (int c = blockIdx.x; c < n_pieces; c += gridDim.x) mine++;
    unsigned long long acc = 0;
    int issued = 0, done = 0, c = blockIdx.x;
    while (done < mine) {
        while (issued < mine && issued - done < stages) {
            const int st = issued % stages;
            mbar_expect_tx(smem_u32(&bars[st]), PIECE);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(smem + (size_t)st * PIECE)), "l"(base + (size_t)order[c] * PIECE), "r"(PIECE), "r"(smem_u32(&bars[st])) : "memory");
            c += gridDim.x;
            issued++;
        }
        const int st = done % stages;
        if (!mbar_wait(smem_u32(&bars[st]), (uint32_t)((done / stages) & 1))) {      // bounded: gives up and says so
            atomicOr(status, MYNAH_ST_TIMEOUT);
            return;
        }
        acc += smem[(size_t)st * PIECE];
        done++;
    }
    if (acc == 0x0123456789abcdefull) *sink = acc;                                  // keeps the reads alive
}

}  // namespace

// Reads n_pieces pieces of 16 KB at base + order[i] * 16 KB with ctas_per_sm CTAs an SM, each keeping `stages`
// (at most 12) copies in flight. The caller times it.
MYNAH_API int mynah_read_probe(const void* base, const int* order, int n_pieces, int ctas_per_sm, int stages,
                               unsigned long long* sink, int* status, cudaStream_t stream) {
    MYNAH_REQUIRE(n_pieces > 0 && ctas_per_sm >= 1 && stages >= 1 && stages <= 12 && ((uintptr_t)base & 15) == 0, "read_probe: bad arguments");
    const size_t smem = (size_t)stages * PIECE;
    MYNAH_REQUIRE(smem * ctas_per_sm <= 220 * 1024, "read_probe: %d CTAs of %d stages do not fit an SM", ctas_per_sm, stages);
    const cudaError_t e = cudaFuncSetAttribute(read_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return mynah_fail("read_probe: %s", cudaGetErrorString(e));
    read_probe_kernel<<<mynah_sm_count() * ctas_per_sm, 32, smem, stream>>>((const unsigned char*)base, order, n_pieces, stages, sink, status);
    return mynah_check_launch("read_probe");
}
