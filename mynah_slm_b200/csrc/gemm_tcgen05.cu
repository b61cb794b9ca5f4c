// bf16 matrix product on the fifth-generation tensor cores:
//   C[M, N] = A[M, K] . W[N, K]^T,  fp32 accumulation in tensor memory.
//
// A persistent kernel: one CTA per SM walks over 128 x BN tiles of C (BN = 128
// or 256). Operand tiles of 64 k (128 bytes per row) are brought into shared
// memory by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a ring of
// stages that runs on across tiles; one elected thread issues tcgen05.mma
// (cta_group::1, kind::f16, M = 128, N = BN, K = 16 per instruction) with
// shared-memory descriptors for both operands (both are K-major: activations
// [M, K] and weights [N, K] as stored). The accumulator lives in tensor
// memory, in two buffers of BN columns, so that the epilogue of one tile
// (tcgen05.ld, conversion, the activation if any, a swizzled staging tile in
// shared memory, a TMA store) runs while the tensor cores work on the next.
//
// Warp roles: 0 TMA producer, 1 MMA issuer and tensor-memory owner, 2..5
// epilogue (one per 32-lane quadrant of tensor memory). Hand-over is by
// mbarriers: TMA completes transactions on `full`; tcgen05.commit arrives on
// `empty` when the instructions that read a stage have finished and on
// `acc_full` when a tile is accumulated; the epilogue warps arrive on
// `acc_empty` when they have read a buffer out.
//
// Epilogues: bf16 rows; fp32 rows (logits); SwiGLU, where the B tile is 128
// gate rows followed by the matching 128 up rows of the fused gate/up matrix,
// so the activation (mynah-slm src/kernels.c:193-205) is applied to the
// accumulator and only [M, F] is ever written.
//
// Every wait on an mbarrier is bounded by a wall-clock limit; a wait that runs
// out sets a status bit and an abort flag, and the CTA still drains the copies
// it started, frees its tensor memory and returns. Rows of A or W beyond the
// matrix are zero-filled by TMA; TMA stores clip what lies outside C.
#include "tcgen05.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int THREADS = 192;
constexpr int STAGING_BYTES = 32 * 128;              // 32 rows x 128 bytes per epilogue warp and buffer

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2, EPI_QKV = 3 };

// Shared-memory operand descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, M = m, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Stages of the operand ring: what fits beside the staging tiles.
__host__ __device__ constexpr int ring_stages(int bn, int ctas) {
    return (227 * 1024 - 4 * 2 * STAGING_BYTES - 2048) / (A_BYTES + bn * BK * 2 / ctas) > 8
               ? 8 : (227 * 1024 - 4 * 2 * STAGING_BYTES - 2048) / (A_BYTES + bn * BK * 2 / ctas);
}

// The stable form of the reference's sigmoid (mynah-slm src/kernels.c:193-205: e^-|v| never overflows), on the
// hardware's base-2 exponential and reciprocal: a relative error of a few 2^-23 in a value that is rounded to
// bf16 right after. The accurate library forms cost four times the instructions and left the epilogue warps,
// not the tensor cores, as the kernel's limit.
__device__ __forceinline__ float sigmoid_stable(float v) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-fabsf(v) * 1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return (v >= 0.f ? 1.0f : e) * r;
}
// What the q/k/v epilogue needs: the product's rows are tokens, its columns the heads of q, then k, then v.
// Each epilogue thread has one token's head in registers (fp32, straight from the accumulator), norms it, rotates
// it and writes it where the attention kernels read it: q rows to q_out, k and v to the token's place in its
// sequence's page. (Norm before rotation, one gain per head position shared by all heads, v neither normed nor
// rotated: mynah-slm src/arch_qwen3.c:208-218, src/kernels.c:130-137, :173-189.)
struct QkvEpilogue {
    int H, KV;
    float eps;
    const float* cos_t;               // [n_pos, HD / 2], or null: no rotation
    const float* sin_t;
    int n_pos;
    VecRef q_gain, k_gain;            // .p null: no per-head norm
    const int* tok_seq;               // [M], -1: padding row
    const int* tok_pos;
    PageTable pt;
    bf16* q_out;                      // [M, ldq]
    int ldq;
    bf16* k_cache;                    // [n_pages, KV, 64, HD], or null: only q is produced
    bf16* v_cache;
};

// Which tile of the output a tile number is. Tiles are numbered band by band: a band is `band` rows of tiles (8 for
// CTA pairs, 16 for single CTAs), and inside a band the numbers run down a column of tiles first. The CTAs of a
// launch work on consecutive numbers at any time, so together they touch a block of about as many rows of A as of
// W, which stays in L2; numbered column by column over all of M, a product of 16,384 rows streamed all of A from
// DRAM once for every column of tiles.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int band, int& m_tile, int& n_tile) {
    const int band_tiles = band * n_tiles;
    const int b = tile / band_tiles, in_band = tile - b * band_tiles;
    const int m0 = b * band;
    const int rows = min(band, m_tiles - m0);                        // the last band may be narrower
    m_tile = m0 + in_band % rows;
    n_tile = in_band / rows;
}

struct GemmShape {
    int M, N, K;          // N: output columns (for SwiGLU: gate rows; the up rows follow up_offset rows later)
    int up_offset;
    int m_tiles, n_tiles; // m_tiles: tiles of 128 rows (one CTA) or 256 rows (a pair of CTAs)
    float* sk_part;       // with SK: a CTA's partial accumulator, [CTAs][128][BN] fp32
    int* sk_flag;         // with SK: [CTAs][4], set by the warp that wrote its 32 rows, cleared by the warp that read them
};

// What a unit works on next: a tile of C and a range of its k-blocks. Without SK that is a whole tile (or, with
// KS, this CTA's half of K), tiles unit, unit + n_units, ... With SK ("stream-K") the k-blocks of all tiles,
// tile after tile, are dealt out evenly: CTA u takes k-blocks [u * I / U, (u + 1) * I / U) of the I in all, so
// every CTA has the same work however the number of tiles relates to the number of SMs. A tile that a boundary
// cuts is accumulated by consecutive CTAs. The one with the tile's first k-block owns it: it finishes the tile.
// The others (`produce`: their range starts inside the tile, so it is the first thing they do) write their
// accumulators to their slot of `sk_part` and raise their flags; the owner, for which the tile is the last thing
// it does, adds the `follow` slots behind its own in order and runs the epilogue. A CTA produces at most once
// (only its first item can start inside a tile), so a slot a CTA suffices. All CTAs of the launch are resident
// (at most one per SM is launched), so the producers run whether or not the owner waits. It is used only when
// there are at least as many tiles as CTAs: a tile then has at most two parts, and the owner fetches the other
// part with one bulk copy a warp into the operand ring, which is idle by then.
struct Item {
    int tile, kb0, kb1;
    int follow;           // an owner's: how many of the next CTAs hold a part of this tile
    bool produce;
};

template <bool SK>
struct ItemIter {
    int nk, unit, n_units, total_tiles, kb_begin, kb_end;
    long long it, it1, total;         // SK: this CTA's range of k-blocks over all tiles
    int tile;                         // not SK: the next tile
    __device__ ItemIter(int nk_, int unit_, int n_units_, int total_tiles_, int kb_begin_, int kb_end_)
        : nk(nk_), unit(unit_), n_units(n_units_), total_tiles(total_tiles_), kb_begin(kb_begin_), kb_end(kb_end_) {
        total = (long long)total_tiles * nk;
        it = SK ? (long long)unit * total / n_units : 0;
        it1 = SK ? (long long)(unit + 1) * total / n_units : 0;
        tile = unit;
    }
    __device__ bool next(Item& w) {
        if (!SK) {
            if (tile >= total_tiles) return false;
            w.tile = tile; w.kb0 = kb_begin; w.kb1 = kb_end; w.follow = 0; w.produce = false;
            tile += n_units;
            return true;
        }
        if (it >= it1) return false;
        w.tile = (int)(it / nk);
        w.kb0 = (int)(it % nk);
        const long long left = it1 - it;
        w.kb1 = left < (long long)(nk - w.kb0) ? w.kb0 + (int)left : nk;
        w.produce = w.kb0 != 0;
        w.follow = 0;
        if (!w.produce && w.kb1 < nk) {
            const long long tile_end = (long long)(w.tile + 1) * nk;
            int m = 1;
            while (unit + m + 1 < n_units && (long long)(unit + m + 1) * total / n_units < tile_end) m++;
            w.follow = m;
        }
        it += w.kb1 - w.kb0;
        return true;
    }
};

// CTAS = 2: two CTAs of a cluster share a tile of 256 x BN. Each brings its own 128 rows of A and half of the
// BN rows of W (for SwiGLU: one the gate rows, the other the up rows), the even CTA issues
// tcgen05.mma.cta_group::2 for both, and each reads its 128 rows of the accumulator out of its own tensor
// memory. A CTA then loads 16 + BN/8 KB a k-block instead of 16 + BN/4, which is what the ring's depth and
// the L2's bandwidth have to cover.
//
// KS = 2 (single CTAs, bf16 rows, BN = 256, one tile a cluster): the two CTAs of a cluster share a tile by halves
// of K. A product with few tiles (a narrow N at a few thousand rows) then still fills the SMs with 256-wide
// tiles, which need fewer operand bytes a flop than the 128-wide ones. When both have accumulated, each sends
// the 128 accumulator columns that the other will finish to the other's idle operand ring (fp32, through
// distributed shared memory), adds what it received to its own 128 columns and stores them.
// With -DMYNAH_GEMM_STAMPS the first CTA of a launch writes its SM's cycle counter at fixed points of every role's
// loop (a diagnostic build; mynah_gemm_tcgen05_stamps copies the table out).
#ifdef MYNAH_GEMM_STAMPS
constexpr int GS_ITEMS = 16, GS_POINTS = 4;
__device__ long long g_gemm_stamps[8][GS_ITEMS][GS_POINTS];
__device__ long long g_gemm_spans[1024][2];                          // every CTA's entry and exit on the global timer (ns)
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define GSTAMP(role, item, p)                                                                               \
    do {                                                                                                    \
        if (blockIdx.x == 0 && (item) < GS_ITEMS) g_gemm_stamps[(role)][(item)][(p)] = clock64();          \
    } while (0)
#else
#define GSTAMP(role, item, p) do { } while (0)
#endif

// mbar_wait that also gives up when another role of the CTA has: the flag is looked at only once polls have
// failed, so a wait that finds its phase complete costs one try_wait.
__device__ __forceinline__ bool mbar_wait_abort(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = now_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) return false;
        }
    }
}

template <int BN, int EPI, int CTAS, int KS = 1, bool SK = false>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, GemmShape g, int* __restrict__ status, const QkvEpilogue qe) {
    constexpr int HD = EPI == EPI_QKV ? 128 : 32;                    // the q/k/v epilogue is built for heads of 128
    __shared__ float gain_s[EPI == EPI_QKV ? 2 : 1][EPI == EPI_QKV ? HD : 1];
    constexpr int B_BYTES = BN * BK * 2 / CTAS;                      // this CTA's rows of W
    constexpr int STAGE = A_BYTES + B_BYTES;
    constexpr int STAGES = ring_stages(BN, CTAS);
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? 128 : BN;           // output columns of a tile
    constexpr int CHUNK = EPI == EPI_F32 ? 32 : 64;                  // output columns per staged store (128 bytes per row)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = smem + STAGES * STAGE;                  // 4 warps x 2 buffers x 4 KB, 1024-aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 4 * 2 * STAGING_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t fix_bar0 = smem_u32(bars + 2 * STAGES + 5);       // SK: one per epilogue warp, used once

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) GSTAMP(7, 0, 0);                             // entry
#ifdef MYNAH_GEMM_STAMPS
    if (threadIdx.x == 0 && blockIdx.x < 1024) g_gemm_spans[blockIdx.x][0] = global_ns();
#endif
    const int nk = (g.K + BK - 1) / BK;
    const int total_tiles = g.m_tiles * g.n_tiles;
    if (EPI == EPI_QKV && threadIdx.x < HD) {                        // the gains, once (ones when there is no per-head norm)
        gain_s[0][threadIdx.x] = qe.q_gain.p != nullptr ? qe.q_gain.at(threadIdx.x) : 1.0f;
        gain_s[EPI == EPI_QKV ? 1 : 0][threadIdx.x] = qe.k_gain.p != nullptr ? qe.k_gain.at(threadIdx.x) : 1.0f;
    }
    static_assert(KS == 1 || (KS == 2 && CTAS == 1 && EPI == EPI_BF16 && BN == 256), "K is split for single CTAs with bf16 rows only");
    static_assert(!SK || (CTAS == 1 && KS == 1 && EPI != EPI_QKV), "k-blocks are dealt out to single CTAs with the plain epilogues only");
    const int rank = CTAS == 2 ? (int)cluster_ctarank() : 0;         // 0 leads
    const int krank = KS == 2 ? (int)cluster_ctarank() : 0;          // which half of K
    const int unit = blockIdx.x / (CTAS * KS), n_units = gridDim.x / (CTAS * KS);   // a unit walks over tiles: a CTA, a pair, or two halves of K
    const int kb_begin = krank == 0 ? 0 : (nk + 1) / 2, kb_end = KS == 2 && krank == 0 ? (nk + 1) / 2 : nk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4 * CTAS);                 // one arrival per epilogue warp (of both CTAs, on the leader's)
        }
        if (SK)
            for (int q = 0; q < 4; q++) mbar_init(fix_bar0 + 8 * q, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        if (CTAS == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();                               // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched behind another kernel with programmatic dependent launch, everything above ran while that kernel was
    // finishing; nothing it wrote is touched before this returns (a no-op for an ordinary launch).
    griddep_wait();
    if (threadIdx.x == 0) GSTAMP(7, 0, 1);                             // set up

    if (warp == 0) {
        if (lane == 0) {                                             // ---- TMA producer
            int it = 0;                                              // k-blocks issued, over all tiles
            bool ok = true;
            ItemIter<SK> items(nk, unit, n_units, total_tiles, kb_begin, kb_end);
            Item w;
            int n_item = 0;
            while (ok && items.next(w)) {
                int m_tile, n_tile;
                tile_coords(w.tile, g.m_tiles, g.n_tiles, CTAS == 2 ? 8 : 16, m_tile, n_tile);
                GSTAMP(0, n_item, 0);
                n_item++;
                for (int kb = w.kb0; kb < w.kb1; kb++, it++) {
                    if (kb == w.kb1 - 1) GSTAMP(0, n_item - 1, 1);
                    if (kb == w.kb0 + 3) GSTAMP(0, n_item - 1, 2);     // the fourth k-block's turn: the ring was empty until here
                    if (kb == w.kb0 + 8) GSTAMP(0, n_item - 1, 3);
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it >= STAGES && !mbar_wait_abort(empty0 + 8 * s, ph ^ 1, abort_flag)) {   // (the ring starts empty)
                        *abort_flag = 1;
                        atomicOr(status, MYNAH_ST_TIMEOUT);
                        ok = false;
                        break;
                    }
                    const uint32_t a_dst = smem_u32(smem + s * STAGE), b_dst = a_dst + A_BYTES;
                    if (CTAS == 2) {
                        // both CTAs' copies complete on the leader's barrier, which expects the bytes of both
                        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE);
                        tma_load_2d_pair(a_dst, &map_a, kb * BK, (m_tile * 2 + rank) * BM, full0 + 8 * s);
                        const int w_row = EPI == EPI_SWIGLU ? (rank == 0 ? n_tile * 128 : g.up_offset + n_tile * 128)
                                                            : n_tile * BN + rank * (BN / 2);
                        tma_load_2d_pair(b_dst, &map_b, kb * BK, w_row, full0 + 8 * s);
                        continue;
                    }
                    if (it == 1) GSTAMP(3, 0, 0);
                    mbar_expect_tx(full0 + 8 * s, STAGE);
                    if (it == 1) GSTAMP(3, 0, 1);
                    tma_load_2d(a_dst, &map_a, kb * BK, m_tile * BM, full0 + 8 * s);
                    if (it == 1) GSTAMP(3, 0, 2);
                    if (EPI == EPI_SWIGLU) {                         // 128 gate rows, then their 128 up rows
                        tma_load_2d(b_dst, &map_b, kb * BK, n_tile * 128, full0 + 8 * s);
                        tma_load_2d(b_dst + 128 * BK * 2, &map_b, kb * BK, g.up_offset + n_tile * 128, full0 + 8 * s);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 128; j++)
                            tma_load_2d(b_dst + j * 128 * BK * 2, &map_b, kb * BK, n_tile * BN + j * 128, full0 + 8 * s);
                    }
                    if (it == 1) GSTAMP(3, 0, 3);
                }
            }
            // every operand of this CTA has been asked for: what follows on the stream may begin its own set-up
            griddep_launch_late();
            if (!ok && rank == 0) {
                // copies that were started still land in shared memory: wait for them (bounded)
                for (int j = max(0, it - STAGES); j < it; j++) mbar_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                                // ---- MMA issuer (of the pair: the leader's)
            constexpr uint32_t idesc = umma_idesc(BM * CTAS, BN);
            int it = 0, local = 0;
            bool ok = true;
            ItemIter<SK> items(nk, unit, n_units, total_tiles, kb_begin, kb_end);
            Item w;
            for (; ok && items.next(w); local++) {
                const int buf = local & 1;
                const uint32_t use = (local >> 1) & 1;
                if (local >= 2 && !mbar_wait_abort(acc_empty0 + 8 * buf, use ^ 1, abort_flag)) {   // the epilogue has read this buffer out
                    *abort_flag = 1;
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                    break;
                }
                tc_fence_after();
                GSTAMP(1, local, 0);
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = w.kb0; kb < w.kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_abort(full0 + 8 * s, ph, abort_flag)) {
                        *abort_flag = 1;
                        atomicOr(status, MYNAH_ST_TIMEOUT);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    if (kb == w.kb0) GSTAMP(1, local, 1);
                    const uint32_t a_addr = smem_u32(smem + s * STAGE), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
                        if (CTAS == 2) tc_mma_pair(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (kb | k) != 0);
                        else tc_mma(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, ((kb - w.kb0) | k) != 0);
                    }
                    // the stage is free (in both CTAs) once these have read it
                    if (CTAS == 2) tc_commit_pair(empty0 + 8 * s); else tc_commit(empty0 + 8 * s);
                }
                // arrives when the tile is accumulated
                if (CTAS == 2) tc_commit_pair(acc_full0 + 8 * buf); else tc_commit(acc_full0 + 8 * buf);
                GSTAMP(1, local, 2);
            }
        }
    } else if (KS == 2) {                                            // ---- epilogue warps, K split: the tile is accumulated (this half)
        if (unit < total_tiles && !mbar_wait_abort(acc_full0, 0, abort_flag)) {
            if (lane == 0) {
                *abort_flag = 1;
                atomicOr(status, MYNAH_ST_TIMEOUT);
            }
        }
        if (warp == 2 && lane == 0) GSTAMP(2, 0, 0);
    } else {                                                         // ---- epilogue: warps 2..5 -> lane quadrants 2,3,0,1
        const int quad = warp & 3;
        unsigned char* my_stage = staging + quad * 2 * STAGING_BYTES;
        int local = 0, n_store = 0;
        ItemIter<SK> items(nk, unit, n_units, total_tiles, kb_begin, kb_end);
        Item w;
        for (; items.next(w); local++) {
            int m_tile, n_tile;
            tile_coords(w.tile, g.m_tiles, g.n_tiles, CTAS == 2 ? 8 : 16, m_tile, n_tile);
            const int buf = local & 1;
            const uint32_t use = (local >> 1) & 1;
            if (!mbar_wait_abort(acc_full0 + 8 * buf, use, abort_flag)) {
                if (lane == 0) {
                    *abort_flag = 1;
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                }
                break;
            }
            tc_fence_after();
            if (warp == 2 && lane == 0) GSTAMP(2, local, 0);
            const uint32_t t_row = tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16);
            const int row0 = (m_tile * CTAS + rank) * BM + quad * 32;
            if (SK && w.produce) {
                // this CTA's part of a tile that the CTA before it owns: the accumulator goes to this CTA's slot
                float* mine = g.sk_part + ((size_t)unit * BM + quad * 32 + lane) * BN;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(t_row + c0, r);
                    // 16-byte pieces, eight at a time swizzled by the row: the owner reads them from shared memory a
                    // thread a row without meeting in a bank
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        __stcg(reinterpret_cast<float4*>(mine + c0) + (j ^ (lane & 7)), make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                }
                __syncwarp();
                if (lane == 0) {
                    __threadfence();                                 // the warp's rows before its flag
                    atomicExch(g.sk_flag + unit * 4 + quad, 1);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
                continue;
            }
            const float* part_s = reinterpret_cast<const float*>(smem) + (size_t)(quad * 32 + lane) * BN;   // this thread's row of the fetched part
            if (SK && w.follow > 0) {
                // The owner of a tile whose other part the next CTA holds: when that CTA's warp of this quadrant has
                // raised its flag, its 32 rows (one contiguous block) come into the operand ring, which is idle now
                // (this is the CTA's last item and its products are done), with one bulk copy.
                int got = 1;
                if (lane == 0) {
                    const unsigned long long t0 = now_ns();
                    const volatile int* f = g.sk_flag + (unit + 1) * 4 + quad;
                    for (uint32_t spin = 0; *f == 0; spin++) {
                        if ((spin & 255u) == 255u && (now_ns() - t0 > WAIT_LIMIT_NS || *abort_flag)) {
                            got = 0;
                            break;
                        }
                    }
                    if (got && w.follow == 1) {
                        __threadfence();                             // the flag before the rows it announces
                        constexpr uint32_t BYTES = 32 * BN * 4;
                        mbar_expect_tx(fix_bar0 + 8 * quad, BYTES);
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(smem_u32(smem) + quad * BYTES), "l"(g.sk_part + ((size_t)(unit + 1) * BM + quad * 32) * BN),
                                       "r"(BYTES), "r"(fix_bar0 + 8 * quad) : "memory");
                    } else {
                        got = 0;                                     // (more than two parts a tile are not launched)
                    }
                }
                got = __shfl_sync(0xffffffffu, got, 0);
                if (got && !mbar_wait(fix_bar0 + 8 * quad, 0)) got = 0;
                if (!__all_sync(0xffffffffu, got) && lane == 0) {
                    *abort_flag = 1;
                    atomicOr(status, MYNAH_ST_TIMEOUT);
                }
            }
            // adds the other part to 32 accumulator columns from `col` on
            auto add_parts = [&](uint32_t (&r)[32], int col) {
                if (SK && w.follow > 0) {
                    const float4* src = reinterpret_cast<const float4*>(part_s + col);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float4 v = src[j ^ (lane & 7)];
                        r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
                        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
                        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
                        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
                    }
                }
            };
            if (EPI == EPI_QKV) {
                // ---- a token a thread: its heads of this tile, one after the other
                const int row = row0 + lane;
                const int seq = row < g.M ? qe.tok_seq[row] : -1;
                const int pos = seq >= 0 ? qe.tok_pos[row] : 0;
                bool live = seq >= 0;
                if (live && qe.cos_t != nullptr && (pos < 0 || pos >= qe.n_pos)) {
                    atomicOr(status, MYNAH_ST_POS_RANGE);
                    live = false;
                }
                size_t cache_row = 0;
                bool paged = false;
                if (live && qe.k_cache != nullptr) {
                    const int page = page_of(qe.pt, seq, pos);
                    if (page < 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
                    else {
                        paged = true;
                        cache_row = (size_t)page * qe.KV * PAGE_TOKENS + pos % PAGE_TOKENS;
                    }
                }
#pragma unroll 1
                for (int hh = 0; hh < BN / HD; hh++) {
                    const int col0 = n_tile * BN + hh * HD;
                    if (col0 >= g.N) break;                          // uniform over the warp
                    const int head = col0 / HD;
                    const bool is_q = head < qe.H, is_k = !is_q && head < qe.H + qe.KV;
                    float v[HD];
                    __syncwarp();                                    // the loads from tensor memory need the whole warp together
#pragma unroll
                    for (int c = 0; c < HD / 32; c++) tc_ld32(t_row + hh * HD + c * 32, reinterpret_cast<uint32_t(&)[32]>(v[c * 32]));
                    bf16* dst = nullptr;
                    if (live) {
                        if (is_q) dst = qe.q_out + (size_t)row * qe.ldq + (size_t)head * HD;
                        else if (paged) dst = (is_k ? qe.k_cache : qe.v_cache) + (cache_row + (size_t)(head - qe.H - (is_k ? 0 : qe.KV)) * PAGE_TOKENS) * HD;
                    }
                    if (dst != nullptr) {
                        if (is_q || is_k) {
                            if (qe.q_gain.p != nullptr) {
                                float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int j = 0; j < HD; j++) s4[j & 3] = fmaf(v[j], v[j], s4[j & 3]);
                                const float sc = 1.0f / sqrtf(((s4[0] + s4[1]) + (s4[2] + s4[3])) / (float)HD + qe.eps);
                                const float* gn = gain_s[is_q ? 0 : 1];
#pragma unroll
                                for (int j = 0; j < HD; j++) v[j] = v[j] * (sc * gn[j]);
                            }
                            if (qe.cos_t != nullptr) {
                                const float4* c4 = reinterpret_cast<const float4*>(qe.cos_t + (size_t)pos * (HD / 2));
                                const float4* s4p = reinterpret_cast<const float4*>(qe.sin_t + (size_t)pos * (HD / 2));
#pragma unroll
                                for (int i4 = 0; i4 < HD / 8; i4++) {
                                    const float4 c = c4[i4], sn = s4p[i4];
                                    const float cc[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                                    for (int e = 0; e < 4; e++) {
                                        const int i = i4 * 4 + e;
                                        const float a0 = v[i], b0 = v[i + HD / 2];
                                        v[i] = a0 * cc[e] - b0 * ss[e];
                                        v[i + HD / 2] = b0 * cc[e] + a0 * ss[e];
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int j = 0; j < HD / 8; j++)
                            reinterpret_cast<uint4*>(dst)[j] = make_uint4(pack2(v[8 * j], v[8 * j + 1]), pack2(v[8 * j + 2], v[8 * j + 3]),
                                                                          pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
                    }
                }
            } else
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += CHUNK, n_store++) {
                unsigned char* st = my_stage + (n_store & 1) * STAGING_BYTES;
                // the store that last read this staging buffer must have finished reading it
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
                unsigned char* my_row = st + lane * 128;
                if (EPI == EPI_F32) {
                    uint32_t r[32];
                    tc_ld32(t_row + c0, r);
                    add_parts(r, c0);
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        *reinterpret_cast<uint4*>(my_row + ((j ^ (lane & 7)) * 16)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                } else if (EPI == EPI_BF16) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t r[32];
                        tc_ld32(t_row + c0 + half * 32, r);
                        add_parts(r, c0 + half * 32);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint4 v = make_uint4(pack2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                                                       pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                                       pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                                       pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
                            *reinterpret_cast<uint4*>(my_row + (((half * 4 + j) ^ (lane & 7)) * 16)) = v;
                        }
                    }
                } else {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t gt[32], up[32];
                        tc_ld32(t_row + c0 + half * 32, gt);
                        tc_ld32(t_row + 128 + c0 + half * 32, up);
                        add_parts(gt, c0 + half * 32);
                        add_parts(up, 128 + c0 + half * 32);
                        float o[32];
#pragma unroll
                        for (int e = 0; e < 32; e++) {
                            // gate and up rounded to bf16 first, as when they are stored before the activation
                            const float gv = round_to<bf16>(__uint_as_float(gt[e])), uv = round_to<bf16>(__uint_as_float(up[e]));
                            o[e] = (gv * sigmoid_stable(gv)) * uv;
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint4 v = make_uint4(pack2(o[8 * j], o[8 * j + 1]), pack2(o[8 * j + 2], o[8 * j + 3]),
                                                       pack2(o[8 * j + 4], o[8 * j + 5]), pack2(o[8 * j + 6], o[8 * j + 7]));
                            *reinterpret_cast<uint4*>(my_row + (((half * 4 + j) ^ (lane & 7)) * 16)) = v;
                        }
                    }
                }
                fence_async_smem();                                  // the staged rows become visible to the TMA engine
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&map_c, smem_u32(st), n_tile * OUT_COLS + c0, row0);
                    tma_store_commit();
                }
            }
            // this warp has read its quadrant of the buffer out
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (SK)                                              // the parts are read: their flags are clear for the next launch
                    for (int p = 1; p <= w.follow; p++) g.sk_flag[(unit + p) * 4 + quad] = 0;
                if (CTAS == 2) mbar_arrive_leader(acc_empty0 + 8 * buf); else mbar_arrive(acc_empty0 + 8 * buf);
            }
            if (warp == 2 && lane == 0) GSTAMP(2, local, 1);
        }
        if (lane == 0) tma_store_wait_all();
        if (warp == 2 && lane == 0) GSTAMP(2, 0, 2);
    }
    if (KS == 2) {
        // Both CTAs are past their last product (or gave up): their operand rings are idle and may be written.
        tc_fence_before();
        __syncthreads();
        cluster_sync_all();
        tc_fence_after();
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                            // of the tile; epilogue warps only
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
        const bool work = warp >= 2 && unit < total_tiles;
        if (work) {
            // the other CTA's 128 columns of this CTA's accumulator, as fp32 rows of 512 bytes, 16-byte pieces
            // swizzled by the row so that neither these stores nor the loads below meet in a bank
            const uint32_t there = cluster_map(smem_u32(smem), (uint32_t)(krank ^ 1)) + (uint32_t)row * 512u;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                uint32_t r[32];
                tc_ld32(t_row + (krank ^ 1) * 128 + c * 32, r);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    st_cluster_v4(there + (uint32_t)(((c * 8 + j) ^ (lane & 7)) * 16), r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            }
        }
        if (warp == 2 && lane == 0) GSTAMP(2, 0, 1);
        cluster_sync_all();                                          // what the other CTA sent has arrived
        if (warp == 2 && lane == 0) GSTAMP(2, 0, 2);
        if (work) {
            int m_tile, n_tile;
            tile_coords(unit, g.m_tiles, g.n_tiles, 16, m_tile, n_tile);
            const int row0 = m_tile * BM + quad * 32;
            unsigned char* my_stage = staging + quad * 2 * STAGING_BYTES;
            const unsigned char* got = smem + (size_t)row * 512;
#pragma unroll 1
            for (int c0 = 0, n_store = 0; c0 < 128; c0 += 64, n_store++) {
                unsigned char* st = my_stage + (n_store & 1) * STAGING_BYTES;
                unsigned char* my_row = st + lane * 128;
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t r[32];
                    tc_ld32(t_row + krank * 128 + c0 + half * 32, r);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int piece = (c0 + half * 32 + 8 * j) / 4;
                        const float4 pa = *reinterpret_cast<const float4*>(got + ((piece ^ (lane & 7)) * 16));
                        const float4 pb = *reinterpret_cast<const float4*>(got + (((piece + 1) ^ (lane & 7)) * 16));
                        const uint4 v = make_uint4(pack2(__uint_as_float(r[8 * j]) + pa.x, __uint_as_float(r[8 * j + 1]) + pa.y),
                                                   pack2(__uint_as_float(r[8 * j + 2]) + pa.z, __uint_as_float(r[8 * j + 3]) + pa.w),
                                                   pack2(__uint_as_float(r[8 * j + 4]) + pb.x, __uint_as_float(r[8 * j + 5]) + pb.y),
                                                   pack2(__uint_as_float(r[8 * j + 6]) + pb.z, __uint_as_float(r[8 * j + 7]) + pb.w));
                        *reinterpret_cast<uint4*>(my_row + (((half * 4 + j) ^ (lane & 7)) * 16)) = v;
                    }
                }
                fence_async_smem();                                  // the staged rows become visible to the TMA engine
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&map_c, smem_u32(st), n_tile * BN + krank * 128 + c0, row0);
                    tma_store_commit();
                }
            }
            if (lane == 0) tma_store_wait_all();
            if (warp == 2 && lane == 0) GSTAMP(2, 0, 3);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) GSTAMP(7, 0, 2);                             // all roles done
#ifdef MYNAH_GEMM_STAMPS
    if (threadIdx.x == 0 && blockIdx.x < 1024) g_gemm_spans[blockIdx.x][1] = global_ns();
#endif
    if (CTAS == 2) cluster_sync_all();                               // neither CTA leaves while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        if (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

#ifdef MYNAH_GEMM_STAMPS
// out: [8 roles][16 items][4 points] of the stamped CTA's cycle counts (host memory).
MYNAH_API int mynah_gemm_tcgen05_stamps(long long* out) {
    return cudaMemcpyFromSymbol(out, g_gemm_stamps, sizeof(g_gemm_stamps)) == cudaSuccess ? 0 : -1;
}
// out: [1024 CTAs][entry, exit] in nanoseconds of the device's global timer.
MYNAH_API int mynah_gemm_tcgen05_spans(long long* out) {
    return cudaMemcpyFromSymbol(out, g_gemm_spans, sizeof(g_gemm_spans)) == cudaSuccess ? 0 : -1;
}
#endif

// The stream-K workspace of the current device: a slot of 128 x 256 floats and four flags a CTA, allocated at the
// first launch that needs it (never during a graph capture: a captured step has run once before).
// (One workspace a device: stream-K products of one device must not overlap in time, which holds for the
// single stream that the engine launches on.)
float* part_d[64] = {};
int* flag_d[64] = {};
int ctas_d[64] = {};

int sk_workspace(int n_ctas, float** part, int** flag) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return mynah_fail("gemm_tcgen05: no current device");
    if (ctas_d[dev] < n_ctas) {
        float* pnew = nullptr;
        int* fnew = nullptr;
        cudaError_t e = cudaMalloc(&pnew, (size_t)n_ctas * BM * 256 * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&fnew, (size_t)n_ctas * 4 * sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(fnew, 0, (size_t)n_ctas * 4 * sizeof(int));
        if (e != cudaSuccess) return mynah_fail("gemm_tcgen05: workspace for %d CTAs: %s", n_ctas, cudaGetErrorString(e));
        // (an earlier, smaller workspace may still be in use by a captured graph: it is kept)
        part_d[dev] = pnew; flag_d[dev] = fnew; ctas_d[dev] = n_ctas;
    }
    *part = part_d[dev];
    *flag = flag_d[dev];
    return 0;
}

template <int BN, int EPI, int CTAS, int KS = 1, bool SK = false>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, int M, int N, int K, int up_offset,
                int sm_count, int* status, cudaStream_t stream, const QkvEpilogue& qe = QkvEpilogue{}) {
    constexpr int STAGES = ring_stages(BN, CTAS);
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2 / CTAS) + 4 * 2 * STAGING_BYTES + 256 + 1024;
    auto kern = gemm_tcgen05_kernel<BN, EPI, CTAS, KS, SK>;
    static bool opted = false;
    if (!opted) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return mynah_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
        opted = true;
    }
    GemmShape g;
    g.M = M; g.N = N; g.K = K; g.up_offset = up_offset;
    g.m_tiles = ceil_div(M, BM * CTAS);
    g.n_tiles = EPI == EPI_SWIGLU ? ceil_div(N, 128) : ceil_div(N, BN);
    const long long tiles = (long long)g.m_tiles * g.n_tiles;
    MYNAH_REQUIRE(tiles < (1ll << 30), "gemm_tcgen05: too many tiles");
    const int max_units = sm_count / (CTAS * KS);
    const int units = (int)(tiles < max_units && !SK ? tiles : max_units);     // with SK every SM takes its share of the k-blocks
    g.sk_part = nullptr;
    g.sk_flag = nullptr;
    if (SK && sk_workspace(units, &g.sk_part, &g.sk_flag)) return -1;
    MYNAH_REQUIRE(KS == 1 || tiles <= max_units, "gemm_tcgen05: K is split only when every tile has a cluster of its own");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units * CTAS * KS);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (CTAS * KS == 2) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = CTAS * KS;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    if (mynah_pdl_enabled()) {                                       // the kernel's set-up may run under the kernel before it
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, g, status, qe);
    if (e != cudaSuccess) return mynah_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
    return mynah_check_launch("gemm_tcgen05");
}

// 1 (default): products of 256 rows or more run on pairs of CTAs (cta_group::2) where that measured faster.
// MYNAH_GEMM_PAIR=0 keeps single CTAs, 2 takes pairs for every product of 256 rows or more.
int pair_mode() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("MYNAH_GEMM_PAIR");
        v = e == nullptr ? 1 : (e[0] == '0' ? 0 : (e[0] == '2' ? 2 : 1));
    }
    return v;
}

}  // namespace

// After a launch that gave up on a wait (status bit 16) a stream-K flag may have been left raised: clears them,
// behind whatever the stream still holds.
MYNAH_API int mynah_gemm_tcgen05_reset(cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || flag_d[dev] == nullptr) return 0;
    const cudaError_t e = cudaMemsetAsync(flag_d[dev], 0, (size_t)ctas_d[dev] * 4 * sizeof(int), stream);
    if (e != cudaSuccess) return mynah_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
    return 0;
}

MYNAH_API int mynah_gemm_tcgen05_supported(int M, int N, int K) {
    return M >= 1 && N >= 8 && N % 8 == 0 && K >= 8 && K % 8 == 0;      // rows of 16-byte multiples for TMA
}

// Whether the bf16-rows product of this shape is run as two halves of K (its sums then differ in rounding from
// the product run whole). MYNAH_GEMM_KSPLIT=0 keeps whole tiles.
MYNAH_API int mynah_gemm_tcgen05_splits_k(int M, int N, int K, int sm_count) {
    static const bool on = [] { const char* e = getenv("MYNAH_GEMM_KSPLIT"); return !(e != nullptr && e[0] == '0'); }();
    if (sm_count <= 0) sm_count = mynah_sm_count();
    // (the exchange costs about 4 us; a k-block about 0.34 us on a 128-wide tile, 0.39 us on half of a 256-wide one)
    return on && ceil_div(K, BK) >= 32 && (long long)ceil_div(M, BM) * ceil_div(N, 256) <= sm_count / 2;
}

// epilogue 0: C bf16 [M, N]; 1: C fp32 [M, N]; 2: SwiGLU, W holds N gate rows then N up rows, C bf16 [M, N].
// A [M, K] and W [rows, K] are bf16, row-major, 16-byte aligned; ldc is C's row pitch in elements. `status`
// receives MYNAH_ST_TIMEOUT if a wait inside the kernel ran out.
MYNAH_API int mynah_gemm_tcgen05(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int epilogue,
                                 int sm_count, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    MYNAH_REQUIRE(mynah_gemm_tcgen05_supported(M, N, K), "gemm_tcgen05: M=%d N=%d K=%d is not taken (N and K must be multiples of 8)", M, N, K);
    MYNAH_REQUIRE(epilogue >= 0 && epilogue <= 2 && ldc >= N, "gemm_tcgen05: bad epilogue or output stride");
    const int csize = epilogue == EPI_F32 ? 4 : 2;
    MYNAH_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)C & 15) == 0 && (ldc * csize) % 16 == 0,
                  "gemm_tcgen05: operands must be 16-byte aligned and the output pitch a multiple of 16 bytes");
    MYNAH_REQUIRE(status != nullptr, "gemm_tcgen05: a status word is required");
    if (sm_count <= 0) sm_count = mynah_sm_count();
    // Pairs pay once a unit has tiles to run one after the other (the ring then stays full across tiles); with
    // one tile a unit, as for a 2,048-token prompt of a small model, single CTAs measured the same or better.
    const long long pair_tiles = (long long)ceil_div(M, 2 * BM) * (epilogue == EPI_SWIGLU ? ceil_div(N, 128) : ceil_div(N, 256));
    const bool pair = M >= 2 * BM && sm_count >= 2 &&
                      (pair_mode() == 2 || (pair_mode() == 1 && pair_tiles >= 2 * (sm_count / 2)));
    // The k-blocks of all tiles dealt out evenly (stream-K) where whole tiles would leave SMs idle in their last
    // wave and the k-blocks saved are worth more than the fix-up. MYNAH_GEMM_SK=0: never, 2: wherever it can run.
    static const int sk_mode = [] { const char* e = getenv("MYNAH_GEMM_SK"); return e == nullptr ? 1 : (e[0] == '0' ? 0 : (e[0] == '2' ? 2 : 1)); }();
    if (epilogue != EPI_SWIGLU && !pair && sk_mode != 0) {
        const long long tiles_w = (long long)ceil_div(M, BM) * ceil_div(N, 256);
        const int nk = ceil_div(K, BK);
        const long long waves = (tiles_w + sm_count - 1) / sm_count;
        // k-blocks a CTA with whole tiles and with the k-blocks dealt out; a k-block takes about 0.39 us, the fix-up about 3 us
        const long long kb_whole = waves * nk, kb_dealt = (tiles_w * nk + sm_count - 1) / sm_count;
        const bool fits = tiles_w >= sm_count && nk >= 8;            // at most two parts a tile
        // (dealt out, CTAs no longer walk the same k-blocks of neighbouring tiles at the same time, which costs L2
        // hits: 2,048 x 4,096 x 12,288 got slower with 13% fewer k-blocks a CTA, 2,048 x 2,560 x 9,728 faster with 45%)
        if (fits && (sk_mode == 2 || ((kb_whole - kb_dealt) * 39 > 600 && (kb_whole - kb_dealt) * 4 >= kb_whole))) {
            CUtensorMap ma, mb, mc;
            if (make_map(&ma, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, K, 128, BK)) return -1;
            if (make_map(&mb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, K, 128, BK)) return -1;
            if (epilogue == EPI_F32) {
                if (make_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32)) return -1;
                return launch_gemm<256, EPI_F32, 1, 1, true>(ma, mb, mc, M, N, K, 0, sm_count, status, stream);
            }
            if (make_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 32, 64)) return -1;
            return launch_gemm<256, EPI_BF16, 1, 1, true>(ma, mb, mc, M, N, K, 0, sm_count, status, stream);
        }
    }
    // Few tiles even at 256 columns (a narrow N): two CTAs a tile, a half of K each.
    if (epilogue == EPI_BF16 && !pair && mynah_gemm_tcgen05_splits_k(M, N, K, sm_count)) {
        CUtensorMap ma, mb, mc;
        if (make_map(&ma, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, K, 128, BK)) return -1;
        if (make_map(&mb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, K, 128, BK)) return -1;
        if (make_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 32, 64)) return -1;
        return launch_gemm<256, EPI_BF16, 1, 2>(ma, mb, mc, M, N, K, 0, sm_count, status, stream);
    }
    // wide tiles unless they would leave most SMs idle
    const long long units = pair ? sm_count / 2 : sm_count;
    const bool wide = epilogue == EPI_SWIGLU || (long long)ceil_div(N, 256) * ceil_div(M, pair ? 2 * BM : BM) * 10 >= units * 8 || N > 4096;
    const int w_box_rows = pair ? (wide ? 128 : 64) : 128;           // rows of W that one copy brings
    CUtensorMap ma, mb, mc;
    if (make_map(&ma, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, K, 128, BK)) return -1;
    if (make_map(&mb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, epilogue == EPI_SWIGLU ? 2LL * N : N, K, K, w_box_rows, BK)) return -1;
    if (epilogue == EPI_F32) {
        if (make_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32)) return -1;
    } else {
        if (make_map(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 32, 64)) return -1;
    }
#define MYNAH_GEMM_GO(BN_, EPI_) \
    (pair ? launch_gemm<BN_, EPI_, 2>(ma, mb, mc, M, N, K, epilogue == EPI_SWIGLU ? N : 0, sm_count, status, stream) \
          : launch_gemm<BN_, EPI_, 1>(ma, mb, mc, M, N, K, epilogue == EPI_SWIGLU ? N : 0, sm_count, status, stream))
    if (epilogue == EPI_SWIGLU) return MYNAH_GEMM_GO(256, EPI_SWIGLU);
    if (epilogue == EPI_F32) return wide ? MYNAH_GEMM_GO(256, EPI_F32) : MYNAH_GEMM_GO(128, EPI_F32);
    return wide ? MYNAH_GEMM_GO(256, EPI_BF16) : MYNAH_GEMM_GO(128, EPI_BF16);
#undef MYNAH_GEMM_GO
}

// The q/k/v projection of a prompt step with its epilogue: C = A . W^T as above (W rows: H heads of q, KV of k,
// KV of v, head_dim 128), then per token and head the per-head RMSNorm (gains may be null), the rotation of the
// whole head (tables may be null) and the writes: q to q_out [M, ldq], k and v to the token's row of its
// sequence's page (k_cache null: W holds q only). tok_seq [M] (-1: padding row), tok_pos [M].
MYNAH_API int mynah_gemm_qkv_rope_supported(int M, int H, int KV, int HD, int K) {
    return M >= 1 && HD == 128 && H >= 1 && KV >= 1 && K >= 8 && K % 8 == 0;
}

MYNAH_API int mynah_gemm_qkv_rope(const void* A, const void* W, int M, int H, int KV, int HD, int K,
                                  const void* q_gain, const void* k_gain, int gain_dtype, float eps,
                                  const float* cos_t, const float* sin_t, int n_pos,
                                  const int* tok_seq, const int* tok_pos,
                                  const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
                                  void* q_out, int ldq, void* k_cache, void* v_cache,
                                  int sm_count, int* status, cudaStream_t stream) {
    if (M == 0) return 0;
    MYNAH_REQUIRE(mynah_gemm_qkv_rope_supported(M, H, KV, HD, K), "gemm_qkv_rope: M=%d H=%d KV=%d head_dim=%d K=%d is not taken", M, H, KV, HD, K);
    MYNAH_REQUIRE((k_cache == nullptr) == (v_cache == nullptr) && (cos_t == nullptr) == (sin_t == nullptr) &&
                  (q_gain == nullptr) == (k_gain == nullptr), "gemm_qkv_rope: caches, tables and gains come in pairs");
    MYNAH_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ldq % 8 == 0 && ldq >= H * HD &&
                  ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)cos_t & 15) == 0 && ((uintptr_t)sin_t & 15) == 0,
                  "gemm_qkv_rope: operands must be 16-byte aligned");
    MYNAH_REQUIRE(status != nullptr, "gemm_qkv_rope: a status word is required");
    if (sm_count <= 0) sm_count = mynah_sm_count();
    const int N = (k_cache != nullptr ? H + 2 * KV : H) * HD;
    QkvEpilogue qe;
    qe.H = H; qe.KV = KV; qe.eps = eps; qe.cos_t = cos_t; qe.sin_t = sin_t; qe.n_pos = n_pos;
    qe.q_gain = VecRef{q_gain, gain_dtype}; qe.k_gain = VecRef{k_gain, gain_dtype};
    qe.tok_seq = tok_seq; qe.tok_pos = tok_pos;
    qe.pt = PageTable{page_indptr, page_ids, page_base, n_pages};
    qe.q_out = (bf16*)q_out; qe.ldq = ldq; qe.k_cache = (bf16*)k_cache; qe.v_cache = (bf16*)v_cache;
    const long long pair_tiles = (long long)ceil_div(M, 2 * BM) * ceil_div(N, 256);
    const bool pair = pair_mode() >= 1 && M >= 2 * BM && sm_count >= 2 && pair_tiles >= 2 * (sm_count / 2);
    CUtensorMap ma, mb;
    if (make_map(&ma, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, K, 128, BK)) return -1;
    if (make_map(&mb, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, K, 128, BK)) return -1;
    // the epilogue stores from registers: the third map is not used
    if (pair) return launch_gemm<256, EPI_QKV, 2>(ma, mb, ma, M, N, K, 0, sm_count, status, stream, qe);
    return launch_gemm<256, EPI_QKV, 1>(ma, mb, ma, M, N, K, 0, sm_count, status, stream, qe);
}
