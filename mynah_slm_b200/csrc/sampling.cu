// From logits to a token, on the device: penalties, greedy argmax, and
// temperature sampling with top-k, min-p and top-p, in the reference's order
// (mynah-slm src/sampler.c:116-187; penalties :80-106; ring :73-78; the
// generator is splitmix64, :40-46).
//
// The reference sorts the whole vocabulary by (probability descending, id
// ascending) and works on prefixes of that order. Every filter keeps a prefix
// and the draw walks a prefix, so no sort is needed here: a prefix is found by
// a radix search over the bits of the probabilities (three passes of 11, 11
// and 10 bits) with a histogram of counts and of probability mass per digit.
// Mass is summed as 2^-60 fixed point in 64-bit integers: integer sums do not
// depend on the order of the additions, so the same logits and the same
// generator state give the same token in every run.
#include "common.cuh"

#include <cooperative_groups.h>

namespace {

namespace cg = cooperative_groups;

constexpr int THREADS = 1024;
constexpr int ROW_CTAS = 8;            // CTAs (one cluster) that share a row of a large vocabulary
constexpr int LOADS = 8;               // loads of a row that a thread keeps in flight
constexpr int BINS = 2048;

__device__ __forceinline__ unsigned long long mass_of(float p) {
    return __double2ull_rd((double)p * 1152921504606846976.0);     // p * 2^60
}

struct Prefix {            // a prefix of the sorted order
    unsigned int value;    // bits of the probability at which it ends
    unsigned int above;    // elements with a larger probability
    unsigned int ties;     // elements equal to `value` that belong to it (by ascending id)
    unsigned long long mass;   // its total mass
};

struct Shared {
    unsigned int count[BINS];
    // a digit's mass (2^-60 fixed point) as two 32-bit words: 32-bit adds are native atomics in shared memory,
    // 64-bit ones are compare-and-swap loops that crawl when many warps hit one digit
    unsigned int mass_lo[BINS], mass_hi[BINS];
    unsigned int warp_count[32];
    unsigned long long warp_mass[32];
    // results handed from the finding thread to the block (and, in a cluster, read by the other CTAs); two
    // sets used in turn, so that one pass's results can still be read while the next pass starts
    unsigned int found_digit[2], found_above[2], found_count[2];
    unsigned long long found_mass[2];
    unsigned int turn;                 // passes done so far (selects the set)
    double part_d;                     // this CTA's share of a sum over the row
    unsigned long long part_m;         // this CTA's share of the row's mass
    unsigned int part_u;
    float red_f[32];
    int red_i[32];
    double red_d[32];
    unsigned int scan_u[32];
};

__device__ __forceinline__ void add_mass(Shared& sh, unsigned int d, unsigned long long m) {
    const unsigned int lo = (unsigned int)m;
    unsigned int hi = (unsigned int)(m >> 32);
    if (lo != 0) {
        const unsigned int old = atomicAdd(&sh.mass_lo[d], lo);
        hi += old > 0xffffffffu - lo;                      // the low word wrapped: carry
    }
    if (hi != 0) atomicAdd(&sh.mass_hi[d], hi);
}
__device__ __forceinline__ unsigned long long mass_at(const Shared& sh, int d) {
    return ((unsigned long long)sh.mass_hi[d] << 32) | sh.mass_lo[d];
}

// A row is shared by NC CTAs (NC = 1, or the ROW_CTAS CTAs of a cluster): CTA r works on the elements
// [r * chunk, (r + 1) * chunk) and the CTAs meet through distributed shared memory. Every CTA of a row runs
// the same code with the same decisions, so the cluster barriers below are reached by all of them.
template <int NC>
struct RowShare {
    int rank, begin, end;                                   // this CTA's elements
    __device__ RowShare(int V) {
        if (NC == 1) {
            rank = 0; begin = 0; end = V;
        } else {
            rank = (int)cg::this_cluster().block_rank();
            const int chunk = ((V + NC - 1) / NC + 3) & ~3;
            begin = min(V, rank * chunk);
            end = min(V, begin + chunk);
        }
    }
    __device__ __forceinline__ void sync() const {
        if (NC == 1) __syncthreads();
        else cg::this_cluster().sync();
    }
    template <typename T> __device__ __forceinline__ T* at(T* mine, int r) const {
        return NC == 1 ? mine : cg::this_cluster().map_shared_rank(mine, r);
    }
};

struct Found {
    unsigned int digit, above, count;                       // the digit, the elements in larger digits, those in it
    unsigned long long mass;                                // mass of the elements in larger digits
};

// Finds the digit where the running (count, mass), taken from the largest digit down, first satisfies the
// target, among elements whose higher bits equal `prefix_bits` under `prefix_mask`. by_mass: cum_mass >=
// target_mass; else cum_count >= target_count. The carried count and mass are those of the elements in larger
// digits of earlier passes. Every thread of every CTA of the row gets the result.
template <int NC>
__device__ Found radix_pass(const float* __restrict__ p, const RowShare<NC>& rs, unsigned int prefix_bits, unsigned int prefix_mask,
                            int shift, int n_bins, bool by_mass, unsigned int target_count,
                            unsigned long long target_mass, unsigned int carry_count, unsigned long long carry_mass,
                            Shared& sh, float scale = 1.0f) {                // the elements are p[i] * scale (1: as stored)
    for (int i = threadIdx.x; i < BINS; i += THREADS) {
        sh.count[i] = 0;
        sh.mass_lo[i] = 0;
        sh.mass_hi[i] = 0;
    }
    __syncthreads();                                        // (the previous pass's advance of `turn` is visible from here on)
    const unsigned int set = sh.turn & 1u;                  // advanced only after this pass's last barrier
    if (threadIdx.x == 0) {
        sh.found_digit[set] = 0;                            // the smallest digit, when the target is never met
        sh.found_above[set] = 0xffffffffu;
    }
    // Probabilities crowd into a few digits where the digit is the exponent (the first pass): a warp whose 32
    // elements fall into at most four digits adds each digit's count and mass up with shuffles and lets one lane
    // do the atomics; a warp whose elements are spread out (the mantissa passes) uses plain atomics. Counts
    // and masses are integers, so the order of the additions does not matter. A row of a large vocabulary
    // comes from L2, a round trip a load: eight loads a thread are issued together.
    const int lane_h = threadIdx.x & 31;
    for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {    // the same number of turns for every thread
        float vals[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            vals[u] = i < rs.end ? p[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            if (base0 + u * THREADS >= rs.end) break;             // uniform
            bool on = false;
            unsigned int d = 0xffffffffu;
            unsigned long long ms = 0;
            if (i < rs.end) {
                const float v = vals[u] * scale;
                const unsigned int bits = __float_as_uint(v);
                if ((bits & prefix_mask) == prefix_bits) {
                    on = true;
                    d = (bits >> shift) & (n_bins - 1);
                    ms = mass_of(v);
                }
            }
            const unsigned int peers = __match_any_sync(0xffffffffu, d);
            const bool leader = on && lane_h == __ffs(peers) - 1;
            const unsigned int leaders = __ballot_sync(0xffffffffu, leader);
            if (__popc(leaders) <= 4) {
                unsigned int rem = leaders;
                while (rem) {                                     // uniform over the warp
                    const int src = __ffs(rem) - 1;
                    rem &= rem - 1;
                    const unsigned int grp = __shfl_sync(0xffffffffu, peers, src);
                    unsigned long long m = ((grp >> lane_h) & 1u) ? ms : 0ull;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) m += __shfl_xor_sync(0xffffffffu, m, o);
                    if (lane_h == src) {
                        atomicAdd(&sh.count[d], (unsigned int)__popc(grp));
                        add_mass(sh, d, m);
                    }
                }
            } else if (on) {
                atomicAdd(&sh.count[d], 1u);
                add_mass(sh, d, ms);
            }
        }
    }
    rs.sync();                                              // every CTA's histogram is complete
    if (NC > 1) {
        // the histograms are added up a slice of digits a CTA (all CTAs at once), the totals go to the leading CTA
        const int per_cta = (n_bins + NC - 1) / NC;
        const int i = rs.rank * per_cta + (int)threadIdx.x;
        const bool mine = (int)threadIdx.x < per_cta && i < n_bins;
        unsigned int ct = 0;
        unsigned long long mt = 0;
        if (mine) {
            unsigned int c[NC], lo[NC], hi[NC];
#pragma unroll
            for (int r = 0; r < NC; r++) {                  // the loads first, all in flight together
                c[r] = *rs.at(&sh.count[i], r);
                lo[r] = *rs.at(&sh.mass_lo[i], r);
                hi[r] = *rs.at(&sh.mass_hi[i], r);
            }
#pragma unroll
            for (int r = 0; r < NC; r++) {
                ct += c[r];
                mt += ((unsigned long long)hi[r] << 32) | lo[r];
            }
        }
        rs.sync();                                          // every digit of every CTA has been read: they may be overwritten
        if (mine) {
            *rs.at(&sh.count[i], 0) = ct;
            *rs.at(&sh.mass_lo[i], 0) = (unsigned int)mt;
            *rs.at(&sh.mass_hi[i], 0) = (unsigned int)(mt >> 32);
        }
        rs.sync();                                          // the leading CTA's histogram holds the row's totals
    }
    if (rs.rank == 0) {
        // scan from the largest digit down: thread t owns digits n_bins-1-2t and n_bins-2-2t
        const int d0 = n_bins - 1 - 2 * (int)threadIdx.x, d1 = d0 - 1;
        const unsigned int c0 = d0 >= 0 ? sh.count[d0] : 0, c1 = d1 >= 0 ? sh.count[d1] : 0;
        const unsigned long long m0 = d0 >= 0 ? mass_at(sh, d0) : 0, m1 = d1 >= 0 ? mass_at(sh, d1) : 0;
        unsigned int cs = c0 + c1;
        unsigned long long ms = m0 + m1;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned int c = __shfl_up_sync(0xffffffffu, cs, o);
            const unsigned long long m = __shfl_up_sync(0xffffffffu, ms, o);
            if (lane >= o) {
                cs += c;
                ms += m;
            }
        }
        if (lane == 31) {
            sh.warp_count[warp] = cs;
            sh.warp_mass[warp] = ms;
        }
        __syncthreads();
        unsigned int cbase = carry_count;
        unsigned long long mbase = carry_mass;
        for (int w = 0; w < warp; w++) {
            cbase += sh.warp_count[w];
            mbase += sh.warp_mass[w];
        }
        // exclusive values before this thread's first digit
        const unsigned int c_before = cbase + cs - (c0 + c1);
        const unsigned long long m_before = mbase + ms - (m0 + m1);
        auto met = [&](unsigned int c, unsigned long long m) {
            return by_mass ? (m >= target_mass) : (c >= target_count);
        };
        if (c0 > 0 && !met(c_before, m_before) && met(c_before + c0, m_before + m0)) {
            sh.found_digit[set] = (unsigned int)d0;
            sh.found_above[set] = c_before;
            sh.found_mass[set] = m_before;
            sh.found_count[set] = c0;
        } else if (c1 > 0 && !met(c_before + c0, m_before + m0) && met(c_before + c0 + c1, m_before + m0 + m1)) {
            sh.found_digit[set] = (unsigned int)d1;
            sh.found_above[set] = c_before + c0;
            sh.found_mass[set] = m_before + m0;
            sh.found_count[set] = c1;
        }
        __syncthreads();
        if (sh.found_above[set] == 0xffffffffu) {
            // target beyond everything (rounding): end at the smallest populated digit
            if (threadIdx.x == 0) {
                int d = 0;
                while (d < n_bins - 1 && sh.count[d] == 0) d++;
                unsigned int c = carry_count;
                unsigned long long m = carry_mass;
                for (int e = n_bins - 1; e > d; e--) {
                    c += sh.count[e];
                    m += mass_at(sh, e);
                }
                sh.found_digit[set] = (unsigned int)d;
                sh.found_above[set] = c;
                sh.found_mass[set] = m;
                sh.found_count[set] = sh.count[d];
            }
        }
    }
    rs.sync();                                              // the result is there (in the leading CTA)
    Found f;
    f.digit = *rs.at(&sh.found_digit[set], 0);
    f.above = *rs.at(&sh.found_above[set], 0);
    f.count = *rs.at(&sh.found_count[set], 0);
    f.mass = *rs.at(&sh.found_mass[set], 0);
    __syncthreads();                                        // all of this CTA's threads have read `turn` and the result
    if (threadIdx.x == 0) sh.turn++;                        // (the other set is used next; this one stays readable for the
    return f;                                               //  CTAs that have not read it yet until the pass after next)
}

// The smallest prefix of the sorted order whose count reaches target_count
// (by_mass false) or whose mass reaches target_mass (by_mass true).
template <int NC>
__device__ Prefix find_prefix(const float* __restrict__ p, const RowShare<NC>& rs, bool by_mass, unsigned int target_count,
                              unsigned long long target_mass, Shared& sh) {
    unsigned int bits = 0, mask = 0, above = 0, n_eq = 0;
    unsigned long long mass = 0;
    if (by_mass && target_mass == 0) target_mass = 1;      // a draw of exactly 0 takes the first element
    if (!by_mass && target_count == 0) target_count = 1;
    const int shifts[3] = {21, 10, 0}, nb[3] = {2048, 2048, 1024};
    for (int r = 0; r < 3; r++) {
        const Found f = radix_pass<NC>(p, rs, bits, mask, shifts[r], nb[r], by_mass, target_count, target_mass, above, mass, sh);
        bits |= f.digit << shifts[r];
        mask |= (unsigned int)(nb[r] - 1) << shifts[r];
        above = f.above;
        mass = f.mass;
        n_eq = f.count;
    }
    // `bits` is the probability at which the prefix ends; n_eq elements have exactly it
    const unsigned long long pm = mass_of(__uint_as_float(bits));
    unsigned int ties;
    if (by_mass) {
        if (pm == 0 || target_mass <= mass) ties = 1;
        else {
            const unsigned long long need = target_mass - mass;
            const unsigned long long t = (need + pm - 1) / pm;
            ties = (unsigned int)(t < 1 ? 1 : (t > n_eq ? n_eq : t));
        }
    } else {
        ties = target_count > above ? target_count - above : 1;
        if (ties > n_eq) ties = n_eq;
    }
    if (ties < 1) ties = 1;
    return Prefix{bits, above, ties, mass + (unsigned long long)ties * pm};
}

// Id of the j-th (1-based) element, by ascending id, whose probability bits equal `value` (-1: there is none).
// The CTAs of a row hold consecutive ranges of ids, so the j-th lies in the first CTA whose running count reaches j.
template <int NC>
__device__ int nth_equal(const float* __restrict__ p, const RowShare<NC>& rs, unsigned int value, unsigned int j, Shared& sh) {
    const int n_mine = rs.end - rs.begin;
    const int per = (n_mine + THREADS - 1) / THREADS;
    const int lo = rs.begin + threadIdx.x * per, hi = min(rs.end, lo + per);
    unsigned int c = 0;
    for (int i = lo; i < hi; i++) c += __float_as_uint(p[i]) == value;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int cs = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned int t = __shfl_up_sync(0xffffffffu, cs, o);
        if (lane >= o) cs += t;
    }
    if (lane == 31) sh.scan_u[warp] = cs;
    if (threadIdx.x == 0) sh.red_i[0] = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int tot = 0;
        for (int w = 0; w < THREADS / 32; w++) tot += sh.scan_u[w];
        sh.part_u = tot;                                    // equal elements in this CTA's range
    }
    rs.sync();
    unsigned int before = cs - c;                           // equal elements before this thread's range
    for (int r = 0; r < rs.rank; r++) before += *rs.at(&sh.part_u, r);
    for (int w = 0; w < warp; w++) before += sh.scan_u[w];
    if (c > 0 && before < j && j <= before + c) {
        unsigned int seen = before;
        for (int i = lo; i < hi; i++) {
            if (__float_as_uint(p[i]) == value && ++seen == j) {
                sh.red_i[0] = i;
                break;
            }
        }
    }
    rs.sync();
    int r = -1;
    for (int k = 0; k < NC; k++) {                          // at most one CTA has found it
        const int v = *rs.at(&sh.red_i[0], k);
        if (v >= 0) r = v;
    }
    rs.sync();                                              // red_i and part_u may be written again
    return r;
}

__device__ __forceinline__ double splitmix_uniform(unsigned long long* state) {
    unsigned long long z = (*state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

struct SampleParams {
    float temp, top_p, min_p;
    int top_k;
};

// First maximum of a row (strict >, lowest index on ties: sampler.c:124-129).
__device__ int block_argmax(const float* __restrict__ row, int V, Shared& sh, float* max_out) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += THREADS) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, bv, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        if (v2 > bv || (v2 == bv && i2 < bi)) {
            bv = v2;
            bi = i2;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
        sh.red_f[warp] = bv;
        sh.red_i[warp] = bi;
    }
    __syncthreads();
    bv = sh.red_f[lane];
    bi = sh.red_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, bv, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        if (v2 > bv || (v2 == bv && i2 < bi)) {
            bv = v2;
            bi = i2;
        }
    }
    __syncthreads();
    *max_out = bv;
    return bi == 0x7fffffff ? 0 : bi;
}

// The first maximum of a row in two steps, for vocabularies that one CTA reads too slowly: ARGMAX_PARTS CTAs
// each take a contiguous piece of the row, then the sampling CTA reduces their results. Ties go to the lowest
// index in both steps, so the result is the one-CTA result.
constexpr int ARGMAX_PARTS = 32;
constexpr int PART_THREADS = 256;

__device__ __forceinline__ void take_first_max(float& bv, int& bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

__global__ void __launch_bounds__(PART_THREADS)
argmax_partial_kernel(const float* __restrict__ logits, int V, int ld, const int* __restrict__ slots,
                      float* __restrict__ part_val, int* __restrict__ part_idx) {
    __shared__ float red_f[PART_THREADS / 32];
    __shared__ int red_i[PART_THREADS / 32];
    griddep_launch();
    griddep_wait();
    const int c = blockIdx.x, b = blockIdx.y;
    if (slots != nullptr && slots[b] < 0) return;          // padding row: the sampling CTA does not look
    const float* row = logits + (size_t)b * ld;
    const int chunk = ((V + ARGMAX_PARTS - 1) / ARGMAX_PARTS + 3) & ~3;
    const int i0 = c * chunk, i1 = min(V, i0 + chunk);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        const int n4 = (i1 - i0) / 4;
        const float4* r4 = reinterpret_cast<const float4*>(row + i0);
        for (int j = threadIdx.x; j < n4; j += PART_THREADS) {
            const float4 v = r4[j];
            const int i = i0 + 4 * j;
            take_first_max(bv, bi, v.x, i);
            take_first_max(bv, bi, v.y, i + 1);
            take_first_max(bv, bi, v.z, i + 2);
            take_first_max(bv, bi, v.w, i + 3);
        }
        for (int i = i0 + 4 * n4 + threadIdx.x; i < i1; i += PART_THREADS) take_first_max(bv, bi, row[i], i);
    } else {
        for (int i = i0 + threadIdx.x; i < i1; i += PART_THREADS) take_first_max(bv, bi, row[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, bv, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
        take_first_max(bv, bi, v2, i2);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        red_f[warp] = bv;
        red_i[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < PART_THREADS / 32; w++) take_first_max(bv, bi, red_f[w], red_i[w]);
        part_val[(size_t)b * ARGMAX_PARTS + c] = bv;
        part_idx[(size_t)b * ARGMAX_PARTS + c] = bi;
    }
}

// The row's first maximum from the pieces' results (every thread of the CTA gets it).
__device__ int argmax_from_parts(const float* __restrict__ part_val, const int* __restrict__ part_idx, int b, Shared& sh, float* max_out) {
    if (threadIdx.x < 32) {
        float bv = part_val[(size_t)b * ARGMAX_PARTS + threadIdx.x];
        int bi = part_idx[(size_t)b * ARGMAX_PARTS + threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(0xffffffffu, bv, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, bi, o);
            take_first_max(bv, bi, v2, i2);
        }
        if (threadIdx.x == 0) {
            sh.red_f[0] = bv;
            sh.red_i[0] = bi;
        }
    }
    __syncthreads();
    const float bv = sh.red_f[0];
    const int bi = sh.red_i[0];
    __syncthreads();
    *max_out = bv;
    return bi == 0x7fffffff ? 0 : bi;
}

// A top-k of at most MAX_CAND entries is drawn by sample_top_k_kernel, everything else by sample_kernel; both are
// launched for every step (the parameters are read on the device) and each leaves at once when the other is due.
constexpr int MAX_CAND = 256;
__device__ __forceinline__ bool small_top_k(const SampleParams& sp, int V) {
    return sp.temp > 0.f && sp.top_k > 0 && sp.top_k <= MAX_CAND && sp.top_k < V;
}

// One CTA a row, or for a large vocabulary the ROW_CTAS CTAs of a cluster (NC), each with a consecutive part of
// the row. The row of logits is overwritten with probabilities when the temperature is positive (the
// reference's sampler also works in place).
template <int NC>
__global__ void __launch_bounds__(THREADS)
sample_kernel(float* __restrict__ logits, int V, int ld, const float* __restrict__ params,
              unsigned long long* __restrict__ rng, const int* __restrict__ slots, int* __restrict__ out,
              const float* __restrict__ part_val, const int* __restrict__ part_idx) {
    __shared__ Shared sh;
    griddep_launch();
    griddep_wait();
    const SampleParams sp{params[0], params[1], params[2], (int)params[3]};
    if (small_top_k(sp, V)) return;          // (every CTA of the launch: sample_top_k_kernel draws this step)
    const int b = NC == 1 ? blockIdx.x : blockIdx.x / NC;
    float* row = logits + (size_t)b * ld;
    const int slot = slots ? slots[b] : b;
    const RowShare<NC> rs(V);
    if (slot < 0) {                          // padding row (all CTAs of the row leave)
        if (threadIdx.x == 0 && rs.rank == 0) out[b] = 0;
        return;
    }
    if (threadIdx.x == 0) sh.turn = 0;
    float mx;
    const int best = part_val != nullptr ? argmax_from_parts(part_val, part_idx, b, sh, &mx) : block_argmax(row, V, sh, &mx);
    if (sp.temp <= 0.f) {
        if (threadIdx.x == 0 && rs.rank == 0) out[b] = best;
        return;
    }
    // p_i = expf((l_i - max) / temp) * (float)(1 / sum), the sum in double (sampler.c:132-143)
    double part = 0.0;
    for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {
        float vals[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            vals[u] = i < rs.end ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            if (i < rs.end) {
                const float e = expf((vals[u] - mx) / sp.temp);
                row[i] = e;
                part += (double)e;                          // in index order within a thread
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) sh.red_d[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        double mine = 0.0;
        for (int w = 0; w < THREADS / 32; w++) mine += sh.red_d[w];
        sh.part_d = mine;
    }
    rs.sync();
    double sum = 0.0;
    for (int r = 0; r < NC; r++) sum += *rs.at(&sh.part_d, r);       // in the CTAs' order: the same value in each of them
    const float inv = (float)(1.0 / sum);
    unsigned int n_floor = 0;
    unsigned long long mass_part = 0;                       // the mass of this thread's probabilities (integers: any order)
    for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {
        float vals[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            vals[u] = i < rs.end ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            if (i < rs.end) {
                const float pr = vals[u] * inv;
                row[i] = pr;
                mass_part += mass_of(pr);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mass_part += __shfl_xor_sync(0xffffffffu, mass_part, o);
    if (lane == 0) sh.warp_mass[warp] = mass_part;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long mine = 0;
        for (int w = 0; w < THREADS / 32; w++) mine += sh.warp_mass[w];
        sh.part_m = mine;
    }
    rs.sync();                                              // the whole row holds probabilities (and part_d has been read)
    unsigned long long row_mass = 0;
    for (int r = 0; r < NC; r++) row_mass += *rs.at(&sh.part_m, r);
    const float p_best = __ldcg(row + best);                // possibly written by another CTA of the row

    // the kept prefix: top-k, then min-p, then top-p (sampler.c:146-175)
    unsigned int n = (unsigned int)V;
    if (sp.top_k > 0 && (unsigned int)sp.top_k < n) n = (unsigned int)sp.top_k;
    if (sp.min_p > 0.f) {
        const float floor_p = sp.min_p * p_best;
        unsigned int c = 0;
        for (int i = rs.begin + (int)threadIdx.x; i < rs.end; i += THREADS) c += row[i] >= floor_p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        if (lane == 0) sh.scan_u[warp] = c;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int mine = 0;
            for (int w = 0; w < THREADS / 32; w++) mine += sh.scan_u[w];
            sh.part_u = mine;
        }
        rs.sync();
        for (int r = 0; r < NC; r++) n_floor += *rs.at(&sh.part_u, r);
        rs.sync();                                          // part_u may be written again
        if (n_floor < 1) n_floor = 1;
        if (n_floor < n) n = n_floor;
    }
    if (sp.top_p < 1.0f) {
        const unsigned long long target = __double2ull_ru((double)sp.top_p * 1152921504606846976.0);
        const Prefix pp = find_prefix<NC>(row, rs, true, 0, target, sh);
        const unsigned int np = pp.above + pp.ties;
        if (np < n) n = np;
    }
    if (n < 1) n = 1;
    // mass of the kept prefix, then the draw r = U * total and the walk (sampler.c:178-186)
    // (with nothing cut off that is the row's mass, which the pass above has added up: three passes fewer)
    const Prefix kept = n == (unsigned int)V ? Prefix{0u, 0u, 0u, row_mass} : find_prefix<NC>(row, rs, false, n, 0, sh);
    unsigned long long state = rng[slot];                   // (rewritten by the leading CTA only after the last barrier)
    const double u = splitmix_uniform(&state);
    const double r = u * (double)kept.mass;
    unsigned long long target = __double2ull_ru(r);
    if (target > kept.mass) target = kept.mass;
    Prefix hit = find_prefix<NC>(row, rs, true, 0, target, sh);
    unsigned int rank = hit.above + hit.ties;              // 1-based place in the sorted order
    unsigned int value = hit.value, j = hit.ties;
    if (rank > n) {                                        // only through rounding: the last kept one
        value = kept.value;
        j = kept.ties;
    }
    const int id = nth_equal<NC>(row, rs, value, j, sh);
    if (threadIdx.x == 0 && rs.rank == 0) {
        out[b] = id >= 0 ? id : best;
        rng[slot] = state;
    }
}

// The draw with a small top-k (sampler.c:132-186, the same decisions in another order). The k largest
// probabilities are found once (a search by count, then the id up to which entries equal to the k-th belong),
// gathered into the leading CTA and sorted by (probability descending, id ascending), which is the order that
// the general kernel walks. min-p, top-p, the kept mass and the drawn place are then prefixes of at most k
// entries, walked by one thread in the same integer arithmetic: three passes over the row (exponentials and their
// sum, the leading bits of the k-th largest, the gather) instead of thirteen; seven for a row with many equal logits.
struct Candidates {
    unsigned long long key[MAX_CAND];      // probability bits above, ~id below: larger keys come first
    unsigned int n;
};

template <int NC>
__global__ void __launch_bounds__(THREADS)
sample_top_k_kernel(float* __restrict__ logits, int V, int ld, const float* __restrict__ params,
                    unsigned long long* __restrict__ rng, const int* __restrict__ slots, int* __restrict__ out,
                    const float* __restrict__ part_val, const int* __restrict__ part_idx) {
    __shared__ Shared sh;
    __shared__ Candidates cand;
    griddep_launch();
    griddep_wait();
    const SampleParams sp{params[0], params[1], params[2], (int)params[3]};
    if (!small_top_k(sp, V)) return;         // (every CTA of the launch)
    const int b = NC == 1 ? blockIdx.x : blockIdx.x / NC;
    float* row = logits + (size_t)b * ld;
    const int slot = slots ? slots[b] : b;
    const RowShare<NC> rs(V);
    if (slot < 0) {                          // padding row (all CTAs of the row leave)
        if (threadIdx.x == 0 && rs.rank == 0) out[b] = 0;
        return;
    }
    if (threadIdx.x == 0) sh.turn = 0;
    float mx;
    const int best = part_val != nullptr ? argmax_from_parts(part_val, part_idx, b, sh, &mx) : block_argmax(row, V, sh, &mx);
    // p_i = expf((l_i - max) / temp) * (float)(1 / sum), the sum in double, as in sample_kernel
    double part = 0.0;
    for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {
        float vals[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            vals[u] = i < rs.end ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            if (i < rs.end) {
                const float e = expf((vals[u] - mx) / sp.temp);
                row[i] = e;
                part += (double)e;
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) sh.red_d[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        double mine = 0.0;
        for (int w = 0; w < THREADS / 32; w++) mine += sh.red_d[w];
        sh.part_d = mine;
    }
    rs.sync();
    double sum = 0.0;
    for (int r = 0; r < NC; r++) sum += *rs.at(&sh.part_d, r);
    const float inv = (float)(1.0 / sum);
    if (threadIdx.x == 0) cand.n = 0;
    for (int i = threadIdx.x; i < MAX_CAND; i += THREADS) cand.key[i] = 0ull;
    rs.sync();                                              // the row holds the exponentials; the leading CTA's list is empty
    const float p_best = __ldcg(row + best) * inv;

    // One pass over the probabilities (the stored exponentials times inv, as the reference forms them) finds the
    // leading eleven bits of the k-th largest. Everything with those bits or larger ones holds the k largest; when
    // that is a short list it is gathered and sorted, and its first k entries are the k largest in the order
    // (probability descending, id ascending). Only a row that crowds more than MAX_CAND entries there (many equal
    // logits) takes the long way: the row normalised in place, the k-th probability to the last bit and the id up
    // to which its equals belong.
    const Found lead = radix_pass<NC>(row, rs, 0u, 0u, 21, 2048, false, (unsigned int)sp.top_k, 0, 0, 0, sh, inv);
    const bool short_list = lead.above + lead.count <= (unsigned int)MAX_CAND;      // the same in every CTA of the row
    Prefix topk{0u, 0u, 0u, 0ull};
    int id_bound = -1;
    float gather_scale = inv;
    if (!short_list) {
        for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {
            float vals[LOADS];
#pragma unroll
            for (int u = 0; u < LOADS; u++) {
                const int i = base0 + u * THREADS + (int)threadIdx.x;
                vals[u] = i < rs.end ? row[i] : 0.f;
            }
#pragma unroll
            for (int u = 0; u < LOADS; u++) {
                const int i = base0 + u * THREADS + (int)threadIdx.x;
                if (i < rs.end) row[i] = vals[u] * inv;
            }
        }
        rs.sync();                                          // the row holds probabilities
        topk = find_prefix<NC>(row, rs, false, (unsigned int)sp.top_k, 0, sh);
        id_bound = nth_equal<NC>(row, rs, topk.value, topk.ties, sh);
        gather_scale = 1.0f;
    }
    unsigned int* cnt = rs.at(&cand.n, 0);
    unsigned long long* keys = rs.at(&cand.key[0], 0);
    for (int base0 = rs.begin; base0 < rs.end; base0 += THREADS * LOADS) {
        float vals[LOADS];
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            vals[u] = i < rs.end ? __ldcg(row + i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < LOADS; u++) {
            const int i = base0 + u * THREADS + (int)threadIdx.x;
            const unsigned int bits = __float_as_uint(vals[u] * gather_scale);    // probabilities are not negative: bits order as values
            const bool take = short_list ? (bits >> 21) >= lead.digit : (bits > topk.value || (bits == topk.value && i <= id_bound));
            if (i < rs.end && take) {
                const unsigned int at = atomicAdd(cnt, 1u);
                if (at < (unsigned int)MAX_CAND) keys[at] = ((unsigned long long)bits << 32) | (0xffffffffu - (unsigned int)i);
            }
        }
    }
    rs.sync();                                              // the list is complete
    if (rs.rank != 0) return;                               // (the leading CTA reads its own memory only from here on)
    // bitonic sort, largest key first: larger probability, then lower id
    for (int size = 2; size <= MAX_CAND; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const int t = threadIdx.x, partner = t ^ stride;
            if (t < MAX_CAND && partner > t) {
                const unsigned long long a = cand.key[t], c = cand.key[partner];
                const bool descending = (t & size) == 0;
                if (descending ? a < c : a > c) {
                    cand.key[t] = c;
                    cand.key[partner] = a;
                }
            }
            __syncthreads();
        }
    }
    if (threadIdx.x != 0) return;
    const unsigned int n_c = min(min(cand.n, (unsigned int)MAX_CAND), (unsigned int)sp.top_k);   // top_k, unless the row has fewer entries
    unsigned int n = n_c;
    if (sp.min_p > 0.f) {
        const float floor_p = sp.min_p * p_best;
        unsigned int c = 0;
        while (c < n_c && __uint_as_float((unsigned int)(cand.key[c] >> 32)) >= floor_p) c++;
        if (c < 1) c = 1;
        if (c < n) n = c;
    }
    if (sp.top_p < 1.0f) {
        unsigned long long target = __double2ull_ru((double)sp.top_p * 1152921504606846976.0);
        if (target == 0) target = 1;
        unsigned long long cum = 0;
        for (unsigned int i = 0; i < n; i++) {
            cum += mass_of(__uint_as_float((unsigned int)(cand.key[i] >> 32)));
            if (cum >= target) {
                n = i + 1;
                break;
            }
        }
    }
    if (n < 1) n = 1;
    unsigned long long total = 0;
    for (unsigned int i = 0; i < n; i++) total += mass_of(__uint_as_float((unsigned int)(cand.key[i] >> 32)));
    unsigned long long state = rng[slot];
    const double u = splitmix_uniform(&state);
    unsigned long long target = __double2ull_ru(u * (double)total);
    if (target > total) target = total;
    if (target == 0) target = 1;
    unsigned int pick = n - 1;                              // (only through rounding: the last kept one)
    unsigned long long cum = 0;
    for (unsigned int i = 0; i < n; i++) {
        cum += mass_of(__uint_as_float((unsigned int)(cand.key[i] >> 32)));
        if (cum >= target) {
            pick = i;
            break;
        }
    }
    out[b] = n_c > 0 ? (int)(0xffffffffu - (unsigned int)cand.key[pick]) : best;
    rng[slot] = state;
}

// One thread per row: the reference's loop over the ring of recent tokens,
// entry by entry (a token that sits in the ring c times is penalised c times).
// The ring rows are `stride` apart; the window in use is params[7] <= stride.
__global__ void penalties_kernel(float* __restrict__ logits, int B, int V, int ld, const int* __restrict__ ring,
                                 const int* __restrict__ ring_n, int stride, const int* __restrict__ slots,
                                 const float* __restrict__ params) {
    griddep_launch();
    griddep_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const float repeat = params[4], freq = params[5], presence = params[6];
    const int window = min((int)params[7], stride);
    if (window <= 0 || (repeat == 1.0f && freq == 0.0f && presence == 0.0f)) return;   // sampler.c:81-84
    const int slot = slots ? slots[b] : b;
    if (slot < 0) return;
    const int n = min(ring_n[slot], window);
    const int* r = ring + (size_t)slot * stride;
    float* row = logits + (size_t)b * ld;
    for (int i = 0; i < n; i++) {
        const int tok = r[i];
        if (tok < 0 || tok >= V) continue;
        int count = 0;
        for (int k = 0; k < n; k++) count += r[k] == tok;
        float l = row[tok];
        if (repeat != 1.0f) l = l > 0.f ? l / repeat : l * repeat;
        l -= freq * (float)count;
        l -= presence;
        row[tok] = l;
    }
}

// ring[slot][head] = token; head advances; the count saturates at the window.
__global__ void accept_kernel(const int* __restrict__ tokens, int B, int* __restrict__ ring, int* __restrict__ ring_n,
                              int* __restrict__ ring_head, int stride, const int* __restrict__ slots,
                              const float* __restrict__ params) {
    griddep_launch();
    griddep_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    const int window = min((int)params[7], stride);
    if (b >= B || window <= 0) return;
    const int slot = slots ? slots[b] : b;
    if (slot < 0) return;
    const int head = ring_head[slot] % window;
    ring[(size_t)slot * stride + head] = tokens[b];
    ring_head[slot] = (head + 1) % window;
    if (ring_n[slot] < window) ring_n[slot]++;
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int ld, int* __restrict__ out) {
    __shared__ Shared sh;
    griddep_launch();
    griddep_wait();
    float mx;
    const int best = block_argmax(logits + (size_t)blockIdx.x * ld, V, sh, &mx);
    if (threadIdx.x == 0) out[blockIdx.x] = best;
}

}  // namespace

MYNAH_API int mynah_argmax(const float* logits, int B, int V, int ld, int* out, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && V > 0 && ld >= V, "argmax: bad sizes B=%d V=%d ld=%d", B, V, ld);
    mynah_launch(argmax_kernel, dim3(B), dim3(THREADS), 0, stream, logits, V, ld, out);
    return mynah_check_launch("argmax");
}

// logits [B, ld] are overwritten. params (device): temp, top_p, min_p, top_k,
// repeat, freq, presence as floats; they are read on the device so that a
// captured step serves every setting. rng: one 64-bit generator state per
// slot; slots [B] maps rows to slots (null: row b is slot b; a negative slot
// marks a padding row). out [B] receives the token ids.
// part_val, part_idx: scratch of B * mynah_argmax_parts() entries each for the two-step maximum, or null.
MYNAH_API int mynah_sample(float* logits, int B, int V, int ld, const float* params,
                           unsigned long long* rng, const int* slots, int* out,
                           float* part_val, int* part_idx, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && V > 0 && ld >= V, "sample: bad sizes B=%d V=%d ld=%d", B, V, ld);
    MYNAH_REQUIRE(params != nullptr && rng != nullptr, "sample: parameters and generator states are required");
    MYNAH_REQUIRE((part_val == nullptr) == (part_idx == nullptr) && B <= 65535, "sample: bad scratch or too many rows");
    if (part_val != nullptr) {
        mynah_launch(argmax_partial_kernel, dim3(ARGMAX_PARTS, B), dim3(PART_THREADS), 0, stream, (const float*)logits, V, ld, slots, part_val, part_idx);
        if (mynah_check_launch("argmax_partial")) return -1;
    }
    if (part_val != nullptr && V >= ROW_CTAS * 4096) {
        // a large vocabulary: a cluster of ROW_CTAS CTAs a row
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)B * ROW_CTAS);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = ROW_CTAS;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_top_k_kernel<ROW_CTAS>, logits, V, ld, params, rng, slots, out,
                                           (const float*)part_val, (const int*)part_idx);
        if (e == cudaSuccess)
            e = cudaLaunchKernelEx(&cfg, sample_kernel<ROW_CTAS>, logits, V, ld, params, rng, slots, out,
                                   (const float*)part_val, (const int*)part_idx);
        if (e != cudaSuccess) return mynah_fail("sample: %s", cudaGetErrorString(e));
        return mynah_check_launch("sample");
    }
    mynah_launch(sample_top_k_kernel<1>, dim3(B), dim3(THREADS), 0, stream, logits, V, ld, params, rng, slots, out,
                 (const float*)part_val, (const int*)part_idx);
    if (mynah_check_launch("sample (top-k)")) return -1;
    mynah_launch(sample_kernel<1>, dim3(B), dim3(THREADS), 0, stream, logits, V, ld, params, rng, slots, out,
                 (const float*)part_val, (const int*)part_idx);
    return mynah_check_launch("sample");
}

MYNAH_API int mynah_argmax_parts() { return ARGMAX_PARTS; }

MYNAH_API int mynah_apply_penalties(float* logits, int B, int V, int ld, const int* ring, const int* ring_n,
                                    int window, const int* slots, const float* params, cudaStream_t stream) {
    if (B == 0 || window == 0) return 0;
    mynah_launch(penalties_kernel, dim3(ceil_div(B, 64)), dim3(64), 0, stream, logits, B, V, ld, ring, ring_n, window, slots, params);
    return mynah_check_launch("apply_penalties");
}

namespace {
// After a sampled decode step: the sampled token becomes the sequence's next
// input, one position further on.
__global__ void decode_advance_kernel(int* __restrict__ tokens, const int* __restrict__ sampled,
                                      int* __restrict__ tok_pos, int* __restrict__ kv_len,
                                      const int* __restrict__ slots, int B) {
    griddep_launch();
    griddep_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B || slots[b] < 0) return;
    tokens[b] = sampled[b];
    tok_pos[b] += 1;
    kv_len[b] += 1;
}
}  // namespace

MYNAH_API int mynah_decode_advance(int* tokens, const int* sampled, int* tok_pos, int* kv_len, const int* slots,
                                   int B, cudaStream_t stream) {
    if (B == 0) return 0;
    mynah_launch(decode_advance_kernel, dim3(ceil_div(B, 64)), dim3(64), 0, stream, tokens, sampled, tok_pos, kv_len, slots, B);
    return mynah_check_launch("decode_advance");
}

MYNAH_API int mynah_sampler_accept(const int* tokens, int B, int* ring, int* ring_n, int* ring_head, int window,
                                   const int* slots, const float* params, cudaStream_t stream) {
    if (B == 0 || window == 0) return 0;
    mynah_launch(accept_kernel, dim3(ceil_div(B, 64)), dim3(64), 0, stream, tokens, B, ring, ring_n, ring_head, window, slots, params);
    return mynah_check_launch("sampler_accept");
}
