// Position encoding and the write into the cache, fused with the per-head
// norm: one pass over the projected q/k/v of a step.
//
//   q head: RMSNorm over head_dim (optional) -> split-half rotation (optional)
//           -> back in place, for the attention kernel
//   k head: same norm and rotation -> the sequence's page at its position
//   v head: copied to the sequence's page
//
// Norm before rotation, one gain vector of head_dim shared by all heads,
// V neither normed nor rotated (mynah-slm src/arch_qwen3.c:208-218,
// src/kernels.c:130-137, :173-189). Norm, angles and rotation are fp32; the
// rotation table is built in double like the reference's
// (src/kernels.c:154-162) and stored as float. Values are rounded to the
// activation or cache type once, when stored.
#include "layout.cuh"
#include "head_prep.cuh"

namespace {

// cos/sin[p][i] = (float) cos/sin(p * theta^(-2i/rotary_dim)), in double.
__global__ void rope_table_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t,
                                  int n_pos, int half, double theta, int rotary_dim) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_pos * half) return;
    const int p = (int)(idx / half), i = (int)(idx % half);
    const double inv = 1.0 / pow(theta, (2.0 * (double)i) / (double)rotary_dim);
    const double a = (double)p * inv;
    cos_t[idx] = (float)cos(a);
    sin_t[idx] = (float)sin(a);
}

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS = 4;

struct QkvArgs {
    int T, H, KV, HD, ld;          // ld: row stride of qkv in elements
    int rotary_dim, n_pos;         // rotation over the first rotary_dim dims; table rows
    float eps;
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(TA* __restrict__ qkv, VecRef q_gain, VecRef k_gain,
                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                          PageTable pt, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                          QkvArgs a, int* __restrict__ status) {
    __shared__ float stage[WARPS][MAX_HEAD_DIM];
    griddep_wait();
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = k_cache != nullptr ? a.H + 2 * a.KV : a.H;   // without storage only q is touched
    const long long unit = (long long)blockIdx.x * WARPS + warp;
    if (unit >= (long long)a.T * heads) return;
    const int t = (int)(unit / heads), h = (int)(unit % heads);
    const int seq = tok_seq[t];
    if (seq < 0) return;                                   // padding token: nothing to do
    const int pos = tok_pos[t];
    const bool is_q = h < a.H, is_k = !is_q && h < a.H + a.KV;
    const int kvh = is_q ? 0 : (is_k ? h - a.H : h - a.H - a.KV);
    TA* src = qkv + (size_t)t * a.ld + (size_t)h * a.HD;

    TC* dst = nullptr;
    if (!is_q) {
        TC* cache = is_k ? k_cache : v_cache;
        const int page = page_of(pt, seq, pos);
        if (page < 0) {
            if (lane == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
            return;
        }
        dst = cache + (((size_t)page * a.KV + kvh) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.HD;
    }

    if (!is_q && !is_k) {                                  // V: copy
        for (int i = lane; i < a.HD; i += 32) dst[i] = from_f32<TC>(to_f32(src[i]));
        return;
    }

    float* s = stage[warp];
    const VecRef gain = is_q ? q_gain : k_gain;
    float ss = 0.f;
    for (int i = lane; i < a.HD; i += 32) {
        const float v = to_f32(src[i]);
        s[i] = v;
        ss += v * v;
    }
    if (gain.p != nullptr) {
        ss = warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss / (float)a.HD + a.eps);
        for (int i = lane; i < a.HD; i += 32) s[i] = s[i] * (sc * gain.at(i));   // x *= s*w, kernels.c:135
    }
    __syncwarp();

    const int half = a.rotary_dim / 2;
    const bool rotate = cos_t != nullptr && half > 0;
    if (rotate && (pos < 0 || pos >= a.n_pos)) {
        if (lane == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    if (rotate) {
        const float* c = cos_t + (size_t)pos * half;
        const float* sn = sin_t + (size_t)pos * half;
        for (int i = lane; i < half; i += 32) {
            const float x0 = s[i], x1 = s[i + half];
            const float o0 = x0 * c[i] - x1 * sn[i];       // kernels.c:181-187
            const float o1 = x1 * c[i] + x0 * sn[i];
            if (is_q) {
                src[i] = from_f32<TA>(o0);
                src[i + half] = from_f32<TA>(o1);
            } else {
                dst[i] = from_f32<TC>(o0);
                dst[i + half] = from_f32<TC>(o1);
            }
        }
    }
    for (int i = (rotate ? a.rotary_dim : 0) + lane; i < a.HD; i += 32) {
        if (is_q) src[i] = from_f32<TA>(s[i]);
        else dst[i] = from_f32<TC>(s[i]);
    }
}

// The same pass for head sizes 32, 64, 128 and 256 with the whole head rotated (or none of it): a head lies
// across head_dim / 8 lanes, eight consecutive elements a lane, so a warp works on 32 / (head_dim / 8) heads
// with every instruction, nothing goes through shared memory and every access is a 16-byte vector (two for
// fp32). A warp takes `hpw` consecutive heads of one token, four passes at a time with their loads in flight
// together; the token's position, page and rotation row are fetched once for all of them.
template <typename T, int HD>
__global__ void __launch_bounds__(WARPS * 32, sizeof(T) == 2 ? 7 : 4)
qk_norm_rope_store_fast_kernel(T* __restrict__ qkv, VecRef q_gain, VecRef k_gain,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                               const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                               PageTable pt, T* __restrict__ k_cache, T* __restrict__ v_cache,
                               QkvArgs a, int hpw, int* __restrict__ status) {
    griddep_launch();
    griddep_wait();
    constexpr int LPH = HeadLanes<HD>::LPH, HPW = HeadLanes<HD>::HPW;
    constexpr int BATCH = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = k_cache != nullptr ? a.H + 2 * a.KV : a.H;
    const int groups = (heads + hpw - 1) / hpw;
    const long long unit = (long long)blockIdx.x * WARPS + warp;
    if (unit >= (long long)a.T * groups) return;
    const int t = (int)(unit / groups), h0 = (int)(unit % groups) * hpw, h1 = min(heads, h0 + hpw);
    const int seq = tok_seq[t];
    if (seq < 0) return;
    const int pos = tok_pos[t];
    const int sub = lane / LPH, li = lane % LPH;           // which of the warp's heads, and where in it
    T* row = qkv + (size_t)t * a.ld + li * 8;
    // the first passes' loads go out before anything that depends on the position
    Raw8<T> in[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; i++) {
        const int h = h0 + i * HPW + sub;
        if (h < h1) in[i].load(row + (size_t)h * HD);
    }
    const bool rotate = cos_t != nullptr;
    if (rotate && (pos < 0 || pos >= a.n_pos)) {
        if (lane == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    float c[8], sn[8];
    if (rotate) load_rotation<HD>(cos_t, sin_t, pos, lane, c, sn);
    const bool has_gain = q_gain.p != nullptr;
    size_t cache_row = 0;
    if (h1 > a.H) {                                        // some head of this warp goes to the cache
        const int page = page_of(pt, seq, pos);
        if (page < 0) {
            if (lane == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
            return;
        }
        cache_row = (size_t)page * a.KV * PAGE_TOKENS + pos % PAGE_TOKENS;
    }
    for (int hb = h0; hb < h1; hb += BATCH * HPW) {
        if (hb != h0) {
#pragma unroll
            for (int i = 0; i < BATCH; i++) {
                const int h = hb + i * HPW + sub;
                if (h < h1) in[i].load(row + (size_t)h * HD);
            }
        }
#pragma unroll
        for (int i = 0; i < BATCH; i++) {
            if (hb + i * HPW >= h1) break;                 // uniform over the warp
            const int h = hb + i * HPW + sub;              // this lane group's head (may lie beyond the warp's heads)
            const bool mine = h < h1;
            if (hb + i * HPW >= a.H + a.KV) {              // uniform: a pass of V heads only is a copy of 16 bytes a lane
                if (mine) in[i].store(v_cache + (cache_row + (size_t)(h - a.H - a.KV) * PAGE_TOKENS) * HD + li * 8);
                continue;
            }
            const bool is_q = h < a.H, is_k = !is_q && h < a.H + a.KV;
            float v[8];
            in[i].to_f32(v);                               // (a lane group without a head works on whatever is there)
            if (mine && !is_q && !is_k) {                  // V: copy (no shuffles inside)
                const int kvh = h - a.H - a.KV;
                store8<T>(v_cache + (cache_row + (size_t)kvh * PAGE_TOKENS) * HD + li * 8, v);
            }
            // every lane takes part in the norm and the rotation; what is not a q or k head is dropped afterwards
            float g[8];                                    // the head's gains: a few hundred bytes that stay in L1
            if (has_gain) load_gain8(is_q ? q_gain : k_gain, li * 8, g);
            head_norm_rotate<HD>(v, has_gain, g, a.eps, rotate, c, sn, lane);
            if (mine && is_q) store8<T>(row + (size_t)h * HD, v);
            else if (mine && is_k) store8<T>(k_cache + (cache_row + (size_t)(h - a.H) * PAGE_TOKENS) * HD + li * 8, v);
        }
    }
}

template <typename T>
bool launch_fast(int HD, cudaStream_t stream, T* qkv, VecRef qg, VecRef kg, const float* cos_t,
                 const float* sin_t, const int* tok_seq, const int* tok_pos, PageTable pt, T* kc, T* vc, QkvArgs a, int* status) {
    if (HD != 32 && HD != 64 && HD != 128 && HD != 256) return false;
    // heads per warp: one pass while the step is small (latency matters), up to eight passes when there are many tokens
    // (a warp's set-up, the token's position, page and rotation row, is then shared by more heads: 2,048 tokens of 32
    // heads of 128 take 19.3, 13.9, 11.8, 10.8 and 13.2 us with 1, 2, 4, 8 and 16 passes)
    const int heads = kc != nullptr ? a.H + 2 * a.KV : a.H;
    const int per_pass = 32 / (HD / 8);
    const long long units1 = (long long)a.T * ((heads + per_pass - 1) / per_pass);
    int passes = 1;
    while (passes < 8 && units1 / passes > (long long)mynah_sm_count() * 16) passes *= 2;
    const int hpw = per_pass * passes;
    const int groups = (heads + hpw - 1) / hpw;
    const unsigned blocks = (unsigned)ceil_div_ll((long long)a.T * groups, WARPS);
    switch (HD) {
        case 32: mynah_launch(qk_norm_rope_store_fast_kernel<T, 32>, dim3(blocks), dim3(WARPS * 32), 0, stream, qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, kc, vc, a, hpw, status); return true;
        case 64: mynah_launch(qk_norm_rope_store_fast_kernel<T, 64>, dim3(blocks), dim3(WARPS * 32), 0, stream, qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, kc, vc, a, hpw, status); return true;
        case 128: mynah_launch(qk_norm_rope_store_fast_kernel<T, 128>, dim3(blocks), dim3(WARPS * 32), 0, stream, qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, kc, vc, a, hpw, status); return true;
        default: mynah_launch(qk_norm_rope_store_fast_kernel<T, 256>, dim3(blocks), dim3(WARPS * 32), 0, stream, qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, kc, vc, a, hpw, status); return true;
    }
}

}  // namespace

MYNAH_API int mynah_rope_table(float* cos_t, float* sin_t, int n_pos, int rotary_dim, double theta,
                               cudaStream_t stream) {
    MYNAH_REQUIRE(n_pos > 0 && rotary_dim > 0 && rotary_dim % 2 == 0,
                  "rope_table: rotary_dim %d must be positive and even", rotary_dim);
    const int half = rotary_dim / 2;
    const long long n = (long long)n_pos * half;
    rope_table_kernel<<<(unsigned)ceil_div_ll(n, 256), 256, 0, stream>>>(cos_t, sin_t, n_pos, half, theta, rotary_dim);
    return mynah_check_launch("rope_table");
}

// dtype: type of qkv and of the cache (the 32-bit path keeps both in fp32).
MYNAH_API int mynah_qk_norm_rope_store(
    void* qkv, int dtype, int T, int H, int KV, int HD, int ld,
    const void* q_gain, const void* k_gain, int gain_dtype, float eps,
    const float* cos_t, const float* sin_t, int rotary_dim, int n_pos,
    const int* tok_seq, const int* tok_pos,
    const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
    void* k_cache, void* v_cache, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && KV > 0 && HD > 0, "qk_norm_rope_store: bad sizes");
    MYNAH_REQUIRE(HD <= MAX_HEAD_DIM, "qk_norm_rope_store: head_dim %d exceeds %d", HD, MAX_HEAD_DIM);
    MYNAH_REQUIRE(rotary_dim % 2 == 0 && rotary_dim <= HD, "qk_norm_rope_store: rotary_dim %d does not fit head_dim %d", rotary_dim, HD);
    MYNAH_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "qk_norm_rope_store: K and V storage go together");
    const int heads = k_cache != nullptr ? H + 2 * KV : H;     // a run that reads another run's cache brings q only
    MYNAH_REQUIRE(ld >= heads * HD, "qk_norm_rope_store: row stride %d is smaller than the row", ld);
    const QkvArgs a{T, H, KV, HD, ld, cos_t ? rotary_dim : 0, n_pos, eps};
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const long long units = (long long)T * heads;
    const unsigned blocks = (unsigned)ceil_div_ll(units, WARPS);
    // the register-only kernel: the whole head rotated (or none of it), rows 16-byte aligned
    const bool fast_ok = (cos_t == nullptr || rotary_dim == HD) && ld % 8 == 0;
    if (fast_ok && dtype == MYNAH_F32 &&
        launch_fast<float>(HD, stream, (float*)qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, a, status))
        return mynah_check_launch("qk_norm_rope_store");
    if (fast_ok && dtype == MYNAH_BF16 &&
        launch_fast<bf16>(HD, stream, (bf16*)qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, a, status))
        return mynah_check_launch("qk_norm_rope_store");
    if (dtype == MYNAH_F32)
        mynah_launch(qk_norm_rope_store_kernel<float, float>, dim3(blocks), dim3(WARPS * 32), 0, stream,
            (float*)qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(qk_norm_rope_store_kernel<bf16, bf16>, dim3(blocks), dim3(WARPS * 32), 0, stream,
            (bf16*)qkv, qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, a, status);
    else
        return mynah_fail("qk_norm_rope_store: unsupported dtype %d", dtype);
    return mynah_check_launch("qk_norm_rope_store");
}
