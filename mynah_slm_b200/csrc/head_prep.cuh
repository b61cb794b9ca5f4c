// Per-head RMSNorm and split-half rotation of a head that lies across the lanes of a warp, shared by the
// rope/store pass and the one-launch decode attention so that both give a row the same bits.
//
// A head of HD elements takes LPH = HD / 8 lanes, eight consecutive elements a lane (one 16-byte load of
// bfloat16), so a warp holds 32 / LPH heads side by side and every instruction below works on all of them.
// The lanes of the first half of a head hold elements [0, HD/2), their rotation partners are LPH / 2 lanes on.
//
// Norm before rotation, one gain per head position shared by all heads (mynah-slm src/arch_qwen3.c:208-218,
// src/kernels.c:130-137, :173-189): out = (x * (1 / sqrt(mean(x^2) + eps))) * w, then
// x[i] = a c - b s, x[i + HD/2] = b c + a s.
#pragma once
#include "common.cuh"

template <int HD>
struct HeadLanes {
    static_assert(HD == 32 || HD == 64 || HD == 128 || HD == 256, "a head of 8 * (4, 8, 16 or 32) elements");
    static constexpr int LPH = HD / 8;            // lanes a head
    static constexpr int HPW = 32 / LPH;          // heads a warp
};

// The lane's eight cosines and sines of the token's position. The first half's lanes and their partners read the
// same entries; the first half's lanes get the sines negated, so that both halves rotate with one expression.
template <int HD>
__device__ __forceinline__ void load_rotation(const float* __restrict__ cos_t, const float* __restrict__ sin_t, int pos, int lane,
                                              float (&c)[8], float (&sn)[8]) {
    constexpr int LPH = HeadLanes<HD>::LPH;
    const int i0 = ((lane % LPH) % (LPH / 2)) * 8;
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)pos * (HD / 2) + i0);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)pos * (HD / 2) + i0);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    if ((lane % LPH) < LPH / 2) {
#pragma unroll
        for (int j = 0; j < 8; j++) sn[j] = -sn[j];
    }
}

// Eight consecutive gains (stored as fp32 or bfloat16) starting at element i0, a multiple of 8.
__device__ __forceinline__ void load_gain8(VecRef g, int i0, float (&out)[8]) {
    if (g.dtype == MYNAH_F32) {
        const float4 a = reinterpret_cast<const float4*>(static_cast<const float*>(g.p) + i0)[0];
        const float4 b = reinterpret_cast<const float4*>(static_cast<const float*>(g.p) + i0)[1];
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    } else {
        const uint4 r = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(g.p) + i0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[2 * j] = __low2float(h[j]);
            out[2 * j + 1] = __high2float(h[j]);
        }
    }
}

// All 32 lanes must call this together (it shuffles); lanes without a head pass anything and ignore the result.
// `c` and `sn` come from load_rotation.
template <int HD>
__device__ __forceinline__ void head_norm_rotate(float (&v)[8], bool norm, const float (&g)[8], float eps,
                                                 bool rotate, const float (&c)[8], const float (&sn)[8], int lane) {
    constexpr int LPH = HeadLanes<HD>::LPH;
    if (norm) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) ss += v[j] * v[j];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float sc = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = v[j] * (sc * g[j]);
    }
    if (rotate) {
        // first half: a c - b s; second half: b c + a s; `sn` carries the sign (load_rotation). One rounded
        // product and one fused multiply-add, written out so that every user rounds alike.
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], LPH / 2);
            v[j] = fmaf(other, sn[j], __fmul_rn(v[j], c[j]));
        }
    }
}

// Eight consecutive elements of a row as they are stored (kept packed while their load is in flight).
template <typename T>
struct Raw8 {
    uint4 q[sizeof(T) == 2 ? 1 : 2];
    __device__ __forceinline__ void load(const T* p) {
        q[0] = reinterpret_cast<const uint4*>(p)[0];
        if (sizeof(T) != 2) q[sizeof(T) == 2 ? 0 : 1] = reinterpret_cast<const uint4*>(p)[1];
    }
    __device__ __forceinline__ void store(T* p) const {
        reinterpret_cast<uint4*>(p)[0] = q[0];
        if (sizeof(T) != 2) reinterpret_cast<uint4*>(p)[1] = q[sizeof(T) == 2 ? 0 : 1];
    }
    __device__ __forceinline__ void to_f32(float (&v)[8]) const {
        if (sizeof(T) == 2) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[0]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[2 * j] = __low2float(h[j]);
                v[2 * j + 1] = __high2float(h[j]);
            }
        } else {
            const float* f = reinterpret_cast<const float*>(&q[0]);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = f[j];
        }
    }
};

// Eight consecutive elements of a row, as fp32, and back (bfloat16: one 16-byte access; fp32: two).
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
    if (sizeof(T) == 2) {
        const uint4 r = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[2 * j] = __low2float(h[j]);
            v[2 * j + 1] = __high2float(h[j]);
        }
    } else {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]) {
    if (sizeof(T) == 2) {
        uint4 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    } else {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}
