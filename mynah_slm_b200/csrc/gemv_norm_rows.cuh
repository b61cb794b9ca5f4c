// The norm prologue of the decode products: the rows of the residual stream, with the pending delta added, are
// normalised by every CTA into its shared memory as bf16, so that neither the sum nor the normalised rows make a
// trip through global memory and no norm kernel stands between two products.
//
// out = (v * s) * w with v = x (+ delta), s = 1 / sqrt(mean(v^2) + eps) (mynah-slm src/kernels.c:118-128).
//
// A warp takes a row (rows warp, warp + 8, ... of the batch). A lane takes the row's chunks of eight elements
// lane, lane + 32, ...: all of their loads are issued before anything is used (a chunk is two 16-byte loads of the
// fp32 row and one of the bf16 delta), so a row costs one round trip to L2 while it has at most 1,024 elements,
// which then stay in registers until the scale is known; longer rows are read a second time. The sum of squares
// is added up in a fixed order (a lane's chunks in order, then the warp's butterfly), so a row's result does not
// depend on what else is in the batch. CTA 0 also writes the updated residual.
#pragma once
#include "common.cuh"
#include "head_prep.cuh"

struct NormRowsArgs {
    const float* x_res;               // [M, K]
    const bf16* delta;                // [M, K] or null
    float* x_res_out;                 // [M, K], written when delta is given (never the same memory as x_res)
    VecRef gain;
    float eps;
    int M, K;
};

__device__ __forceinline__ void add_delta8(float (&v)[8], const uint4& d) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        v[2 * j] += __low2float(h[j]);
        v[2 * j + 1] += __high2float(h[j]);
    }
}

__device__ __forceinline__ float sum_squares8(const float (&v)[8]) {
    return ((v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3])) + ((v[4] * v[4] + v[5] * v[5]) + (v[6] * v[6] + v[7] * v[7]));
}

// xs: [rows][ldx] bf16 in shared memory, ldx a multiple of 8. All warps of the CTA call this; K a multiple of 8.
template <int WARPS_>
__device__ __forceinline__ void norm_rows_to_smem(const NormRowsArgs& a, bf16* xs, int ldx, int warp, int lane) {
    constexpr int BATCH = 4;                                         // chunks a lane has in flight
    const int K = a.K, nch = K >> 3;
    const bool write_back = a.delta != nullptr && blockIdx.x == 0;
    for (int m = warp; m < a.M; m += WARPS_) {
        const float* xr = a.x_res + (size_t)m * K;
        const bf16* dr = a.delta != nullptr ? a.delta + (size_t)m * K : nullptr;
        float* xo = a.x_res_out + (size_t)m * K;
        bf16* out = xs + (size_t)m * ldx;
        float ss = 0.f;
        if (nch <= BATCH * 32) {                                     // uniform: the row stays in registers
            float v[BATCH][8];
            uint4 d[BATCH];
#pragma unroll
            for (int c = 0; c < BATCH; c++) {
                const int ch = lane + c * 32;
                if (ch < nch) {
                    load8(xr + ch * 8, v[c]);
                    d[c] = dr != nullptr ? *reinterpret_cast<const uint4*>(dr + ch * 8) : make_uint4(0u, 0u, 0u, 0u);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[c][j] = 0.f;
                    d[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int c = 0; c < BATCH; c++) {
                add_delta8(v[c], d[c]);                              // (bf16 zero adds nothing)
                ss += sum_squares8(v[c]);
                if (write_back && lane + c * 32 < nch) store8(xo + (lane + c * 32) * 8, v[c]);
            }
            ss = warp_sum(ss);
            const float s = 1.0f / sqrtf(ss / (float)K + a.eps);
#pragma unroll
            for (int c = 0; c < BATCH; c++) {
                const int ch = lane + c * 32;
                if (ch < nch) {
                    float g[8];
                    load_gain8(a.gain, ch * 8, g);
#pragma unroll
                    for (int j = 0; j < 8; j++) v[c][j] = (v[c][j] * s) * g[j];
                    store8(out + ch * 8, v[c]);
                }
            }
        } else {
            for (int c0 = lane; c0 < nch; c0 += BATCH * 32) {
                float v[BATCH][8];
                uint4 d[BATCH];
#pragma unroll
                for (int c = 0; c < BATCH; c++) {
                    const int ch = c0 + c * 32;
                    if (ch < nch) {
                        load8(xr + ch * 8, v[c]);
                        d[c] = dr != nullptr ? *reinterpret_cast<const uint4*>(dr + ch * 8) : make_uint4(0u, 0u, 0u, 0u);
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; j++) v[c][j] = 0.f;
                        d[c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
#pragma unroll
                for (int c = 0; c < BATCH; c++) {
                    add_delta8(v[c], d[c]);
                    ss += sum_squares8(v[c]);
                    if (write_back && c0 + c * 32 < nch) store8(xo + (c0 + c * 32) * 8, v[c]);
                }
            }
            ss = warp_sum(ss);
            const float s = 1.0f / sqrtf(ss / (float)K + a.eps);
            for (int c0 = lane; c0 < nch; c0 += BATCH * 32) {
                float v[BATCH][8];
                uint4 d[BATCH];
#pragma unroll
                for (int c = 0; c < BATCH; c++) {
                    const int ch = c0 + c * 32;
                    if (ch < nch) {
                        load8(xr + ch * 8, v[c]);
                        d[c] = dr != nullptr ? *reinterpret_cast<const uint4*>(dr + ch * 8) : make_uint4(0u, 0u, 0u, 0u);
                    } else {
                        d[c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
#pragma unroll
                for (int c = 0; c < BATCH; c++) {
                    const int ch = c0 + c * 32;
                    if (ch < nch) {
                        add_delta8(v[c], d[c]);
                        float g[8];
                        load_gain8(a.gain, ch * 8, g);
#pragma unroll
                        for (int j = 0; j < 8; j++) v[c][j] = (v[c][j] * s) * g[j];
                        store8(out + ch * 8, v[c]);
                    }
                }
            }
        }
    }
}
