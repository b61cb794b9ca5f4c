// Row-wise kernels around the matrix products: token embedding, RMSNorm with
// the residual add folded in, SwiGLU, and the plain residual add.
//
// The residual stream is fp32 in both precisions. Sums of squares and the
// scale are fp32; the order of every sum is fixed by the thread layout, so a
// row's result does not depend on which other rows share the launch.
#include "common.cuh"
#include "head_prep.cuh"

// ------------------------------------------------------------- embedding
// x[t, :] = E[token_t, :]           (mynah-slm src/arch_qwen3.c:186: no scaling)
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ x, int D, int V) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* out = x + (size_t)t * D;
    if (tok < 0 || tok >= V) {      // refused on the host already; never read out of range
        for (int i = threadIdx.x; i < D; i += blockDim.x) out[i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)tok * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[i] = to_f32(row[i]);
}

MYNAH_API int mynah_embed_gather(const void* table, int table_dtype, const int* tokens, float* x,
                                 int T, int D, int V, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && D > 0 && V > 0, "embed_gather: bad sizes T=%d D=%d V=%d", T, D, V);
    const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : 64);
    if (table_dtype == MYNAH_F32)
        mynah_launch(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, tokens, x, D, V);
    else if (table_dtype == MYNAH_BF16)
        mynah_launch(embed_gather_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)table, tokens, x, D, V);
    else
        return mynah_fail("embed_gather: unsupported table dtype %d", table_dtype);
    return mynah_check_launch("embed_gather");
}

// --------------------------------------------------------------- RMSNorm
// v = x[r] (+ delta[r]);  x[r] = v when delta is given and every row is taken (no `rows`);
// out[i] = (v * s) * w   with   s = 1 / sqrt(mean(v^2) + eps)
// (mynah-slm src/kernels.c:118-128; plain gain, not 1+w). `rows`, when given,
// selects the rows to normalise (the rows whose logits are wanted); out then
// has one row per selected row.
template <typename TA>
__global__ void rmsnorm_kernel(float* __restrict__ x, const TA* __restrict__ delta, VecRef w,
                               const int* __restrict__ rows, TA* __restrict__ out, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * D;
    const TA* dr = delta ? delta + (size_t)r * D : nullptr;
    // the sum is kept in x when every row is normalised once; selected rows may repeat (several CTAs on one
    // row), so with a selection x is only read
    const bool keep = dr != nullptr && rows == nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v += to_f32(dr[i]);
            if (keep) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
    TA* o = out + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = xr[i];
        if (dr && !keep) v += to_f32(dr[i]);
        o[i] = from_f32<TA>((v * s) * w.at(i));
    }
}

// The same norm with the row kept in registers: four consecutive elements per thread, one pass over
// memory. Taken when D is a multiple of 4 and fits (D <= 4 * 1024).
template <typename TA>
__global__ void rmsnorm_vec4_kernel(float* __restrict__ x, const TA* __restrict__ delta, VecRef w,
                                    const int* __restrict__ rows, TA* __restrict__ out, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * D;
    const int i = threadIdx.x * 4;
    const bool on = i < D;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (on) {
        v = *reinterpret_cast<const float4*>(xr + i);
        if (delta) {
            const TA* dr = delta + (size_t)r * D + i;
            v.x += to_f32(dr[0]); v.y += to_f32(dr[1]); v.z += to_f32(dr[2]); v.w += to_f32(dr[3]);
            if (rows == nullptr) *reinterpret_cast<float4*>(xr + i) = v;     // (selected rows may repeat: x is only read)
        }
    }
    float ss = (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
    if (on) {
        TA* o = out + (size_t)blockIdx.x * D + i;
        o[0] = from_f32<TA>((v.x * s) * w.at(i));
        o[1] = from_f32<TA>((v.y * s) * w.at(i + 1));
        o[2] = from_f32<TA>((v.z * s) * w.at(i + 2));
        o[3] = from_f32<TA>((v.w * s) * w.at(i + 3));
    }
}

// Eight consecutive elements per thread: the row, the pending delta, the gains and the result all move as 16-byte
// vectors. Taken when D is a multiple of 8 and fits (D <= 8 * 1024), for any number of rows, so that a row's sum
// has the same order in every step.
template <typename TA>
__global__ void rmsnorm_vec8_kernel(float* __restrict__ x, const TA* __restrict__ delta, VecRef w,
                                    const int* __restrict__ rows, TA* __restrict__ out, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * D;
    const int i = threadIdx.x * 8;
    const bool on = i < D;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (on) {
        load8(xr + i, v);
        if (delta) {
            float d[8];
            load8(delta + (size_t)r * D + i, d);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] += d[j];
            if (rows == nullptr) store8(xr + i, v);        // (selected rows may repeat: x is only read)
        }
    }
    float ss = ((v[0] * v[0] + v[1] * v[1]) + (v[2] * v[2] + v[3] * v[3])) + ((v[4] * v[4] + v[5] * v[5]) + (v[6] * v[6] + v[7] * v[7]));
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
    if (on) {
        float g[8];
        load_gain8(w, i, g);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = (v[j] * s) * g[j];
        store8(out + (size_t)blockIdx.x * D + i, v);
    }
}

MYNAH_API int mynah_rmsnorm(float* x, const void* delta, const void* w, int w_dtype, const int* rows,
                            void* out, int act_dtype, int n_rows, int D, float eps, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    MYNAH_REQUIRE(n_rows > 0 && D > 0, "rmsnorm: bad sizes rows=%d D=%d", n_rows, D);
    MYNAH_REQUIRE(w_dtype == MYNAH_F32 || w_dtype == MYNAH_BF16, "rmsnorm: unsupported gain dtype %d", w_dtype);
    const VecRef wr{w, w_dtype};
    const bool aligned16 = (((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (D % 8 == 0 && D <= 8192 && D >= 256 && aligned16) {
        const int threads = ((D / 8 + 31) / 32) * 32;
        if (act_dtype == MYNAH_F32)
            mynah_launch(rmsnorm_vec8_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, (const float*)delta, wr, rows, (float*)out, D, eps);
        else if (act_dtype == MYNAH_BF16)
            mynah_launch(rmsnorm_vec8_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, (const bf16*)delta, wr, rows, (bf16*)out, D, eps);
        else
            return mynah_fail("rmsnorm: unsupported activation dtype %d", act_dtype);
        return mynah_check_launch("rmsnorm");
    }
    if (D % 4 == 0 && D <= 4096 && D >= 128) {
        const int threads = ((D / 4 + 31) / 32) * 32;
        if (act_dtype == MYNAH_F32)
            mynah_launch(rmsnorm_vec4_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, (const float*)delta, wr, rows, (float*)out, D, eps);
        else if (act_dtype == MYNAH_BF16)
            mynah_launch(rmsnorm_vec4_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, (const bf16*)delta, wr, rows, (bf16*)out, D, eps);
        else
            return mynah_fail("rmsnorm: unsupported activation dtype %d", act_dtype);
        return mynah_check_launch("rmsnorm");
    }
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : (D >= 128 ? 128 : 32));
    if (act_dtype == MYNAH_F32)
        mynah_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, (const float*)delta, wr, rows, (float*)out, D, eps);
    else if (act_dtype == MYNAH_BF16)
        mynah_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, (const bf16*)delta, wr, rows, (bf16*)out, D, eps);
    else
        return mynah_fail("rmsnorm: unsupported activation dtype %d", act_dtype);
    return mynah_check_launch("rmsnorm");
}

// ----------------------------------------------------------- residual add
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ x, const TA* __restrict__ delta, size_t n) {
    griddep_launch();
    griddep_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += to_f32(delta[i]);          // mynah-slm src/kernels.c:222-224
}

MYNAH_API int mynah_residual_add(float* x, const void* delta, int act_dtype, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    const unsigned blocks = (unsigned)ceil_div_ll(n, 256);
    if (act_dtype == MYNAH_F32)
        mynah_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)delta, (size_t)n);
    else if (act_dtype == MYNAH_BF16)
        mynah_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (const bf16*)delta, (size_t)n);
    else
        return mynah_fail("residual_add: unsupported activation dtype %d", act_dtype);
    return mynah_check_launch("residual_add");
}

// ----------------------------------------------------------------- SwiGLU
// a = (g * sigmoid(g)) * u with the sigmoid that never exponentiates a
// positive argument (mynah-slm src/kernels.c:193-205). gate_up is [T, 2F]:
// gate in columns [0, F), up in [F, 2F).
__device__ __forceinline__ float stable_sigmoid(float v) {
    // e^-|v| never overflows; the select keeps both branches of the reference's stable form exact
    const float e = expf(-fabsf(v));
    return (v >= 0.f ? 1.0f : e) / (1.0f + e);
}

template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gate_up, TA* __restrict__ out, int F) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= F) return;
    const TA* row = gate_up + (size_t)t * 2 * F;
    const float g = to_f32(row[i]), u = to_f32(row[F + i]);
    out[(size_t)t * F + i] = from_f32<TA>((g * stable_sigmoid(g)) * u);
}

// Eight elements per thread (16-byte loads and stores) when F is a multiple of 8.
template <typename TA>
__global__ void swiglu_vec8_kernel(const TA* __restrict__ gate_up, TA* __restrict__ out, int F) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (i >= F) return;
    const TA* row = gate_up + (size_t)t * 2 * F;
    float g[8], u[8], o[8];
    load8(row + i, g);
    load8(row + F + i, u);
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = (g[j] * stable_sigmoid(g[j])) * u[j];
    store8(out + (size_t)t * F + i, o);
}

MYNAH_API int mynah_swiglu(const void* gate_up, void* out, int act_dtype, int T, int F, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && F > 0, "swiglu: bad sizes T=%d F=%d", T, F);
    MYNAH_REQUIRE(ceil_div(F, 256) <= 65535, "swiglu: width %d exceeds one launch", F);
    if (F % 8 == 0) {
        const dim3 vgrid(T, ceil_div(F / 8, 128));
        if (act_dtype == MYNAH_F32)
            mynah_launch(swiglu_vec8_kernel<float>, vgrid, dim3(128), 0, stream, (const float*)gate_up, (float*)out, F);
        else if (act_dtype == MYNAH_BF16)
            mynah_launch(swiglu_vec8_kernel<bf16>, vgrid, dim3(128), 0, stream, (const bf16*)gate_up, (bf16*)out, F);
        else
            return mynah_fail("swiglu: unsupported activation dtype %d", act_dtype);
        return mynah_check_launch("swiglu");
    }
    const dim3 grid(T, ceil_div(F, 256));
    if (act_dtype == MYNAH_F32)
        mynah_launch(swiglu_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)gate_up, (float*)out, F);
    else if (act_dtype == MYNAH_BF16)
        mynah_launch(swiglu_kernel<bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, F);
    else
        return mynah_fail("swiglu: unsupported activation dtype %d", act_dtype);
    return mynah_check_launch("swiglu");
}
