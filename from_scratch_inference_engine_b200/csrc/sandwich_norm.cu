// RMS norms on both sides of a sublayer ("sandwich" arrangement) in one pass over the row, and
// the gated activation of feed-forwards whose gate is not SiLU.
//
//   norm_add_norm:   d = delta[s] / sqrt(mean(delta[s]^2) + eps_d) * gain_d      (the sublayer's output, normed)
//                    v = x[s] + d;  if write_x: x[s] = v                          (the 32-bit residual sum)
//                    y[r] = T( v / sqrt(mean(v^2) + eps) * gain )                 (the next sublayer's input)
//   with s = rows[r] (or r).  Without delta the first line falls away (a plain norm of x), without
//   y the last one (the sum alone).  All statistics, both gains and the sum are 32-bit whatever
//   the storage type T of delta and y.
//
//   gated_act:       act[t, i] = f(gu[t, i]) * gu[t, inter + i],  f = SiLU or the tanh form of GELU,
//                    g/2 * (1 + tanh(0.7978845608 * (g + 0.044715 g^3))), in 32-bit.
#include "common.cuh"
#include <math.h>

namespace fsie {

// One block per row; thread i owns the 8-element chunks i, i + blockDim, ... (NCH at most), held in
// registers between the two reductions.  VEC = false: any width, one element at a time, the row
// kept in shared memory.
template <typename T, int NCH>
__global__ void norm_add_norm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                         const float* __restrict__ gain_d, const float* __restrict__ gain,
                                         T* __restrict__ y, const int* __restrict__ rows, int hidden,
                                         float eps_d, float eps, int write_x) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int chunks = hidden / 8;
    grid_dependency_wait();
    grid_dependents_go();
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * hidden;
    float v[NCH][8];
    if (delta) {
        const T* dr = delta + s * hidden;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < chunks) {
                load8(dr + c * 8, v[k]);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
            }
        }
        ss = block_sum(ss, scratch);
        const float scale_d = 1.0f / sqrtf(ss / (float)hidden + eps_d);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < chunks) {
                float xv[8], g[8];
                load8(xr + c * 8, xv);
                load8(gain_d + c * 8, g);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[k][e] = xv[e] + (v[k][e] * scale_d) * g[e];
                if (write_x) store8(xr + c * 8, v[k]);
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < chunks) load8(xr + c * 8, v[k]);
        }
    }
    if (!y) return;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < chunks) {
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
        }
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c < chunks) {
            float g[8], o[8];
            load8(gain + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = (v[k][e] * scale) * g[e];
            store8(yr + c * 8, o);
        }
    }
}

template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                     const float* __restrict__ gain_d, const float* __restrict__ gain,
                                     T* __restrict__ y, const int* __restrict__ rows, int hidden,
                                     float eps_d, float eps, int write_x) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * hidden;
    float scale_d = 0.f;
    if (delta) {
        const T* dr = delta + s * hidden;
        float ss = 0.f;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float d = to_float(dr[c]);
            row_cache[c] = d;
            ss += d * d;
        }
        ss = block_sum(ss, scratch);
        scale_d = 1.0f / sqrtf(ss / (float)hidden + eps_d);
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = xr[c];
        if (delta) {
            v += (row_cache[c] * scale_d) * gain_d[c];
            if (write_x) xr[c] = v;
        }
        row_cache[c] = v;
        ss += v * v;
    }
    if (!y) return;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        yr[c] = from_float<T>((row_cache[c] * scale) * gain[c]);
}

__device__ __forceinline__ float gate_value(float z, int kind) {
    if (kind == 0) return z / (1.0f + expf(-z));
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(inner));
}

template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter,
                                 long long total, int kind) {
    grid_dependency_wait();
    grid_dependents_go();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gu[t * 2 * inter + i]);
    const float u = to_float(gu[t * 2 * inter + inter + i]);
    act[idx] = from_float<T>(gate_value(g, kind) * u);
}

template <typename T>
__global__ void gated_act_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter,
                                     long long chunks, int kind) {
    grid_dependency_wait();
    grid_dependents_go();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= chunks) return;
    const int per_row = inter / 8;
    const long long t = idx / per_row;
    const int i = (int)(idx - t * per_row) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * inter + i, g);
    load8(gu + t * 2 * inter + inter + i, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = gate_value(g[e], kind) * u[e];
    store8(act + t * inter + i, o);
}

template <typename T>
static int norm_add_norm_launch(float* x, const void* delta, const float* gain_d, const float* gain,
                                void* y, const int* rows, int num_rows, int hidden, float eps_d,
                                float eps, int write_x, cudaStream_t stream) {
    const bool aligned = ((((size_t)x) | ((size_t)delta) | ((size_t)y) | ((size_t)gain) | ((size_t)gain_d)) & 31) == 0;
    if (hidden % 8 == 0 && aligned && hidden <= 16384) {
        const int chunks = hidden / 8;
        const int threads = chunks >= 512 ? 512 : (chunks >= 256 ? 256 : (chunks >= 128 ? 128 : (chunks + 31) / 32 * 32));
        const int nch = (chunks + threads - 1) / threads;
#define FSIE_NAN(N)                                                                                       \
    return launch_dependent(norm_add_norm_vec_kernel<T, N>, dim3(num_rows), dim3(threads), 0, stream, x,   \
                            (const T*)delta, gain_d, gain, (T*)y, rows, hidden, eps_d, eps, write_x)
        if (nch <= 1) FSIE_NAN(1);
        if (nch <= 2) FSIE_NAN(2);
        FSIE_NAN(4);
#undef FSIE_NAN
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(norm_add_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    norm_add_norm_kernel<T><<<num_rows, 256, smem, stream>>>(x, (const T*)delta, gain_d, gain, (T*)y, rows,
                                                            hidden, eps_d, eps, write_x);
    return FSIE_LAUNCH_CHECK();
}

// x[s] += a1 * d1[s] + a2 * d2[s] (either may be null); y[r] = T( x[s] / sqrt(mean(x[s]^2) + eps) * gain ).
// The outputs of two mixers that run side by side, each with its weight, meet the 32-bit residual
// stream here without being summed in the storage type first.  VEC: width a multiple of 8, rows on
// 16 bytes, eight columns per thread and trip.
template <typename T, bool VEC>
__global__ void scaled_sum_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ d1, float a1,
                                          const T* __restrict__ d2, float a2, const float* __restrict__ gain,
                                          T* __restrict__ y, const int* __restrict__ rows, int hidden,
                                          float eps, int write_x) {
    extern __shared__ __align__(16) float ssr_row[];
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * hidden;
    const T* p1 = d1 ? d1 + s * hidden : nullptr;
    const T* p2 = d2 ? d2 + s * hidden : nullptr;
    constexpr int STEP = VEC ? 8 : 1;
    float ss = 0.f;
    for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], d[8];
            load8(xr + c, v);
            if (p1) {
                load8(p1 + c, d);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = fmaf(a1, d[e], v[e]);
            }
            if (p2) {
                load8(p2 + c, d);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = fmaf(a2, d[e], v[e]);
            }
            if (write_x) store8(xr + c, v);
            store8(ssr_row + c, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
        } else {
            float v = xr[c];
            if (p1) v = fmaf(a1, to_float(p1[c]), v);
            if (p2) v = fmaf(a2, to_float(p2[c]), v);
            if (write_x) xr[c] = v;
            ssr_row[c] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    if (!y) return;
    const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
    for (int c = threadIdx.x * STEP; c < hidden; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], g[8];
            load8(ssr_row + c, v);
            load8(gain + c, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (v[e] * scale) * g[e];
            store8(yr + c, v);
        } else {
            yr[c] = from_float<T>((ssr_row[c] * scale) * gain[c]);
        }
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// x float32 [*, hidden]; delta and y of storage type `dtype` (either may be null, not both);
// gain_d and gain float32 [hidden].  rows: the rows to work on (y row r comes from x row rows[r]).
int fsie_norm_add_norm(float* x, const void* delta, const float* gain_d, const float* gain, void* y,
                       const int* rows, int num_rows, int hidden, float eps_d, float eps, int write_x,
                       int dtype, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (hidden <= 0 || (!delta && !y) || (delta && !gain_d) || (y && !gain)) return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return norm_add_norm_launch<float>(x, delta, gain_d, gain, y, rows, num_rows, hidden, eps_d, eps,
                                           write_x, stream);
    return norm_add_norm_launch<bf16>(x, delta, gain_d, gain, y, rows, num_rows, hidden, eps_d, eps,
                                      write_x, stream);
}

// kind 0: SiLU, 1: GELU (tanh form)
int fsie_gated_act(const void* gu, void* act, long long tokens, int inter, int kind, int dtype,
                   cudaStream_t stream) {
    const long long total = tokens * inter;
    if (total <= 0) return 0;
    if (kind != 0 && kind != 1) return ERR_BAD_ARGUMENT;
    const int threads = 256;
    const bool aligned = ((((size_t)gu) | ((size_t)act)) & 31) == 0;
    if (inter % 8 == 0 && aligned) {
        const long long chunks = total / 8;
        const unsigned blocks = (unsigned)((chunks + threads - 1) / threads);
        if (dtype == DTYPE_F32)
            return launch_dependent(gated_act_vec_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                                    (const float*)gu, (float*)act, inter, chunks, kind);
        return launch_dependent(gated_act_vec_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream,
                                (const bf16*)gu, (bf16*)act, inter, chunks, kind);
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == DTYPE_F32)
        return launch_dependent(gated_act_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                                (const float*)gu, (float*)act, inter, total, kind);
    return launch_dependent(gated_act_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream,
                            (const bf16*)gu, (bf16*)act, inter, total, kind);
}

// x float32 [*, hidden]; d1, d2 and y of storage type `dtype` (any may be null); gain float32 [hidden].
int fsie_scaled_sum_rmsnorm(float* x, const void* d1, float a1, const void* d2, float a2, const float* gain,
                            void* y, const int* rows, int num_rows, int hidden, float eps, int write_x,
                            int dtype, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (hidden <= 0 || (y && !gain)) return ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const bool vec = hidden % 8 == 0 &&
        ((((size_t)x) | ((size_t)d1) | ((size_t)d2) | ((size_t)y) | ((size_t)gain)) & 15) == 0;
    const int threads = vec ? (hidden >= 4096 ? 512 : (hidden >= 1024 ? 128 : 64))
                            : (hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128));
#define FSIE_SSR(T, V)                                                                                      \
    do {                                                                                                    \
        if (smem > 48 * 1024)                                                                               \
            cudaFuncSetAttribute(scaled_sum_rmsnorm_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem);                                                                \
        return launch_dependent(scaled_sum_rmsnorm_kernel<T, V>, dim3(num_rows), dim3(threads), smem, stream, x, \
                                (const T*)d1, a1, (const T*)d2, a2, gain, (T*)y, rows, hidden, eps, write_x); \
    } while (0)
    if (dtype == DTYPE_F32) { if (vec) FSIE_SSR(float, true); else FSIE_SSR(float, false); }
    if (vec) FSIE_SSR(bf16, true); else FSIE_SSR(bf16, false);
#undef FSIE_SSR
}

}  // extern "C"
