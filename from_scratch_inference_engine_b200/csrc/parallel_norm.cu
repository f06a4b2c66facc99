// Element-wise steps of decoders whose two sublayers read ONE norm of the residual stream and whose
// residual stream can be sent through a product together with the embedding output.
//
//   sum_layernorm   v = x[s] + (d1[s] + d2[s]);  if write_x: x[s] = v;
//                   y[r] = T( (v - mean) / sqrt(mean((v - mean)^2) + eps) * gain + bias )
//                   s = rows ? rows[r] : r; d1, d2, bias and y are optional
//   settle_concat   out[t] = [ T(x[t] + (d1[t] + d2[t])) | T(x0[t]) ]      (two widths side by side)
//   logit_cap       z <- cap * tanh(z * scale / cap)   (cap = 0: z * scale)
//   sigmoid_gate    out[t, c] <- out[t, c] * sigmoid(g[t, c])
//
// Sums, statistics, gain, bias, the cap and the gate are 32-bit whatever the storage type T is.
#include "common.cuh"
#include <math.h>

namespace fsie {

// VEC: the width is a multiple of 8 and every row starts on 16 bytes: eight columns per thread and
// trip, 16-byte accesses (32 bytes of x as two).  The sums run over the same values in another
// order of the threads' partial sums.
template <typename T, bool VEC>
__global__ void sum_layernorm_kernel(float* __restrict__ x, const T* __restrict__ d1,
                                     const T* __restrict__ d2, const float* __restrict__ gain,
                                     const float* __restrict__ bias, const int* __restrict__ rows,
                                     T* __restrict__ y, int width, float eps, int write_x) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * width;
    const T* a = d1 ? d1 + s * width : nullptr;
    const T* b = d2 ? d2 + s * width : nullptr;
    constexpr int STEP = VEC ? 8 : 1;
    float sum = 0.f;
    for (int c = threadIdx.x * STEP; c < width; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], u[8], w[8];
            load8(xr + c, v);
            if (a) load8(a + c, u);
            if (b) load8(b + c, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (a && b) v[i] += u[i] + w[i];
                else if (a) v[i] += u[i];
                else if (b) v[i] += w[i];
                sum += v[i];
            }
            if (write_x && (a || b)) store8(xr + c, v);
            store8(row_cache + c, v);
        } else {
            float v = xr[c];
            if (a && b) v += to_float(a[c]) + to_float(b[c]);
            else if (a) v += to_float(a[c]);
            else if (b) v += to_float(b[c]);
            if (write_x && (a || b)) xr[c] = v;
            row_cache[c] = v;
            sum += v;
        }
    }
    if (!y) return;
    // every thread reads back only what it wrote itself: no barrier is needed before these loops
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.f;
    for (int c = threadIdx.x * STEP; c < width; c += blockDim.x * STEP) {
#pragma unroll
        for (int i = 0; i < STEP; ++i) {
            const float d = row_cache[c + i] - mean;
            sq += d * d;
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    T* yr = y + (size_t)r * width;
    for (int c = threadIdx.x * STEP; c < width; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], g[8], o[8];
            load8(row_cache + c, v);
            load8(gain + c, g);
            if (bias) load8(bias + c, o);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[i] = (v[i] - mean) * inv * g[i];
                if (bias) v[i] += o[i];
            }
            store8(yr + c, v);
        } else {
            float v = (row_cache[c] - mean) * inv * gain[c];
            if (bias) v += bias[c];
            yr[c] = from_float<T>(v);
        }
    }
}

template <typename T, bool VEC>
__global__ void settle_concat_kernel(const float* __restrict__ x, const T* __restrict__ d1,
                                     const T* __restrict__ d2, const float* __restrict__ x0,
                                     T* __restrict__ out, int width) {
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    const float* xr = x + t * width;
    const float* er = x0 + t * width;
    const T* a = d1 ? d1 + t * width : nullptr;
    const T* b = d2 ? d2 + t * width : nullptr;
    T* o = out + t * 2 * width;
    constexpr int STEP = VEC ? 8 : 1;
    for (int c = threadIdx.x * STEP; c < width; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], u[8], w[8];
            load8(xr + c, v);
            if (a) load8(a + c, u);
            if (b) load8(b + c, w);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (a && b) v[i] += u[i] + w[i];
                else if (a) v[i] += u[i];
                else if (b) v[i] += w[i];
            }
            store8(o + c, v);
            load8(er + c, v);
            store8(o + width + c, v);
        } else {
            float v = xr[c];
            if (a && b) v += to_float(a[c]) + to_float(b[c]);
            else if (a) v += to_float(a[c]);
            else if (b) v += to_float(b[c]);
            o[c] = from_float<T>(v);
            o[width + c] = from_float<T>(er[c]);
        }
    }
}

__global__ void logit_cap_kernel(float* __restrict__ z, long long count, float scale, float cap) {
    grid_dependency_wait();
    grid_dependents_go();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = z[i] * scale;
        z[i] = cap > 0.f ? cap * tanhf(v / cap) : v;
    }
}

template <typename T, bool VEC>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, int out_ld, const T* __restrict__ g, int g_ld,
                                    int width) {
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    T* o = out + t * out_ld;
    const T* gr = g + t * g_ld;
    constexpr int STEP = VEC ? 8 : 1;
    for (int c = threadIdx.x * STEP; c < width; c += blockDim.x * STEP) {
        if (VEC) {
            float v[8], z[8];
            load8(o + c, v);
            load8(gr + c, z);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= 1.0f / (1.0f + expf(-z[i]));
            store8(o + c, v);
        } else {
            const float gate = 1.0f / (1.0f + expf(-to_float(gr[c])));
            o[c] = from_float<T>(to_float(o[c]) * gate);
        }
    }
}

}  // namespace fsie

using namespace fsie;

// every pointer given (null ones aside) starts on 16 bytes
template <typename... P>
static bool aligned16(P... pointers) {
    size_t bits = 0;
    ((bits |= reinterpret_cast<size_t>(pointers)), ...);
    return (bits & 15) == 0;
}

extern "C" {

int fsie_sum_layernorm(float* x, const void* d1, const void* d2, const float* gain, const float* bias,
                       const int* rows, void* y, int num_rows, int width, float eps, int write_x,
                       int dtype, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (width <= 0 || !x || (y && !gain)) return ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const bool vec = width % 8 == 0 && aligned16(x, d1, d2, gain, bias, y);
    const int threads = vec ? (width >= 4096 ? 512 : (width >= 1024 ? 256 : 128))
                            : (width >= 2048 ? 512 : (width >= 512 ? 256 : 128));
#define FSIE_NORM(T, V)                                                                                        \
    (smem > 48 * 1024 ? (void)cudaFuncSetAttribute(sum_layernorm_kernel<T, V>,                                 \
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)     \
                      : (void)0,                                                                               \
     launch_dependent(sum_layernorm_kernel<T, V>, num_rows, threads, smem, stream, x, (const T*)d1, (const T*)d2, \
                      gain, bias, rows, (T*)y, width, eps, write_x))
    if (dtype == DTYPE_F32) return vec ? FSIE_NORM(float, true) : FSIE_NORM(float, false);
    return vec ? FSIE_NORM(bf16, true) : FSIE_NORM(bf16, false);
#undef FSIE_NORM
}

int fsie_settle_concat(const float* x, const void* d1, const void* d2, const float* x0, void* out,
                       int tokens, int width, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || !x || !x0 || !out) return ERR_BAD_ARGUMENT;
    const bool vec = width % 8 == 0 && aligned16(x, d1, d2, x0, out);
    const int threads = vec ? (width >= 2048 ? 256 : 128) : (width >= 1024 ? 256 : 128);
#define FSIE_CONCAT(T, V) launch_dependent(settle_concat_kernel<T, V>, tokens, threads, 0, stream, x, (const T*)d1, \
                                           (const T*)d2, x0, (T*)out, width)
    if (dtype == DTYPE_F32) return vec ? FSIE_CONCAT(float, true) : FSIE_CONCAT(float, false);
    return vec ? FSIE_CONCAT(bf16, true) : FSIE_CONCAT(bf16, false);
#undef FSIE_CONCAT
}

int fsie_logit_cap(float* z, long long count, float scale, float cap, cudaStream_t stream) {
    if (count <= 0) return 0;
    const int threads = 256;
    const long long wanted = (count + threads - 1) / threads;
    const unsigned blocks = (unsigned)(wanted > 4096 ? 4096 : wanted);
    return launch_dependent(logit_cap_kernel, blocks, threads, 0, stream, z, count, scale, cap);
}

int fsie_sigmoid_gate(void* out, int out_ld, const void* g, int g_ld, int tokens, int width, int dtype,
                      cudaStream_t stream) {
    if (tokens <= 0 || width <= 0) return 0;
    const bool vec = width % 8 == 0 && out_ld % 8 == 0 && g_ld % 8 == 0 && aligned16(out, g);
    const int threads = vec ? (width >= 2048 ? 256 : 128) : (width >= 1024 ? 256 : 128);
#define FSIE_GATE(T, V) launch_dependent(sigmoid_gate_kernel<T, V>, tokens, threads, 0, stream, (T*)out, out_ld, \
                                         (const T*)g, g_ld, width)
    if (dtype == DTYPE_F32) return vec ? FSIE_GATE(float, true) : FSIE_GATE(float, false);
    return vec ? FSIE_GATE(bf16, true) : FSIE_GATE(bf16, false);
#undef FSIE_GATE
}

}  // extern "C"
