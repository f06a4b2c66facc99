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

template <typename T>
__global__ void sum_layernorm_kernel(float* __restrict__ x, const T* __restrict__ d1,
                                     const T* __restrict__ d2, const float* __restrict__ gain,
                                     const float* __restrict__ bias, const int* __restrict__ rows,
                                     T* __restrict__ y, int width, float eps, int write_x) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * width;
    const T* a = d1 ? d1 + s * width : nullptr;
    const T* b = d2 ? d2 + s * width : nullptr;
    float sum = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = xr[c];
        if (a && b) v += to_float(a[c]) + to_float(b[c]);
        else if (a) v += to_float(a[c]);
        else if (b) v += to_float(b[c]);
        if (write_x && (a || b)) xr[c] = v;
        row_cache[c] = v;
        sum += v;
    }
    if (!y) return;
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row_cache[c] - mean;
        sq += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    T* yr = y + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = (row_cache[c] - mean) * inv * gain[c];
        if (bias) v += bias[c];
        yr[c] = from_float<T>(v);
    }
}

template <typename T>
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
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = xr[c];
        if (a && b) v += to_float(a[c]) + to_float(b[c]);
        else if (a) v += to_float(a[c]);
        else if (b) v += to_float(b[c]);
        o[c] = from_float<T>(v);
        o[width + c] = from_float<T>(er[c]);
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

template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, int out_ld, const T* __restrict__ g, int g_ld,
                                    int width) {
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    T* o = out + t * out_ld;
    const T* gr = g + t * g_ld;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-to_float(gr[c])));
        o[c] = from_float<T>(to_float(o[c]) * gate);
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_sum_layernorm(float* x, const void* d1, const void* d2, const float* gain, const float* bias,
                       const int* rows, void* y, int num_rows, int width, float eps, int write_x,
                       int dtype, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (width <= 0 || !x || (y && !gain)) return ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(sum_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(sum_layernorm_kernel<float>, num_rows, threads, smem, stream, x, (const float*)d1,
                                (const float*)d2, gain, bias, rows, (float*)y, width, eps, write_x);
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(sum_layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(sum_layernorm_kernel<bf16>, num_rows, threads, smem, stream, x, (const bf16*)d1,
                            (const bf16*)d2, gain, bias, rows, (bf16*)y, width, eps, write_x);
}

int fsie_settle_concat(const float* x, const void* d1, const void* d2, const float* x0, void* out,
                       int tokens, int width, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (width <= 0 || !x || !x0 || !out) return ERR_BAD_ARGUMENT;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == DTYPE_F32)
        return launch_dependent(settle_concat_kernel<float>, tokens, threads, 0, stream, x, (const float*)d1,
                                (const float*)d2, x0, (float*)out, width);
    return launch_dependent(settle_concat_kernel<bf16>, tokens, threads, 0, stream, x, (const bf16*)d1,
                            (const bf16*)d2, x0, (bf16*)out, width);
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
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == DTYPE_F32)
        return launch_dependent(sigmoid_gate_kernel<float>, tokens, threads, 0, stream, (float*)out, out_ld,
                                (const float*)g, g_ld, width);
    return launch_dependent(sigmoid_gate_kernel<bf16>, tokens, threads, 0, stream, (bf16*)out, out_ld,
                            (const bf16*)g, g_ld, width);
}

}  // extern "C"
