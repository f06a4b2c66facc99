// The steps around the recurrence of a state-space mixer (the "state-space duality" form):
//
//   proj = [ z (inner) | u (channels = inner + 2 groups n) | dt (heads) ]          one product
//   c_t  = silu(bias + sum_j w[., j] u_(t - taps + 1 + j))          causal convolution per channel,
//          zeros before the sequence starts; c = [ x (heads x vdim) | B (groups x n) | C (groups x n) ]
//   dt_t = softplus(dt_t + dt_bias)   a_t = exp(-exp(A_log) dt_t)                  per head
//   S_t  = a_t S_(t-1) + B_t (dt_t x_t)^T      o_t = S_t^T C_t                     the scan (lightning.cu)
//   y_t  = (o_t + D x_t) * silu(z_t), divided by its root mean square in `parts` equal parts, times a gain
//
// ssd_prep writes, per token, c (32-bit), dt x (32-bit) and a (32-bit) for the scan, which then runs
// with a decay per token and head and with the B and C columns of a group shared by its heads.  The
// last taps - 1 inputs u of a request live in its state slot behind the matrix S (ssd_tails moves
// them on after ssd_prep has read them).  Everything but the stored projection is 32-bit.
#include "common.cuh"
#include <math.h>

namespace fsie {

__device__ __forceinline__ float ssd_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float ssd_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int SSD_MAX_TAPS = 16;

// One block per token.  act [tokens, act_ld] = [ c (channels) | dt x (inner) ]; decay [tokens, heads].
// VEC: channels, the head size, the offsets and the row strides are multiples of 8 and the rows start
// on 16 bytes: a thread owns eight neighbouring channels (all of one head), 16-byte loads per tap;
// the weights then come from conv_wt [taps, channels], the transposed table.
template <typename T, bool VEC>
__global__ void ssd_prep_kernel(const T* __restrict__ proj, int ld, int conv_off, int dt_off,
                                const int* __restrict__ item_qstart, const int* __restrict__ item_qlen,
                                const int* __restrict__ item_slots, int items,
                                const float* __restrict__ state, long long state_stride, long long tail_off,
                                const float* __restrict__ conv_w, const float* __restrict__ conv_b, int taps,
                                int channels, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                int heads, int vdim, float* __restrict__ act, int act_ld,
                                float* __restrict__ decay, const float* __restrict__ conv_wt) {
    extern __shared__ float ssd_dt[];                  // [heads]
    __shared__ int found;
    grid_dependency_wait();
    grid_dependents_go();
    const int t = blockIdx.x;
    if (threadIdx.x == 0) found = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < items; i += blockDim.x)
        if (t >= item_qstart[i] && t < item_qstart[i] + item_qlen[i]) found = i;
    __syncthreads();
    const int item = found;
    if (item < 0) return;
    const int slot = item_slots[item];
    if (slot < 0) return;                              // a padding entry of a fixed-size batch
    const int r = t - item_qstart[item];               // the token's place among the request's new tokens
    const T* row = proj + (size_t)t * ld;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float dt = ssd_softplus(to_float(row[dt_off + h]) + dt_bias[h]);
        ssd_dt[h] = dt;
        decay[(size_t)t * heads + h] = expf(-expf(a_log[h]) * dt);
    }
    __syncthreads();
    const float* tail = state + (size_t)slot * state_stride + tail_off;     // [taps - 1][channels], oldest first
    const int inner = heads * vdim;
    float* out = act + (size_t)t * act_ld;
    if (VEC) {
        for (int c = threadIdx.x * 8; c < channels; c += blockDim.x * 8) {
            float sum[8], u[8], w[8];
            if (conv_b) load8(conv_b + c, sum);
            else {
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] = 0.f;
            }
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j;
                if (back <= r) load8(proj + (size_t)(t - back) * ld + conv_off + c, u);
                else load8(tail + (size_t)(taps - 1 + r - back) * channels + c, u);
                load8(conv_wt + (size_t)j * channels + c, w);         // the taps' weights, tap by tap
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] = fmaf(w[i], u[i], sum[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) sum[i] = ssd_silu(sum[i]);
            store8(out + c, sum);
            if (c < inner) {
                const float dt = ssd_dt[c / vdim];
#pragma unroll
                for (int i = 0; i < 8; ++i) sum[i] *= dt;
                store8(out + channels + c, sum);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float sum = conv_b ? conv_b[c] : 0.f;
        const float* w = conv_w + (size_t)c * taps;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;             // how many tokens before this one
            float u;
            if (back <= r) u = to_float(proj[(size_t)(t - back) * ld + conv_off + c]);
            else u = tail[(size_t)(taps - 1 + r - back) * channels + c];
            sum = fmaf(w[j], u, sum);
        }
        const float v = ssd_silu(sum);
        out[c] = v;
        if (c < inner) out[channels + c] = v * ssd_dt[c / vdim];
    }
}

// One block per request: the last taps - 1 inputs of (what the slot held, then the step's tokens).
template <typename T>
__global__ void ssd_tails_kernel(const T* __restrict__ proj, int ld, int conv_off,
                                 const int* __restrict__ item_qstart, const int* __restrict__ item_qlen,
                                 const int* __restrict__ item_slots, float* __restrict__ state,
                                 long long state_stride, long long tail_off, int taps, int channels) {
    grid_dependency_wait();
    grid_dependents_go();
    const int item = blockIdx.x;
    const int slot = item_slots[item];
    if (slot < 0) return;
    const int start = item_qstart[item], n = item_qlen[item], keep = taps - 1;
    float* tail = state + (size_t)slot * state_stride + tail_off;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float next[SSD_MAX_TAPS];
#pragma unroll
        for (int j = 0; j < SSD_MAX_TAPS; ++j) {
            if (j >= keep) break;
            const int at = n + j;                      // index into (old tail, then the new tokens)
            next[j] = at < keep ? tail[(size_t)at * channels + c]
                                : to_float(proj[(size_t)(start + at - keep) * ld + conv_off + c]);
        }
#pragma unroll
        for (int j = 0; j < SSD_MAX_TAPS; ++j) {
            if (j >= keep) break;
            tail[(size_t)j * channels + c] = next[j];
        }
    }
}

// grid (tokens, parts): y = T( v / sqrt(mean over the part of v^2 + eps) * gain ),
// v = (o + D[head] x) * silu(z).  o [tokens, inner] float; x = act[., 0 .. inner); z = proj[., z_off ..).
template <typename T>
__global__ void ssd_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ act, int act_ld,
                                     const T* __restrict__ proj, int ld, int z_off,
                                     const float* __restrict__ skip, const float* __restrict__ gain,
                                     T* __restrict__ y, int inner, int vdim, int parts, float eps) {
    extern __shared__ float ssd_row[];                 // [inner / parts]
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    const int width = inner / parts, c0 = blockIdx.y * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int c = c0 + i;
        const float z = to_float(proj[t * ld + z_off + c]);
        const float v = (o[t * inner + c] + skip[c / vdim] * act[t * act_ld + c]) * ssd_silu(z);
        ssd_row[i] = v;
        sq += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        y[t * inner + c0 + i] = from_float<T>(ssd_row[i] * inv * gain[c0 + i]);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_ssd_max_taps() { return SSD_MAX_TAPS; }

// proj [tokens, ld] of the storage type; state [slots, state_stride] float, a request's inputs of
// the last taps - 1 tokens at tail_off; conv_w [channels, taps], conv_b [channels] or null, dt_bias,
// a_log [heads] float; act [tokens, act_ld >= channels + heads * vdim] and decay [tokens, heads] float;
// conv_wt [taps, channels] float or null: conv_w transposed, for the form that takes eight channels at once.
int fsie_ssd_prep(const void* proj, int ld, int conv_off, int dt_off, const int* item_qstart,
                  const int* item_qlen, const int* item_slots, int items, const float* state,
                  long long state_stride, long long tail_off, const float* conv_w, const float* conv_b,
                  int taps, int channels, const float* dt_bias, const float* a_log, int heads, int vdim,
                  float* act, int act_ld, float* decay, const float* conv_wt, int tokens, int dtype,
                  cudaStream_t stream) {
    if (tokens <= 0 || items <= 0) return 0;
    if (taps < 1 || taps > SSD_MAX_TAPS || channels < heads * vdim || heads <= 0 || vdim <= 0 ||
        act_ld < channels + heads * vdim || (taps > 1 && !state))
        return ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)heads * sizeof(float);
    if (smem > 40 * 1024) return ERR_UNSUPPORTED;
    const bool vec = conv_wt && channels % 8 == 0 && vdim % 8 == 0 && conv_off % 8 == 0 && ld % 8 == 0 && act_ld % 8 == 0 &&
        (taps == 1 || (state_stride % 8 == 0 && tail_off % 8 == 0)) &&
        ((((size_t)proj) | ((size_t)act) | ((size_t)state) | ((size_t)conv_b) | ((size_t)conv_wt)) & 31) == 0;
    const int threads = vec ? (channels >= 2048 ? 256 : (channels >= 1024 ? 128 : 64))
                            : (channels >= 2048 ? 512 : (channels >= 512 ? 256 : 128));
#define FSIE_SSD_PREP(T, V)                                                                                        \
    launch_dependent(ssd_prep_kernel<T, V>, tokens, threads, smem, stream, (const T*)proj, ld, conv_off, dt_off,    \
                     item_qstart, item_qlen, item_slots, items, state, state_stride, tail_off, conv_w, conv_b, taps, \
                     channels, dt_bias, a_log, heads, vdim, act, act_ld, decay, conv_wt)
    if (dtype == DTYPE_F32) return vec ? FSIE_SSD_PREP(float, true) : FSIE_SSD_PREP(float, false);
    return vec ? FSIE_SSD_PREP(bf16, true) : FSIE_SSD_PREP(bf16, false);
#undef FSIE_SSD_PREP
}

int fsie_ssd_tails(const void* proj, int ld, int conv_off, const int* item_qstart, const int* item_qlen,
                   const int* item_slots, int items, float* state, long long state_stride, long long tail_off,
                   int taps, int channels, int dtype, cudaStream_t stream) {
    if (items <= 0 || taps <= 1) return 0;
    if (taps > SSD_MAX_TAPS || channels <= 0 || !state) return ERR_BAD_ARGUMENT;
    const int threads = channels >= 512 ? 256 : 128;
    if (dtype == DTYPE_F32)
        return launch_dependent(ssd_tails_kernel<float>, items, threads, 0, stream, (const float*)proj, ld,
                                conv_off, item_qstart, item_qlen, item_slots, state, state_stride, tail_off, taps,
                                channels);
    return launch_dependent(ssd_tails_kernel<bf16>, items, threads, 0, stream, (const bf16*)proj, ld, conv_off,
                            item_qstart, item_qlen, item_slots, state, state_stride, tail_off, taps, channels);
}

// o [tokens, inner] float; act [tokens, act_ld] float with x in its first inner columns; proj of the
// storage type with z at z_off; skip [heads], gain [inner] float; y [tokens, inner] of the storage type.
int fsie_ssd_gate_norm(const float* o, const float* act, int act_ld, const void* proj, int ld, int z_off,
                       const float* skip, const float* gain, void* y, int tokens, int inner, int vdim,
                       int parts, float eps, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (inner <= 0 || vdim <= 0 || inner % vdim || parts <= 0 || inner % parts || parts > 65535)
        return ERR_BAD_ARGUMENT;
    const int width = inner / parts;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    const dim3 grid(tokens, parts);
    if (dtype == DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(ssd_gate_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(ssd_gate_norm_kernel<float>, grid, dim3(threads), smem, stream, o, act, act_ld,
                                (const float*)proj, ld, z_off, skip, gain, (float*)y, inner, vdim, parts, eps);
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(ssd_gate_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(ssd_gate_norm_kernel<bf16>, grid, dim3(threads), smem, stream, o, act, act_ld,
                            (const bf16*)proj, ld, z_off, skip, gain, (bf16*)y, inner, vdim, parts, eps);
}

}  // extern "C"
