// The steps of attention over a latent cache that are neither a plain matrix product nor the
// attention itself.  Per token the cache keeps ONE row shared by all heads: a normed latent vector
// c (rank columns) and a rotated key part (rope columns).  A head's unrotated keys and its values
// are linear in c (k_h = U_h c, v_h = V_h c), so they are never formed: the query takes U_h over
// (q_h . U_h c = (U_h^T q_h) . c) and V_h is applied to the attention's output over c.
//
//   latent_prep    proj[t] = [ q: heads x (dim | rope) | lat: rank | kr: rope ]
//                  c  = lat / sqrt(mean(lat^2) + eps) * gain          -> cache row columns [0, rank)
//                  kr rotated (pairs 2i, 2i + 1 of the leading rotary_dim, or - `half_pairs` - pairs
//                  i, i + rotary_dim / 2)                              -> columns [rank, rank + rope)
//                  each head's rope part of q, rotated the same way     -> qa[t, h, rank ...]
//   head_product   out[t, h, :] = W[h] x[t, h, :]   for W [heads, n, k]: U_h^T before the attention
//                  (x = the unrotated part of q, out = qa[t, h, 0 .. rank)), V_h after it.
//
// Norm statistics, angles and the products' sums are 32-bit; storage type T for proj, cache and qa.
#include "common.cuh"
#include <math.h>

namespace fsie {

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                   const float* __restrict__ cos_sin, int table_len,
                                   const int* __restrict__ slot_of, T* __restrict__ pages,
                                   long long page_stride, int page_size, const float* __restrict__ gain,
                                   float eps, T* __restrict__ qa, int heads, int dim, int rope, int rank,
                                   int rotary_dim, int half_pairs, int* __restrict__ error) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependents_go();
    const int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;       // cos of pair i at [i], sin at [half + i]
    const T* row = proj + (size_t)t * ld;
    const int qd = dim + rope, row_width = rank + rope;
    // queries: the rope part of every head, rotated, behind the rank columns the product will fill
    for (int e = threadIdx.x; e < heads * rope; e += blockDim.x) {
        const int h = e / rope, d = e - h * rope;
        const T* src = row + h * qd + dim;
        float val = to_float(src[d]);
        if (d < rotary_dim) {
            // the pair's index, whether d is its second member, and where the other member sits
            const int i = half_pairs ? (d < half ? d : d - half) : d >> 1;
            const bool second = half_pairs ? d >= half : (d & 1);
            const int mate = half_pairs ? (second ? d - half : d + half) : d ^ 1;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(src[mate]);
            val = second ? val * c + other * s : val * c - other * s;
        }
        qa[((size_t)t * heads + h) * row_width + rank + d] = from_float<T>(val);
    }
    const int slot = slot_of ? slot_of[t] : -1;
    const T* lat = row + heads * qd;
    float ss = 0.f;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        const float v = to_float(lat[d]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    if (slot < 0) return;
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    T* dst = pages + (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * row_width;
    for (int d = threadIdx.x; d < rank; d += blockDim.x)
        dst[d] = from_float<T>((to_float(lat[d]) * scale) * gain[d]);
    const T* kr = lat + rank;
    for (int d = threadIdx.x; d < rope; d += blockDim.x) {
        float val = to_float(kr[d]);
        if (d < rotary_dim) {
            // the pair's index, whether d is its second member, and where the other member sits
            const int i = half_pairs ? (d < half ? d : d - half) : d >> 1;
            const bool second = half_pairs ? d >= half : (d & 1);
            const int mate = half_pairs ? (second ? d - half : d + half) : d ^ 1;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(kr[mate]);
            val = second ? val * c + other * s : val * c - other * s;
        }
        dst[rank + d] = from_float<T>(val);
    }
}

// out[t, h, n] = sum_k x[t, h, k] w[h, n, k]; a block owns 64 tokens x 64 outputs of one head,
// a thread 4 x 4 of them; k in steps of 16 through shared memory.
constexpr int HP_TILE = 64, HP_K = 16;

template <typename T>
__global__ void __launch_bounds__(256) head_product_kernel(const T* __restrict__ x, long long x_ld, int x_head,
                                                           const T* __restrict__ w, T* __restrict__ out,
                                                           long long out_ld, int out_head, int tokens,
                                                           int n, int k) {
    __shared__ float xs[HP_K][HP_TILE + 4];
    __shared__ float ws[HP_K][HP_TILE + 4];
    const int h = blockIdx.z, t0 = blockIdx.x * HP_TILE, n0 = blockIdx.y * HP_TILE;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    grid_dependency_wait();
    grid_dependents_go();
    const T* xh = x + (size_t)h * x_head;
    const T* wh = w + (size_t)h * n * k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < k; k0 += HP_K) {
        for (int e = threadIdx.x; e < HP_TILE * HP_K; e += 256) {
            const int r = e / HP_K, kk = e - r * HP_K;
            const int t = t0 + r, c = n0 + r, kc = k0 + kk;
            xs[kk][r] = (t < tokens && kc < k) ? to_float(xh[(size_t)t * x_ld + kc]) : 0.f;
            ws[kk][r] = (c < n && kc < k) ? to_float(wh[(size_t)c * k + kc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HP_K; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < n) out[(size_t)t * out_ld + (size_t)h * out_head + c] = from_float<T>(acc[i][j]);
        }
    }
}


// ---- the same product for steps of few tokens (up to HF_TOKENS): the weights stream once, a warp
// owns one output row of one head at a time, its lanes side by side along k; the step's rows of x
// wait in shared memory as floats.
constexpr int HF_TOKENS = 16, HF_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(HF_WARPS * 32) head_product_few_kernel(
        const T* __restrict__ x, long long x_ld, int x_head, const T* __restrict__ w, T* __restrict__ out,
        long long out_ld, int out_head, int tokens, int n, int k) {
    extern __shared__ __align__(16) float hf_x[];               // [tokens][k]
    const int h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * HF_WARPS + warp;
    // this warp's weight row is asked for before the kernel that produces x has finished
    const T* wr = w + ((size_t)h * n + min(c, n - 1)) * k;
    float first[8];
    const bool wide = k % 8 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (wide && lane * 8 < k) load8(wr + lane * 8, first);
    grid_dependency_wait();
    grid_dependents_go();
    for (int e = threadIdx.x; e < tokens * k; e += blockDim.x) {
        const int t = e / k, kk = e - t * k;
        hf_x[e] = to_float(x[(size_t)t * x_ld + (size_t)h * x_head + kk]);
    }
    __syncthreads();
    if (c >= n) return;
    float acc[HF_TOKENS];
#pragma unroll
    for (int t = 0; t < HF_TOKENS; ++t) acc[t] = 0.f;
    if (wide) {
        for (int kk = lane * 8; kk < k; kk += 256) {
            float wv[8];
            if (kk == lane * 8) {
#pragma unroll
                for (int e = 0; e < 8; ++e) wv[e] = first[e];
            } else {
                load8(wr + kk, wv);
            }
#pragma unroll
            for (int t = 0; t < HF_TOKENS; ++t) {
                if (t >= tokens) break;
                const float4 a = *reinterpret_cast<const float4*>(hf_x + t * k + kk);
                const float4 b = *reinterpret_cast<const float4*>(hf_x + t * k + kk + 4);
                acc[t] += wv[0] * a.x + wv[1] * a.y + wv[2] * a.z + wv[3] * a.w +
                          wv[4] * b.x + wv[5] * b.y + wv[6] * b.z + wv[7] * b.w;
            }
        }
    } else {
        for (int kk = lane; kk < k; kk += 32) {
            const float wv = to_float(wr[kk]);
#pragma unroll
            for (int t = 0; t < HF_TOKENS; ++t) {
                if (t >= tokens) break;
                acc[t] = fmaf(wv, hf_x[t * k + kk], acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < HF_TOKENS; ++t) {
        if (t >= tokens) break;
        const float total = warp_sum(acc[t]);
        if (lane == 0) out[(size_t)t * out_ld + (size_t)h * out_head + c] = from_float<T>(total);
    }
}

// ---- and on the tensor cores for steps of many tokens in bfloat16 (mma.sync m16n8k16): a block of
// four warps owns 64 tokens x 64 outputs of one head, a warp 16 tokens; x and w travel by cp.async in
// chunks of 64 k-elements into two slots.
constexpr int HM_TILE = 64, HM_K = 64, HM_LD = HM_K + 8;

__device__ __forceinline__ uint32_t hm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void hm_ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(hm_smem_u32(p)));
}
__device__ __forceinline__ void hm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void hm_cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(hm_smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(128) head_product_mma_kernel(
        const bf16* __restrict__ x, long long x_ld, int x_head, const bf16* __restrict__ w,
        bf16* __restrict__ out, long long out_ld, int out_head, int tokens, int n, int k) {
    __shared__ __align__(16) bf16 xs[2][HM_TILE][HM_LD];
    __shared__ __align__(16) bf16 ws[2][HM_TILE][HM_LD];
    const int h = blockIdx.z, t0 = blockIdx.x * HM_TILE, n0 = blockIdx.y * HM_TILE;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bf16* xh = x + (size_t)h * x_head;
    const bf16* wh = w + (size_t)h * n * k;
    grid_dependency_wait();
    grid_dependents_go();
    // a thread copies half a row (four 16-byte pieces) of x and of w per chunk
    auto issue = [&](int stage, int k0) {
        const int r = tid >> 1, c0 = (tid & 1) * 4;
#pragma unroll
        for (int c = c0; c < c0 + 4; ++c) {
            const int kc = k0 + c * 8;
            const bool xin = t0 + r < tokens && kc < k, win = n0 + r < n && kc < k;
            hm_cp16(&xs[stage][r][c * 8], xh + (xin ? (size_t)(t0 + r) * x_ld + kc : 0), xin);
            hm_cp16(&ws[stage][r][c * 8], wh + (win ? (size_t)(n0 + r) * k + kc : 0), win);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    issue(0, 0);
    int it = 0;
    for (int k0 = 0; k0 < k; k0 += HM_K, ++it) {
        const int stage = it & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (k0 + HM_K < k) issue(stage ^ 1, k0 + HM_K);
        const bf16* xa = &xs[stage][warp * 16 + (lane & 15)][(lane >> 4) * 8];
        const bf16* wb = &ws[stage][(lane & 7) + (lane >> 4) * 8][((lane >> 3) & 1) * 8];
#pragma unroll
        for (int kk = 0; kk < HM_K; kk += 16) {
            uint32_t a[4];
            hm_ldsm_x4(a, xa + kk);
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                uint32_t b[4];
                hm_ldsm_x4(b, wb + nb * 16 * HM_LD + kk);
                hm_mma(acc[2 * nb], a, b[0], b[1]);
                hm_mma(acc[2 * nb + 1], a, b[2], b[3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int tok = t0 + warp * 16 + g + 8 * i;
        if (tok >= tokens) continue;
        bf16* o = out + (size_t)tok * out_ld + (size_t)h * out_head + n0 + 2 * t;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = n0 + j * 8 + 2 * t;
            if (c + 1 < n) *reinterpret_cast<__nv_bfloat162*>(o + j * 8) = __floats2bfloat162_rn(acc[j][2 * i], acc[j][2 * i + 1]);
            else if (c < n) o[j * 8] = __float2bfloat16_rn(acc[j][2 * i]);
        }
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// proj [tokens, ld]; pages: the cache entry's rows of rank + rope columns, `page_size` per page;
// qa [tokens, heads, rank + rope]; gain float32 [rank]; cos_sin [table_len, rotary_dim].
int fsie_latent_prep(const void* proj, int ld, const int* positions, const float* cos_sin, int table_len,
                     const int* slot_of, void* pages, long long page_stride, int page_size,
                     const float* gain, float eps, void* qa, int tokens, int heads, int dim, int rope,
                     int rank, int rotary_dim, int half_pairs, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || dim < 0 || rope < 0 || rank <= 0 || rotary_dim < 0 || rotary_dim > rope ||
        (rotary_dim & 1) || ld < heads * (dim + rope) + rank + rope)
        return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return launch_dependent(latent_prep_kernel<float>, dim3(tokens), dim3(256), 0, stream,
                                (const float*)proj, ld, positions, cos_sin, table_len, slot_of, (float*)pages,
                                page_stride, page_size, gain, eps, (float*)qa, heads, dim, rope, rank,
                                rotary_dim, half_pairs, error);
    return launch_dependent(latent_prep_kernel<bf16>, dim3(tokens), dim3(256), 0, stream,
                            (const bf16*)proj, ld, positions, cos_sin, table_len, slot_of, (bf16*)pages,
                            page_stride, page_size, gain, eps, (bf16*)qa, heads, dim, rope, rank,
                            rotary_dim, half_pairs, error);
}

// x: head h of token t at t * x_ld + h * x_head (k columns); w [heads, n, k]; out: head h of token t
// at t * out_ld + h * out_head (n columns).
int fsie_head_product(const void* x, long long x_ld, int x_head, const void* w, void* out, long long out_ld,
                      int out_head, int tokens, int heads, int n, int k, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || n <= 0) return 0;
    if (heads <= 0 || k <= 0 || heads > 65535) return ERR_BAD_ARGUMENT;
    if (tokens <= HF_TOKENS && (size_t)tokens * k * sizeof(float) <= 96 * 1024) {
        // few tokens: the weights stream once, a warp per output row
        const dim3 few((n + HF_WARPS - 1) / HF_WARPS, heads);
        const size_t smem = (size_t)tokens * k * sizeof(float);
        if (dtype == DTYPE_F32) {
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(head_product_few_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            return launch_dependent(head_product_few_kernel<float>, few, dim3(HF_WARPS * 32), smem, stream, (const float*)x,
                                    x_ld, x_head, (const float*)w, (float*)out, out_ld, out_head, tokens, n, k);
        }
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(head_product_few_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(head_product_few_kernel<bf16>, few, dim3(HF_WARPS * 32), smem, stream, (const bf16*)x,
                                x_ld, x_head, (const bf16*)w, (bf16*)out, out_ld, out_head, tokens, n, k);
    }
    if (dtype == DTYPE_BF16 && k % 8 == 0 && x_ld % 8 == 0 && x_head % 8 == 0 && out_ld % 2 == 0 && out_head % 2 == 0 &&
        ((((size_t)x) | ((size_t)w)) & 15) == 0 && (((size_t)out) & 3) == 0) {
        const dim3 tiles((tokens + HM_TILE - 1) / HM_TILE, (n + HM_TILE - 1) / HM_TILE, heads);
        if (tiles.y > 65535) return ERR_UNSUPPORTED;
        return launch_dependent(head_product_mma_kernel, tiles, dim3(128), 0, stream, (const bf16*)x, x_ld, x_head,
                                (const bf16*)w, (bf16*)out, out_ld, out_head, tokens, n, k);
    }
    const dim3 grid((tokens + HP_TILE - 1) / HP_TILE, (n + HP_TILE - 1) / HP_TILE, heads);
    if (grid.y > 65535) return ERR_UNSUPPORTED;
    if (dtype == DTYPE_F32)
        return launch_dependent(head_product_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, x_ld,
                                x_head, (const float*)w, (float*)out, out_ld, out_head, tokens, n, k);
    return launch_dependent(head_product_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, x_ld,
                            x_head, (const bf16*)w, (bf16*)out, out_ld, out_head, tokens, n, k);
}

}  // extern "C"
