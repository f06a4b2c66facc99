// A feed-forward of routed experts: every token chooses `top` of `experts` small gated
// feed-forwards and adds their outputs with weights.
//
//   route      z = W_r y (32-bit), s = sigmoid(z) (or softmax over the experts), choice = s + correction;
//              experts form `groups` equal groups of neighbours, a group's score is the sum of its two
//              largest choices, only experts of the `keep` best groups can be chosen (the others
//              count as minus infinity); the `top` largest choices are taken; their weights are
//              s / (sum of the chosen s + 1e-20) * scale (normalise = 0: s * scale)
//   align      (token, choice) pairs sorted by expert, cut into tiles of rows that share an expert
//   gate_up    act[r] = f(W_gate[e] y[t(r)]) * (W_up[e] y[t(r)])       r in sorted order
//   down       out[pair(r)] = W_down[e] act[r]
//   combine    y_out[t] = sum_j weight[t, j] * out[t, j] (+ what a shared expert gave for t)
//
// The number of rows per expert is known only on the device, so the grids are sized for the worst
// case (pairs / tile + experts tiles) and blocks beyond the tile count leave at once: a step
// launches the same kernels whatever the routing says.  The router, its scores, the choice and the
// weights are 32-bit; the products add in 32-bit.
#include "common.cuh"
#include <math.h>

namespace fsie {

constexpr int MOE_TILE = 64;          // rows (and output columns) per tile of the tiled products

// -------------------------------------------------------------------------------- router
// (value, index) maximum over a shared array by one warp; ties go to the lower index.
__device__ __forceinline__ int warp_argmax(const float* v, const unsigned char* taken, int n, int lane) {
    float best = -INFINITY;
    int at = -1;
    for (int i = lane; i < n; i += 32) {
        if (taken[i]) continue;
        if (at < 0 || v[i] > best) { best = v[i]; at = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    return at;
}

// y == nullptr: the router's logits were computed by a matrix product and wait in `logits`
// [tokens, experts]; the block (one warp then) only scores, chooses and weighs.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ y, int y_ld, const float* __restrict__ w_router,
                                 const float* __restrict__ logits,
                                 const float* __restrict__ correction, int* __restrict__ ids,
                                 float* __restrict__ weights, int width, int experts, int top, int groups,
                                 int keep, float scale, int softmax_scores, int normalise, int group_max) {
    extern __shared__ float route_smem[];
    float* row = route_smem;                       // [width]
    float* score = row + width;                    // [experts] s
    float* choice = score + experts;               // [experts] s + correction
    float* group_score = choice + experts;         // [groups]
    unsigned char* taken = reinterpret_cast<unsigned char*>(group_score + groups);   // [experts]
    unsigned char* group_taken = taken + experts;                                     // [groups]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    grid_dependency_wait();
    grid_dependents_go();
    if (y) {
        const T* yr = y + (size_t)t * y_ld;
        for (int c = threadIdx.x; c < width; c += blockDim.x) row[c] = to_float(yr[c]);
        __syncthreads();
        for (int e = warp; e < experts; e += warps) {
            const float* wr = w_router + (size_t)e * width;
            float acc = 0.f;
            for (int c = lane; c < width; c += 32) acc = fmaf(wr[c], row[c], acc);
            acc = warp_sum(acc);
            if (lane == 0) score[e] = acc;
        }
    } else {
        for (int e = threadIdx.x; e < experts; e += blockDim.x) score[e] = logits[(size_t)t * experts + e];
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax_scores) {
        float m = -INFINITY;
        for (int e = lane; e < experts; e += 32) m = fmaxf(m, score[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < experts; e += 32) sum += expf(score[e] - m);
        sum = warp_sum(sum);
        for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - m) / sum;
    } else {
        for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    for (int e = lane; e < experts; e += 32) {
        choice[e] = score[e] + (correction ? correction[e] : 0.f);
        taken[e] = 0;
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        const int per = experts / groups;
        for (int g = lane; g < groups; g += 32) {
            float first = -INFINITY, second = -INFINITY;
            for (int i = 0; i < per; ++i) {
                const float v = choice[g * per + i];
                if (v > first) { second = first; first = v; }
                else if (v > second) second = v;
            }
            group_score[g] = (per > 1 && !group_max) ? first + second : first;
            group_taken[g] = 0;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            const int g = warp_argmax(group_score, group_taken, groups, lane);
            if (lane == 0 && g >= 0) group_taken[g] = 1;
            __syncwarp();
        }
        for (int e = lane; e < experts; e += 32)
            if (!group_taken[e / per]) taken[e] = 1;       // outside the kept groups: never chosen
        __syncwarp();
    }
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
        const int e = warp_argmax(choice, taken, experts, lane);
        if (lane == 0) {
            ids[(size_t)t * top + k] = e < 0 ? 0 : e;
            if (e >= 0) taken[e] = 1;
        }
        sum += e < 0 ? 0.f : score[e];
        __syncwarp();
    }
    if (lane == 0) {
        for (int k = 0; k < top; ++k) {
            const float s = score[ids[(size_t)t * top + k]];
            weights[(size_t)t * top + k] = normalise ? s / (sum + 1e-20f) * scale : s * scale;
        }
    }
}

// ------------------------------------------------------------------- pairs sorted by expert
// One block.  Compact layout: offsets[e] .. offsets[e + 1] are the rows of expert e in `sorted`
// (pair = token * top + choice); tiles: (expert, first row) of every tile of `tile` rows; meta[0] =
// their number.  Padded layout (`padded`): every expert's rows start on a multiple of `tile`, rows
// that no pair owns hold -1, offsets[e] is the expert's first row, and place[pair] is the pair's row.
__global__ void moe_align_kernel(const int* __restrict__ ids, int pairs, int experts, int tile, int padded,
                                 int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ tile_expert,
                                 int* __restrict__ tile_row0, int* __restrict__ meta, int* __restrict__ place) {
    extern __shared__ int align_smem[];
    int* count = align_smem;                    // [experts]
    int* start = count + experts;               // [experts + 1]
    int* tile_start = start + experts + 1;      // [experts + 1]
    grid_dependency_wait();
    grid_dependents_go();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            start[e] = padded ? tiles * tile : rows;
            tile_start[e] = tiles;
            rows += count[e];
            tiles += (count[e] + tile - 1) / tile;
        }
        start[experts] = padded ? tiles * tile : rows;
        tile_start[experts] = tiles;
        meta[0] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = start[e];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int n = tile_start[e + 1] - tile_start[e];
        for (int i = 0; i < n; ++i) {
            tile_expert[tile_start[e] + i] = e;
            tile_row0[tile_start[e] + i] = start[e] + i * tile;
        }
        count[e] = 0;                           // from here on: how many rows of e are placed
    }
    if (padded)
        for (int r = threadIdx.x; r < start[experts]; r += blockDim.x) sorted[r] = -1;
    __syncthreads();
    // a pair's place among its expert's rows: in the order the threads arrive.  Each row of a
    // product is summed on its own, so the order of an expert's rows changes no result.
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e < 0 || e >= experts) continue;
        const int at = start[e] + atomicAdd(&count[e], 1);
        sorted[at] = p;
        if (place) place[p] = at;
    }
}

// x_sorted[r] = x[sorted[r] / top] for the rows of the used tiles (zeros where no pair owns the row):
// the rows of the step's tokens in the padded order, for a product that reads whole tiles.
__global__ void moe_gather_kernel(const bf16* __restrict__ x, long long x_ld, const int* __restrict__ sorted,
                                  const int* __restrict__ meta, int tile, int top, bf16* __restrict__ out, int k) {
    grid_dependency_wait();
    grid_dependents_go();
    const int r = blockIdx.x;
    if (r >= meta[0] * tile) return;
    const int pair = sorted[r];
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * k);
    if (pair < 0) {
        for (int c = threadIdx.x; c < k / 8; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / top) * x_ld);
    for (int c = threadIdx.x; c < k / 8; c += blockDim.x) dst[c] = src[c];
}

// --------------------------------------------------------------- tiled products, any type
// A block owns one tile (expert e, 64 rows) x 64 output columns; a thread 4 x 4 of them; k in
// steps of 16 through shared memory.  GATED: the 64 columns are 32 of the gate and the same 32 of
// the up projection (a thread holds two of each), the result is f(gate) * up, rows are read at
// token = pair / top and written in sorted order.  Not GATED: rows are read in sorted order and
// written at their pair.
__device__ __forceinline__ float gate_fn(float g, int kind) {
    if (kind == 2) { const float r = fmaxf(g, 0.f); return r * r; }      // the square of relu
    if (kind == 1) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) moe_product_kernel(
        const T* __restrict__ x, long long x_ld, const T* __restrict__ w, T* __restrict__ out, long long out_ld,
        const int* __restrict__ offsets, const int* __restrict__ sorted, const int* __restrict__ tile_expert,
        const int* __restrict__ tile_row0, const int* __restrict__ meta, int top, int n, int k, int gate_kind) {
    constexpr bool GATED = MODE == 1, FIRST = MODE != 0;
    __shared__ float xs[16][MOE_TILE + 4];
    __shared__ float ws[16][MOE_TILE + 4];
    __shared__ int src[MOE_TILE], dst[MOE_TILE];
    grid_dependency_wait();
    grid_dependents_go();
    const int tile = blockIdx.x;
    if (tile >= meta[0]) return;
    const int e = tile_expert[tile], r0 = tile_row0[tile];
    const int rows = min(MOE_TILE, offsets[e + 1] - r0);
    constexpr int COLS = GATED ? MOE_TILE / 2 : MOE_TILE;     // distinct outputs per block
    const int n0 = blockIdx.y * COLS;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    if (threadIdx.x < MOE_TILE) {
        const int r = threadIdx.x;
        const int pair = r < rows ? sorted[r0 + r] : -1;
        src[r] = pair < 0 ? -1 : (FIRST ? pair / top : r0 + r);
        dst[r] = pair < 0 ? -1 : (FIRST ? r0 + r : pair);
    }
    __syncthreads();
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * n * k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < k; k0 += 16) {
        for (int idx = threadIdx.x; idx < MOE_TILE * 16; idx += 256) {
            const int r = idx / 16, kk = idx - r * 16, kc = k0 + kk;
            const int s = src[r];
            xs[kk][r] = (s >= 0 && kc < k) ? to_float(x[(size_t)s * x_ld + kc]) : 0.f;
            // column r of the tile: which row of the expert's matrix
            int wrow;
            if (GATED) {
                const int c = n0 + (r >> 2) * 2 + (r & 1);
                wrow = c < n ? ((r & 2) ? n + c : c) : -1;
            } else {
                wrow = n0 + r < n ? n0 + r : -1;
            }
            ws[kk][r] = (wrow >= 0 && kc < k) ? to_float(we[(size_t)wrow * k + kc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
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
        const int d = dst[ty * 4 + i];
        if (d < 0) continue;
        T* o = out + (size_t)d * out_ld;
        if (GATED) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = n0 + tx * 2 + j;
                // gate and up are rounded to the storage type before the activation, as a product
                // that stored them in between would have
                const float g = to_float(from_float<T>(acc[i][j])), u = to_float(from_float<T>(acc[i][2 + j]));
                if (c < n) o[c] = from_float<T>(gate_fn(g, gate_kind) * u);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = n0 + tx * 4 + j;
                if (c < n) o[c] = MODE == 2 ? from_float<T>(gate_fn(to_float(from_float<T>(acc[i][j])), gate_kind))
                                            : from_float<T>(acc[i][j]);
            }
        }
    }
}

// ------------------------------------------------- the same on the tensor cores (bfloat16)
// mma.sync m16n8k16: a block of four warps owns a tile of 64 rows x 64 columns (GATED: 32 of the
// gate, then the same 32 of the up projection; a thread's fragments j and j + 4 are a gate and its
// up), a warp 16 rows; x and w travel by cp.async in chunks of 64 k-elements into two slots.
constexpr int MM_K = 64, MM_LD = MM_K + 8;

__device__ __forceinline__ uint32_t mm_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mm_ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(mm_smem_u32(p)));
}
__device__ __forceinline__ void mm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mm_cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(mm_smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(128) moe_product_mma_kernel(
        const bf16* __restrict__ x, long long x_ld, const bf16* __restrict__ w, bf16* __restrict__ out,
        long long out_ld, const int* __restrict__ offsets, const int* __restrict__ sorted,
        const int* __restrict__ tile_expert, const int* __restrict__ tile_row0, const int* __restrict__ meta,
        int top, int n, int k, int gate_kind) {
    constexpr bool GATED = MODE == 1, FIRST = MODE != 0;
    __shared__ __align__(16) bf16 xs[2][MOE_TILE][MM_LD];
    __shared__ __align__(16) bf16 ws[2][MOE_TILE][MM_LD];
    __shared__ int src[MOE_TILE], dst[MOE_TILE];
    grid_dependency_wait();
    grid_dependents_go();
    const int tile = blockIdx.x;
    if (tile >= meta[0]) return;
    const int e = tile_expert[tile], r0 = tile_row0[tile];
    const int rows = min(MOE_TILE, offsets[e + 1] - r0);
    constexpr int COLS = GATED ? MOE_TILE / 2 : MOE_TILE;
    const int n0 = blockIdx.y * COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    if (tid < MOE_TILE) {
        const int pair = tid < rows ? sorted[r0 + tid] : -1;
        src[tid] = pair < 0 ? -1 : (FIRST ? pair / top : r0 + tid);
        dst[tid] = pair < 0 ? -1 : (FIRST ? r0 + tid : pair);
    }
    __syncthreads();
    const bf16* we = w + (size_t)e * (GATED ? 2 : 1) * n * k;
    // a thread copies half a row (four 16-byte pieces) of x and of w per chunk
    const int cr = tid >> 1, c0 = (tid & 1) * 4;
    const int xrow = src[cr];
    int wrow;
    if (GATED) {
        const int c = n0 + (cr & 31);
        wrow = c < n ? (cr >= 32 ? n + c : c) : -1;
    } else {
        wrow = n0 + cr < n ? n0 + cr : -1;
    }
    auto issue = [&](int stage, int k0) {
#pragma unroll
        for (int c = c0; c < c0 + 4; ++c) {
            const int kc = k0 + c * 8;
            const bool xin = xrow >= 0 && kc < k, win = wrow >= 0 && kc < k;
            mm_cp16(&xs[stage][cr][c * 8], x + (xin ? (size_t)xrow * x_ld + kc : 0), xin);
            mm_cp16(&ws[stage][cr][c * 8], we + (win ? (size_t)wrow * k + kc : 0), win);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    issue(0, 0);
    int it = 0;
    for (int k0 = 0; k0 < k; k0 += MM_K, ++it) {
        const int stage = it & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (k0 + MM_K < k) issue(stage ^ 1, k0 + MM_K);
        if (warp * 16 < rows) {
            const bf16* xa = &xs[stage][warp * 16 + (lane & 15)][(lane >> 4) * 8];
            const bf16* wb = &ws[stage][(lane & 7) + (lane >> 4) * 8][((lane >> 3) & 1) * 8];
#pragma unroll
            for (int kk = 0; kk < MM_K; kk += 16) {
                uint32_t a[4];
                mm_ldsm_x4(a, xa + kk);
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    uint32_t b[4];
                    mm_ldsm_x4(b, wb + nb * 16 * MM_LD + kk);
                    mm_mma(acc[2 * nb], a, b[0], b[1]);
                    mm_mma(acc[2 * nb + 1], a, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int d = dst[warp * 16 + g + 8 * i];
        if (d < 0) continue;
        bf16* o = out + (size_t)d * out_ld;
        if (GATED) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = n0 + j * 8 + 2 * t + h;
                    const float gt = __bfloat162float(__float2bfloat16_rn(acc[j][2 * i + h]));
                    const float up = __bfloat162float(__float2bfloat16_rn(acc[j + 4][2 * i + h]));
                    if (c < n) o[c] = __float2bfloat16_rn(gate_fn(gt, gate_kind) * up);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = n0 + j * 8 + 2 * t + h;
                    if (c < n)
                        o[c] = MODE == 2 ? __float2bfloat16_rn(gate_fn(__bfloat162float(__float2bfloat16_rn(acc[j][2 * i + h])), gate_kind))
                                         : __float2bfloat16_rn(acc[j][2 * i + h]);
                }
            }
        }
    }
}

// -------------------------------------------------------------------------------- combine
template <typename T, bool VEC>
__global__ void moe_combine_kernel(const T* __restrict__ expert_out, const float* __restrict__ weights,
                                   const T* __restrict__ shared, const int* __restrict__ place,
                                   T* __restrict__ out, int width, int top, const int* __restrict__ ids,
                                   int experts, const T* __restrict__ y, long long y_ld) {
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    // a choice at or beyond `experts` is an identity expert: its output is the token's input row
    if (VEC) {          // eight columns per thread, 16-byte accesses; the sums run in the same order
        for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, v[8];
            for (int j = 0; j < top; ++j) {
                const float w = weights[t * top + j];
                if (ids && ids[t * top + j] >= experts) {
                    load8(y + t * y_ld + c, v);
                } else {
                    const size_t row = place ? (size_t)place[t * top + j] : t * top + j;
                    load8(expert_out + row * width + c, v);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, v[i], acc[i]);
            }
            if (shared) {
                load8(shared + t * width + c, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += v[i];
            }
            store8(out + t * width + c, acc);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            if (ids && ids[t * top + j] >= experts) {
                acc = fmaf(weights[t * top + j], to_float(y[t * y_ld + c]), acc);
                continue;
            }
            const size_t row = place ? (size_t)place[t * top + j] : t * top + j;
            acc = fmaf(weights[t * top + j], to_float(expert_out[row * width + c]), acc);
        }
        if (shared) acc += to_float(shared[t * width + c]);
        out[t * width + c] = from_float<T>(acc);
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_moe_tile_rows() { return MOE_TILE; }

// y [tokens, y_ld] of the storage type; w_router float32 [experts, width]; correction float32
// [experts] or null; ids int32 / weights float32 [tokens, top].
int fsie_moe_route(const void* y, int y_ld, const float* w_router, const float* logits, const float* correction, int* ids,
                   float* weights, int tokens, int width, int experts, int top, int groups, int keep,
                   float scale, int softmax_scores, int normalise, int group_max, int dtype,
                   cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if ((y && width <= 0) || experts <= 0 || top <= 0 || top > experts || groups <= 0 || experts % groups ||
        keep <= 0 || keep > groups || top > keep * (experts / groups))
        return ERR_BAD_ARGUMENT;
    if (!y && !logits) return ERR_BAD_ARGUMENT;
    if (!y) width = 0;
    const int threads = y ? 128 : 32;
    const size_t smem = ((size_t)width + 2 * experts + groups) * sizeof(float) + experts + groups + 8;
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    if (dtype == DTYPE_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(moe_route_kernel<float>, tokens, threads, smem, stream, (const float*)y, y_ld, w_router,
                                logits, correction, ids, weights, width, experts, top, groups, keep, scale,
                                softmax_scores, normalise, group_max);
    }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(moe_route_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(moe_route_kernel<bf16>, tokens, threads, smem, stream, (const bf16*)y, y_ld, w_router,
                            logits, correction, ids, weights, width, experts, top, groups, keep, scale, softmax_scores,
                            normalise, group_max);
}

// offsets [experts + 1], sorted [pairs] (padded: [(pairs / tile + experts) * tile]), tile_expert /
// tile_row0 [pairs / tile + experts], meta [1], place [pairs] or null
int fsie_moe_align(const int* ids, int pairs, int experts, int tile, int padded, int* offsets, int* sorted,
                   int* tile_expert, int* tile_row0, int* meta, int* place, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (experts <= 0 || tile <= 0 || (!padded && tile != MOE_TILE)) return ERR_BAD_ARGUMENT;
    const size_t smem = (3 * (size_t)experts + 2) * sizeof(int);
    if (smem > 40 * 1024) return ERR_UNSUPPORTED;
    const int threads = pairs >= 4096 ? 1024 : (pairs >= 512 ? 256 : 64);
    return launch_dependent(moe_align_kernel, 1, threads, smem, stream, ids, pairs, experts, tile, padded, offsets,
                            sorted, tile_expert, tile_row0, meta, place);
}

// out [rows of the padded layout, k] bf16 = the tokens' rows of x in that order; `rows` is the room
// there is (pairs / tile + experts tiles).
int fsie_moe_gather(const void* x, long long x_ld, const int* sorted, const int* meta, int tile, int top,
                    void* out, int rows, int k, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (k <= 0 || k % 8 || x_ld % 8 || ((((size_t)x) | ((size_t)out)) & 15)) return ERR_BAD_ARGUMENT;
    return launch_dependent(moe_gather_kernel, rows, k >= 2048 ? 256 : 128, 0, stream, (const bf16*)x, x_ld, sorted,
                            meta, tile, top, (bf16*)out, k);
}

// gated = 1: x [tokens, x_ld] read at pair / top, w [experts, 2 n, k] (gate rows, then up rows), out
// [pairs, out_ld] in sorted order.  gated = 2: the same rows in and out, w [experts, n, k], out = f(x w^T)
// (an expert without a gate: gate_kind names f).  gated = 0: x [pairs, x_ld] in sorted order, w [experts, n, k], out
// written at the pair's own row.
int fsie_moe_product(const void* x, long long x_ld, const void* w, void* out, long long out_ld,
                     const int* offsets, const int* sorted, const int* tile_expert, const int* tile_row0,
                     const int* meta, int pairs, int experts, int top, int n, int k, int gated, int gate_kind,
                     int dtype, cudaStream_t stream) {
    if (pairs <= 0 || n <= 0) return 0;
    if (k <= 0 || experts <= 0 || top <= 0 || gated < 0 || gated > 2) return ERR_BAD_ARGUMENT;
    const int cols = gated == 1 ? MOE_TILE / 2 : MOE_TILE;
    const dim3 grid(pairs / MOE_TILE + experts, (n + cols - 1) / cols);
    if (grid.y > 65535) return ERR_UNSUPPORTED;
    if (dtype == DTYPE_BF16 && k % 8 == 0 && x_ld % 8 == 0 && ((((size_t)x) | ((size_t)w)) & 15) == 0) {
#define FSIE_MOE_MMA(M)                                                                                      \
        launch_dependent(moe_product_mma_kernel<M>, grid, dim3(128), 0, stream, (const bf16*)x, x_ld,              \
                         (const bf16*)w, (bf16*)out, out_ld, offsets, sorted, tile_expert, tile_row0, meta, top, n, \
                         k, gate_kind)
        return gated == 1 ? FSIE_MOE_MMA(1) : (gated == 2 ? FSIE_MOE_MMA(2) : FSIE_MOE_MMA(0));
#undef FSIE_MOE_MMA
    }
#define FSIE_MOE(T, G)                                                                                      \
    launch_dependent(moe_product_kernel<T, G>, grid, dim3(256), 0, stream, (const T*)x, x_ld, (const T*)w, \
                     (T*)out, out_ld, offsets, sorted, tile_expert, tile_row0, meta, top, n, k, gate_kind)
    if (dtype == DTYPE_F32) return gated == 1 ? FSIE_MOE(float, 1) : (gated == 2 ? FSIE_MOE(float, 2) : FSIE_MOE(float, 0));
    return gated == 1 ? FSIE_MOE(bf16, 1) : (gated == 2 ? FSIE_MOE(bf16, 2) : FSIE_MOE(bf16, 0));
#undef FSIE_MOE
}

// ids [tokens, top] with `experts` and y [tokens, y_ld] (or all null): a choice at or beyond `experts` is an
// identity expert, whose output is the token's row of y.
// expert_out [tokens * top, width] at the pairs' rows (or, with `place`, pair p at row place[p]);
// weights float32 [tokens, top]; shared [tokens, width] or null; out [tokens, width].
int fsie_moe_combine(const void* expert_out, const float* weights, const void* shared, const int* place, void* out,
                     int tokens, int width, int top, const int* ids, int experts, const void* y, long long y_ld,
                     int dtype, cudaStream_t stream) {
    if (tokens <= 0 || width <= 0) return 0;
    if (ids && !y) return ERR_BAD_ARGUMENT;
    const bool vec = width % 8 == 0 && (!ids || y_ld % 8 == 0) &&
        (((size_t)expert_out | (size_t)shared | (size_t)out | (size_t)y) & 15) == 0;
    const int threads = vec ? (width >= 2048 ? 256 : (width >= 1024 ? 128 : 64)) : (width >= 1024 ? 256 : 128);
#define FSIE_COMBINE(T, V) launch_dependent(moe_combine_kernel<T, V>, tokens, threads, 0, stream, (const T*)expert_out, \
                                            weights, (const T*)shared, place, (T*)out, width, top, ids, experts, \
                                            (const T*)y, y_ld)
    if (dtype == DTYPE_F32) return vec ? FSIE_COMBINE(float, true) : FSIE_COMBINE(float, false);
    return vec ? FSIE_COMBINE(bf16, true) : FSIE_COMBINE(bf16, false);
#undef FSIE_COMBINE
}

}  // extern "C"
