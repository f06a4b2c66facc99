// Linear attention with a per-head decay ("lightning attention") over per-request state.
//
//   q_t, k_t = silu(projected q, k)  [heads, dim]     v_t = silu(projected v)  [heads, vdim]
//   S_t = decay_h * S_{t-1} + k_t v_t^T               o_t = S_t^T q_t
//   y_t = T( o_t / sqrt(mean(o_t^2) + eps) * gain * sigmoid(g_t) )      over all heads together
//
// The state S [heads, dim, vdim] of a request is 32-bit and lives in its state slot; a step
// carries it on from where the step before left it, token by token in the order of the
// sequence, so the result does not depend on how the tokens were cut into steps beyond rounding
// (long prompts sum chunk by chunk).  The activations, the decay, the state and the output o are
// 32-bit whatever the storage type.
//
// The scan also serves recurrences of the same form with a decay per token and head (`decay_tok`
// [tokens, heads] in place of the constant per head) and with q and k columns that `share` heads
// read together (head h reads the q and k of column group h / share): a state-space mixer's
// S_t = a_t S_(t-1) + B_t (dt_t x_t)^T, o_t = S_t^T C_t.  A request's state starts `state_stride`
// floats after the one before it (a slot may hold more than S).
#include "common.cuh"

namespace fsie {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

constexpr int SCAN_COLS = 32;      // value columns of one block
constexpr int SCAN_ROW_GROUPS = 16;// threads that share four columns; thread r owns rows r DR .. r DR + DR - 1
constexpr int SCAN_TOKENS = 16;    // tokens staged in shared memory at a time

// where row d of a staged q or k vector lives: the DR rows of a thread are contiguous (one or
// more 16-byte loads) and the groups are four floats apart in the banks
template <int DR> __device__ __forceinline__ int scan_row_at(int d) {
    constexpr int PAD = DR >= 4 ? DR + 4 : DR;
    return (d / DR) * PAD + d % DR;
}

// grid (column slices of 32, heads, segments), 128 threads.  Thread (row group r, column group c)
// keeps the DR x 4 patch S[r DR + i][4 c + x] in registers: a staged k or q value serves four
// columns and a v value DR rows, so the arithmetic, not shared memory, sets the pace; the
// output's sum over the rows is finished by shuffles among the 16 row groups.
//
// A block works on one segment of one request: the whole of its new tokens (seg_item == nullptr:
// segment z is request z, the state comes from and goes back to the request's slot), or one
// chunk of them.  Chunks make a long prompt parallel: every chunk first sums its own tokens
// from a zero state (`chunk_states` receives the sum, nothing else is written), a second kernel
// chains the sums into the state at every chunk's start, and every chunk then runs again from
// that state and writes the outputs.
template <int DR>
__global__ void __launch_bounds__(SCAN_COLS / 4 * SCAN_ROW_GROUPS)
lightning_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                      const int* __restrict__ item_qstart, const int* __restrict__ item_qlen,
                      const int* __restrict__ item_slots, float* __restrict__ state,
                      const float* __restrict__ decay, float* __restrict__ out, int heads, int dim,
                      int vdim, const int* __restrict__ seg_item, const int* __restrict__ seg_row0,
                      int seg_tokens, float* __restrict__ chunk_states, int phase, int share,
                      const float* __restrict__ decay_tok, long long state_stride,
                      float* __restrict__ chunk_decay) {
    constexpr int PAD = DR >= 4 ? DR + 4 : DR;
    constexpr int ROW_LEN = SCAN_ROW_GROUPS * PAD;
    __shared__ __align__(16) float qs[SCAN_TOKENS * ROW_LEN];
    __shared__ __align__(16) float ks[SCAN_TOKENS * ROW_LEN];
    __shared__ __align__(16) float vs[SCAN_TOKENS * SCAN_COLS];
    __shared__ float ls[SCAN_TOKENS];                  // the decay of each staged token
    grid_dependency_wait();
    grid_dependents_go();
    const int item = seg_item ? seg_item[blockIdx.z] : blockIdx.z, head = blockIdx.y;
    const int slot = item_slots[item];
    if (slot < 0) return;                              // a padding entry of a fixed-size batch
    const int row0 = seg_item ? seg_row0[blockIdx.z] : 0;
    const int start = item_qstart[item] + row0;
    const int count = seg_item ? min(seg_tokens, item_qlen[item] - row0) : item_qlen[item];
    // phase 0: from the slot, outputs, back to the slot; 1: from zero, the sum to chunk_states;
    // 2: from chunk_states (the state at the chunk's start), outputs
    const bool from_zero = phase == 1, write_out = phase != 1;
    const int rg = threadIdx.x & (SCAN_ROW_GROUPS - 1), cg = threadIdx.x / SCAN_ROW_GROUPS;
    const int col0 = blockIdx.x * SCAN_COLS + cg * 4;
    const bool wide = (vdim & 3) == 0 && (state_stride & 3) == 0;                 // rows of the state start on 16 bytes
    // q and k rows of a head start on 16 bytes and end on them: staged four values at a time
    const bool vec = DR * SCAN_ROW_GROUPS >= 4 && ((dim | ld | q_off | k_off) & 3) == 0;
    float* mine = (phase == 0 ? state + (size_t)slot * state_stride + ((size_t)head * dim) * vdim
                              : chunk_states + (((size_t)blockIdx.z * heads + head) * dim) * vdim);
    const float head_decay = decay ? decay[head] : 1.f;
    const int qk_head = head / share;                  // `share` heads read the same q and k columns
    float through = 1.f;                               // the product of the chunk's decays (phase 1)
    float s[DR][4];
#pragma unroll
    for (int i = 0; i < DR; ++i) {
        const int d = rg * DR + i;
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        if (from_zero || d >= dim || col0 >= vdim) continue;
        const float* at = mine + (size_t)d * vdim + col0;
        if (wide) {
            const float4 v = *reinterpret_cast<const float4*>(at);
            s[i][0] = v.x; s[i][1] = v.y; s[i][2] = v.z; s[i][3] = v.w;
        } else {
#pragma unroll
            for (int x = 0; x < 4; ++x) if (col0 + x < vdim) s[i][x] = at[x];
        }
    }
    for (int t0 = 0; t0 < count; t0 += SCAN_TOKENS) {
        const int n = min(SCAN_TOKENS, count - t0);
        __syncthreads();
        if (vec) {
            constexpr int CHUNKS = SCAN_ROW_GROUPS * DR / 4 > 0 ? SCAN_ROW_GROUPS * DR / 4 : 1;
            for (int idx = threadIdx.x; idx < n * CHUNKS; idx += blockDim.x) {
                const int t = idx / CHUNKS, d = (idx - t * CHUNKS) * 4;
                const float* row = proj + (size_t)(start + t0 + t) * ld + qk_head * dim + d;
                const int at = t * ROW_LEN + scan_row_at<DR>(d);
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                if (write_out)
                    *reinterpret_cast<float4*>(qs + at) = d < dim ? *reinterpret_cast<const float4*>(row + q_off) : zero;
                *reinterpret_cast<float4*>(ks + at) = d < dim ? *reinterpret_cast<const float4*>(row + k_off) : zero;
            }
        } else {
            for (int idx = threadIdx.x; idx < n * SCAN_ROW_GROUPS * DR; idx += blockDim.x) {
                const int t = idx / (SCAN_ROW_GROUPS * DR), d = idx - t * (SCAN_ROW_GROUPS * DR);
                const float* row = proj + (size_t)(start + t0 + t) * ld + qk_head * dim + d;
                const int at = t * ROW_LEN + scan_row_at<DR>(d);
                if (write_out) qs[at] = d < dim ? row[q_off] : 0.f;
                ks[at] = d < dim ? row[k_off] : 0.f;
            }
        }
        for (int idx = threadIdx.x; idx < n * SCAN_COLS; idx += blockDim.x) {
            const int t = idx / SCAN_COLS, c = idx - t * SCAN_COLS;
            const int cc = blockIdx.x * SCAN_COLS + c;
            vs[idx] = cc < vdim ? proj[(size_t)(start + t0 + t) * ld + v_off + head * vdim + cc] : 0.f;
        }
        if (threadIdx.x < n)
            ls[threadIdx.x] = decay_tok ? decay_tok[(size_t)(start + t0 + threadIdx.x) * heads + head] : head_decay;
        __syncthreads();
        for (int t = 0; t < n; ++t) {
            const float lambda = ls[t];
            through *= lambda;
            const float4 v4 = *reinterpret_cast<const float4*>(vs + t * SCAN_COLS + cg * 4);
            const float v[4] = {v4.x, v4.y, v4.z, v4.w};
            float kk[DR], qq[DR];
            const float* kr = ks + t * ROW_LEN + rg * PAD;
            const float* qr = qs + t * ROW_LEN + rg * PAD;
            if (DR >= 4) {
#pragma unroll
                for (int i = 0; i < DR; i += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(kr + i);
                    kk[i] = a.x; kk[i + 1] = a.y; kk[i + 2] = a.z; kk[i + 3] = a.w;
                    if (write_out) {
                        const float4 b = *reinterpret_cast<const float4*>(qr + i);
                        qq[i] = b.x; qq[i + 1] = b.y; qq[i + 2] = b.z; qq[i + 3] = b.w;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < DR; ++i) {
                    kk[i] = kr[i];
                    if (write_out) qq[i] = qr[i];
                }
            }
            float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < DR; ++i)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    s[i][x] = lambda * s[i][x] + kk[i] * v[x];
                    if (write_out) o[x] += s[i][x] * qq[i];
                }
            if (!write_out) continue;
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                o[x] += __shfl_xor_sync(0xffffffffu, o[x], 1);
                o[x] += __shfl_xor_sync(0xffffffffu, o[x], 2);
                o[x] += __shfl_xor_sync(0xffffffffu, o[x], 4);
                o[x] += __shfl_xor_sync(0xffffffffu, o[x], 8);
            }
            if (rg == 0 && col0 < vdim) {
                float* dst = out + (size_t)(start + t0 + t) * heads * vdim + head * vdim + col0;
                if (wide) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                else {
#pragma unroll
                    for (int x = 0; x < 4; ++x) if (col0 + x < vdim) dst[x] = o[x];
                }
            }
        }
    }
    if (phase == 1 && chunk_decay && blockIdx.x == 0 && threadIdx.x == 0)
        chunk_decay[(size_t)blockIdx.z * heads + head] = through;
    if (phase != 2 && col0 < vdim) {
#pragma unroll
        for (int i = 0; i < DR; ++i) {
            const int d = rg * DR + i;
            if (d >= dim) continue;
            float* at = mine + (size_t)d * vdim + col0;
            if (wide) *reinterpret_cast<float4*>(at) = make_float4(s[i][0], s[i][1], s[i][2], s[i][3]);
            else {
#pragma unroll
                for (int x = 0; x < 4; ++x) if (col0 + x < vdim) at[x] = s[i][x];
            }
        }
    }
}

// act[t, c] = silu(proj[t, c]) for the first `width` columns (q, k and v), widened to 32-bit: the
// scan reads every value several times (once per column slice and walk), the activation is
// taken once.
template <typename T>
__global__ void silu_rows_kernel(const T* __restrict__ proj, int ld, int width, float* __restrict__ act,
                                 long long count) {
    grid_dependency_wait();
    grid_dependents_go();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / width;
        const int c = (int)(i - t * width);
        act[i] = silu_f(to_float(proj[t * ld + c]));
    }
}

// Chains the chunks' sums of every request: chunk_states[c] (on entry the sum of chunk c's own
// tokens from a zero state) becomes the state at the start of chunk c, and the request's slot
// receives the state after its last chunk.  S_after = decay^len * S_before + sum.  One thread per
// state element; chunks are listed request by request, in order.
__global__ void lightning_chain_kernel(const int* __restrict__ item_qstart, const int* __restrict__ item_qlen,
                                       const int* __restrict__ item_slots,
                                       int items, float* __restrict__ state, const float* __restrict__ decay,
                                       float* __restrict__ chunk_states, int seg_tokens, int heads,
                                       int dim, int vdim, const float* __restrict__ chunk_decay,
                                       long long state_stride) {
    const int item = blockIdx.y;
    const int slot = item_slots[item];
    if (slot < 0) return;
    const size_t per_head = (size_t)dim * vdim, per_state = per_head * heads;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_state) return;
    int first = 0;                                         // index of this request's first chunk
    for (int i = 0; i < item; ++i) first += (item_qlen[i] + seg_tokens - 1) / seg_tokens;
    const int count = item_qlen[item];
    const int chunks = (count + seg_tokens - 1) / seg_tokens;
    const int head = (int)(e / per_head);
    const float lambda = decay ? decay[head] : 1.f;
    float s = state[(size_t)slot * state_stride + e];
    for (int c = 0; c < chunks; ++c) {
        const int len = min(seg_tokens, count - c * seg_tokens);
        float* at = chunk_states + (size_t)(first + c) * per_state + e;
        const float sum = *at;
        *at = s;
        float power = 1.f;                                 // decay^len by the same products as the scan
        if (chunk_decay) power = chunk_decay[(size_t)(first + c) * heads + head];     // (what the chunk's walk multiplied)
        else for (int t = 0; t < len; ++t) power *= lambda;
        s = power * s + sum;
    }
    state[(size_t)slot * state_stride + e] = s;
}

// One block per token: y = T( o * rsqrt(mean(o^2) + eps) * gain * sigmoid(gate) ).
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ proj, int ld,
                                     int g_off, const float* __restrict__ gain, T* __restrict__ y,
                                     int width, float eps) {
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    const float* row = o + t * width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sq += row[c] * row[c];
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    const T* gate = proj + t * ld + g_off;
    T* yr = y + t * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float g = to_float(gate[c]);
        yr[c] = from_float<T>(row[c] * inv * gain[c] * (1.0f / (1.0f + expf(-g))));
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_silu_rows(const void* proj, int ld, int width, float* act, int tokens, int dtype,
                   cudaStream_t stream) {
    const long long count = (long long)tokens * width;
    if (count <= 0) return 0;
    const long long wanted = (count + 255) / 256;
    const unsigned blocks = (unsigned)(wanted > 8192 ? 8192 : wanted);
    if (dtype == DTYPE_F32)
        return launch_dependent(silu_rows_kernel<float>, blocks, 256, 0, stream, (const float*)proj, ld,
                                width, act, count);
    return launch_dependent(silu_rows_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)proj, ld, width,
                            act, count);
}

// proj [tokens, ld] (float: the activations that fsie_silu_rows left) holds q at q_off, k at k_off
// (heads * dim each) and v at v_off (heads * vdim); state [slots, heads, dim, vdim]; out [tokens,
// heads * vdim] (float).
//
// With seg_item / seg_row0 (num_segs chunks of seg_tokens tokens, listed request by request) and
// chunk_states [num_segs, heads, dim, vdim] (with decay_tok: and num_segs * heads floats more) the
// requests run chunk-parallel in three launches.
int fsie_lightning_scan(const float* proj, int ld, int q_off, int k_off, int v_off,
                        const int* item_qstart, const int* item_qlen, const int* item_slots,
                        int items, float* state, const float* decay, float* out, int heads,
                        int dim, int vdim, const int* seg_item, const int* seg_row0, int num_segs,
                        int seg_tokens, float* chunk_states, int share, const float* decay_tok,
                        long long state_stride, cudaStream_t stream) {
    if (items <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || heads > 65535 || items > 65535 || share <= 0 ||
        heads % share || (!decay && !decay_tok) || state_stride < (long long)heads * dim * vdim)
        return ERR_BAD_ARGUMENT;
    if (dim > SCAN_ROW_GROUPS * 16) return ERR_UNSUPPORTED;
    const bool chunked = seg_item != nullptr;
    if (chunked && (!seg_row0 || !chunk_states || num_segs <= 0 || num_segs > 65535 || seg_tokens <= 0))
        return ERR_BAD_ARGUMENT;
    // decays per token: every chunk's walk leaves the product of its decays behind its sums, for the chain
    float* chunk_decay = chunked && decay_tok ? chunk_states + (size_t)num_segs * heads * dim * vdim : nullptr;
    dim3 grid((vdim + SCAN_COLS - 1) / SCAN_COLS, heads, chunked ? num_segs : items);
    int phase = chunked ? 1 : 0;
    const int threads = SCAN_COLS / 4 * SCAN_ROW_GROUPS;
    const int per_thread = (dim + SCAN_ROW_GROUPS - 1) / SCAN_ROW_GROUPS;
    int launch_code = 0;
#define FSIE_SCAN(T, DPT)                                                                        \
    launch_code = launch_dependent(lightning_scan_kernel<DPT>, grid, threads, 0, stream,         \
        proj, ld, q_off, k_off, v_off, item_qstart, item_qlen, item_slots, state,      \
        decay, out, heads, dim, vdim, seg_item, seg_row0, seg_tokens, chunk_states, phase, share, \
        decay_tok, state_stride, chunk_decay)
#define FSIE_SCAN_BY_SIZE(T)                                                                     \
    do {                                                                                         \
        if (per_thread <= 1) FSIE_SCAN(T, 1);                                                    \
        else if (per_thread <= 2) FSIE_SCAN(T, 2);                                               \
        else if (per_thread <= 4) FSIE_SCAN(T, 4);                                               \
        else if (per_thread <= 8) FSIE_SCAN(T, 8);                                               \
        else FSIE_SCAN(T, 16);                                                                   \
    } while (0)
    FSIE_SCAN_BY_SIZE(float);
    if (launch_code) return launch_code;
    if (chunked) {
        int code;
        const size_t per_state = (size_t)heads * dim * vdim;
        lightning_chain_kernel<<<dim3((unsigned)((per_state + 255) / 256), items), 256, 0, stream>>>(
            item_qstart, item_qlen, item_slots, items, state, decay, chunk_states, seg_tokens, heads, dim, vdim,
            chunk_decay, state_stride);
        code = FSIE_LAUNCH_CHECK();
        if (code) return code;
        phase = 2;
        FSIE_SCAN_BY_SIZE(float);
    }
#undef FSIE_SCAN_BY_SIZE
#undef FSIE_SCAN
    return launch_code;
}

int fsie_gated_rmsnorm(const float* o, const void* proj, int ld, int g_off, const float* gain,
                       void* y, int tokens, int width, float eps, int dtype, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == DTYPE_F32)
        return launch_dependent(gated_rmsnorm_kernel<float>, tokens, threads, 0, stream, o,
                                (const float*)proj, ld, g_off, gain, (float*)y, width, eps);
    return launch_dependent(gated_rmsnorm_kernel<bf16>, tokens, threads, 0, stream, o,
                            (const bf16*)proj, ld, g_off, gain, (bf16*)y, width, eps);
}

}  // extern "C"
