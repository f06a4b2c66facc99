// Causal softmax attention over the paged cache with a scale per query head, keys and values of
// different widths, and optionally values that ARE the leading columns of the key rows (a cache
// that stores one latent row per token, read by every head as key and as value).  32-bit
// arithmetic on the CUDA cores for any sizes; storage type T (float or bfloat16) for q, the pages
// and the output.
//
//   s_h(i, j) = (q_h,i . k_g(h),j) * head_scale[h]      visible: j <= i and (window == 0 or i - j < window)
//                                                       and (chunk == 0 or i / chunk == j / chunk)
//   o_h,i     = sum_j softmax_j(s_h(i, .)) v_g(h),j      g(h) = h / (heads / kv_heads)
//
// Work is cut as in attention_generic.cu: a tile is up to ROWS query rows of one request and one
// key/value head, a row being (token, head of the group): row = token * group + head_in_group; a
// tile's key range may be split over blockIdx.z and merged by sa_combine_kernel.
//
// The file also holds the step before it for projections q | k | v laid out head by head:
// rotation of q and k over the leading `rotary_dim` of each head (pairs i, i + rotary_dim / 2),
// blending of v with the values another layer computed for the same token, and the cache write.
#include "common.cuh"
#include <math.h>

namespace fsie {

constexpr int SA_ROWS = 32;
constexpr int SA_WARPS = 8;
constexpr int SA_RPW = SA_ROWS / SA_WARPS;
constexpr int SA_KT = 32;

struct ScaledAttnParams {
    const void* q; int q_ld;                  // head h of token t at t * q_ld + h * key_dim
    const float* head_scale;                  // [heads]
    const void* k_pages; const void* v_pages;
    long long page_stride; int page_size;
    int key_dim, value_dim, value_ld;         // value rows are value_ld apart (key_dim when they live in the key rows)
    const int* block_tables; int bt_stride;
    const int* tile_item; const int* tile_row0;
    const int* item_qstart; const int* item_qlen; const int* item_pos0; const int* item_slots;
    void* out; int out_ld;                    // head h of token t at t * out_ld + h * value_dim
    float* part_o; float* part_ml;            // [nsplit, tokens, heads, value_dim], [nsplit, tokens, heads, 2]
    int tokens, heads, kv_heads, window, nsplit;
    int chunk;                                // > 0: a query sees only the keys of its own chunk of this many positions
    int* error;
};

// The first key that the query at `pos` sees: the window's start, or the start of its chunk.
__device__ __forceinline__ int sa_first_key(const ScaledAttnParams& p, int pos) {
    int first = p.window > 0 ? pos - p.window + 1 : 0;
    if (p.chunk > 0) first = max(first, pos - pos % p.chunk);
    return max(first, 0);
}

template <typename T, int DPL, bool SHARED_V>
__global__ void __launch_bounds__(SA_WARPS * 32) scaled_attention_kernel(const ScaledAttnParams p) {
    extern __shared__ __align__(16) float sa_smem[];
    const int dk = p.key_dim, dv = p.value_dim;
    const int dk4 = (dk + 3) & ~3;
    float* qs = sa_smem;                              // [ROWS][dk4]
    float* ks = qs + SA_ROWS * dk4;                   // [KT][dk4 + 1]
    float* vs = ks + SA_KT * (dk4 + 1);               // [KT][dv] unless the values live in the key rows
    __shared__ long long key_base[SA_KT];
    __shared__ long long value_base[SA_KT];

    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    grid_dependency_wait();
    grid_dependents_go();
    const int item = p.tile_item[tile];
    if (p.item_slots && p.item_slots[item] < 0) return;      // a padding entry of a fixed-size batch
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(SA_ROWS, qlen * group - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* q = (const T*)p.q;
    const T* kp = (const T*)p.k_pages;
    const T* vp = (const T*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    // the tile's query rows, multiplied by their head's scale, zero beyond the tile and the key size
    for (int r = warp; r < SA_ROWS; r += SA_WARPS) {
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        const float sc = r < nrows ? p.head_scale[h] : 0.f;
        for (int d = lane; d < dk4; d += 32)
            qs[r * dk4 + d] = (r < nrows && d < dk) ? to_float(q[(size_t)tok * p.q_ld + (size_t)h * dk + d]) * sc : 0.f;
    }

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = sa_first_key(p, pos_first);
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + SA_KT - 1) / SA_KT) * SA_KT;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }

    float m[SA_RPW], l[SA_RPW], acc[SA_RPW][DPL];
    int pos[SA_RPW], first_key[SA_RPW];
#pragma unroll
    for (int i = 0; i < SA_RPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
        const int r = warp * SA_RPW + i;
        pos[i] = r < nrows ? pos0 + (row0 + r) / group : -1;       // -1: no row, sees nothing
        first_key[i] = sa_first_key(p, pos[i]);
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[i][c] = 0.f;
    }

    for (int k0 = kbegin; k0 < kend; k0 += SA_KT) {
        __syncthreads();
        if (tid < SA_KT) {
            const int kj = k0 + tid;
            long long kb = -1, vb = -1;
            if (kj < kend) {
                const int page = bt[kj / p.page_size];
                if (page >= 0) {
                    const long long at = (long long)kvh * p.page_size + kj % p.page_size;
                    kb = (long long)page * p.page_stride + at * dk;
                    vb = (long long)page * p.page_stride + at * p.value_ld;
                } else if (kj <= pos_last && kj >= sa_first_key(p, pos_first) && p.error) {
                    atomicExch(p.error, 3);            // some row of the tile sees this key, and its page was given back
                }
            }
            key_base[tid] = kb;
            value_base[tid] = vb;
        }
        __syncthreads();
        for (int j = warp; j < SA_KT; j += SA_WARPS) {
            const long long kb = key_base[j];
            for (int d = lane; d < dk4; d += 32)
                ks[j * (dk4 + 1) + d] = (kb >= 0 && d < dk) ? to_float(kp[kb + d]) : 0.f;
            if (!SHARED_V) {
                const long long vb = value_base[j];
                for (int d = lane; d < dv; d += 32) vs[j * dv + d] = vb >= 0 ? to_float(vp[vb + d]) : 0.f;
            }
        }
        __syncthreads();
        if (warp * SA_RPW >= nrows) continue;          // a warp without rows (it still took part in the copies)
        const int kj = k0 + lane;
        const bool key_ok = kj < kend && key_base[lane] >= 0;
        float s[SA_RPW];
#pragma unroll
        for (int i = 0; i < SA_RPW; ++i) s[i] = 0.f;
        const float* kr = ks + lane * (dk4 + 1);
        const float* qr = qs + warp * SA_RPW * dk4;
        for (int d = 0; d < dk4; d += 4) {
            const float k0v = kr[d], k1v = kr[d + 1], k2v = kr[d + 2], k3v = kr[d + 3];
#pragma unroll
            for (int i = 0; i < SA_RPW; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(qr + i * dk4 + d);
                s[i] = fmaf(qq.x, k0v, s[i]);
                s[i] = fmaf(qq.y, k1v, s[i]);
                s[i] = fmaf(qq.z, k2v, s[i]);
                s[i] = fmaf(qq.w, k3v, s[i]);
            }
        }
        float pj[SA_RPW];
        bool any = false;
#pragma unroll
        for (int i = 0; i < SA_RPW; ++i) {
            const bool seen = key_ok && kj <= pos[i] && kj >= first_key[i];
            const float si = seen ? s[i] : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(si));
            if (m_new == -INFINITY) { pj[i] = 0.f; continue; }       // uniform over the warp
            const float corr = expf(m[i] - m_new);
            pj[i] = seen ? expf(si - m_new) : 0.f;
            l[i] = l[i] * corr + warp_sum(pj[i]);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[i][c] *= corr;
            any = true;
        }
        if (!any) continue;
        const int nk = min(SA_KT, kend - k0);
        for (int j = 0; j < nk; ++j) {
            float pw[SA_RPW];
#pragma unroll
            for (int i = 0; i < SA_RPW; ++i) pw[i] = __shfl_sync(0xffffffffu, pj[i], j);
            const float* vr = SHARED_V ? ks + j * (dk4 + 1) : vs + j * dv;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                const float v = d < dv ? vr[d] : 0.f;
#pragma unroll
                for (int i = 0; i < SA_RPW; ++i) acc[i][c] = fmaf(pw[i], v, acc[i][c]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < SA_RPW; ++i) {
        const int r = warp * SA_RPW + i;
        if (r >= nrows) continue;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            T* o = (T*)p.out + (size_t)tok * p.out_ld + (size_t)h * dv;
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) o[d] = from_float<T>(acc[i][c] * inv);
            }
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* o = p.part_o + idx * dv;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) o[d] = acc[i][c];
            }
            if (lane == 0) { p.part_ml[idx * 2] = m[i]; p.part_ml[idx * 2 + 1] = l[i]; }
        }
    }
}

// ------------------------------------------------------------------------------------------
// The same attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit sums) for
// key sizes that are multiples of 16 and value sizes of 64, 128, 192, 256, 384 or 512.  A block
// owns the same tile of up to 32 query rows; its eight warps are two groups of 16 rows times four
// quarters.  Of a tile of 64 keys a warp first forms the scores of its 16 rows with ITS 16 keys
// over the whole key size, the four quarters exchange the rows' maxima through shared memory, the
// weights e^(s - m) go to shared memory as two bfloat16 halves (the weight and what rounding it
// lost, so that they stay 32-bit weights), and then the warp adds all 64 keys into ITS quarter of
// the value columns - with values 512 wide a warp still holds only 16 x 128 sums.  Keys and values
// come by cp.async into two slots: the next tile travels while this one is multiplied.  (A key whose
// page was given back arrives as zeros and sets the error flag; the exponentials are the fast ones.)
constexpr int TM_KT = 64;          // keys per tile
constexpr int TM_PAD = 8;          // elements between rows in shared memory beyond their width

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory; zeros when `valid` is false (nothing is read then)
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct MmaLayout {
    int ldk, ldv, ldp;
    size_t q_bytes, k_bytes, v_bytes, p_bytes, total;
    __host__ __device__ MmaLayout(int dk, int dv, bool shared_v) {
        ldk = dk + TM_PAD; ldv = dv + TM_PAD; ldp = TM_KT + TM_PAD;
        q_bytes = (size_t)SA_ROWS * ldk * 2;
        k_bytes = (size_t)2 * TM_KT * ldk * 2;
        v_bytes = shared_v ? 0 : (size_t)2 * TM_KT * ldv * 2;
        p_bytes = (size_t)2 * SA_ROWS * ldp * 2;
        total = q_bytes + k_bytes + v_bytes + p_bytes + 2 * SA_ROWS * 4 * sizeof(float) + 2 * TM_KT * sizeof(int);
    }
};

template <int NV, bool SHARED_V>
__global__ void __launch_bounds__(SA_WARPS * 32) scaled_attention_mma_kernel(const ScaledAttnParams p) {
    extern __shared__ __align__(16) unsigned char tm_smem[];
    const int dk = p.key_dim, dv = p.value_dim;
    const MmaLayout L(dk, dv, SHARED_V);
    bf16* Qs = reinterpret_cast<bf16*>(tm_smem);                                   // [32][ldk]
    bf16* Ks = reinterpret_cast<bf16*>(tm_smem + L.q_bytes);                       // [2][64][ldk]
    bf16* Vs = reinterpret_cast<bf16*>(tm_smem + L.q_bytes + L.k_bytes);           // [2][64][ldv]
    bf16* Ph = reinterpret_cast<bf16*>(tm_smem + L.q_bytes + L.k_bytes + L.v_bytes);   // [32][ldp] weights
    bf16* Pl = Ph + SA_ROWS * L.ldp;                                               //           and what rounding lost
    float* pmax = reinterpret_cast<float*>(Pl + SA_ROWS * L.ldp);                  // [32][4]
    float* psum = pmax + SA_ROWS * 4;                                              // [32][4]
    int* key_ok = reinterpret_cast<int*>(psum + SA_ROWS * 4);                      // [2][64]

    // blocks start in the order of the grid: the last tiles of a prompt see the most keys and go first
    const int kvh = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    grid_dependency_wait();
    grid_dependents_go();
    const int item = p.tile_item[tile];
    if (p.item_slots && p.item_slots[item] < 0) return;
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(SA_ROWS, qlen * group - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mi = warp >> 2, vi = warp & 3;             // which 16 rows; which quarter of keys / value columns
    const int g = lane >> 2, t = lane & 3;
    const bf16* q = (const bf16*)p.q;
    const bf16* kp = (const bf16*)p.k_pages;
    const bf16* vp = (const bf16*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = sa_first_key(p, pos_first);
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + TM_KT - 1) / TM_KT) * TM_KT;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }

    // one tile of keys (and values) on its way into slot `stage`: THREADS / 64 threads share a row, so
    // that all 64 page lookups are under way at once
    // the page of this thread's key in the tile that starts at k0 (asked for a tile ahead of its use)
    auto page_of = [&](int k0) {
        const int kj = k0 + tid / ((SA_WARPS * 32) / TM_KT);
        return kj < kend ? bt[kj / p.page_size] : -1;
    };
    auto issue_tile = [&](int stage, int k0, int page) {
        constexpr int TPR = (SA_WARPS * 32) / TM_KT;
        const int j = tid / TPR, part = tid % TPR;
        const int kj = k0 + j;
        if (kj < kend && page < 0 && part == 0 && p.error && kj <= pos_last &&
            kj >= sa_first_key(p, pos_first))
            atomicExch(p.error, 3);                // some row of the tile sees this key, and its page was given back
        const bool ok = page >= 0;
        const long long at = (long long)kvh * p.page_size + kj % p.page_size;
        const bf16* ksrc = kp + (ok ? (long long)page * p.page_stride + at * dk : 0);
        bf16* kdst = Ks + ((size_t)stage * TM_KT + j) * L.ldk;
        for (int c = part; c < dk / 8; c += TPR) cp_async16(kdst + c * 8, ksrc + c * 8, ok);
        if (!SHARED_V) {
            const bf16* vsrc = vp + (ok ? (long long)page * p.page_stride + at * p.value_ld : 0);
            bf16* vdst = Vs + ((size_t)stage * TM_KT + j) * L.ldv;
            for (int c = part; c < dv / 8; c += TPR) cp_async16(vdst + c * 8, vsrc + c * 8, ok);
        }
        if (part == 0) key_ok[stage * TM_KT + j] = ok;
        cp_async_commit();
    };
    if (kbegin < kend) issue_tile(0, kbegin, page_of(kbegin));
    int page_ahead = page_of(kbegin + TM_KT);

    // the tile's query rows as they are (the head's scale meets the scores), zero beyond the tile
    for (int r = warp; r < SA_ROWS; r += SA_WARPS) {
        const int row = row0 + r;
        const bf16* src = q + (size_t)(qstart + row / group) * p.q_ld + (size_t)(kvh * group + row % group) * dk;
        for (int c = lane; c < dk / 8; c += 32) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < nrows) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(Qs + r * L.ldk + c * 8) = v;
        }
    }

    // this thread's two rows: g and g + 8 of its group of 16
    int pos[2], first_key[2];
    float sc[2], m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = mi * 16 + g + 8 * i;
        pos[i] = r < nrows ? pos0 + (row0 + r) / group : -1;
        first_key[i] = sa_first_key(p, pos[i]);
        sc[i] = r < nrows ? p.head_scale[kvh * group + (row0 + r) % group] : 0.f;
        m[i] = -INFINITY; l[i] = 0.f;
    }
    float acc[NV][4];
#pragma unroll
    for (int n = 0; n < NV; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const int dvq = NV * 8;                              // value columns of this warp: vi * dvq ...
    const int ldvv = SHARED_V ? L.ldk : L.ldv;

    int it = 0;
    for (int k0 = kbegin; k0 < kend; k0 += TM_KT, ++it) {
        const int stage = it & 1;
        cp_async_wait_all();
        __syncthreads();                 // this tile has arrived; everybody is done with the tile before it
        if (k0 + TM_KT < kend) {
            issue_tile(stage ^ 1, k0 + TM_KT, page_ahead);
            page_ahead = page_of(k0 + 2 * TM_KT);
        }
        // ---- scores of 16 rows x 16 keys over the whole key size
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        {
            const bf16* qa = Qs + (mi * 16 + (lane & 15)) * L.ldk + (lane >> 4) * 8;
            const bf16* kb = Ks + ((size_t)stage * TM_KT + vi * 16 + (lane & 7) + (lane >> 4) * 8) * L.ldk + ((lane >> 3) & 1) * 8;
            for (int kk = 0; kk < dk; kk += 16) {
                uint32_t a[4], b[4];
                ldsm_x4(a, qa + kk);
                ldsm_x4(b, kb + kk);
                mma_bf16(s[0], a, b[0], b[1]);
                mma_bf16(s[1], a, b[2], b[3]);
            }
        }
        bool seen[2][4];
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int j = vi * 16 + n * 8 + 2 * t + (e & 1);
                const int kj = k0 + j;
                seen[n][e] = kj < kend && kj <= pos[i] && kj >= first_key[i];
                s[n][e] = seen[n][e] ? s[n][e] * sc[i] : -INFINITY;
                tmax[i] = fmaxf(tmax[i], s[n][e]);
            }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            if (t == 0) pmax[(mi * 16 + g + 8 * i) * 4 + vi] = tmax[i];
        }
        __syncthreads();                 // the four quarters' maxima of every row
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float4 q4 = *reinterpret_cast<const float4*>(pmax + (mi * 16 + g + 8 * i) * 4);
            const float m_new = fmaxf(m[i], fmaxf(fmaxf(q4.x, q4.y), fmaxf(q4.z, q4.w)));
            corr[i] = m_new == -INFINITY ? 1.f : __expf(m[i] - m_new);
            m[i] = m_new;
            l[i] *= corr[i];
        }
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            float pw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pw[e] = seen[n][e] ? __expf(s[n][e] - m[e >> 1]) : 0.f;
                l[e >> 1] += pw[e];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const __nv_bfloat162 hi = __floats2bfloat162_rn(pw[2 * i], pw[2 * i + 1]);
                const float2 back = __bfloat1622float2(hi);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(pw[2 * i] - back.x, pw[2 * i + 1] - back.y);
                const int at = (mi * 16 + g + 8 * i) * L.ldp + vi * 16 + n * 8 + 2 * t;
                *reinterpret_cast<__nv_bfloat162*>(Ph + at) = hi;
                *reinterpret_cast<__nv_bfloat162*>(Pl + at) = lo;
            }
        }
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            acc[n][0] *= corr[0]; acc[n][1] *= corr[0];
            acc[n][2] *= corr[1]; acc[n][3] *= corr[1];
        }
        __syncthreads();                 // the weights of all 64 keys
        // ---- 16 rows x this warp's value columns += weights x values, for both halves of the weights
        {
            const bf16* pa = Ph + (mi * 16 + (lane & 15)) * L.ldp + (lane >> 4) * 8;
            const bf16* pb = Pl + (mi * 16 + (lane & 15)) * L.ldp + (lane >> 4) * 8;
            const bf16* vbase = (SHARED_V ? Ks + (size_t)stage * TM_KT * L.ldk : Vs + (size_t)stage * TM_KT * L.ldv) +
                                ((lane & 7) + ((lane >> 3) & 1) * 8) * ldvv + vi * dvq + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < TM_KT; kk += 16) {
                uint32_t ah[4], al[4];
                ldsm_x4(ah, pa + kk);
                ldsm_x4(al, pb + kk);
#pragma unroll
                for (int np = 0; np < NV / 2; ++np) {
                    uint32_t b[4];
                    ldsm_x4_trans(b, vbase + (size_t)kk * ldvv + np * 16);
                    mma_bf16(acc[2 * np], ah, b[0], b[1]);
                    mma_bf16(acc[2 * np], al, b[0], b[1]);
                    mma_bf16(acc[2 * np + 1], ah, b[2], b[3]);
                    mma_bf16(acc[2 * np + 1], al, b[2], b[3]);
                }
            }
        }
    }

    // the rows' sums: over the four lanes that share a row, then over the four quarters
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        if (t == 0) psum[(mi * 16 + g + 8 * i) * 4 + vi] = l[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = mi * 16 + g + 8 * i;
        if (r >= nrows) continue;
        const float4 q4 = *reinterpret_cast<const float4*>(psum + r * 4);
        const float total = (q4.x + q4.y) + (q4.z + q4.w);
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            const float inv = total > 0.f ? 1.0f / total : 0.f;
            bf16* o = (bf16*)p.out + (size_t)tok * p.out_ld + (size_t)h * dv + vi * dvq + 2 * t;
#pragma unroll
            for (int n = 0; n < NV; ++n)
                *reinterpret_cast<__nv_bfloat162*>(o + n * 8) =
                    __floats2bfloat162_rn(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* o = p.part_o + idx * dv + vi * dvq + 2 * t;
#pragma unroll
            for (int n = 0; n < NV; ++n)
                *reinterpret_cast<float2*>(o + n * 8) = make_float2(acc[n][2 * i], acc[n][2 * i + 1]);
            if (vi == 0 && t == 0) { p.part_ml[idx * 2] = m[i]; p.part_ml[idx * 2 + 1] = total; }
        }
    }
}

// ------------------------------------------------------------------------------------------
// The tensor-core form for value sizes up to 256: a warp owns 16 query rows with ALL their value
// columns, so the weights never leave its registers (the score tile's accumulator layout is the
// layout of the next product's first operand) and the warps of a block meet only where a tile of
// keys changes hands.  A block is four warps = a tile of up to 64 query rows.
constexpr int TR_ROWS = 64, TR_WARPS = 4;

struct RowsLayout {
    int ldk, ldv;
    size_t q_bytes, k_bytes, v_bytes, total;
    __host__ __device__ RowsLayout(int dk, int dv, bool shared_v) {
        ldk = dk + TM_PAD; ldv = dv + TM_PAD;
        q_bytes = (size_t)TR_ROWS * ldk * 2;
        k_bytes = (size_t)2 * TM_KT * ldk * 2;
        v_bytes = shared_v ? 0 : (size_t)2 * TM_KT * ldv * 2;
        total = q_bytes + k_bytes + v_bytes + 2 * TM_KT * sizeof(int);
    }
};

template <int NVT, bool SHARED_V>
__global__ void __launch_bounds__(TR_WARPS * 32) scaled_attention_rows_kernel(const ScaledAttnParams p) {
    extern __shared__ __align__(16) unsigned char tr_smem[];
    const int dk = p.key_dim, dv = p.value_dim;
    const RowsLayout L(dk, dv, SHARED_V);
    bf16* Qs = reinterpret_cast<bf16*>(tr_smem);                                   // [64][ldk]
    bf16* Ks = reinterpret_cast<bf16*>(tr_smem + L.q_bytes);                       // [2][64][ldk]
    bf16* Vs = reinterpret_cast<bf16*>(tr_smem + L.q_bytes + L.k_bytes);           // [2][64][ldv]
    int* key_ok = reinterpret_cast<int*>(tr_smem + L.q_bytes + L.k_bytes + L.v_bytes);   // [2][64]

    // blocks start in the order of the grid: the last tiles of a prompt see the most keys and go first
    const int kvh = blockIdx.x, tile = gridDim.y - 1 - blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    grid_dependency_wait();
    grid_dependents_go();
    const int item = p.tile_item[tile];
    if (p.item_slots && p.item_slots[item] < 0) return;
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(TR_ROWS, qlen * group - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bf16* q = (const bf16*)p.q;
    const bf16* kp = (const bf16*)p.k_pages;
    const bf16* vp = (const bf16*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = sa_first_key(p, pos_first);
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + TM_KT - 1) / TM_KT) * TM_KT;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }

    // one tile of keys (and values) on its way into slot `stage`: THREADS / 64 threads share a row, so
    // that all 64 page lookups are under way at once
    // the page of this thread's key in the tile that starts at k0 (asked for a tile ahead of its use)
    auto page_of = [&](int k0) {
        const int kj = k0 + tid / ((TR_WARPS * 32) / TM_KT);
        return kj < kend ? bt[kj / p.page_size] : -1;
    };
    auto issue_tile = [&](int stage, int k0, int page) {
        constexpr int TPR = (TR_WARPS * 32) / TM_KT;
        const int j = tid / TPR, part = tid % TPR;
        const int kj = k0 + j;
        if (kj < kend && page < 0 && part == 0 && p.error && kj <= pos_last &&
            kj >= sa_first_key(p, pos_first))
            atomicExch(p.error, 3);                // some row of the tile sees this key, and its page was given back
        const bool ok = page >= 0;
        const long long at = (long long)kvh * p.page_size + kj % p.page_size;
        const bf16* ksrc = kp + (ok ? (long long)page * p.page_stride + at * dk : 0);
        bf16* kdst = Ks + ((size_t)stage * TM_KT + j) * L.ldk;
        for (int c = part; c < dk / 8; c += TPR) cp_async16(kdst + c * 8, ksrc + c * 8, ok);
        if (!SHARED_V) {
            const bf16* vsrc = vp + (ok ? (long long)page * p.page_stride + at * p.value_ld : 0);
            bf16* vdst = Vs + ((size_t)stage * TM_KT + j) * L.ldv;
            for (int c = part; c < dv / 8; c += TPR) cp_async16(vdst + c * 8, vsrc + c * 8, ok);
        }
        if (part == 0) key_ok[stage * TM_KT + j] = ok;
        cp_async_commit();
    };
    if (kbegin < kend) issue_tile(0, kbegin, page_of(kbegin));
    int page_ahead = page_of(kbegin + TM_KT);

    for (int r = warp; r < TR_ROWS; r += TR_WARPS) {
        const int row = row0 + r;
        const bf16* src = q + (size_t)(qstart + row / group) * p.q_ld + (size_t)(kvh * group + row % group) * dk;
        for (int c = lane; c < dk / 8; c += 32) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < nrows) v = *reinterpret_cast<const uint4*>(src + c * 8);
            *reinterpret_cast<uint4*>(Qs + r * L.ldk + c * 8) = v;
        }
    }

    int pos[2], first_key[2];
    float sc[2], m[2], l[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 16 + g + 8 * i;
        pos[i] = r < nrows ? pos0 + (row0 + r) / group : -1;
        first_key[i] = sa_first_key(p, pos[i]);
        sc[i] = r < nrows ? p.head_scale[kvh * group + (row0 + r) % group] : 0.f;
        m[i] = -INFINITY; l[i] = 0.f;
    }
    // the latest position among this warp's rows: tiles of keys beyond it are none of its business
    const int warp_rows = min(16, nrows - warp * 16);
    const int warp_last = warp_rows > 0 ? pos0 + (row0 + warp * 16 + warp_rows - 1) / group : -1;
    const int warp_first = warp_rows > 0 ? pos0 + (row0 + warp * 16) / group : 0;
    float acc[NVT][4];
#pragma unroll
    for (int n = 0; n < NVT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const int ldvv = SHARED_V ? L.ldk : L.ldv;

    int it = 0;
    for (int k0 = kbegin; k0 < kend; k0 += TM_KT, ++it) {
        const int stage = it & 1;
        cp_async_wait_all();
        __syncthreads();                 // this tile has arrived; everybody is done with the tile before it
        if (k0 + TM_KT < kend) {
            issue_tile(stage ^ 1, k0 + TM_KT, page_ahead);
            page_ahead = page_of(k0 + 2 * TM_KT);
        }
        if (k0 > warp_last || k0 + TM_KT - 1 < sa_first_key(p, warp_first)) continue;
        // ---- scores of 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
        {
            const bf16* qa = Qs + (warp * 16 + (lane & 15)) * L.ldk + (lane >> 4) * 8;
            const bf16* kb = Ks + ((size_t)stage * TM_KT + (lane & 7) + (lane >> 4) * 8) * L.ldk + ((lane >> 3) & 1) * 8;
            for (int kk = 0; kk < dk; kk += 16) {
                uint32_t a[4];
                ldsm_x4(a, qa + kk);
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    uint32_t b[4];
                    ldsm_x4(b, kb + (size_t)nb * 16 * L.ldk + kk);
                    mma_bf16(s[2 * nb], a, b[0], b[1]);
                    mma_bf16(s[2 * nb + 1], a, b[2], b[3]);
                }
            }
        }
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int j = n * 8 + 2 * t + (e & 1);
                const int kj = k0 + j;
                const bool seen = kj < kend && kj <= pos[i] && kj >= first_key[i];
                s[n][e] = seen ? s[n][e] * sc[i] : -INFINITY;
                tmax[i] = fmaxf(tmax[i], s[n][e]);
            }
        float corr[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float m_new = fmaxf(m[i], tmax[i]);
            corr[i] = m_new == -INFINITY ? 1.f : __expf(m[i] - m_new);
            m[i] = m_new;
            l[i] *= corr[i];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[n][e] = s[n][e] == -INFINITY ? 0.f : __expf(s[n][e] - m[e >> 1]);
                l[e >> 1] += s[n][e];
            }
#pragma unroll
        for (int n = 0; n < NVT; ++n) {
            acc[n][0] *= corr[0]; acc[n][1] *= corr[0];
            acc[n][2] *= corr[1]; acc[n][3] *= corr[1];
        }
        // ---- 16 rows x all value columns += weights x values; the weights as two bfloat16 halves
        const bf16* vbase = (SHARED_V ? Ks + (size_t)stage * TM_KT * L.ldk : Vs + (size_t)stage * TM_KT * L.ldv) +
                            ((lane & 7) + ((lane >> 3) & 1) * 8) * ldvv + (lane >> 4) * 8;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t ah[4], al[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const float w0 = s[2 * kk + (x >> 1)][2 * (x & 1)], w1 = s[2 * kk + (x >> 1)][2 * (x & 1) + 1];
                const __nv_bfloat162 hi = __floats2bfloat162_rn(w0, w1);
                const float2 back = __bfloat1622float2(hi);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(w0 - back.x, w1 - back.y);
                ah[x] = *reinterpret_cast<const uint32_t*>(&hi);
                al[x] = *reinterpret_cast<const uint32_t*>(&lo);
            }
#pragma unroll
            for (int np = 0; np < NVT / 2; ++np) {
                uint32_t b[4];
                ldsm_x4_trans(b, vbase + (size_t)kk * 16 * ldvv + np * 16);
                mma_bf16(acc[2 * np], ah, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], ah, b[2], b[3]);
                mma_bf16(acc[2 * np], al, b[0], b[1]);
                mma_bf16(acc[2 * np + 1], al, b[2], b[3]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        const int r = warp * 16 + g + 8 * i;
        if (r >= nrows) continue;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
            bf16* o = (bf16*)p.out + (size_t)tok * p.out_ld + (size_t)h * dv + 2 * t;
#pragma unroll
            for (int n = 0; n < NVT; ++n)
                *reinterpret_cast<__nv_bfloat162*>(o + n * 8) =
                    __floats2bfloat162_rn(acc[n][2 * i] * inv, acc[n][2 * i + 1] * inv);
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* o = p.part_o + idx * dv + 2 * t;
#pragma unroll
            for (int n = 0; n < NVT; ++n)
                *reinterpret_cast<float2*>(o + n * 8) = make_float2(acc[n][2 * i], acc[n][2 * i + 1]);
            if (t == 0) { p.part_ml[idx * 2] = m[i]; p.part_ml[idx * 2 + 1] = l[i]; }
        }
    }
}

// o = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M) over the key ranges z of one (token, head)
template <typename T>
__global__ void sa_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  T* __restrict__ out, int out_ld, int tokens, int heads, int dv,
                                  int nsplit) {
    const int tok = blockIdx.x, h = blockIdx.y;
    float mmax = -INFINITY;
    for (int z = 0; z < nsplit; ++z)
        mmax = fmaxf(mmax, part_ml[(((size_t)z * tokens + tok) * heads + h) * 2]);
    float denom = 0.f;
    for (int z = 0; z < nsplit; ++z) {
        const size_t idx = ((size_t)z * tokens + tok) * heads + h;
        const float mz = part_ml[idx * 2];
        if (mz != -INFINITY) denom += part_ml[idx * 2 + 1] * expf(mz - mmax);
    }
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < nsplit; ++z) {
            const size_t idx = ((size_t)z * tokens + tok) * heads + h;
            const float mz = part_ml[idx * 2];
            if (mz != -INFINITY) o += part_o[idx * dv + d] * expf(mz - mmax);
        }
        out[(size_t)tok * out_ld + (size_t)h * dv + d] = from_float<T>(o * inv);
    }
}

// One block per token of proj = [ q (heads x dim) | k (kv_heads x dim) | v (kv_heads x vdim) ].
//   q, k   pairs (i, i + rotary_dim / 2) of every head turn by the token's angles (cos | sin rows of
//          the table); q in place, k into its page
//   v      mix_mode 1: also copied as it is into v_first[t];  2: v <- (1 - mix) v + mix v_first[t];
//          then into its page.  mix is one float on the device.
template <typename T>
__global__ void rotate_mix_write_kernel(T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                        const float* __restrict__ cos_sin, int table_len,
                                        const int* __restrict__ slot_of, T* __restrict__ k_pages,
                                        T* __restrict__ v_pages, long long page_stride, int page_size,
                                        int heads, int kv_heads, int dim, int vdim, int rotary_dim,
                                        int mix_mode, const float* __restrict__ mix, T* __restrict__ v_first,
                                        int* __restrict__ error) {
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependents_go();
    const int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    T* row = proj + (size_t)t * ld;
    const int slot = slot_of ? slot_of[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int off = slot >= 0 ? slot % page_size : 0;
    // queries: rotated in place
    for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        T* a = row + h * dim + i;
        const float u = to_float(a[0]), v = to_float(a[half]);
        const float c = cs[i], s = cs[half + i];
        a[0] = from_float<T>(u * c - v * s);
        a[half] = from_float<T>(v * c + u * s);
    }
    if (slot < 0) return;
    // keys: rotated pairs and the columns that pass unchanged, into the page
    const T* k = row + heads * dim;
    for (int e = threadIdx.x; e < kv_heads * dim; e += blockDim.x) {
        const int g = e / dim, d = e - g * dim;
        float val = to_float(k[e]);
        if (d < rotary_dim) {
            const int i = d < half ? d : d - half;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(k[g * dim + (d < half ? d + half : d - half)]);
            val = d < half ? val * c - other * s : val * c + other * s;
        }
        k_pages[page * page_stride + ((long long)g * page_size + off) * dim + d] = from_float<T>(val);
    }
    // values: blended with the first blending layer's, into the page
    const T* v = k + kv_heads * dim;
    const float lambda = mix_mode == 2 ? mix[0] : 0.f;
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) {
        const int g = e / vdim, d = e - g * vdim;
        float val = to_float(v[e]);
        if (mix_mode == 1) v_first[(size_t)t * kv_heads * vdim + e] = v[e];
        if (mix_mode == 2) val = (1.0f - lambda) * val + lambda * to_float(v_first[(size_t)t * kv_heads * vdim + e]);
        v_pages[page * page_stride + ((long long)g * page_size + off) * vdim + d] = from_float<T>(val);
    }
}

// One block per token of proj = [ q (heads x dim) | k (kv_heads x dim) | v (kv_heads x vdim) | ... ],
// a warp per head of q and k in turn.
//   q, k   with gains (q_gain, k_gain [dim], shared by the heads): every head divided by its root
//          mean square (eps inside the root) times the gain, in 32-bit, BEFORE the rotation;
//          then pairs (i, i + rotary_dim / 2) turn by the token's angles; q in place, k into its page
//   v      into its page as it is
template <typename T>
__global__ void norm_rotate_write_kernel(T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                         const float* __restrict__ cos_sin, int table_len,
                                         const int* __restrict__ slot_of, T* __restrict__ k_pages,
                                         T* __restrict__ v_pages, long long page_stride, int page_size,
                                         int heads, int kv_heads, int dim, int vdim, int rotary_dim,
                                         const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                         float eps, int* __restrict__ error) {
    extern __shared__ float nr_smem[];                 // [warps][dim]
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependents_go();
    const int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    T* row = proj + (size_t)t * ld;
    const int slot = slot_of ? slot_of[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int off = slot >= 0 ? slot % page_size : 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float* mine = nr_smem + (size_t)warp * dim;
    for (int h = warp; h < heads + kv_heads; h += warps) {
        const bool is_q = h < heads;
        if (!is_q && slot < 0) continue;               // nothing to store (uniform over the warp)
        T* src = row + (size_t)h * dim;
        const float* gain = is_q ? q_gain : k_gain;
        float sq = 0.f;
        for (int d = lane; d < dim; d += 32) {
            const float v = to_float(src[d]);
            mine[d] = v;
            sq += v * v;
        }
        if (gain) {
            const float inv = 1.0f / sqrtf(warp_sum(sq) / (float)dim + eps);
            for (int d = lane; d < dim; d += 32) mine[d] = mine[d] * inv * gain[d];
        }
        __syncwarp();
        T* dst = is_q ? src : k_pages + page * page_stride + ((long long)(h - heads) * page_size + off) * dim;
        for (int d = lane; d < dim; d += 32) {
            float val = mine[d];
            if (d < rotary_dim) {
                const int i = d < half ? d : d - half;
                const float c = cs[i], sn = cs[half + i];
                const float other = mine[d < half ? d + half : d - half];
                val = d < half ? val * c - other * sn : val * c + other * sn;
            }
            dst[d] = from_float<T>(val);
        }
        __syncwarp();
    }
    if (slot < 0) return;
    const T* v = row + (size_t)(heads + kv_heads) * dim;
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) {
        const int g = e / vdim, d = e - g * vdim;
        v_pages[page * page_stride + ((long long)g * page_size + off) * vdim + d] = v[e];
    }
}

// out[t, h, :] <- out[t, h, :] * sigmoid(gate[t, h]): one number per token and head.  VEC: vdim a
// multiple of 8 and rows on 16 bytes, eight columns per thread and trip.
template <typename T, bool VEC>
__global__ void head_gate_kernel(T* __restrict__ out, int out_ld, const T* __restrict__ gate, int gate_ld,
                                 int heads, int vdim) {
    grid_dependency_wait();
    grid_dependents_go();
    const size_t t = blockIdx.x;
    T* o = out + t * out_ld;
    const T* g = gate + t * gate_ld;
    if (VEC) {
        for (int c = threadIdx.x * 8; c < heads * vdim; c += blockDim.x * 8) {
            const float s = 1.0f / (1.0f + expf(-to_float(g[c / vdim])));
            float v[8];
            load8(o + c, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= s;
            store8(o + c, v);
        }
        return;
    }
    for (int c = threadIdx.x; c < heads * vdim; c += blockDim.x) {
        const float s = 1.0f / (1.0f + expf(-to_float(g[c / vdim])));
        o[c] = from_float<T>(to_float(o[c]) * s);
    }
}

template <typename T, int DPL>
static int scaled_attention_launch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const int dk4 = (p.key_dim + 3) & ~3;
    const size_t smem = sizeof(float) * ((size_t)SA_ROWS * dk4 + (size_t)SA_KT * (dk4 + 1) +
                                         (shared_v ? 0 : (size_t)SA_KT * p.value_dim));
    if (smem > 220 * 1024) return ERR_UNSUPPORTED;
    const dim3 grid(p.kv_heads, tiles, p.nsplit);
    if (shared_v) {
        cudaFuncSetAttribute(scaled_attention_kernel<T, DPL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(scaled_attention_kernel<T, DPL, true>, grid, dim3(SA_WARPS * 32), smem, stream, p);
    }
    cudaFuncSetAttribute(scaled_attention_kernel<T, DPL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(scaled_attention_kernel<T, DPL, false>, grid, dim3(SA_WARPS * 32), smem, stream, p);
}

template <typename T>
static int scaled_attention_dispatch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const int dpl = (p.value_dim + 31) / 32;
    if (dpl <= 2) return scaled_attention_launch<T, 2>(p, tiles, shared_v, stream);
    if (dpl <= 4) return scaled_attention_launch<T, 4>(p, tiles, shared_v, stream);
    if (dpl <= 8) return scaled_attention_launch<T, 8>(p, tiles, shared_v, stream);
    if (dpl <= 16) return scaled_attention_launch<T, 16>(p, tiles, shared_v, stream);
    return ERR_UNSUPPORTED;
}


template <int NV>
static int scaled_attention_mma_launch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const size_t smem = MmaLayout(p.key_dim, p.value_dim, shared_v).total;
    const dim3 grid(p.kv_heads, tiles, p.nsplit);
    if (shared_v) {
        cudaFuncSetAttribute(scaled_attention_mma_kernel<NV, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(scaled_attention_mma_kernel<NV, true>, grid, dim3(SA_WARPS * 32), smem, stream, p);
    }
    cudaFuncSetAttribute(scaled_attention_mma_kernel<NV, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(scaled_attention_mma_kernel<NV, false>, grid, dim3(SA_WARPS * 32), smem, stream, p);
}

template <int NVT>
static int scaled_attention_rows_launch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const size_t smem = RowsLayout(p.key_dim, p.value_dim, shared_v).total;
    const dim3 grid(p.kv_heads, tiles, p.nsplit);
    if (shared_v) {
        cudaFuncSetAttribute(scaled_attention_rows_kernel<NVT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(scaled_attention_rows_kernel<NVT, true>, grid, dim3(TR_WARPS * 32), smem, stream, p);
    }
    cudaFuncSetAttribute(scaled_attention_rows_kernel<NVT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(scaled_attention_rows_kernel<NVT, false>, grid, dim3(TR_WARPS * 32), smem, stream, p);
}

// whether the tensor-core form of a warp per 16 rows takes these sizes (value sizes up to 256)
static bool scaled_attention_rows_takes(int key_dim, int value_dim, bool shared_v) {
    return value_dim <= 256 && RowsLayout(key_dim, value_dim, shared_v).total <= 227 * 1024;
}

// whether the tensor-core form takes these sizes and addresses
static bool scaled_attention_mma_takes(const ScaledAttnParams& p, int dtype, bool shared_v) {
    const int dv = p.value_dim;
    if (dtype != DTYPE_BF16 || p.key_dim % 16 || !(dv == 64 || dv == 128 || dv == 192 || dv == 256 || dv == 384 || dv == 512))
        return false;
    if (p.page_stride % 8 || p.q_ld % 8 || p.out_ld % 2 || p.value_ld % 8) return false;
    if (((size_t)p.q | (size_t)p.k_pages | (size_t)p.v_pages) & 15 || ((size_t)p.out & 3)) return false;
    return MmaLayout(p.key_dim, dv, shared_v).total <= 227 * 1024;
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_scaled_attention_rows() { return SA_ROWS; }

// Query rows of one tile for these sizes: 64 where a warp of the tensor-core kernel owns 16 rows
// with all their value columns (bfloat16, key sizes in steps of 16, value sizes 64, 128, 192, 256;
// form 0 or 2), else 32.  The caller cuts its tile list accordingly.  form 3 asks for the
// tensor-core kernel whose warps split the value columns at any value size it takes.
int fsie_scaled_attention_tile_rows(int dtype, int key_dim, int value_dim, int values_in_keys, int form) {
    if (dtype != DTYPE_BF16 || form == 1 || form == 3 || key_dim % 16 || value_dim % 64) return SA_ROWS;
    return scaled_attention_rows_takes(key_dim, value_dim, values_in_keys != 0) ? TR_ROWS : SA_ROWS;
}

// values_in_keys != 0: v_pages is ignored, a key row's first value_dim columns are its value row.
// form 0: the tensor-core kernel where it takes the sizes (bfloat16), else the 32-bit one; 1: the
// 32-bit kernel; 2: a tensor-core kernel or refusal; 3: the tensor-core kernel whose warps split the
// value columns, or refusal.  The tiles hold fsie_scaled_attention_tile_rows(...) rows.
// With nsplit > 1 the caller gives part_o [nsplit, tokens, heads, value_dim] and part_ml
// [nsplit, tokens, heads, 2] (float); the ranges are merged after the launch.
int fsie_scaled_attention(const void* q, int q_ld, const float* head_scale, const void* k_pages,
                          const void* v_pages, long long page_stride, int page_size, int key_dim,
                          int value_dim, int values_in_keys, const int* block_tables, int bt_stride,
                          const int* tile_item, const int* tile_row0, int tiles, const int* item_qstart,
                          const int* item_qlen, const int* item_pos0, const int* item_slots, void* out,
                          int out_ld, float* part_o, float* part_ml, int tokens, int heads, int kv_heads,
                          int window, int chunk, int nsplit, int dtype, int form, int* error,
                          cudaStream_t stream) {
    if (tokens <= 0 || tiles <= 0) return 0;
    if (tiles > 65535 || nsplit > 65535) return ERR_UNSUPPORTED;
    if (key_dim <= 0 || value_dim <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 ||
        page_size <= 0 || window < 0 || chunk < 0 || (values_in_keys && value_dim > key_dim))
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    ScaledAttnParams p;
    p.q = q; p.q_ld = q_ld; p.head_scale = head_scale;
    p.k_pages = k_pages; p.v_pages = values_in_keys ? k_pages : v_pages;
    p.page_stride = page_stride; p.page_size = page_size;
    p.key_dim = key_dim; p.value_dim = value_dim; p.value_ld = values_in_keys ? key_dim : value_dim;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0; p.item_slots = item_slots;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.window = window; p.nsplit = nsplit;
    p.chunk = chunk;
    p.error = error;
    int rc;
    const int tile_rows = fsie_scaled_attention_tile_rows(dtype, key_dim, value_dim, values_in_keys, form);
    if (tile_rows == TR_ROWS) {
        // the caller has cut tiles of 64 rows: no other kernel may take them
        if (!scaled_attention_mma_takes(p, dtype, values_in_keys != 0)) return ERR_UNSUPPORTED;
        switch (value_dim / 64) {
            case 1: rc = scaled_attention_rows_launch<8>(p, tiles, values_in_keys != 0, stream); break;
            case 2: rc = scaled_attention_rows_launch<16>(p, tiles, values_in_keys != 0, stream); break;
            case 3: rc = scaled_attention_rows_launch<24>(p, tiles, values_in_keys != 0, stream); break;
            default: rc = scaled_attention_rows_launch<32>(p, tiles, values_in_keys != 0, stream); break;
        }
    } else if (form != 1 && scaled_attention_mma_takes(p, dtype, values_in_keys != 0)) {
        switch (value_dim / 32) {
            case 2: rc = scaled_attention_mma_launch<2>(p, tiles, values_in_keys != 0, stream); break;
            case 4: rc = scaled_attention_mma_launch<4>(p, tiles, values_in_keys != 0, stream); break;
            case 6: rc = scaled_attention_mma_launch<6>(p, tiles, values_in_keys != 0, stream); break;
            case 8: rc = scaled_attention_mma_launch<8>(p, tiles, values_in_keys != 0, stream); break;
            case 12: rc = scaled_attention_mma_launch<12>(p, tiles, values_in_keys != 0, stream); break;
            default: rc = scaled_attention_mma_launch<16>(p, tiles, values_in_keys != 0, stream); break;
        }
    } else if (form >= 2) {
        return ERR_UNSUPPORTED;
    } else {
        rc = dtype == DTYPE_F32 ? scaled_attention_dispatch<float>(p, tiles, values_in_keys != 0, stream)
                                : scaled_attention_dispatch<bf16>(p, tiles, values_in_keys != 0, stream);
    }
    if (rc != 0 || nsplit == 1) return rc;
    const dim3 cgrid(tokens, heads);
    const int threads = value_dim >= 128 ? 128 : (value_dim >= 64 ? 64 : 32);
    if (dtype == DTYPE_F32)
        sa_combine_kernel<float><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (float*)out, out_ld, tokens, heads, value_dim, nsplit);
    else
        sa_combine_kernel<bf16><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (bf16*)out, out_ld, tokens, heads, value_dim, nsplit);
    return FSIE_LAUNCH_CHECK();
}

// proj [tokens, ld] = q | k | v head by head; cos_sin [table_len, rotary_dim]; slot_of [tokens]
// (page * page_size + offset, -1: store nothing).  mix_mode 0: values as they are; 1: values also
// copied to v_first [tokens, kv_heads * vdim]; 2: values blended with v_first by *mix.
int fsie_rotate_mix_write(void* proj, int ld, const int* positions, const float* cos_sin, int table_len,
                          const int* slot_of, void* k_pages, void* v_pages, long long page_stride,
                          int page_size, int tokens, int heads, int kv_heads, int dim, int vdim,
                          int rotary_dim, int mix_mode, const float* mix, void* v_first, int dtype,
                          int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dim || (rotary_dim & 1) || mix_mode < 0 || mix_mode > 2 ||
        (mix_mode != 0 && !v_first) || (mix_mode == 2 && !mix) || ld < (heads + kv_heads) * dim + kv_heads * vdim)
        return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return launch_dependent(rotate_mix_write_kernel<float>, dim3(tokens), dim3(256), 0, stream,
                                (float*)proj, ld, positions, cos_sin, table_len, slot_of, (float*)k_pages,
                                (float*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim,
                                rotary_dim, mix_mode, mix, (float*)v_first, error);
    return launch_dependent(rotate_mix_write_kernel<bf16>, dim3(tokens), dim3(256), 0, stream,
                            (bf16*)proj, ld, positions, cos_sin, table_len, slot_of, (bf16*)k_pages,
                            (bf16*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim,
                            rotary_dim, mix_mode, mix, (bf16*)v_first, error);
}


// proj [tokens, ld] = q | k | v head by head (more columns may follow); q_gain / k_gain [dim] float or
// null (no norm of that side); cos_sin [table_len, rotary_dim]; slot_of [tokens] (page * page_size +
// offset, -1: store nothing).
int fsie_norm_rotate_write(void* proj, int ld, const int* positions, const float* cos_sin, int table_len,
                           const int* slot_of, void* k_pages, void* v_pages, long long page_stride,
                           int page_size, int tokens, int heads, int kv_heads, int dim, int vdim,
                           int rotary_dim, const float* q_gain, const float* k_gain, float eps, int dtype,
                           int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dim || (rotary_dim & 1) || dim <= 0 ||
        ld < (heads + kv_heads) * dim + kv_heads * vdim)
        return ERR_BAD_ARGUMENT;
    const int warps = 8;
    const size_t smem = (size_t)warps * dim * sizeof(float);
    if (smem > 48 * 1024) return ERR_UNSUPPORTED;
    if (dtype == DTYPE_F32)
        return launch_dependent(norm_rotate_write_kernel<float>, dim3(tokens), dim3(warps * 32), smem, stream,
                                (float*)proj, ld, positions, cos_sin, table_len, slot_of, (float*)k_pages,
                                (float*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim, rotary_dim,
                                q_gain, k_gain, eps, error);
    return launch_dependent(norm_rotate_write_kernel<bf16>, dim3(tokens), dim3(warps * 32), smem, stream,
                            (bf16*)proj, ld, positions, cos_sin, table_len, slot_of, (bf16*)k_pages,
                            (bf16*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim, rotary_dim,
                            q_gain, k_gain, eps, error);
}

// out [tokens, out_ld] holds heads x vdim columns per token, gate [tokens, gate_ld] one column per head.
int fsie_head_gate(void* out, int out_ld, const void* gate, int gate_ld, int tokens, int heads, int vdim,
                   int dtype, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0 || vdim <= 0) return 0;
    const bool vec = vdim % 8 == 0 && out_ld % 8 == 0 && (((size_t)out) & (dtype == DTYPE_F32 ? 31 : 15)) == 0;
    const int threads = vec ? (heads * vdim >= 2048 ? 256 : 128) : (heads * vdim >= 1024 ? 256 : 128);
#define FSIE_HEAD_GATE(T, V) launch_dependent(head_gate_kernel<T, V>, dim3(tokens), dim3(threads), 0, stream, (T*)out, \
                                              out_ld, (const T*)gate, gate_ld, heads, vdim)
    if (dtype == DTYPE_F32) return vec ? FSIE_HEAD_GATE(float, true) : FSIE_HEAD_GATE(float, false);
    return vec ? FSIE_HEAD_GATE(bf16, true) : FSIE_HEAD_GATE(bf16, false);
#undef FSIE_HEAD_GATE
}

}  // extern "C"
