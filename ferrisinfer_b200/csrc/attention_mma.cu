// Attention over the paged bf16 cache on the tensor cores, for head sizes 64 and 128 and pages of a
// multiple of 16 tokens: a split-KV kernel for steps of single tokens (decode) with its merge, and a
// kernel for portions of prompts (prefill).  Both stream 16-key tiles of K and V from the pages by
// TMA (128-byte swizzle, boxes addressed through the request's block table), form q.k with
// mma.sync m16n8k16 (bf16 in, fp32 out), keep the softmax (scale, running maximum, sum) in fp32,
// and share one tile routine.
//
// The formulas are those of the reference's streaming attention
// (crates/ferrisinfer-kernel/src/cpu/attention.rs:729-781, 1125-1155): query head hq reads kv head
// hq / (nh / nkv); s = (q . k) * scale; the query at position P attends keys lo..P (lo = 0, or
// P - window + 1); out = sum softmax(s) v.  The rows of an MMA tile are (token, head of the group)
// pairs that share one kv head, so the keys and values of a group are loaded once for all its heads.
//
// Every mbarrier wait is bounded; a wait that runs out records its place in the status word and
// the kernel runs on to its end with a wrong result instead of hanging.
#include <limits.h>
#include <stdlib.h>

#include <type_traits>
#include <math.h>

#include "common.cuh"
#include "sm100.cuh"

namespace {

constexpr int TILE_KEYS = 16;
constexpr int WARPS = 4;
constexpr int ROW_CACHE = 64;  // block-table look-ups a warp keeps ahead
constexpr int MAX_CLUSTER = 16;  // key ranges that one thread-block cluster merges (more than 8: not portable, but B200's)

// Position limits of one thread's two rows (g and g + 8 of the warp's 16-row slab).
struct RowLimits {
    int hi[2];  // last key a row may see (its own position); -1 for a row that does not exist
    int lo[2];  // first key it may see
};

template <int D>
struct WarpState {
    uint32_t q[D / 16][4];  // A fragments of the 16 x D query slab
    float o[D / 8][4];      // output accumulators
    float m[2], l[2];       // running maximum and (per-thread partial) sum of rows g and g + 8
};

template <int D>
__device__ __forceinline__ void init_state(WarpState<D>& st) {
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[n][e] = 0.0f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
}

// Load the query fragments of rows g and g + 8; row pointers may be null (rows that do not exist).
template <int D>
__device__ __forceinline__ void load_q(WarpState<D>& st, const bf16* row0, const bf16* row1) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int c = ks * 16 + 2 * t;
        st.q[ks][0] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c) : 0u;
        st.q[ks][1] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c) : 0u;
        st.q[ks][2] = row0 ? *reinterpret_cast<const uint32_t*>(row0 + c + 8) : 0u;
        st.q[ks][3] = row1 ? *reinterpret_cast<const uint32_t*>(row1 + c + 8) : 0u;
    }
}

// One tile of 16 keys starting at absolute key `key0`; K and V tiles lie in shared memory as D/64
// swizzled boxes of 16 rows x 128 bytes each (box c = columns 64c .. 64c+63).
// CS: bytes between the 64-column boxes of one tile (2048 when the boxes of K lie together and those of V after them;
// 4096 when each box of K is followed by the box of V of the same columns).
template <int D, int CS = 2048>
__device__ __forceinline__ void attend_tile(WarpState<D>& st, uint32_t k_smem, uint32_t v_smem, int key0,
                                            const RowLimits& lim, float scale) {
    const int lane = threadIdx.x & 31;
    const int t = lane & 3;
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;

    // scores: S[16 x 16] = Q[16 x D] K^T
    {
        const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
                const int cc = 2 * ks + mi;  // 16-byte chunk of the row: k columns 8cc .. 8cc+7
                uint32_t r[4];
                ldmatrix_x4(r, k_smem + (cc >> 3) * CS + swizzle128(8 * j + r8, cc & 7));
                mma_bf16_16816(s[j], st.q[ks], r[0], r[1]);
                mma_bf16_16816(s[j], st.q[ks + 1], r[2], r[3]);
            }
        }
    }
    // scale, mask, running maximum
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = e >> 1;
            const int key = key0 + 8 * j + 2 * t + (e & 1);
            const bool ok = key <= lim.hi[row] && key >= lim.lo[row];
            s[j][e] = ok ? s[j][e] * scale : -INFINITY;
            mx[row] = fmaxf(mx[row], s[j][e]);
        }
    float corr[2], base[2];
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
        const float m_new = fmaxf(st.m[row], mx[row]);
        base[row] = m_new == -INFINITY ? 0.0f : m_new;  // a row that has seen no key yet
        corr[row] = st.m[row] == -INFINITY ? 0.0f : expf(st.m[row] - base[row]);
        st.m[row] = m_new;
        st.l[row] *= corr[row];
    }
    uint32_t p[4];
    {
        float e00 = expf(s[0][0] - base[0]), e01 = expf(s[0][1] - base[0]);
        float e02 = expf(s[0][2] - base[1]), e03 = expf(s[0][3] - base[1]);
        float e10 = expf(s[1][0] - base[0]), e11 = expf(s[1][1] - base[0]);
        float e12 = expf(s[1][2] - base[1]), e13 = expf(s[1][3] - base[1]);
        st.l[0] += (e00 + e01) + (e10 + e11);
        st.l[1] += (e02 + e03) + (e12 + e13);
        p[0] = pack_bf16(e00, e01);
        p[1] = pack_bf16(e02, e03);
        p[2] = pack_bf16(e10, e11);
        p[3] = pack_bf16(e12, e13);
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        st.o[n][0] *= corr[0];
        st.o[n][1] *= corr[0];
        st.o[n][2] *= corr[1];
        st.o[n][3] *= corr[1];
    }
    // O[16 x D] += P[16 x 16] V[16 x D]
    {
        const int mi = lane >> 3, r8 = lane & 7;
        const int row = (mi & 1) * 8 + r8;
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            const int cc = n + (mi >> 1);
            uint32_t r[4];
            ldmatrix_x4_trans(r, v_smem + (cc >> 3) * CS + swizzle128(row, cc & 7));
            mma_bf16_16816(st.o[n], p, r[0], r[1]);
            mma_bf16_16816(st.o[n + 1], p, r[2], r[3]);
        }
    }
}

// NT consecutive 16-key tiles (16 NT keys from `key0`) at once: one running-maximum update and one
// rescale of the output per block, and NT independent score tiles in flight.  The tiles lie
// `tile_bytes` apart in shared memory, each laid out as attend_tile expects.
template <int D, int NT, int CS = 2048, int VOFF = (D / 64) * 2048>
__device__ __forceinline__ void attend_block(WarpState<D>& st, uint32_t base, uint32_t tile_bytes, int key0,
                                             const RowLimits& lim, float scale) {
    const int lane = threadIdx.x & 31;
    const int t = lane & 3;
    const int mi = lane >> 3, r8 = lane & 7;
    float s[2 * NT][4];
#pragma unroll
    for (int j = 0; j < 2 * NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
    for (int k = 0; k < NT; ++k) {
        const uint32_t k_smem = base + k * tile_bytes;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
                const int cc = 2 * ks + mi;
                uint32_t r[4];
                ldmatrix_x4(r, k_smem + (cc >> 3) * CS + swizzle128(8 * j + r8, cc & 7));
                mma_bf16_16816(s[2 * k + j], st.q[ks], r[0], r[1]);
                mma_bf16_16816(s[2 * k + j], st.q[ks + 1], r[2], r[3]);
            }
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    const bool interior = key0 + 16 * NT - 1 <= min(lim.hi[0], lim.hi[1]) && key0 >= max(lim.lo[0], lim.lo[1]) &&
                          lim.hi[0] >= 0 && lim.hi[1] >= 0;
    if (__all_sync(0xffffffffu, interior)) {
#pragma unroll
        for (int j = 0; j < 2 * NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[j][e] *= scale;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
            }
    } else {
#pragma unroll
        for (int j = 0; j < 2 * NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = e >> 1;
                const int key = key0 + 8 * j + 2 * t + (e & 1);
                const bool ok = key <= lim.hi[row] && key >= lim.lo[row];
                s[j][e] = ok ? s[j][e] * scale : -INFINITY;
                mx[row] = fmaxf(mx[row], s[j][e]);
            }
    }
    float corr[2], sub[2];
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
        mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
        const float m_new = fmaxf(st.m[row], mx[row]);
        sub[row] = m_new == -INFINITY ? 0.0f : m_new;
        corr[row] = st.m[row] == -INFINITY ? 0.0f : expf(st.m[row] - sub[row]);
        st.m[row] = m_new;
        st.l[row] *= corr[row];
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        st.o[n][0] *= corr[0];
        st.o[n][1] *= corr[0];
        st.o[n][2] *= corr[1];
        st.o[n][3] *= corr[1];
    }
#pragma unroll
    for (int k = 0; k < NT; ++k) {
        uint32_t p[4];
        {
            const float e00 = expf(s[2 * k][0] - sub[0]), e01 = expf(s[2 * k][1] - sub[0]);
            const float e02 = expf(s[2 * k][2] - sub[1]), e03 = expf(s[2 * k][3] - sub[1]);
            const float e10 = expf(s[2 * k + 1][0] - sub[0]), e11 = expf(s[2 * k + 1][1] - sub[0]);
            const float e12 = expf(s[2 * k + 1][2] - sub[1]), e13 = expf(s[2 * k + 1][3] - sub[1]);
            st.l[0] += (e00 + e01) + (e10 + e11);
            st.l[1] += (e02 + e03) + (e12 + e13);
            p[0] = pack_bf16(e00, e01);
            p[1] = pack_bf16(e02, e03);
            p[2] = pack_bf16(e10, e11);
            p[3] = pack_bf16(e12, e13);
        }
        const uint32_t v_smem = base + k * tile_bytes + VOFF;
        const int row = (mi & 1) * 8 + r8;
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            const int cc = n + (mi >> 1);
            uint32_t r[4];
            ldmatrix_x4_trans(r, v_smem + (cc >> 3) * CS + swizzle128(row, cc & 7));
            mma_bf16_16816(st.o[n], p, r[0], r[1]);
            mma_bf16_16816(st.o[n + 1], p, r[2], r[3]);
        }
    }
}

// Sum the per-thread partial sums of a row over the four threads that share it.
template <int D>
__device__ __forceinline__ void finish_rows(WarpState<D>& st) {
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        st.l[row] += __shfl_xor_sync(0xffffffffu, st.l[row], 1);
        st.l[row] += __shfl_xor_sync(0xffffffffu, st.l[row], 2);
    }
}

// ---------------------------------------------------------------------------------------------
// The same for a group of at most 8 query heads (the decode kernel's case at every published size), TRANSPOSED:
// the 16 keys of a tile are the rows of the MMA and the query heads its 8 columns,
//   S^T [16 keys x 8 heads] = K [16 x D] Q^T,        O^T [D x 8 heads] += V^T [D x 16 keys] P^T,
// which halves the MMAs and the exponentials (no rows 8 to 15 that belong to no head).  A thread holds columns
// 2 t and 2 t + 1 (t = lane % 4) of every row it has a share in: the running maximum and sum are per COLUMN, reduced
// over the lanes that differ in lane / 4; P^T becomes the B operand of the second product through movmatrix.
// ---------------------------------------------------------------------------------------------
template <int D>
struct WarpStateT {
    uint32_t q[D / 16][2];  // B fragments of Q^T: head lane / 4, columns 16 ks + 2 t (+ 8)
    float o[D / 16][4];     // O^T: rows 16 i + lane / 4 (+ 8), columns 2 t, 2 t + 1
    float m[2], l[2];       // running maximum and (per-thread partial) sum of heads 2 t and 2 t + 1
};

template <int D>
__device__ __forceinline__ void init_state(WarpStateT<D>& st) {
#pragma unroll
    for (int i = 0; i < D / 16; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[i][e] = 0.0f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
}

// The query fragments of head lane / 4; ``row`` null: no such head (zeros).
template <int D>
__device__ __forceinline__ void load_q(WarpStateT<D>& st, const bf16* row) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        st.q[ks][0] = row ? *reinterpret_cast<const uint32_t*>(row + ks * 16 + 2 * t) : 0u;
        st.q[ks][1] = row ? *reinterpret_cast<const uint32_t*>(row + ks * 16 + 2 * t + 8) : 0u;
    }
}

// NT consecutive 16-key tiles of which the first ``valid`` exist (the same for the whole warp), keys from ``key0``;
// the token sees keys lo..hi.  Layout of the tiles as for attend_block.
template <int D, int NT, int CS, int VOFF>
__device__ __forceinline__ void attend_block_t(WarpStateT<D>& st, uint32_t base, uint32_t tile_bytes, int key0, int valid,
                                               int lo, int hi, float scale) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int mi = lane >> 3, r8 = lane & 7;
    float s[NT][4];
#pragma unroll
    for (int k = 0; k < NT; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[k][e] = 0.0f;
    // S^T = K Q^T: A fragments of K by ldmatrix (keys 0-7 | 8-15 of the tile x columns 0-7 | 8-15 of the K step)
#pragma unroll
    for (int k = 0; k < NT; ++k) {
        if (k >= valid) continue;
        const uint32_t k_smem = base + k * tile_bytes;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int cc = 2 * ks + (mi >> 1);
            uint32_t a[4];
            ldmatrix_x4(a, k_smem + (cc >> 3) * CS + swizzle128((mi & 1) * 8 + r8, cc & 7));
            mma_bf16_16816(s[k], a, st.q[ks][0], st.q[ks][1]);
        }
    }
    // scale, mask (per key = per row), maximum per column
    float mx[2] = {-INFINITY, -INFINITY};
    const bool interior = valid == NT && key0 + 16 * NT - 1 <= hi && key0 >= lo;
    if (interior) {
#pragma unroll
        for (int k = 0; k < NT; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[k][e] *= scale;
                mx[e & 1] = fmaxf(mx[e & 1], s[k][e]);
            }
    } else {
#pragma unroll
        for (int k = 0; k < NT; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + 16 * k + g + ((e & 2) ? 8 : 0);
                const bool ok = k < valid && key <= hi && key >= lo;
                s[k][e] = ok ? s[k][e] * scale : -INFINITY;
                mx[e & 1] = fmaxf(mx[e & 1], s[k][e]);
            }
    }
    float corr[2], sub[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 4));
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 8));
        mx[c] = fmaxf(mx[c], __shfl_xor_sync(0xffffffffu, mx[c], 16));
        const float m_new = fmaxf(st.m[c], mx[c]);
        sub[c] = m_new == -INFINITY ? 0.0f : m_new;
        corr[c] = st.m[c] == -INFINITY ? 0.0f : expf(st.m[c] - sub[c]);
        st.m[c] = m_new;
        st.l[c] *= corr[c];
    }
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
        st.o[i][0] *= corr[0];
        st.o[i][1] *= corr[1];
        st.o[i][2] *= corr[0];
        st.o[i][3] *= corr[1];
    }
#pragma unroll
    for (int k = 0; k < NT; ++k) {
        if (k >= valid) continue;
        const float e0 = expf(s[k][0] - sub[0]), e1 = expf(s[k][1] - sub[1]);
        const float e2 = expf(s[k][2] - sub[0]), e3 = expf(s[k][3] - sub[1]);
        st.l[0] += e0 + e2;
        st.l[1] += e1 + e3;
        // P^T as the B operand: keys 2 t, 2 t + 1 (+ 8) of head lane / 4
        const uint32_t b0 = movmatrix_trans(pack_bf16(e0, e1));
        const uint32_t b1 = movmatrix_trans(pack_bf16(e2, e3));
        const uint32_t v_smem = base + k * tile_bytes + VOFF;
        // A fragments of V^T by transposing ldmatrix: columns 16 i .. of the head x the tile's 16 keys
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            const int cc = 2 * i + (mi & 1);
            uint32_t a[4];
            ldmatrix_x4_trans(a, v_smem + (cc >> 3) * CS + swizzle128((mi >> 1) * 8 + r8, cc & 7));
            mma_bf16_16816(st.o[i], a, b0, b1);
        }
    }
}

// The per-thread partial sums of a column, over the eight threads that share it.
template <int D>
__device__ __forceinline__ void finish_rows(WarpStateT<D>& st) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        st.l[c] += __shfl_xor_sync(0xffffffffu, st.l[c], 4);
        st.l[c] += __shfl_xor_sync(0xffffffffu, st.l[c], 8);
        st.l[c] += __shfl_xor_sync(0xffffffffu, st.l[c], 16);
    }
}

// The first 1024-byte boundary of the shared address space at or after p (swizzled TMA tiles need it).
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) { return p + ((1024u - (smem_u32(p) & 1023u)) & 1023u); }

// Issue the TMA loads of one 16-key tile of K and of V into a stage (2 x D/64 boxes of 2 KB).
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* stage, const CUtensorMap* mk, const CUtensorMap* mv, int cache_row,
                                          uint64_t* bar) {
    mbar_expect_tx(bar, 2 * TILE_KEYS * D * 2);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(stage + c * 2048, mk, 64 * c, cache_row, bar);
        tma_load_2d(stage + (D / 64) * 2048 + c * 2048, mv, 64 * c, cache_row, bar);
    }
}

// Row of the cache's 2-D view [pages * kv heads * page_size, D] that holds key `key` of a request.
__device__ __forceinline__ int cache_row_of(const int* table, int key, int page_size, int nkv, int hk) {
    const int page = table[key / page_size];
    return (page * nkv + hk) * page_size + key % page_size;
}

// What the decode kernel needs to take over the rotary-position / cache-write kernel's work for a step of
// single tokens: it rotates q in its registers, and the warp that owns the tile of the token's own position
// rotates k, copies v, stores both to the cache and patches them into the tile it has just loaded.
// inv_freq == nullptr: nothing is fused (q is rotated and the cache written already).
struct FusedRope {
    const float* inv_freq;    // [D / 2]; the whole head is rotated (rotary dims == D)
    const int* slot_mapping;  // [rows of the step]: page * page_size + slot of the token; < 0: the token's k and v are
                              // used but not stored; null: the cache holds them already (q alone is rotated)
    bf16* k_cache;
    bf16* v_cache;
};

__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

// Rotate the query fragments of rows g and g + 8 (both of the token whose angles `cos_sin` holds: (cos, sin) of
// pos * inv_freq[i] for i < D/2):
// pairs (i, i + D/2): lo' = lo cos - hi sin, hi' = hi cos + lo sin (crates/ferrisinfer-kernel/src/cpu/attention.rs:1288-1291).
template <int D>
__device__ __forceinline__ void rotate_q(WarpState<D>& st, const float2* cos_sin) {
    constexpr int HS = D / 32;  // k-steps per half of the head
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < HS; ++ks) {
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
            const int c = 16 * ks + 2 * t + 8 * e2;
            const float2 a0 = cos_sin[c], a1 = cos_sin[c + 1];
#pragma unroll
            for (int rowsel = 0; rowsel < 2; ++rowsel) {
                const int e = 2 * e2 + rowsel;
                const float2 lo = unpack_bf16(st.q[ks][e]), hi = unpack_bf16(st.q[ks + HS][e]);
                st.q[ks][e] = pack_bf16(lo.x * a0.x - hi.x * a0.y, lo.y * a1.x - hi.y * a1.y);
                st.q[ks + HS][e] = pack_bf16(hi.x * a0.x + lo.x * a0.y, hi.y * a1.x + lo.y * a1.y);
            }
        }
    }
}

// The same for the transposed fragments (head lane / 4 only).
template <int D>
__device__ __forceinline__ void rotate_q(WarpStateT<D>& st, const float2* cos_sin) {
    constexpr int HS = D / 32;
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int ks = 0; ks < HS; ++ks) {
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
            const int c = 16 * ks + 2 * t + 8 * e2;
            const float2 a0 = cos_sin[c], a1 = cos_sin[c + 1];
            const float2 lo = unpack_bf16(st.q[ks][e2]), hi = unpack_bf16(st.q[ks + HS][e2]);
            st.q[ks][e2] = pack_bf16(lo.x * a0.x - hi.x * a0.y, lo.y * a1.x - hi.y * a1.y);
            st.q[ks + HS][e2] = pack_bf16(hi.x * a0.x + lo.x * a0.y, hi.y * a1.x + lo.y * a1.y);
        }
    }
}

// =============================================================================================
// Decode: one CTA per (split, kv head, token).  Its NW warps take the 16-key tiles of the
// split's key range in turn, each with a pipeline of its own; their results are merged through
// shared memory and written as the final output, as one partial (m, l, O) per split, or sent to
// the CTAs of the cluster that the splits of a (token, kv head) form.
// =============================================================================================
// PAIR: the key and the value cache are two planes of one tensor, and `map_k` is a 3-D map over both: one copy brings
// the 64-column box of K and the box of V of the same 16 keys and columns (4 KB instead of two copies of 2 KB; a
// copy costs the TMA unit ~30 ns whatever it brings, and a CTA of a long context issues hundreds).  A tile then lies
// in shared memory as (K box, V box) per 64 columns instead of all K boxes followed by all V boxes.
// TR: the group has at most 8 query heads and the warps work on the transposed products (attend_block_t).
template <int D, int STAGES, bool PAIR, int NW, bool TR>
__global__ void __launch_bounds__(NW * 32)
    decode_attention_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const bf16* q, int ldq, bf16* __restrict__ out, int ldo,
                            float* __restrict__ part_o, float* __restrict__ part_ml, const int* __restrict__ block_tables,
                            int max_blocks, const int* __restrict__ token_seq, const int* __restrict__ positions,
                            const int* __restrict__ token_list, int nh, int nkv, int page_size, int window, float scale,
                            int splits, const FusedRope rope, int cluster_merge, int* status) {
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[NW][STAGES];
    __shared__ int tile_rows[NW][ROW_CACHE];  // cache rows of this warp's next tiles, looked up in one go
    __shared__ float2 cos_sin[D / 2];            // (cos, sin) of the token's rotation angles, when the rotation is fused
    uint8_t* smem = align1024(smem_raw);
    constexpr int NT = D == 64 ? 4 : 2;  // 16-key tiles per pipeline stage and per softmax update
    constexpr int TILE_BYTES = 2 * TILE_KEYS * D * 2;
    constexpr int STAGE_BYTES = NT * TILE_BYTES;
    constexpr int BLOCK_CACHE = ROW_CACHE / NT;  // blocks whose rows the cache holds
    constexpr int CS = PAIR ? 4096 : 2048;             // bytes between the 64-column boxes of a tile
    constexpr int VOFF = PAIR ? 2048 : (D / 64) * 2048;  // where a tile's V boxes begin

    const int split = blockIdx.x, hk = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = nh / nkv;
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_k);
        tma_prefetch_descriptor(&map_v);
    }
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[warp][s], 1);
    }
    mbar_fence_init();
    __syncthreads();
    pdl_launch_dependents();
    if (splits > 1 && cluster_merge) cluster_arrive_relaxed();  // first phase of the cluster's barrier: "this CTA runs"
    // A kernel that rotates AND writes the cache reads nothing from the cache that this step wrote before it (the
    // token's own key and value come from its qkv row, which it patches into the tile), and the step's metadata was
    // uploaded before the step began: it requests its first tiles BEFORE the wait, which only the queries need.
    // What such a tile holds was written by an EARLIER step.  A launch of this chain begins no sooner than every CTA
    // of the launch before it has begun, and none of those CTAs ends before the launch before IT has ended; so for
    // this kernel to run while a kernel of the previous step is unfinished, every CTA of the ~120 launches between
    // them would have to be resident at once, which the SMs cannot hold (32 CTAs each at most).  Between a graph
    // replay and the next step the stream orders everything.
    // A kernel that only rotates q (a layer that reads another layer's cache: no slot mapping) reads position P as
    // its owner wrote it a few launches ago in THIS step: it waits first and patches nothing.
    const bool fused = rope.inv_freq != nullptr;
    const bool patches = fused && rope.slot_mapping != nullptr;
    const bool early = patches;
    if (!early) {
        pdl_wait();
        FERRIS_TL_BEGIN();
    }
    // with a token list, only the listed rows of the step are attended (the others belong to another kernel)
    const int tok = token_list ? token_list[blockIdx.z] : (int)blockIdx.z;
    const int seq = token_seq[tok];
    const int P = positions[tok];
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    const int* table = block_tables + (size_t)seq * max_blocks;

    // key tiles of this split, in blocks of NT; the warps take the blocks in turn
    const int first_tile = lo / TILE_KEYS, last_tile = P / TILE_KEYS;
    const int n_tiles = last_tile - first_tile + 1;
    const int per_split = (n_tiles + splits - 1) / splits;
    const int t_begin = first_tile + split * per_split;
    const int t_end = min(t_begin + per_split, last_tile + 1);
    const int n_blocks = t_end > t_begin ? (t_end - t_begin + NT - 1) / NT : 0;
    const int my_count = n_blocks > warp ? (n_blocks - warp + NW - 1) / NW : 0;

    typename std::conditional<TR, WarpStateT<D>, WarpState<D>>::type st;
    init_state(st);
    RowLimits lim;
    auto load_queries = [&]() {
        const int g = lane >> 2;
        const bf16* qrow = q + (size_t)tok * ldq + (size_t)hk * G * D;
        if constexpr (TR) {
            load_q(st, g < G ? qrow + (size_t)g * D : nullptr);
        } else {
            load_q(st, g < G ? qrow + (size_t)g * D : nullptr, g + 8 < G ? qrow + (size_t)(g + 8) * D : nullptr);
        }
        if (rope.inv_freq) rotate_q<D>(st, cos_sin);
        lim.hi[0] = g < G ? P : -1;
        lim.hi[1] = g + 8 < G ? P : -1;
        lim.lo[0] = lim.lo[1] = lo;
    };
    if (!fused) load_queries();
    uint8_t* my_stages = smem + (size_t)warp * STAGES * STAGE_BYTES;
    auto first_tile_of = [&](int i) { return t_begin + (warp + i * NW) * NT; };
    // the block-table look-ups of the warp's tiles are independent loads, issued together
    auto fill_rows = [&](int first_block) {
        for (int e = lane; e < ROW_CACHE; e += 32) {
            const int i = first_block + e / NT, tile = first_tile_of(i) + e % NT;
            if (i < my_count && tile < t_end) tile_rows[warp][e] = cache_row_of(table, tile * TILE_KEYS, page_size, nkv, hk);
        }
        __syncwarp();
    };
    auto issue = [&](int i) {
        const int tile0 = first_tile_of(i);
        const int valid = min(NT, t_end - tile0);
        uint64_t* bar = &full[warp][i % STAGES];
        uint8_t* stage = my_stages + (i % STAGES) * STAGE_BYTES;
        mbar_expect_tx(bar, valid * TILE_BYTES);
        for (int k = 0; k < valid; ++k) {
            const int row = tile_rows[warp][(i % BLOCK_CACHE) * NT + k];
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                if (PAIR) {
                    tma_load_3d(stage + k * TILE_BYTES + c * CS, &map_k, 64 * c, row, 0, bar);
                } else {
                    tma_load_2d(stage + k * TILE_BYTES + c * 2048, &map_k, 64 * c, row, bar);
                    tma_load_2d(stage + k * TILE_BYTES + (D / 64) * 2048 + c * 2048, &map_v, 64 * c, row, bar);
                }
            }
        }
    };
    fill_rows(0);
    if (lane == 0)
        for (int i = 0; i < STAGES && i < my_count; ++i) issue(i);
    // marks of the timeline build: thread 0 of the CTA of the last key range of token 0, kv head 0
    [[maybe_unused]] const bool tl_mark = threadIdx.x == 0 && blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && blockIdx.z == 0;
    // the warp whose tiles include the token's own position (in the CTA of the last key range) will rotate k and copy v
    const int own_block = (last_tile >= t_begin && last_tile < t_end) ? (last_tile - t_begin) / NT : -1;
    const bool owns_token = patches && own_block >= 0 && own_block % NW == warp;
    float k_lo[D / 64], k_hi[D / 64];
    bf16 v_own[D / 32];
    // where the token's k and v go in the cache: step metadata, read before the wait as well
    const int own_slot = owns_token ? rope.slot_mapping[tok] : -1;
    if (fused) {
        // the angles depend on the position alone: formed before the wait, off the step's critical path
        for (int i = threadIdx.x; i < D / 2; i += NW * 32) {
            float sn, cs;
            sincosf((float)P * rope.inv_freq[i], &sn, &cs);
            cos_sin[i] = make_float2(cs, sn);
        }
        __syncthreads();
        if (early) {
            pdl_wait();
            FERRIS_TL_BEGIN();
        }
        FERRIS_TL_MARK(tl_mark, 9);
        if (owns_token) {
            // the token's own k and v (from the q/k/v product that has just finished) are requested with the queries
            const bf16* krow = q + (size_t)tok * ldq + (size_t)(nh + hk) * D;
            const bf16* vrow = q + (size_t)tok * ldq + (size_t)(nh + nkv + hk) * D;
#pragma unroll
            for (int j = 0; j < D / 64; ++j) {
                k_lo[j] = __bfloat162float(krow[lane + 32 * j]);
                k_hi[j] = __bfloat162float(krow[lane + 32 * j + D / 2]);
            }
#pragma unroll
            for (int j = 0; j < D / 32; ++j) v_own[j] = vrow[lane + 32 * j];
        }
        load_queries();
    }
    FERRIS_TL_MARK(tl_mark, 0);
    for (int i = 0; i < my_count; ++i) {
        const int s = i % STAGES;
        // the row cache holds blocks [c, c + BLOCK_CACHE), c a multiple of BLOCK_CACHE; block i + STAGES is
        // issued below, and everything before it has been issued, so its window may be filled now
        if ((i + STAGES) % BLOCK_CACHE == 0 && i + STAGES < my_count) {
            __syncwarp();
            fill_rows(i + STAGES);
        }
        if (!mbar_wait(&full[warp][s], (i / STAGES) & 1, status, 1)) break;
        FERRIS_TL_MARK(tl_mark && i == 0, 1);
        const uint32_t base = smem_u32(my_stages + s * STAGE_BYTES);
        const int tile0 = first_tile_of(i);
        if (patches && last_tile >= tile0 && last_tile < tile0 + NT && last_tile < t_end) {
            // this warp holds the tile of the token's own position: its key (rotated) and value come from the
            // step's qkv row, go to the cache for the steps to come, and into the tile just loaded
            uint8_t* tb = my_stages + s * STAGE_BYTES + (last_tile - tile0) * TILE_BYTES;
            const int r = P % TILE_KEYS;
            const int slot = own_slot;
            const size_t crow = slot >= 0 ? ((size_t)(slot / page_size) * nkv + hk) * page_size + slot % page_size : 0;
            auto put = [&](uint8_t* tile, bf16* cache, int c, bf16 v) {
                *reinterpret_cast<bf16*>(tile + (c >> 6) * CS + swizzle128(r, (c & 63) >> 3) + (c & 7) * 2) = v;
                if (slot >= 0) cache[crow * D + c] = v;
            };
#pragma unroll
            for (int j = 0; j < D / 64; ++j) {
                const int i2 = lane + 32 * j;
                const float2 a = cos_sin[i2];
                put(tb, rope.k_cache, i2, __float2bfloat16_rn(k_lo[j] * a.x - k_hi[j] * a.y));
                put(tb, rope.k_cache, i2 + D / 2, __float2bfloat16_rn(k_hi[j] * a.x + k_lo[j] * a.y));
            }
#pragma unroll
            for (int j = 0; j < D / 32; ++j) put(tb + VOFF, rope.v_cache, lane + 32 * j, v_own[j]);
            fence_proxy_async();
            __syncwarp();
        }
        if constexpr (TR) {
            attend_block_t<D, NT, CS, VOFF>(st, base, TILE_BYTES, tile0 * TILE_KEYS, min(NT, t_end - tile0), lo, P, scale);
        } else if (tile0 + NT <= t_end) {
            attend_block<D, NT, CS, VOFF>(st, base, TILE_BYTES, tile0 * TILE_KEYS, lim, scale);
        } else {
            for (int k = 0; tile0 + k < t_end; ++k)
                attend_tile<D, CS>(st, base + k * TILE_BYTES, base + k * TILE_BYTES + VOFF, (tile0 + k) * TILE_KEYS, lim,
                                   scale);
        }
        __syncwarp();
        if (lane == 0 && i + STAGES < my_count) issue(i + STAGES);
    }
    finish_rows(st);
    FERRIS_TL_MARK(tl_mark, 2);

    // merge the warps through shared memory (the stages are no longer read)
    __syncthreads();
    FERRIS_TL_MARK(tl_mark, 3);
    float* merge = reinterpret_cast<float*>(smem);  // [NW][16][D + 2]
    if constexpr (TR) {
        // a thread holds heads 2 t and 2 t + 1: of each, the output columns 16 i + lane / 4 (+ 8)
        const int g = lane >> 2, t = lane & 3;
        float* mine = merge + (size_t)warp * 16 * (D + 2);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float* r = mine + (2 * t + c) * (D + 2);
            if (g == 0) {
                r[0] = st.m[c];
                r[1] = st.l[c];
            }
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
                r[2 + 16 * i + g] = st.o[i][c];
                r[2 + 16 * i + g + 8] = st.o[i][2 + c];
            }
        }
    } else {
        const int g = lane >> 2, t = lane & 3;
        float* mine = merge + (size_t)warp * 16 * (D + 2);
#pragma unroll
        for (int row = 0; row < 2; ++row) {
            float* r = mine + (g + 8 * row) * (D + 2);
            if (t == 0) {
                r[0] = st.m[row];
                r[1] = st.l[row];
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                r[2 + 8 * n + 2 * t] = st.o[n][2 * row];
                r[2 + 8 * n + 2 * t + 1] = st.o[n][2 * row + 1];
            }
        }
    }
    __syncthreads();
    // per row: the maximum over the warps, each warp's factor e^{m_w - M}, and the sum; one thread per row
    __shared__ float warp_factor[NW][16], row_m[16], row_l[16];
    if ((int)threadIdx.x < G) {
        const int r = threadIdx.x;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) mm = fmaxf(mm, merge[(size_t)(w * 16 + r) * (D + 2)]);
        float ll = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float* rw = merge + (size_t)(w * 16 + r) * (D + 2);
            const float f = rw[0] == -INFINITY ? 0.0f : expf(rw[0] - mm);
            warp_factor[w][r] = f;
            ll += rw[1] * f;
        }
        row_m[r] = mm;
        row_l[r] = ll;
    }
    __syncthreads();
    // With a cluster, element idx of the G x D outputs belongs to the CTA idx / share of the cluster: every key range
    // sends its (maximum, sum) of every row and its unnormalised output elements to the owners' shared memory
    // (a region of its own behind the stages: a peer may still be in its key loop), one barrier follows, and the
    // owner adds the ranges in their order (the sums of decode_merge_kernel): no scratch in global memory, no
    // merge launch, and after the barrier a CTA reads its own shared memory only.
    const bool pushes = splits > 1 && cluster_merge;
    const int share = (G * D + splits - 1) / splits;
    const uint32_t recv_ml = smem_u32(smem + (size_t)NW * STAGES * STAGE_BYTES);  // [splits][G][2]
    const uint32_t recv_o = recv_ml + (uint32_t)(splits * G * 2) * 4u;             // [splits][share]
    if (pushes) {
        cluster_wait();  // first phase: every CTA of the cluster runs
        for (int i = threadIdx.x; i < G * splits; i += NW * 32) {
            const int r = i % G, owner = i / G;
            const uint32_t at = recv_ml + (uint32_t)((split * G + r) * 2) * 4u;
            st_peer_shared_f32(at, (uint32_t)owner, row_m[r]);
            st_peer_shared_f32(at + 4u, (uint32_t)owner, row_l[r]);
        }
    }
    for (int idx = threadIdx.x; idx < G * D; idx += NW * 32) {
        const int r = idx / D, c = idx % D;
        float oo = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) oo += merge[(size_t)(w * 16 + r) * (D + 2) + 2 + c] * warp_factor[w][r];
        const int head = hk * G + r;
        if (splits == 1) {
            out[(size_t)tok * ldo + (size_t)head * D + c] = __float2bfloat16_rn(oo / row_l[r]);
        } else if (cluster_merge) {
            const int owner = idx / share;
            st_peer_shared_f32(recv_o + (uint32_t)(split * share + idx - owner * share) * 4u, (uint32_t)owner, oo);
        } else {
            // partial results are indexed by the row's place in this launch (blockIdx.z), not in the step
            const size_t slot = ((size_t)blockIdx.z * nh + head) * splits + split;
            part_o[slot * D + c] = oo;
            if (c == 0) {
                part_ml[slot * 2] = row_m[r];
                part_ml[slot * 2 + 1] = row_l[r];
            }
        }
    }
    if (pushes) {
        FERRIS_TL_MARK(tl_mark, 5);
        cluster_arrive_release();
        cluster_wait();
        FERRIS_TL_MARK(tl_mark, 6);
        const float* my_ml = reinterpret_cast<const float*>(smem + (size_t)NW * STAGES * STAGE_BYTES);
        const float* my_o = my_ml + splits * G * 2;
        const int begin = split * share, end = min(begin + share, G * D);
        for (int idx = begin + threadIdx.x; idx < end; idx += NW * 32) {
            const int r = idx / D;
            float ms[MAX_CLUSTER], ls[MAX_CLUSTER], os[MAX_CLUSTER];
#pragma unroll
            for (int sp = 0; sp < MAX_CLUSTER; ++sp) {
                const bool have = sp < splits;
                ms[sp] = have ? my_ml[(sp * G + r) * 2] : -INFINITY;
                ls[sp] = have ? my_ml[(sp * G + r) * 2 + 1] : 0.0f;
                os[sp] = have ? my_o[sp * share + idx - begin] : 0.0f;
            }
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < MAX_CLUSTER; ++sp) mm = fmaxf(mm, ms[sp]);
            float ll = 0.0f, oo = 0.0f;
#pragma unroll
            for (int sp = 0; sp < MAX_CLUSTER; ++sp) {
                if (sp >= splits) continue;
                const float f = ms[sp] == -INFINITY ? 0.0f : expf(ms[sp] - mm);
                ll += ls[sp] * f;
                oo += os[sp] * f;
            }
            out[(size_t)tok * ldo + (size_t)(hk * G) * D + idx] = __float2bfloat16_rn(oo / ll);
        }
    }
#ifdef FERRIS_TIMELINE
    __syncthreads();
#endif
    FERRIS_TL_MARK(tl_mark, 4);
    FERRIS_TL_END(4);
}

// Merge of the splits: out = sum_s O_s e^{m_s - M} / sum_s l_s e^{m_s - M}.  One block per (token, head).
template <int D>
__global__ void decode_merge_kernel(const float* part_o, const float* part_ml,
                                    bf16* __restrict__ out, int ldo, const int* __restrict__ token_list, int nh,
                                    int splits) {
    pdl_wait();
    pdl_launch_dependents();
    const int tok = token_list ? token_list[blockIdx.x] : (int)blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)blockIdx.x * nh + head) * splits;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float ll = 0.0f, oo = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float ms = part_ml[(base + s) * 2];
            const float f = ms == -INFINITY ? 0.0f : expf(ms - mm);
            ll += part_ml[(base + s) * 2 + 1] * f;
            oo += part_o[(base + s) * D + c] * f;
        }
        out[(size_t)tok * ldo + (size_t)head * D + c] = __float2bfloat16_rn(oo / ll);
    }
}

// =============================================================================================
// Prefill: one CTA per (row block, kv head, request).  The rows of a request's portion are
// (token, head of the group) pairs, 64 to a CTA (16 per warp).  A fifth warp streams 64-key
// stages of K and V for the CTA; each consumer warp skips the 16-key tiles that none of its rows
// can see.
// =============================================================================================
constexpr int PF_ROWS = 64;
constexpr int PF_STAGE_TILES = 4;  // 64 keys per stage

template <int D, int STAGES>
__global__ void __launch_bounds__((WARPS + 1) * 32)
    prefill_attention_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const bf16* q, int ldq, bf16* __restrict__ out, int ldo,
                             const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ seq_q_start,
                             const int* __restrict__ seq_start_pos, int nh, int nkv, int page_size, int window,
                             float scale, int skip_single, int* status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[STAGES], empty[STAGES];
    uint8_t* smem = align1024(smem_raw);
    constexpr int TILE_BYTES = 2 * TILE_KEYS * D * 2;
    constexpr int STAGE_BYTES = PF_STAGE_TILES * TILE_BYTES;

    const int G = nh / nkv;
    const int seq = blockIdx.z, hk = blockIdx.y;
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int q_start = seq_q_start[seq], q_len = seq_q_start[seq + 1] - q_start;
    if (skip_single && q_len == 1) {  // single tokens are the decode kernel's
        FERRIS_TL_END(7);
        return;
    }
    const int rows_total = q_len * G;
    // heavy row blocks (the last tokens see the most keys) first
    const int n_blocks = (rows_total + PF_ROWS - 1) / PF_ROWS;
    if ((int)blockIdx.x >= n_blocks) {
        FERRIS_TL_END(7);
        return;
    }
    const int block = n_blocks - 1 - blockIdx.x;
    const int row0 = block * PF_ROWS;
    const int start_pos = seq_start_pos[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_tables + (size_t)seq * max_blocks;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_k);
        tma_prefetch_descriptor(&map_v);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], WARPS);
        }
    }
    mbar_fence_init();
    __syncthreads();

    // key range of the block: from the first key its first token may see to its last token's position
    const int tok_first = row0 / G;
    const int tok_last = min(row0 + PF_ROWS - 1, rows_total - 1) / G;
    const int p_first = start_pos + tok_first, p_last = start_pos + tok_last;
    const int lo_block = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int stage_keys = PF_STAGE_TILES * TILE_KEYS;
    const int s_begin = lo_block / stage_keys, s_end = p_last / stage_keys + 1;  // stages of 64 keys
    const int n_stages = s_end - s_begin;

    if (warp == WARPS) {
        // producer
        if (lane == 0) {
            for (int i = 0; i < n_stages; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, status, 2)) break;
                const int key_base = (s_begin + i) * stage_keys;
                int tiles = 0;
                for (int k = 0; k < PF_STAGE_TILES; ++k)
                    if (key_base + k * TILE_KEYS <= p_last) ++tiles;
                mbar_expect_tx(&full[s], tiles * TILE_BYTES);
                for (int k = 0; k < tiles; ++k) {
                    uint8_t* dst = smem + (size_t)s * STAGE_BYTES + k * TILE_BYTES;
                    const int row = cache_row_of(table, key_base + k * TILE_KEYS, page_size, nkv, hk);
#pragma unroll
                    for (int c = 0; c < D / 64; ++c) {
                        tma_load_2d(dst + c * 2048, &map_k, 64 * c, row, &full[s]);
                        tma_load_2d(dst + (D / 64) * 2048 + c * 2048, &map_v, 64 * c, row, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // consumers
    WarpState<D> st;
    init_state(st);
    RowLimits lim;
    int my_lo = INT_MAX, my_hi = -1;
    const bf16* qrow[2];
    bf16* orow[2];
    {
        const int g = lane >> 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = row0 + warp * 16 + g + 8 * r;
            if (row < rows_total) {
                const int tok = row / G, head = hk * G + row % G;
                const int pos = start_pos + tok;
                lim.hi[r] = pos;
                lim.lo[r] = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
                qrow[r] = q + (size_t)(q_start + tok) * ldq + (size_t)head * D;
                orow[r] = out + (size_t)(q_start + tok) * ldo + (size_t)head * D;
            } else {
                lim.hi[r] = -1;
                lim.lo[r] = 0;
                qrow[r] = nullptr;
                orow[r] = nullptr;
            }
        }
        load_q(st, qrow[0], qrow[1]);
        // key range that any row of this warp can see
        const int wr0 = row0 + warp * 16, wr1 = min(wr0 + 15, rows_total - 1);
        if (wr0 < rows_total) {
            const int pa = start_pos + wr0 / G, pb = start_pos + wr1 / G;
            my_lo = (window > 0 && pa - window + 1 > 0) ? pa - window + 1 : 0;
            my_hi = pb;
        }
    }
    for (int i = 0; i < n_stages; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full[s], (i / STAGES) & 1, status, 3)) break;
        const int key_base = (s_begin + i) * stage_keys;
        if (key_base + stage_keys - 1 <= my_hi && key_base >= my_lo - (TILE_KEYS - 1)) {
            // all four tiles hold keys that rows of this warp see: one pass over the 64 keys
            attend_block<D, PF_STAGE_TILES>(st, smem_u32(smem + (size_t)s * STAGE_BYTES), TILE_BYTES, key_base, lim, scale);
        } else {
#pragma unroll
            for (int k = 0; k < PF_STAGE_TILES; ++k) {
                const int key0 = key_base + k * TILE_KEYS;
                if (key0 > my_hi || key0 + TILE_KEYS - 1 < my_lo) continue;
                const uint32_t base = smem_u32(smem + (size_t)s * STAGE_BYTES + k * TILE_BYTES);
                attend_tile<D>(st, base, base + (D / 64) * 2048, key0, lim, scale);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    finish_rows(st);
    {
        const int t = lane & 3;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (!orow[r]) continue;
            const float inv = 1.0f / st.l[r];
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<uint32_t*>(orow[r] + 8 * n + 2 * t) =
                    pack_bf16(st.o[n][2 * r] * inv, st.o[n][2 * r + 1] * inv);
        }
    }
#ifdef FERRIS_TIMELINE
    __syncthreads();
#endif
    FERRIS_TL_END(7);
}

struct MapCacheEntry {
    const void* base;
    uint64_t rows;
    int d;
    CUtensorMap map;
};

// =============================================================================================
// Prefill on the 5th-generation tensor cores (head sizes 64 and 128): one CTA per block of 128 rows ((token,
// head of the group) pairs of one kv head) and a loop over blocks of 128 keys:
//   S = Q K^T      tcgen05.mma 128 x 128 x 64 from shared memory (Q written once by the CTA, K by TMA) into
//                  tensor memory;
//   softmax        eight warps, two threads per row: tcgen05.ld of S, scale, causal / window mask, running
//                  maximum and sum in fp32 (base-2 exponentials of scores pre-multiplied by log2 e), P as
//                  bf16 into shared memory in the layout of an MMA A operand;
//   PV = P V       tcgen05.mma 128 x 64 x 128 with V as TMA wrote it (keys x head size: an MN-major B
//                  operand) into a second accumulator, folded into the thread's fp32 output row
//                  (o = (o + PV_before) * correction) one block later.
// A TMA warp streams K and V blocks through a ring of stages; an MMA warp issues S of the next block as soon
// as the softmax warps have read the current one, so the tensor core works while they exponentiate.
// One CTA per SM (shared memory and registers are each more than half an SM).  Measured with two per SM, by giving
// K a single stage and capping registers at 96: batches of short prompts gain 10 %, but one long prompt loses 15 %,
// because its time is that of the CTA of its last rows, which then shares its SM.
// Head size 64 runs two groups of softmax warps and four stages, head size 128 one group and two stages (what
// fits in shared memory).  Per block of keys the one-group chain costs about 2,600 cycles (wait for S 260, maximum
// and exchange 400, fold 400, exponentials and P 1,500, of which 1,024 is the special-function unit's time for
// 16,384 exponentials); two groups take about 4,400 cycles for two blocks (the second group's wait for the tensor
// core and the shared special-function unit keep it from halving): 2,048-token prompt 31.2 -> 29.8 us, a portion of
// 512 at the end of 4,096 keys 53.4 -> 44.9 us, 8,192-token prompt 326 -> 281 us.
// Measured and not kept: a ring of K blocks apart from a ring of V blocks, so that a K stage is free as soon as
// its scores are done (8,192-token prompt 281 -> 322 us at head size 64, 2,048 tokens at head size 128 43.7 -> 46.9 us).
// =============================================================================================
// 2^x by the special-function unit (ex2.approx: about two units in the last place; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int T5_ROWS = 128;
constexpr int T5_KEYS = 128;
constexpr int T5_GROUP_WARPS = 8;  // softmax warps of a group, two threads per row: warps 0-3 take keys 0-63 of a block, warps 4-7 keys 64-127
constexpr int t5_threads(int groups) { return (T5_GROUP_WARPS * groups + 2) * 32; }  // + a TMA warp and an MMA warp

// GROUPS = 2: two groups of softmax warps work on the SAME 128 rows, group g on the key blocks g, g + 2, ...,
// each with its own score and product accumulators in tensor memory, its own P tile and its own running
// (maximum, sum, output row); the two are merged through shared memory at the end.  A row block's time is that
// of its chain of key blocks (wait for S, maximum, exchange, fold, exponentials, one after the other: about
// 1.4 us per block, of which the exponentials' share of the special-function unit is 0.54 us), and the kernel
// lasts as long as the CTA of the prompt's last rows: two chains side by side shorten it.
template <int D, int GROUPS, int STAGES>
__global__ void __launch_bounds__(t5_threads(GROUPS), 1)
    prefill_attention_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                 const bf16* q, int ldq, bf16* __restrict__ out, int ldo,
                                 const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ seq_q_start,
                                 const int* __restrict__ seq_start_pos, int nh, int nkv, int page_size, int window,
                                 float scale, int skip_single, int* status) {
    constexpr int ATOMS = D / 64;                      // 64-wide column groups of a head (one 128-byte swizzle row each)
    constexpr int TILE = TILE_KEYS * 64 * 2;           // one 16-key x 64-column box of K or of V: 2 KB
    constexpr int ATOM_BYTES = T5_KEYS * 64 * 2;       // 128 rows x 64 columns: 16 KB
    constexpr int BLOCK_BYTES = ATOMS * ATOM_BYTES;    // 128 keys of K or of V
    constexpr int P_BYTES = 32768;                     // a group's P tile: [2 halves of 64 keys][128 rows][64] bf16
    constexpr int SW = T5_GROUP_WARPS * GROUPS;        // softmax warps; then the TMA warp and the MMA warp
    constexpr int TMEM_COLS = GROUPS == 1 ? 256 : 512; // per group 128 columns of scores and D of the product
    static_assert(GROUPS == 1 || GROUPS == 2, "one or two softmax groups");
    static_assert(128 * GROUPS + D * GROUPS <= TMEM_COLS, "tensor memory");
    static_assert(GROUPS == 1 || T5_ROWS * D * 4 <= P_BYTES, "the merge goes through a P tile");
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t kv_full[STAGES], kv_empty[STAGES], q_ready, s_ready[GROUPS], s_free[GROUPS], p_ready[GROUPS],
        pv_done[GROUPS];
    __shared__ uint32_t tmem_base;
    __shared__ float row_share[GROUPS][2][2][T5_ROWS];  // [group][block parity][key half][row]: what the two threads of a row tell each other
    __shared__ float merge_ml[2][T5_ROWS];              // maximum and sum of the second group's rows
    uint8_t* smem = align1024(smem_raw);
    uint8_t* q_smem = smem;                                  // [column group][128 rows][64] bf16, 128-byte swizzle
    uint8_t* p_smem = smem + BLOCK_BYTES;                    // per group: a P tile
    uint8_t* kv_smem = smem + BLOCK_BYTES + GROUPS * P_BYTES;  // stages x (K block, V block), each [column group][128 keys][64]

    const int G = nh / nkv;
    const int seq = blockIdx.z, hk = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int q_start = seq_q_start[seq], q_len = seq_q_start[seq + 1] - q_start;
    const int rows_total = q_len * G;
    const int n_blocks = (rows_total + T5_ROWS - 1) / T5_ROWS;
    if ((skip_single && q_len == 1) || (int)blockIdx.x >= n_blocks) {  // single tokens are the decode kernel's
        FERRIS_TL_END(8);
        return;
    }
    const int block = n_blocks - 1 - blockIdx.x;  // heavy row blocks (the last tokens see the most keys) first
    const int row0 = block * T5_ROWS;
    const int start_pos = seq_start_pos[seq];
    const int* table = block_tables + (size_t)seq * max_blocks;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_k);
        tma_prefetch_descriptor(&map_v);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        mbar_init(&q_ready, 4);
        for (int g = 0; g < GROUPS; ++g) {
            mbar_init(&s_ready[g], 1);
            mbar_init(&s_free[g], T5_GROUP_WARPS);
            mbar_init(&p_ready[g], T5_GROUP_WARPS);
            mbar_init(&pv_done[g], 1);
        }
        mbar_fence_init();
    }
    if (warp == SW + 1) tmem_alloc(&tmem_base, TMEM_COLS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_s = tmem_base, tmem_pv = tmem_base + 128 * GROUPS;  // group g: scores at + 128 g, product at + D g

    // keys of the block: from the first key its first token may see to its last token's position
    const int tok_first = row0 / G;
    const int tok_last = min(row0 + T5_ROWS - 1, rows_total - 1) / G;
    const int p_first = start_pos + tok_first, p_last = start_pos + tok_last;
    const int lo_block = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int kb_begin = lo_block / T5_KEYS, n_kb = p_last / T5_KEYS + 1 - kb_begin;

    if (warp == SW) {
        if (lane == 0) {
            constexpr int TILES = T5_KEYS / TILE_KEYS;
            const int last_tile_key = (p_last / TILE_KEYS) * TILE_KEYS;
            // the block-table look-ups of a block are independent loads issued together, one block ahead of its copies
            int rows[TILES], next_rows[TILES];
            auto look_up = [&](int i, int (&into)[TILES]) {
#pragma unroll
                for (int t = 0; t < TILES; ++t) {
                    // tiles past the last key anybody sees repeat the last one that holds keys (they are masked,
                    // but what the MMA multiplies by zero must be finite)
                    const int key0 = min((kb_begin + i) * T5_KEYS + t * TILE_KEYS, last_tile_key);
                    into[t] = cache_row_of(table, key0, page_size, nkv, hk);
                }
            };
            look_up(0, rows);
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                if (i + 1 < n_kb) look_up(i + 1, next_rows);
                if (i >= STAGES && !mbar_wait(&kv_empty[s], ((i / STAGES) - 1) & 1, status, 40)) break;
                uint8_t* ks = kv_smem + (size_t)s * 2 * BLOCK_BYTES;
                uint8_t* vs = ks + BLOCK_BYTES;
                mbar_expect_tx(&kv_full[s], 2 * BLOCK_BYTES);
#pragma unroll
                for (int t = 0; t < TILES; ++t) {
#pragma unroll
                    for (int a = 0; a < ATOMS; ++a) {
                        tma_load_2d(ks + a * ATOM_BYTES + t * TILE, &map_k, 64 * a, rows[t], &kv_full[s]);
                        tma_load_2d(vs + a * ATOM_BYTES + t * TILE, &map_v, 64 * a, rows[t], &kv_full[s]);
                    }
                }
#pragma unroll
                for (int t = 0; t < TILES; ++t) rows[t] = next_rows[t];
            }
        }
    } else if (warp == SW + 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = umma_idesc_bf16(T5_ROWS, T5_KEYS);
            const uint32_t idesc_pv = umma_idesc_bf16(T5_ROWS, D) | (1u << 16);  // B = V is MN-major (keys x head size)
            bool ok = mbar_wait(&q_ready, 0, status, 41);
            // block i belongs to group i % GROUPS and is that group's block number i / GROUPS
            auto issue_qk = [&](int i) {
                const int s = i % STAGES, g = i % GROUPS, j = i / GROUPS;
                if (!mbar_wait(&kv_full[s], (i / STAGES) & 1, status, 42)) return false;
                if (j > 0 && !mbar_wait(&s_free[g], (j - 1) & 1, status, 43)) return false;
                tcgen05_fence_after();
                const uint32_t k_addr = smem_u32(kv_smem + (size_t)s * 2 * BLOCK_BYTES);
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    // 16 columns of Q and of K: 32 bytes along the row within the column group of 64
                    const uint64_t qd = umma_desc_k_major_sw128(smem_u32(q_smem) + (k >> 2) * ATOM_BYTES) + (uint64_t)(2 * (k & 3));
                    const uint64_t kd = umma_desc_k_major_sw128(k_addr + (k >> 2) * ATOM_BYTES) + (uint64_t)(2 * (k & 3));
                    tcgen05_mma_bf16(tmem_s + 128 * g, qd, kd, idesc_qk, k > 0 ? 1u : 0u);
                }
                tcgen05_commit(&s_ready[g]);
                return true;
            };
            auto issue_pv = [&](int i) {
                const int s = i % STAGES, g = i % GROUPS;
                tcgen05_fence_after();
                // V as an MN-major operand: column groups of 64 lie ATOM_BYTES apart (the leading byte offset)
                const uint64_t v_desc = umma_desc_mn_major_sw128(smem_u32(kv_smem + (size_t)s * 2 * BLOCK_BYTES + BLOCK_BYTES), ATOM_BYTES);
#pragma unroll
                for (int k = 0; k < T5_KEYS / 16; ++k) {
                    // A: 16 keys of P = 32 bytes along the row within the half of 64 keys; B: 16 rows of V = 2 KB further
                    const uint64_t a = umma_desc_k_major_sw128(smem_u32(p_smem + g * P_BYTES + (k >> 2) * 16384)) + (uint64_t)(2 * (k & 3));
                    tcgen05_mma_bf16(tmem_pv + D * g, a, v_desc + (uint64_t)(k * (TILE >> 4)), idesc_pv, k > 0 ? 1u : 0u);
                }
                tcgen05_commit(&pv_done[g]);
                tcgen05_commit(&kv_empty[s]);
            };
            // In block order: the scores of block i + GROUPS as soon as its group has read those of block i, then the
            // product of block i.  (Measured for two groups: serving whichever group is ready first, by polling the
            // barriers, is 5 % slower; a group mostly waits for the tensor core, not for its turn.)
            for (int i = 0; i < GROUPS && i < n_kb && ok; ++i) ok = issue_qk(i);
            for (int i = 0; i < n_kb && ok; ++i) {
                if (i + GROUPS < n_kb) ok = issue_qk(i + GROUPS);
                if (!ok || !mbar_wait(&p_ready[i % GROUPS], (i / GROUPS) & 1, status, 44)) break;
                issue_pv(i);
            }
        }
    } else {
        // softmax: two threads per row; this one takes the keys [64 kh, 64 kh + 64) of its group's blocks and the
        // output columns [D/2 kh, D/2 kh + D/2)
        const int g = warp / T5_GROUP_WARPS, gw = warp % T5_GROUP_WARPS;
        const int wq = gw & 3, kh = gw >> 2;  // a warp reads the TMEM lanes 32 (warp % 4) ..: T5_GROUP_WARPS is a multiple of 4
        const int r = wq * 32 + lane;
        const int R = row0 + r;
        const bool valid = R < rows_total;
        const int tok = valid ? R / G : 0, head = hk * G + (valid ? R % G : 0);
        const int pos = start_pos + tok;
        const int hi = valid ? pos : -1;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        if (g == 0 && kh == 0) {
            const uint4* src = reinterpret_cast<const uint4*>(q + (size_t)(q_start + tok) * ldq + (size_t)head * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                *reinterpret_cast<uint4*>(q_smem + (c >> 3) * ATOM_BYTES + swizzle128(r, c & 7)) =
                    valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_ready);
        }
        const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
        const uint32_t my_s = tmem_s + 128 * g + lane_addr + 64 * kh;
        const uint32_t my_pv = tmem_pv + D * g + lane_addr + (D / 2) * kh;
        const float scale2 = scale * 1.4426950408889634f;  // scores in units of log 2
        float m = -INFINITY, l = 0.0f;
        float o[D / 2];
#pragma unroll
        for (int j = 0; j < D / 2; ++j) o[j] = 0.0f;
        const int n_own = n_kb > g ? (n_kb - g + GROUPS - 1) / GROUPS : 0;  // this group's key blocks: g, g + GROUPS, ...
        // timeline build: where the first thread of the heaviest CTA spends its cycles
        [[maybe_unused]] const bool tl_probe = threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        long long t_wait_s = 0, t_max = 0, t_fold = 0, t_exp = 0, c0 = FERRIS_TL_CLOCK(), c1;
        for (int j = 0; j < n_own; ++j) {
            const int i = j * GROUPS + g;
            if (!mbar_wait(&s_ready[g], j & 1, status, 45)) break;
            tcgen05_fence_after();
            c1 = FERRIS_TL_CLOCK();
            t_wait_s += c1 - c0;
            c0 = c1;
            const int key_base = (kb_begin + i) * T5_KEYS + 64 * kh;
            const bool interior = key_base >= lo && key_base + 63 <= hi;
            // One group: this thread's 64 scores are read once and kept, so that the next block's scores may overwrite
            // them while the exponentials are taken.  Two groups (18 warps leave a thread 96 registers): the scores
            // stay in tensor memory, read in chunks for the maximum and again for the exponentials; the other group
            // keeps the tensor core busy meanwhile.
            constexpr int KEEP = GROUPS == 1 ? 64 : 1;
            uint32_t sv[KEEP];
            float mx = -INFINITY;
            if constexpr (GROUPS == 1) {
                tmem_load_32x64(my_s, reinterpret_cast<uint32_t (&)[64]>(sv));
                tmem_load_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_free[g]);
                if (interior) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(sv[c % KEEP]));
                } else {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int key = key_base + c;
                        mx = fmaxf(mx, (key <= hi && key >= lo) ? __uint_as_float(sv[c % KEEP]) : -INFINITY);
                    }
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t sc[32];
                    tmem_load_32x32(my_s + 32 * h, sc);
                    tmem_load_wait();
                    if (interior) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) mx = fmaxf(mx, __uint_as_float(sc[c]));
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int key = key_base + 32 * h + c;
                            mx = fmaxf(mx, (key <= hi && key >= lo) ? __uint_as_float(sc[c]) : -INFINITY);
                        }
                    }
                }
            }
            mx *= scale2;  // the scale is positive: the maximum of the scaled scores
            // the row's maximum over both halves of the block
            row_share[g][j & 1][kh][r] = mx;
            if (g == 0)
                asm volatile("bar.sync 1, 256;" ::: "memory");
            else
                asm volatile("bar.sync 2, 256;" ::: "memory");
            mx = fmaxf(mx, row_share[g][j & 1][kh ^ 1][r]);
            c1 = FERRIS_TL_CLOCK();
            t_max += c1 - c0;
            c0 = c1;
            const float m_new = fmaxf(m, mx);
            const float base = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = m == -INFINITY ? 0.0f : fast_exp2(m - base);
            if (j > 0) {
                // the product of the group's block before (relative to its maximum m) joins the row before the row is rescaled
                if (!mbar_wait(&pv_done[g], (j - 1) & 1, status, 46)) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t pv[32];
                    tmem_load_32x32(my_pv + 32 * c, pv);
                    tmem_load_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[32 * c + e] = (o[32 * c + e] + __uint_as_float(pv[e])) * corr;
                }
            }
            l *= corr;
            c1 = FERRIS_TL_CLOCK();
            t_fold += c1 - c0;
            c0 = c1;
            {
                float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // four partial sums: the additions do not wait for one another
                uint8_t* half = p_smem + g * P_BYTES + kh * 16384;
#pragma unroll
                for (int h = 0; h < 4; ++h) {  // 16 keys at a time
                    uint32_t sc[16], packed[8];
                    if constexpr (GROUPS == 1) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) sc[c] = sv[(16 * h + c) % KEEP];
                    } else {
                        tmem_load_32x16(my_s + 16 * h, sc);
                        tmem_load_wait();
                    }
                    if (interior) {
#pragma unroll
                        for (int c = 0; c < 16; c += 2) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(sc[c]), scale2, -base));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(sc[c + 1]), scale2, -base));
                            sum4[(c >> 1) & 3] += p0 + p1;
                            packed[c >> 1] = pack_bf16(p0, p1);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 16; c += 2) {
                            const int key = key_base + 16 * h + c;
                            const float e0 = fast_exp2(fmaf(__uint_as_float(sc[c]), scale2, -base));
                            const float e1 = fast_exp2(fmaf(__uint_as_float(sc[c + 1]), scale2, -base));
                            const float p0 = (key <= hi && key >= lo) ? e0 : 0.0f;
                            const float p1 = (key + 1 <= hi && key + 1 >= lo) ? e1 : 0.0f;
                            sum4[(c >> 1) & 3] += p0 + p1;
                            packed[c >> 1] = pack_bf16(p0, p1);
                        }
                    }
                    *reinterpret_cast<uint4*>(half + swizzle128(r, 2 * h)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    *reinterpret_cast<uint4*>(half + swizzle128(r, 2 * h + 1)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
                l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            }
            if constexpr (GROUPS == 2) {
                // the scores have been read for the last time: the group's next block may overwrite them
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_free[g]);
            }
            m = m_new;
            fence_proxy_async();  // the MMA reads P through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[g]);
            c1 = FERRIS_TL_CLOCK();
            t_exp += c1 - c0;
            c0 = c1;
        }
        FERRIS_TL_VALUE(tl_probe, 0, (unsigned long long)t_wait_s);
        FERRIS_TL_VALUE(tl_probe, 1, (unsigned long long)t_max);
        FERRIS_TL_VALUE(tl_probe, 2, (unsigned long long)t_fold);
        FERRIS_TL_VALUE(tl_probe, 3, (unsigned long long)t_exp);
        FERRIS_TL_VALUE(tl_probe, 4, (unsigned long long)n_own);
        // the row's sum over both halves of the keys
        row_share[g][n_own & 1][kh][r] = l;
        if (g == 0)
            asm volatile("bar.sync 1, 256;" ::: "memory");
        else
            asm volatile("bar.sync 2, 256;" ::: "memory");
        l += row_share[g][n_own & 1][kh ^ 1][r];
        // the group's last product joins the row (still relative to m, not yet divided by the sum)
        bool done = true;
        if (n_own > 0) {
            done = mbar_wait(&pv_done[g], (n_own - 1) & 1, status, 47);
            if (done) {
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < D / 64; ++c) {
                    uint32_t pv[32];
                    tmem_load_32x32(my_pv + 32 * c, pv);
                    tmem_load_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[32 * c + e] += __uint_as_float(pv[e]);
                }
            }
        }
        if constexpr (GROUPS == 2) {
            // the second group hands its rows over through its own P tile (its last product has been read out of
            // it): [output column][row] fp32, so that a warp's 32 rows are 32 consecutive words
            float* merge_o = reinterpret_cast<float*>(p_smem + P_BYTES);
            if (g == 1) {
#pragma unroll
                for (int c = 0; c < D / 2; ++c) merge_o[((D / 2) * kh + c) * T5_ROWS + r] = o[c];
                if (kh == 0) {
                    merge_ml[0][r] = m;
                    merge_ml[1][r] = l;
                }
            }
            asm volatile("bar.sync 3, 512;" ::: "memory");
            if (g == 0) {
                const float m1 = merge_ml[0][r], l1 = merge_ml[1][r];
                const float mm = fmaxf(m, m1);
                const float a0 = m == -INFINITY ? 0.0f : fast_exp2(m - mm);
                const float a1 = m1 == -INFINITY ? 0.0f : fast_exp2(m1 - mm);
                l = l * a0 + l1 * a1;
#pragma unroll
                for (int c = 0; c < D / 2; ++c) o[c] = o[c] * a0 + merge_o[((D / 2) * kh + c) * T5_ROWS + r] * a1;
            }
        }
        if (g == 0 && done && n_kb > 0 && valid) {
            uint32_t packed[D / 4];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
            for (int c = 0; c < D / 2; c += 2) packed[c >> 1] = pack_bf16(o[c] * inv, o[c + 1] * inv);
            uint4* dst = reinterpret_cast<uint4*>(out + (size_t)(q_start + tok) * ldo + (size_t)head * D + (D / 2) * kh);
#pragma unroll
            for (int u = 0; u < D / 16; ++u) dst[u] = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == SW + 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    FERRIS_TL_END(8);
}

constexpr int MAP_CACHE = 512;
MapCacheEntry g_maps[MAP_CACHE];
int g_map_count = 0;

// Tensor maps are cached by (base address, extent): a cache tensor keeps both for its lifetime.
int cache_map(const void* base, uint64_t rows, int d, CUtensorMap* out) {
    for (int i = 0; i < g_map_count; ++i)
        if (g_maps[i].base == base && g_maps[i].rows == rows && g_maps[i].d == d) {
            *out = g_maps[i].map;
            return FERRIS_OK;
        }
    CUtensorMap m;
    int rc = ferris_make_tensor_map_2d(&m, base, rows, (uint64_t)d, (uint64_t)d, TILE_KEYS, 64);
    if (rc != FERRIS_OK) return rc;
    const int slot = g_map_count < MAP_CACHE ? g_map_count++ : 0;
    g_maps[slot] = {base, rows, d, m};
    *out = m;
    return FERRIS_OK;
}

// One map over the key cache and the value cache when they are two planes of one tensor (the value plane begins where
// the key plane ends): dims (d, rows, 2), box (64, 16, 2).  Returns false when they are not, or the map cannot be made.
MapCacheEntry g_pair_maps[MAP_CACHE];
int g_pair_map_count = 0;
bool cache_pair_map(const void* k_base, const void* v_base, uint64_t rows, int d, CUtensorMap* out) {
    const uint64_t plane = rows * (uint64_t)d * 2;
    if ((const uint8_t*)v_base != (const uint8_t*)k_base + plane) return false;
    for (int i = 0; i < g_pair_map_count; ++i)
        if (g_pair_maps[i].base == k_base && g_pair_maps[i].rows == rows && g_pair_maps[i].d == d) {
            *out = g_pair_maps[i].map;
            return true;
        }
    CUtensorMap m;
    if (ferris_make_tensor_map_planes(&m, k_base, rows, (uint64_t)d, plane, TILE_KEYS) != FERRIS_OK) return false;
    const int slot = g_pair_map_count < MAP_CACHE ? g_pair_map_count++ : 0;
    g_pair_maps[slot] = {k_base, rows, d, m};
    *out = m;
    return true;
}

int check_common(int nh, int nkv, int d, int page_size, int max_blocks) {
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) FERRIS_REFUSE("attention: %d heads over %d kv heads", nh, nkv);
    if (nh / nkv > 16) FERRIS_REFUSE("tensor-core attention takes groups of at most 16 heads, not %d", nh / nkv);
    if (d != 64 && d != 128) FERRIS_REFUSE("tensor-core attention takes head sizes 64 and 128, not %d", d);
    if (page_size <= 0 || page_size % TILE_KEYS) FERRIS_REFUSE("tensor-core attention takes pages of a multiple of 16 tokens, not %d", page_size);
    if (max_blocks <= 0) FERRIS_REFUSE("attention: max_blocks=%d", max_blocks);
    return FERRIS_OK;
}

// Prefill runs the tcgen05 kernel unless the environment says FERRIS_ATTN_TCGEN05=0 (then the mma.sync kernel);
// FERRIS_ATTN_TCGEN05=2: the tcgen05 kernel with one softmax group at every head size.
int g_prefill_tc5 = -1;
bool prefill_on_tcgen05() {
    if (g_prefill_tc5 < 0) {
        const char* v = getenv("FERRIS_ATTN_TCGEN05");
        g_prefill_tc5 = (v && (v[0] == '0' || v[0] == '2')) ? v[0] - '0' : 1;
    }
    return g_prefill_tc5 != 0;
}

template <typename F>
int set_smem(F kernel, size_t bytes) {
    return ferris_allow_dynamic_smem((const void*)kernel, bytes);
}

}  // namespace

// Floats of scratch that decode attention with `splits` > 1 needs: partial outputs and (m, l) pairs.
FERRIS_API long long ferris_decode_attention_scratch_floats(int tokens, int nh, int d, int splits) {
    if (splits <= 1) return 0;
    return (long long)tokens * nh * splits * (d + 2);
}

// The decode kernel's shape, warps * 10 + stages of 16 KB per warp.  A warp works a block of keys (64 of head size 64,
// 32 of head size 128) off in a dependent chain, one block after the other, so a CTA with many blocks wants many warps
// (8 or 12 warps with one stage each hold as many bytes in flight as 4 warps with three); every warp adds to the merge
// at the end.
// Groups of at most 8 heads (the transposed products, half the work a block): eight warps with one stage each were the
// fastest or within half a percent of it wherever measured (ms a decode step at the 0.5B sizes, 4 x 3 / 8 x 1 / 12 x 1
// warps x stages): batch 1 of 4,096 keys . / 0.702 / 0.738; batch 4 0.727 / 0.692 / 0.710; batch 8 0.771 / 0.744 /
// 0.741; batch 16 0.963 / 0.924 / 0.961; batch 32 1.491 / 1.437 / 1.433; batch 64 1.847 / 1.750 / 1.781; batch 8 of
// 512 keys 0.657 / 0.653 / 0.675; batch 8 of 16,384 keys 1.050 / 0.989 / 0.986.  Stages of 96 keys instead of 64 (eight
// warps then hold 192 KB, and the tiles of a key range divide more evenly among them) were slower at every batch but
// one (batch 1 / 4 / 8 / 16 / 64: 0.747 / 0.721 / 0.741 / 0.965 / 1.794 against 0.703 / 0.692 / 0.744 / 0.924 / 1.750):
// a CTA of 129 KB shares its SM with the launches before and after it, one of 197 KB does not.
// Larger groups (16 rows a warp): by the blocks a CTA may get (from the width of the block tables, which is up to
// twice what the requests hold); measured with the 16-row products at a group of 7: batch 8 of 512 keys 0.683 /
// 0.691 / 0.709; batch 1 of 4,096 keys 0.783 / 0.748 / 0.778; batch 8 0.798 / 0.792 / 0.784; batch 32 1.498 / 1.477
// / 1.461; batch 64 1.887 / 1.866 / 1.849; batch 8 of 16,384 keys 1.096 / 1.098 / 1.055.
static int decode_shape(int group, int blocks, int ctas) {
    if (group <= 8) return 81;
    return blocks <= 4 ? 43 : ((blocks < 10 || ctas <= 64) ? 81 : 121);
}

static int decode_attention_impl(const void* q, int ldq, void* out, int ldo, const void* k_cache, const void* v_cache,
                                 long long cache_pages, const int* block_tables, int max_blocks, const int* token_seq,
                                 const int* positions, const int* token_list, int tokens, int nh, int nkv, int d,
                                 int page_size, int window, float scale, int splits, float* scratch, void* stream,
                                 const float* inv_freq = nullptr, const int* slot_mapping = nullptr, int merge = 1) {
    if (tokens <= 0) return FERRIS_OK;
    int rc = check_common(nh, nkv, d, page_size, max_blocks);
    if (rc != FERRIS_OK) return rc;
    if (splits < 1 || splits > 65535) FERRIS_REFUSE("decode attention: %d splits", splits);
    if (splits > 1 && !scratch && merge != 3) FERRIS_REFUSE("decode attention: splitting the keys needs scratch memory");
    if (nkv > 65535 || tokens > 65535) FERRIS_REFUSE("decode attention: %d tokens x %d kv heads exceed one launch", tokens, nkv);
    const uint64_t rows = (uint64_t)cache_pages * nkv * page_size;
    CUtensorMap mk, mv;
    if ((rc = cache_map(k_cache, rows, d, &mk)) != FERRIS_OK) return rc;
    if ((rc = cache_map(v_cache, rows, d, &mv)) != FERRIS_OK) return rc;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)tokens * nh * splits * d : nullptr;
    dim3 grid(splits, nkv, tokens);
    cudaStream_t s = (cudaStream_t)stream;
    int* status = ferris_status_ptr();
    FusedRope rope;
    rope.inv_freq = inv_freq;
    rope.slot_mapping = slot_mapping;
    rope.k_cache = (bf16*)const_cast<void*>(k_cache);
    rope.v_cache = (bf16*)const_cast<void*>(v_cache);
    const int cluster = (merge == 3 && splits > 1) ? 1 : 0;
    if (cluster && splits > MAX_CLUSTER)
        FERRIS_REFUSE("decode attention: a cluster merges at most %d key ranges, not %d", MAX_CLUSTER, splits);
    cudaError_t e = cudaSuccess;
    CUtensorMap mkv;
    const bool pair = cache_pair_map(k_cache, v_cache, rows, d, &mkv);
    if (pair) mk = mkv;
    // warps x stages of 16 KB each (4 tiles of head size 64, 2 of head size 128)
    long long keys = (long long)max_blocks * page_size;
    if (window > 0 && window + TILE_KEYS < keys) keys = window + TILE_KEYS;
    const int tiles_per_range = (int)(((keys + TILE_KEYS - 1) / TILE_KEYS + splits - 1) / splits);
    const int tiles_per_block = d == 64 ? 4 : 2;
    const int shape = decode_shape(nh / nkv, (tiles_per_range + tiles_per_block - 1) / tiles_per_block, splits * nkv * tokens);
    const int nw = shape / 10, st = shape % 10;
    // behind the stages: what the key ranges of a cluster send each other, [splits][G][2] + [splits][share] fp32
    const int G = nh / nkv;
    const size_t recv_bytes = cluster ? (size_t)splits * (2 * G + (G * d + splits - 1) / splits) * 4 : 0;
    const size_t smem = (size_t)nw * st * 16384 + 1024 + recv_bytes;
    auto launch = [&](auto kernel) -> cudaError_t {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(nw * 32);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        int n = 0;
        if (cluster) {
            attr[n].id = cudaLaunchAttributeClusterDimension;
            attr[n].val.clusterDim.x = (unsigned)splits;
            attr[n].val.clusterDim.y = 1;
            attr[n].val.clusterDim.z = 1;
            ++n;
            if (splits > 8) {
                const cudaError_t allowed = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                if (allowed != cudaSuccess) return allowed;
            }
        }
        if (ferris_pdl_enabled()) {
            attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[n].val.programmaticStreamSerializationAllowed = 1;
            ++n;
        }
        cfg.attrs = attr;
        cfg.numAttrs = n;
        return cudaLaunchKernelEx(&cfg, kernel, mk, mv, (const bf16*)q, ldq, (bf16*)out, ldo, part_o, part_ml, block_tables,
                                  max_blocks, token_seq, positions, token_list, nh, nkv, page_size, window, scale, splits,
                                  rope, cluster, status);
    };
#define FERRIS_DECODE_LAUNCH_AS(DD, PP, NWW, STT)                                                                \
    do {                                                                                                         \
        if (G <= 8) {                                                                                            \
            if ((rc = set_smem(decode_attention_kernel<DD, STT, PP, NWW, true>, smem)) != FERRIS_OK) return rc;  \
            e = launch(decode_attention_kernel<DD, STT, PP, NWW, true>);                                         \
        } else {                                                                                                 \
            if ((rc = set_smem(decode_attention_kernel<DD, STT, PP, NWW, false>, smem)) != FERRIS_OK) return rc; \
            e = launch(decode_attention_kernel<DD, STT, PP, NWW, false>);                                        \
        }                                                                                                        \
    } while (0)
#define FERRIS_DECODE_LAUNCH(DD, PP)                              \
    do {                                                          \
        if (shape == 121) FERRIS_DECODE_LAUNCH_AS(DD, PP, 12, 1); \
        else if (shape == 81) FERRIS_DECODE_LAUNCH_AS(DD, PP, 8, 1); \
        else FERRIS_DECODE_LAUNCH_AS(DD, PP, 4, 3);               \
    } while (0)
    if (d == 64) {
        if (pair) FERRIS_DECODE_LAUNCH(64, true);
        else FERRIS_DECODE_LAUNCH(64, false);
        if (e == cudaSuccess && splits > 1 && merge == 1) ferris_launch(decode_merge_kernel<64>, dim3(tokens, nh), dim3(64), 0, s, part_o, part_ml, (bf16*)out, ldo, token_list, nh, splits);
    } else {
        if (pair) FERRIS_DECODE_LAUNCH(128, true);
        else FERRIS_DECODE_LAUNCH(128, false);
        if (e == cudaSuccess && splits > 1 && merge == 1) ferris_launch(decode_merge_kernel<128>, dim3(tokens, nh), dim3(128), 0, s, part_o, part_ml, (bf16*)out, ldo, token_list, nh, splits);
    }
#undef FERRIS_DECODE_LAUNCH_AS
#undef FERRIS_DECODE_LAUNCH
    if (e != cudaSuccess) {
        ferris_set_error("decode attention: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

// Single-token steps.  scratch: fp32 [tokens * nh * splits * (d + 2)] when splits > 1.
FERRIS_API int ferris_decode_attention(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                       const void* v_cache, long long cache_pages, const int* block_tables,
                                       int max_blocks, const int* token_seq, const int* positions, int tokens, int nh,
                                       int nkv, int d, int page_size, int window, float scale, int splits, float* scratch,
                                       void* stream) {
    return decode_attention_impl(q, ldq, out, ldo, k_cache, v_cache, cache_pages, block_tables, max_blocks, token_seq,
                                 positions, nullptr, tokens, nh, nkv, d, page_size, window, scale, splits, scratch, stream);
}

// The same for the rows of a step that `token_list` (int32 [tokens]) names: the single tokens of a step
// that also carries portions of prompts.  The scratch is indexed by place in the list.
FERRIS_API int ferris_decode_attention_listed(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                              const void* v_cache, long long cache_pages, const int* block_tables,
                                              int max_blocks, const int* token_seq, const int* positions,
                                              const int* token_list, int tokens, int nh, int nkv, int d, int page_size,
                                              int window, float scale, int splits, float* scratch, void* stream) {
    if (!token_list) FERRIS_REFUSE("decode attention: no token list");
    return decode_attention_impl(q, ldq, out, ldo, k_cache, v_cache, cache_pages, block_tables, max_blocks, token_seq,
                                 positions, token_list, tokens, nh, nkv, d, page_size, window, scale, splits, scratch, stream);
}

// Single-token steps whose q and k have NOT been rotated and whose k and v are NOT in the cache yet: the kernel
// does the work of the rotary / cache-write kernel on its way (every dim of a head rotated: rotary dims == d).
// qkv: the step's [tokens, (nh + 2 nkv) d] rows; slot_mapping null: rotate q only (a layer that reads another
// layer's cache).  merge: 1 a merge kernel follows; 0 with splits > 1: the partial results of the key ranges stay
// in scratch, `out` is not written, and the caller merges them (ferris_decode_merge, or the product that follows
// does it on its way); 3: the key ranges of a (token, kv head) form a thread-block cluster (at most 8 ranges) that
// merges them through its distributed shared memory, without scratch (ferris_decode_cluster_splits says how many
// ranges).  A merge by the CTA that finishes last among the ranges (a fence, a counter in global memory) was measured
// too: it cost the decode step of 8 tokens 8.6 us a layer, twice what the merge kernel costs.
FERRIS_API int ferris_decode_attention_rope(const void* qkv, int ldq, void* out, int ldo, void* k_cache, void* v_cache,
                                            long long cache_pages, const int* block_tables, int max_blocks,
                                            const int* token_seq, const int* positions, const float* inv_freq,
                                            const int* slot_mapping, int tokens, int nh, int nkv, int d, int page_size,
                                            int window, float scale, int splits, float* scratch, int merge,
                                            void* stream) {
    if (!inv_freq) FERRIS_REFUSE("decode attention with rotation: no frequency table");
    if (merge != 0 && merge != 1 && merge != 3) FERRIS_REFUSE("decode attention with rotation: merge mode %d", merge);
    return decode_attention_impl(qkv, ldq, out, ldo, k_cache, v_cache, cache_pages, block_tables, max_blocks, token_seq,
                                 positions, nullptr, tokens, nh, nkv, d, page_size, window, scale, splits, scratch, stream,
                                 inv_freq, slot_mapping, merge);
}

// Into how many key ranges a step of `tokens` single tokens is cut when a cluster merges them (merge mode 3): at
// most 8 (a portable cluster), or up to 16 where the block tables span 16,384 keys or more (one or two requests
// with long contexts: 16 CTAs instead of 8 stream each kv head's keys); no more than fill the SMs once, at least
// eight 16-key tiles each, and only as many as the GPU holds clusters of that size at once (the CTAs of a cluster
// share a GPC; a cluster that has to wait for one costs a second round).  0: this head size has no such kernel.
FERRIS_API int ferris_decode_cluster_splits(int tokens, int nkv, int d, int max_kv_len) {
    if (tokens <= 0 || nkv <= 0 || (d != 64 && d != 128)) return 0;
    static int fits[2][MAX_CLUSTER + 1] = {};  // clusters of size s that are resident at once, by head size; 0 = not asked yet
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        sms = 148;
    const int groups = tokens * nkv;
    int want = sms / groups;
    const int cap = max_kv_len >= 16384 ? MAX_CLUSTER : 8;
    if (want > cap) want = cap;
    const int most = (max_kv_len / TILE_KEYS) / 8;
    if (want > most) want = most;
    if (want < 1) want = 1;
    for (int sp = want; sp > 1; --sp) {
        int& have = fits[d == 64 ? 0 : 1][sp];
        if (have == 0) {
            have = -1;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sp, 1, 1);
            // every shape of the kernel takes more than half an SM's shared memory: one CTA per SM; asked for the
            // shape with the most threads and bytes
            cfg.blockDim = dim3(12 * 32);
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)sp;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            cudaError_t e = cudaSuccess;
            cfg.dynamicSmemBytes = (size_t)12 * 16384 + 1024 + (size_t)(MAX_CLUSTER * 2 * 16 + 16 * d + MAX_CLUSTER) * 4;
            if (sp > 8) {
                if (d == 64) cudaFuncSetAttribute(decode_attention_kernel<64, 1, true, 12, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                else cudaFuncSetAttribute(decode_attention_kernel<128, 1, true, 12, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            }
            if (d == 64) {
                set_smem(decode_attention_kernel<64, 1, true, 12, true>, cfg.dynamicSmemBytes);
                e = cudaOccupancyMaxActiveClusters(&clusters, decode_attention_kernel<64, 1, true, 12, true>, &cfg);
            } else {
                set_smem(decode_attention_kernel<128, 1, true, 12, true>, cfg.dynamicSmemBytes);
                e = cudaOccupancyMaxActiveClusters(&clusters, decode_attention_kernel<128, 1, true, 12, true>, &cfg);
            }
            if (e == cudaSuccess && clusters > 0) have = clusters;
            else cudaGetLastError();
        }
        if (have >= groups) return sp;
    }
    return 1;
}

// The merge alone, for partial results that ferris_decode_attention_rope left in scratch (merge == 0):
// out [tokens, nh * d] bf16 from scratch = [tokens, nh, splits, d] followed by [tokens, nh, splits, 2].
FERRIS_API int ferris_decode_merge(const float* scratch, void* out, int ldo, int tokens, int nh, int d, int splits,
                                   void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (!scratch || splits < 1 || nh <= 0 || nh > 65535) FERRIS_REFUSE("decode merge: %d heads, %d splits", nh, splits);
    if (d != 64 && d != 128) FERRIS_REFUSE("decode merge: head size %d (64 or 128)", d);
    const float* part_o = scratch;
    const float* part_ml = scratch + (size_t)tokens * nh * splits * d;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 64)
        ferris_launch(decode_merge_kernel<64>, dim3(tokens, nh), dim3(64), 0, s, part_o, part_ml, (bf16*)out, ldo, (const int*)nullptr, nh, splits);
    else
        ferris_launch(decode_merge_kernel<128>, dim3(tokens, nh), dim3(128), 0, s, part_o, part_ml, (bf16*)out, ldo, (const int*)nullptr, nh, splits);
    FERRIS_LAUNCH_CHECK();
}

// Which prefill kernel runs: 1 the tcgen05 kernel (the default), 0 the mma.sync kernel, 2 the tcgen05 kernel with
// one softmax group at every head size.
FERRIS_API int ferris_set_prefill_tcgen05(int on) {
    g_prefill_tc5 = (on >= 0 && on <= 2) ? on : 1;
    return FERRIS_OK;
}

// Portions of prompts (and anything else: a request with one token is a portion of one, unless
// skip_single leaves those to the decode kernel).
FERRIS_API int ferris_prefill_attention(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                        const void* v_cache, long long cache_pages, const int* block_tables,
                                        int max_blocks, const int* seq_q_start, const int* seq_start_pos, int num_seqs,
                                        int max_q_len, int nh, int nkv, int d, int page_size, int window, float scale,
                                        int skip_single, void* stream) {
    if (num_seqs <= 0 || max_q_len <= 0) return FERRIS_OK;
    int rc = check_common(nh, nkv, d, page_size, max_blocks);
    if (rc != FERRIS_OK) return rc;
    if (nkv > 65535 || num_seqs > 65535) FERRIS_REFUSE("prefill attention: %d requests x %d kv heads exceed one launch", num_seqs, nkv);
    const uint64_t rows = (uint64_t)cache_pages * nkv * page_size;
    CUtensorMap mk, mv;
    if ((rc = cache_map(k_cache, rows, d, &mk)) != FERRIS_OK) return rc;
    if ((rc = cache_map(v_cache, rows, d, &mv)) != FERRIS_OK) return rc;
    const int G = nh / nkv;
    cudaStream_t s = (cudaStream_t)stream;
    int* status = ferris_status_ptr();
    if (prefill_on_tcgen05()) {
        dim3 grid5(((size_t)max_q_len * G + T5_ROWS - 1) / T5_ROWS, nkv, num_seqs);
        // Q, a P tile per softmax group, stages of (K block, V block).  Head size 64: two groups and four stages
        // (209 KB); head size 128: one group and two stages (193 KB), two groups would not fit.
        auto bytes = [&](int groups, int stages) {
            return (size_t)T5_ROWS * d * 2 + (size_t)groups * 32768 + (size_t)stages * 2 * T5_KEYS * d * 2 + 1024;
        };
#define FERRIS_T5_LAUNCH(DD, GG, SS)                                                                                       \
    do {                                                                                                                   \
        const size_t smem = bytes(GG, SS);                                                                                 \
        if ((rc = set_smem(prefill_attention_tc5_kernel<DD, GG, SS>, smem)) != FERRIS_OK) return rc;                       \
        ferris_launch(prefill_attention_tc5_kernel<DD, GG, SS>, grid5, dim3(t5_threads(GG)), smem, s, mk, mv, (const bf16*)q, \
                      ldq, (bf16*)out, ldo, block_tables, max_blocks, seq_q_start, seq_start_pos, nh, nkv, page_size,      \
                      window, scale, skip_single, status);                                                                 \
    } while (0)
        if (d == 64 && g_prefill_tc5 != 2)
            FERRIS_T5_LAUNCH(64, 2, 4);
        else if (d == 64)
            FERRIS_T5_LAUNCH(64, 1, 4);
        else
            FERRIS_T5_LAUNCH(128, 1, 2);
#undef FERRIS_T5_LAUNCH
        FERRIS_LAUNCH_CHECK();
    }
    dim3 grid(((size_t)max_q_len * G + PF_ROWS - 1) / PF_ROWS, nkv, num_seqs);
    if (d == 64) {
        constexpr int ST = 3;
        const size_t smem = (size_t)ST * PF_STAGE_TILES * 2 * TILE_KEYS * 64 * 2 + 1024;
        if ((rc = set_smem(prefill_attention_kernel<64, ST>, smem)) != FERRIS_OK) return rc;
        ferris_launch(prefill_attention_kernel<64, ST>, grid, dim3((WARPS + 1) * 32), smem, s, mk, mv, (const bf16*)q, ldq, (bf16*)out, ldo, block_tables, max_blocks, seq_q_start, seq_start_pos, nh, nkv,
            page_size, window, scale, skip_single, status);
    } else {
        constexpr int ST = 2;
        const size_t smem = (size_t)ST * PF_STAGE_TILES * 2 * TILE_KEYS * 128 * 2 + 1024;
        if ((rc = set_smem(prefill_attention_kernel<128, ST>, smem)) != FERRIS_OK) return rc;
        ferris_launch(prefill_attention_kernel<128, ST>, grid, dim3((WARPS + 1) * 32), smem, s, mk, mv, (const bf16*)q, ldq, (bf16*)out, ldo, block_tables, max_blocks, seq_q_start, seq_start_pos, nh, nkv,
            page_size, window, scale, skip_single, status);
    }
    FERRIS_LAUNCH_CHECK();
}

// =============================================================================================
// The same decode attention for callers that cannot allocate: the partial results of the splits go
// to a fixed array in the device image instead of a buffer that the caller brings (no_alloc.h).
// =============================================================================================
#include "no_alloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_static_scratch[FERRIS_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_ptr[MAX_DEVICES] = {};

// Device address of the array on the current device; looked up once per device.
int static_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        ferris_set_error("static scratch: %s", cudaGetErrorString(e));
        return (int)e;
    }
    if (dev < 0 || dev >= MAX_DEVICES) FERRIS_REFUSE("static scratch: device %d is beyond the %d this build tracks", dev, MAX_DEVICES);
    if (!g_static_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) {
            ferris_set_error("static scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : FERRIS_BAD_ARGUMENT;
        }
        g_static_scratch_ptr[dev] = (float*)p;
    }
    *out = g_static_scratch_ptr[dev];
    return FERRIS_OK;
}
}  // namespace

int ferris_decode_attention_static_scratch(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                           const void* v_cache, long long cache_pages, const int* block_tables,
                                           int max_blocks, const int* token_seq, const int* positions, int tokens,
                                           int nh, int nkv, int d, int page_size, int window, float scale, int splits,
                                           void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (splits < 1) FERRIS_REFUSE("decode attention: %d splits", splits);
    const long long need = ferris_decode_attention_scratch_floats(tokens, nh, d, splits);
    if (need > (long long)FERRIS_STATIC_SCRATCH_FLOATS)
        FERRIS_REFUSE("decode attention without allocation: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of "
                      "partial results exceed the built-in scratch of %u floats; use fewer splits or tokens, or the "
                      "entry point that takes a scratch buffer",
                      tokens, nh, splits, d, need, FERRIS_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc != FERRIS_OK) return rc;
    return ferris_decode_attention(q, ldq, out, ldo, k_cache, v_cache, cache_pages, block_tables, max_blocks, token_seq,
                                   positions, tokens, nh, nkv, d, page_size, window, scale, splits, scratch, stream);
}

FERRIS_TIMELINE_TU(attention_mma)
