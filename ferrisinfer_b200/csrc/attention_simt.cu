// Attention over the paged cache, general form: any head size up to 256, any page size, any
// number of heads and groups, an optional window; fp32 arithmetic throughout whatever the
// storage type.  One block per (token, query head); the warps of a block split the keys and keep
// a running maximum, sum and weighted value sum each, merged at the end.
//
//   query head hq uses kv head hq / (nh / nkv); s_j = (q . k_j) * scale; the query at absolute
//   position P attends keys lo..P, lo = 0 or P - window + 1; softmax over them; out = sum w_j v_j.
//   With `slopes` (one per query head; a position encoding that acts on the scores, not on q and k):
//   s_j += slopes[hq] * (j - P), a penalty linear in the distance.
// (crates/ferrisinfer-kernel/src/cpu/attention.rs:729-781, 1125-1155: streaming softmax with a
// running maximum, which this kernel keeps per warp).  The step's own keys are already in the
// cache when this runs, so prompts, portions of prompts and single decoded tokens are one case.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ATT_THREADS = 128;
constexpr int ATT_WARPS = ATT_THREADS / 32;
constexpr int MAX_PER_LANE = 8;  // head size up to 256

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
    paged_attention_simt_kernel(const T* q, int ldq, T* __restrict__ out, int ldo, const T* k_cache, const T* v_cache,
                                const int* __restrict__ block_tables, int max_blocks,
                                const int* __restrict__ token_seq, const int* __restrict__ positions, int nh,
                                int nkv, int d, int page_size, int window, float scale,
                                const float* __restrict__ slopes) {
    extern __shared__ float smem[];  // per warp: m, z, acc[d]
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, hq = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int hk = hq / (nh / nkv);
    const int seq = token_seq[t];
    const int P = positions[t];
    const int lo = (window > 0 && P - window + 1 > 0) ? P - window + 1 : 0;
    const int* table = block_tables + (size_t)seq * max_blocks;
    const float slope = slopes ? slopes[hq] : 0.0f;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = q + (size_t)t * ldq + (size_t)hq * d;
#pragma unroll
    for (int r = 0; r < MAX_PER_LANE; ++r) {
        const int i = lane + 32 * r;
        qv[r] = i < d ? to_float(qrow[i]) : 0.0f;
        acc[r] = 0.0f;
    }
    float m = -INFINITY, z = 0.0f;
    for (int j = lo + warp; j <= P; j += ATT_WARPS) {
        const int page = table[j / page_size];
        if (page < 0) continue;  // a hole in the table: never reached for keys inside the window
        const size_t base = (((size_t)page * nkv + hk) * page_size + (j % page_size)) * d;
        float dot = 0.0f;
#pragma unroll
        for (int r = 0; r < MAX_PER_LANE; ++r) {
            const int i = lane + 32 * r;
            if (i < d) dot = fmaf(qv[r], to_float(k_cache[base + i]), dot);
        }
        const float s = slopes ? fmaf(slope, (float)(j - P), warp_sum(dot) * scale) : warp_sum(dot) * scale;
        float wgt;
        if (s > m) {
            const float rescale = expf(m - s);  // exp(-inf) = 0 on the first key
#pragma unroll
            for (int r = 0; r < MAX_PER_LANE; ++r) acc[r] *= rescale;
            z = z * rescale + 1.0f;
            m = s;
            wgt = 1.0f;
        } else {
            wgt = expf(s - m);
            z += wgt;
        }
#pragma unroll
        for (int r = 0; r < MAX_PER_LANE; ++r) {
            const int i = lane + 32 * r;
            if (i < d) acc[r] = fmaf(wgt, to_float(v_cache[base + i]), acc[r]);
        }
    }
    float* mine = smem + warp * (d + 2);
    if (lane == 0) {
        mine[0] = m;
        mine[1] = z;
    }
#pragma unroll
    for (int r = 0; r < MAX_PER_LANE; ++r) {
        const int i = lane + 32 * r;
        if (i < d) mine[2 + i] = acc[r];
    }
    __syncthreads();
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) mm = fmaxf(mm, smem[w * (d + 2)]);
    float zz = 0.0f;
    float f[ATT_WARPS];
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
        const float mw = smem[w * (d + 2)];
        f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
        zz += smem[w * (d + 2) + 1] * f[w];
    }
    const float inv = 1.0f / zz;
    T* orow = out + (size_t)t * ldo + (size_t)hq * d;
    for (int i = threadIdx.x; i < d; i += ATT_THREADS) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) o += smem[w * (d + 2) + 2 + i] * f[w];
        orow[i] = from_float<T>(o * inv);
    }
}

}  // namespace

FERRIS_API int ferris_paged_attention_simt(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                           const void* v_cache, int dtype, const int* block_tables, int max_blocks,
                                           const int* token_seq, const int* positions, int tokens, int nh, int nkv,
                                           int d, int page_size, int window, float scale, const float* slopes,
                                           void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) FERRIS_REFUSE("attention: %d heads over %d kv heads", nh, nkv);
    if (d <= 0 || d > 32 * MAX_PER_LANE) FERRIS_REFUSE("attention: head size %d not in 1..%d", d, 32 * MAX_PER_LANE);
    if (page_size <= 0 || max_blocks <= 0) FERRIS_REFUSE("attention: page_size=%d max_blocks=%d", page_size, max_blocks);
    if (nh > 65535) FERRIS_REFUSE("attention: %d heads are more than one launch takes", nh);
    dim3 grid(tokens, nh);
    const size_t smem = (size_t)ATT_WARPS * (d + 2) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(paged_attention_simt_kernel<float>, grid, dim3(ATT_THREADS), smem, s, (const float*)q, ldq, (float*)out, ldo, (const float*)k_cache, (const float*)v_cache, block_tables,
            max_blocks, token_seq, positions, nh, nkv, d, page_size, window, scale, slopes);
    else if (dtype == FERRIS_BF16)
        ferris_launch(paged_attention_simt_kernel<bf16>, grid, dim3(ATT_THREADS), smem, s, (const bf16*)q, ldq, (bf16*)out, ldo, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks,
            token_seq, positions, nh, nkv, d, page_size, window, scale, slopes);
    else
        FERRIS_REFUSE("attention: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}
