// bf16 matrix product on the 5th-generation tensor cores:  out[t, n] = sum_k x[t, k] * w[n, k]  (+ bias[n]).
//
// Both operands are K-major as the model folder and the activations store them, so nothing is
// transposed.  The WEIGHT rows are the M side of the MMA (128 per tile) and the TOKENS its N side
// (16 to 256 per tile): a decode step of a few tokens fills a whole 128-row MMA with weights, which is
// what streams from HBM, and a prefill step uses the same kernel with wide token tiles.
//
// One CTA per (weight tile, token tile, K split); 10 warps:
//   warp 0    TMA producer: 64-wide K slices of the weight tile(s) and the token tile into a ring of
//             shared-memory stages (128-byte swizzle), completion on mbarriers;
//   warp 1    allocates tensor memory, issues tcgen05.mma (one thread) from shared-memory descriptors
//             into fp32 accumulators in TMEM, frees each stage with tcgen05.commit;
//   warps 2-9 epilogue: tcgen05.ld of their lane quarter (lane = weight row), then bias / store /
//             fp32 residual accumulation / SwiGLU, or a partial for the K split.
// With a K split, the CTA that finishes last adds the partials in split order (a fixed order, so
// the result does not depend on timing) and runs the epilogue.
//
// SwiGLU mode keeps TWO accumulators (gate rows and up rows of the same outputs, two MMAs per K
// slice) so that silu(g) * u is formed in the epilogue and the [T, 2I] intermediate never exists.
//
// Formula of the product: crates/ferrisinfer-kernel/src/cpu/matmul.rs:46-118; bias:
// crates/ferrisinfer-runtime/src/reference.rs:1132-1191; SwiGLU: crates/ferrisinfer-runtime/src/reference.rs:346-360.
#include <stdlib.h>

#include "common.cuh"
#include "sm100.cuh"

namespace {

constexpr int BLOCK_N = 128;  // weight rows per tile (MMA M)
constexpr int BLOCK_K = 64;   // one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int THREADS = 320;  // TMA warp, MMA warp, eight epilogue warps
constexpr int MAX_STAGES = 8;

enum Mode { STORE_BF16 = 0, STORE_F32 = 1, ACCUM_F32 = 2, SWIGLU_BF16 = 3, QKV_ROPE_BF16 = 4, ARGMAX_F32 = 5 };

// Mode ARGMAX_F32 (the output head of a step whose rows all take the greatest logit): no logits are stored.  Every
// tile of 128 outputs leaves, per token, the sort key of its best (value, index) pair, its maximum and its sum of
// exp(value - maximum) (16 bytes: key high word, key low word, maximum, sum), and a small kernel merges the tiles'
// entries: the lowest index among equal maxima, probability 1 / sum exp(l - max), as the sampling kernel's greedy
// rows (crates/ferrisinfer-kernel/src/cpu/matmul.rs:190-274 is the reference's fused product + argmax).
// The key orders (value, index) pairs: greater value first, then lower index; a NaN sorts last.
__device__ __forceinline__ uint32_t argmax_key_hi(float v) {
    const uint32_t u = __float_as_uint(v);
    return v != v ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));
}

// Where the q/k/v product of a long step leaves its output (mode QKV_ROPE_BF16 of the token-major kernel): the
// columns are heads of d values, nh query heads, then nkv key heads, then nkv value heads.  Query and key heads are
// rotated by the token's position (pairs (i, i + d/2), whole-head rotation); queries go to the output rows, keys
// and values straight into the paged cache [pages][nkv][page_size][d] at the token's slot.
struct RopeEpilogue {
    const float2* angles;  // [T][d/2] (cos, sin) of position x frequency, fp32
    const int* slots;      // [T] cache slot of each token; null or < 0: keys and values are not stored
    bf16* k_cache;
    bf16* v_cache;
    int nh, nkv, d, page_size;
};

struct Params {
    void* out;
    const float* bias;
    float* scratch;     // [splits][accumulators][T][N] fp32 partials when splits > 1
    int* counters;      // one per (weight tile, token tile); zero between launches
    int T, N, K, ldo;
    int bt;             // tokens per tile
    int stages;
    int kblocks;        // ceil(K / 64)
    int splits;
    int up_row_offset;  // SwiGLU: row of the weight matrix where the up rows start
    int cluster;        // 1: the K splits of a tile form a cluster and add their partials through shared memory
    // RMSNorm fused into the token operand (steps of at most 16 tokens): the kernel reads the fp32 residual rows
    // norm_h [T, K] and builds x = bf16((h * rstd) * norm_w) in shared memory itself instead of loading x by TMA
    const float* norm_h;
    const float* norm_w;
    float norm_eps;
    // Merge of split-KV attention fused into the token operand (same limits): x[t, head * d + c] =
    // sum_s O_s[c] e^{m_s - M} / sum_s l_s e^{m_s - M} from the partial results of the splits,
    // merge_o [T, heads, splits, d] and merge_ml [T, heads, splits, 2] = (m, l); K = heads * d
    const float* merge_o;
    const float* merge_ml;
    int merge_splits, merge_heads, merge_d;
    float* out_prob;    // mode ARGMAX_F32: out is int32 [T] (the tokens), this fp32 [T], scratch the tiles' entries
    int* status;
};

__device__ __forceinline__ float silu_mul(float g, float u) { return u * (g * (1.0f / (1.0f + expf(-g)))); }

// a: the product (the gate's in SwiGLU mode), b: the up product, bias_v: bias[n] or 0.
template <int MODE>
__device__ __forceinline__ void write_out(const Params& p, int t, int n, float a, float b, float bias_v) {
    if (MODE == STORE_BF16) {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(a + bias_v);
    } else if (MODE == STORE_F32) {
        reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = a + bias_v;
    } else if (MODE == ACCUM_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)t * p.ldo + n;
        *o = *o + (a + bias_v);
    } else {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(silu_mul(a, b));
    }
}

// WIDE: the K split's cluster may have up to 16 CTAs (beyond the portable size) instead of 8.  A kernel of its own:
// the narrow kernel's sum of eight peers is sensitive to every change (the other eight reads merely predicated, or
// in a loop that it jumps over, cost a decode step of 24 to 64 rows 13 to 37 us).
template <int MODE, bool WIDE = false>
__global__ void __launch_bounds__(THREADS)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                        const Params p) {
    constexpr int ACCS = MODE == SWIGLU_BF16 ? 2 : 1;
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[MAX_STAGES], empty[MAX_STAGES], accum_full;
    __shared__ uint32_t tmem_base;
    __shared__ int is_last;
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BLOCK_N, t0 = blockIdx.y * p.bt, split = blockIdx.z;
    const int a_bytes = BLOCK_N * BLOCK_K * 2, b_bytes = p.bt * BLOCK_K * 2;
    const int stage_bytes = ACCS * a_bytes + b_bytes;
    const int per_split = (p.kblocks + p.splits - 1) / p.splits;
    const int kb0 = split * per_split, kb1 = min(kb0 + per_split, p.kblocks);
    const int n_kb = max(kb1 - kb0, 0);
    uint32_t tmem_cols = 32;
    while (tmem_cols < (uint32_t)(ACCS * p.bt)) tmem_cols <<= 1;
    const bool built = p.norm_h || p.merge_o;  // the kernel forms the token tiles itself

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_w);
        tma_prefetch_descriptor(&map_x);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], built ? 2 : 1);  // the weight tiles' TMA (+ the token tile built in the kernel)
            mbar_init(&empty[s], 1);
        }
        mbar_init(&accum_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base, tmem_cols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = tmem_base;
    // Everything above touched no global memory: it may overlap the tail of the kernel before this one.
    // The WEIGHTS do not depend on that kernel either: the producer requests the first ring of weight tiles
    // before it waits, so their trip from HBM overlaps the wait; the token tiles follow after it.
    pdl_launch_dependents();
    if (warp == 0 && lane == 0) {
        const int first = min(n_kb, p.stages);
        for (int i = 0; i < first; ++i) {
            uint8_t* st = smem + (size_t)i * stage_bytes;
            const int k = (kb0 + i) * BLOCK_K;
            mbar_expect_tx(&full[i], built ? ACCS * a_bytes : stage_bytes);
            tma_load_2d(st, &map_w, k, n0, &full[i]);
            if (ACCS == 2) tma_load_2d(st + a_bytes, &map_w, k, p.up_row_offset + n0, &full[i]);
        }
    }
    pdl_wait();
    FERRIS_TL_BEGIN();
    // marks of the timeline build: the first epilogue thread of CTA (0, 0, 0)
    [[maybe_unused]] const bool tl_mark = threadIdx.x == 64 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    FERRIS_TL_MARK(tl_mark, 9);  // this thread is past the wait

    if (p.norm_h && warp >= 2) {
        // RMSNorm of the step's rows, then the token tiles of all of this CTA's K slices, written where TMA
        // would have put them (rows of 128 bytes, 16-byte chunks swizzled).  ms = sum(x^2) / K;
        // r = 1 / sqrt(ms + eps); y = (x r) w  (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41).
        __shared__ float rstd_s[64];
        const int e = warp - 2;
        for (int t = e; t < p.bt; t += 8) {
            float ss = 0.0f;
            if (t < p.T) {
                const float4* row = reinterpret_cast<const float4*>(p.norm_h + (size_t)t * p.K);
                for (int i = lane; i < p.K / 4; i += 32) {
                    const float4 v = row[i];
                    ss = fmaf(v.x, v.x, ss);
                    ss = fmaf(v.y, v.y, ss);
                    ss = fmaf(v.z, v.z, ss);
                    ss = fmaf(v.w, v.w, ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[t] = 1.0f / sqrtf(ss / (float)p.K + p.norm_eps);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const int et = threadIdx.x - 64;  // 0..255
        const int per_kb = p.bt * 8;      // 16-byte chunks of one token tile
        for (int idx = et; idx < n_kb * per_kb; idx += 256) {
            const int i = idx / per_kb, t = (idx % per_kb) >> 3, c = idx & 7;
            const int k = (kb0 + i) * BLOCK_K + 8 * c;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (t < p.T && k < p.K) {  // K is a multiple of 8: a chunk is inside or outside as a whole
                const float4 h0 = *reinterpret_cast<const float4*>(p.norm_h + (size_t)t * p.K + k);
                const float4 h1 = *reinterpret_cast<const float4*>(p.norm_h + (size_t)t * p.K + k + 4);
                const float4 w0 = *reinterpret_cast<const float4*>(p.norm_w + k);
                const float4 w1 = *reinterpret_cast<const float4*>(p.norm_w + k + 4);
                const float r = rstd_s[t];
                packed.x = pack_bf16((h0.x * r) * w0.x, (h0.y * r) * w0.y);
                packed.y = pack_bf16((h0.z * r) * w0.z, (h0.w * r) * w0.w);
                packed.z = pack_bf16((h1.x * r) * w1.x, (h1.y * r) * w1.y);
                packed.w = pack_bf16((h1.z * r) * w1.z, (h1.w * r) * w1.w);
            }
            *reinterpret_cast<uint4*>(smem + (size_t)i * stage_bytes + ACCS * a_bytes + swizzle128(t, c)) = packed;
        }
        fence_proxy_async();  // the MMA reads these tiles through the async proxy
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64)
            for (int i = 0; i < n_kb; ++i) mbar_arrive(&full[i]);
    }

    if (p.merge_o && warp >= 2) {
        // The attention rows of the step from the partial results of the key ranges (the merge of the split-KV
        // attention kernel, same order of sums), written as the token tiles of this CTA's K slices.
        const int et = threadIdx.x - 64;  // 0..255
        const int S = p.merge_splits, d = p.merge_d;
        const int per_kb = p.bt * 8;  // 16-byte chunks of one token tile
        for (int idx = et; idx < n_kb * per_kb; idx += 256) {
            const int i = idx / per_kb, t = (idx % per_kb) >> 3, c = idx & 7;
            const int k = (kb0 + i) * BLOCK_K + 8 * c;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (t < p.T && k < p.K) {  // d is a multiple of 8: a chunk lies within one head
                const int head = k / d, col = k - head * d;
                const size_t base = ((size_t)t * p.merge_heads + head) * S;
                const float2* ml = reinterpret_cast<const float2*>(p.merge_ml) + base;
                float mm = -INFINITY;
                for (int sp = 0; sp < S; ++sp) mm = fmaxf(mm, ml[sp].x);
                float ll = 0.0f, o[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                for (int sp = 0; sp < S; ++sp) {
                    const float2 v = ml[sp];
                    const float f = v.x == -INFINITY ? 0.0f : expf(v.x - mm);
                    const float4* po = reinterpret_cast<const float4*>(p.merge_o + (base + sp) * d + col);
                    const float4 o0 = po[0], o1 = po[1];
                    ll += v.y * f;
                    o[0] += o0.x * f;
                    o[1] += o0.y * f;
                    o[2] += o0.z * f;
                    o[3] += o0.w * f;
                    o[4] += o1.x * f;
                    o[5] += o1.y * f;
                    o[6] += o1.z * f;
                    o[7] += o1.w * f;
                }
                packed.x = pack_bf16(o[0] / ll, o[1] / ll);
                packed.y = pack_bf16(o[2] / ll, o[3] / ll);
                packed.z = pack_bf16(o[4] / ll, o[5] / ll);
                packed.w = pack_bf16(o[6] / ll, o[7] / ll);
            }
            *reinterpret_cast<uint4*>(smem + (size_t)i * stage_bytes + ACCS * a_bytes + swizzle128(t, c)) = packed;
        }
        fence_proxy_async();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (threadIdx.x == 64)
            for (int i = 0; i < n_kb; ++i) mbar_arrive(&full[i]);
    }

    FERRIS_TL_MARK(tl_mark, 0);  // token tiles built (or nothing to build)
    if (warp == 0) {
        if (lane == 0) {
            const int first = min(n_kb, p.stages);
            for (int i = 0; i < first && !built; ++i)
                tma_load_2d(smem + (size_t)i * stage_bytes + ACCS * a_bytes, &map_x, (kb0 + i) * BLOCK_K, t0, &full[i]);
            for (int i = first; i < n_kb; ++i) {
                const int s = i % p.stages;
                if (!mbar_wait(&empty[s], ((i / p.stages) - 1) & 1, p.status, 10)) break;
                uint8_t* st = smem + (size_t)s * stage_bytes;
                const int k = (kb0 + i) * BLOCK_K;
                mbar_expect_tx(&full[s], stage_bytes);
                tma_load_2d(st, &map_w, k, n0, &full[s]);
                if (ACCS == 2) tma_load_2d(st + a_bytes, &map_w, k, p.up_row_offset + n0, &full[s]);
                tma_load_2d(st + ACCS * a_bytes, &map_x, k, t0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(BLOCK_N, p.bt);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % p.stages;
                ok = mbar_wait(&full[s], (i / p.stages) & 1, p.status, 11);
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
                const uint64_t a_desc = umma_desc_k_major_sw128(st);
                const uint64_t a2_desc = umma_desc_k_major_sw128(st + a_bytes);
                const uint64_t b_desc = umma_desc_k_major_sw128(st + ACCS * a_bytes);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);  // 32 bytes per K step, in 16-byte units
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    tcgen05_mma_bf16(tmem, a_desc + adv, b_desc + adv, idesc, acc);
                    if (ACCS == 2) tcgen05_mma_bf16(tmem + p.bt, a2_desc + adv, b_desc + adv, idesc, acc);
                }
                tcgen05_commit(&empty[s]);  // the stage is free once these MMAs have read it
            }
            tcgen05_commit(&accum_full);
        }
    } else {
        // epilogue: eight warps; warp e reads TMEM lane quarter (warp % 4) (lane = weight row) and every
        // second 16-column chunk (column = token)
        const int e = warp - 2;
        const int quarter = warp & 3, half = e >> 2;
        const int n = n0 + quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const bool have = n_kb > 0 && mbar_wait(&accum_full, 0, p.status, 12);
        tcgen05_fence_after();
        FERRIS_TL_MARK(tl_mark, 1);  // accumulator ready
        const bool n_ok = n < p.N;
        const float bias_v = (p.bias && n_ok) ? p.bias[n] : 0.0f;
        if constexpr (MODE == ARGMAX_F32) {
            // per token: best key, maximum and sum over this warp's 32 outputs, then over the tile's four lane quarters
            __shared__ float4 quarter_best[4][128];
            // Both warps of a lane quarter read every chunk of 16 tokens and take every second token of it.  Three
            // warp reductions a token, all on integers (redux.sync): the key's high word (the value), its low word
            // among the lanes that hold that value (the index), and the sum of exp(value - maximum) in fixed point
            // (24 fractional bits: 32 terms of at most 1 fit a word; the sum is good to 2^-24 of its largest term).
            for (int c0 = 0; c0 < p.bt && t0 + c0 < p.T; c0 += 16) {
                uint32_t ra[16];
                if (have) {
                    tmem_load_32x16(lane_addr + c0, ra);
                    tmem_load_wait();
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    if ((c & 1) != half || t0 + c0 + c >= p.T) continue;  // the same for the whole warp
                    const float x = (have && n_ok) ? __uint_as_float(ra[c]) : -INFINITY;
                    const uint32_t hi = n_ok ? argmax_key_hi(x) : 0u;
                    const uint32_t best_hi = __reduce_max_sync(0xffffffffu, hi);
                    const uint32_t best_lo = __reduce_max_sync(0xffffffffu, (n_ok && hi == best_hi) ? 0xFFFFFFFFu - (uint32_t)n : 0u);
                    // the maximum itself, back from its key (0: no lane holds a number)
                    const float m = best_hi == 0u ? -INFINITY
                                                  : __uint_as_float((best_hi & 0x80000000u) ? (best_hi & 0x7FFFFFFFu) : ~best_hi);
                    const float e = (x == x && m != -INFINITY) ? expf(x - m) : 0.0f;  // exp(-inf - m) = 0
                    const uint32_t fixed = __reduce_add_sync(0xffffffffu, (uint32_t)(e * 16777216.0f + 0.5f));
                    if (lane == 0)
                        quarter_best[quarter][c0 + c] =
                            make_float4(__uint_as_float(best_hi), __uint_as_float(best_lo), m, (float)fixed * (1.0f / 16777216.0f));
                }
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const int tl = threadIdx.x - 64;
            if (tl < p.bt && t0 + tl < p.T) {
                uint32_t bh = 0u, bl = 0u;
                float m = -INFINITY;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v = quarter_best[q][tl];
                    const uint32_t h = __float_as_uint(v.x), l = __float_as_uint(v.y);
                    if (h > bh || (h == bh && l > bl)) bh = h, bl = l;
                    m = fmaxf(m, v.z);
                }
                float sum = 0.0f;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v = quarter_best[q][tl];
                    sum += v.z == -INFINITY ? 0.0f : v.w * expf(v.z - m);
                }
                reinterpret_cast<float4*>(p.scratch)[(size_t)blockIdx.x * p.T + t0 + tl] =
                    make_float4(__uint_as_float(bh), __uint_as_float(bl), m, sum);
            }
        } else if (p.splits == 1) {
            if (have) {
                for (int c0 = half * 16; c0 < p.bt; c0 += 32) {
                    uint32_t ra[16], rb[16];
                    tmem_load_32x16(lane_addr + c0, ra);
                    if (ACCS == 2) tmem_load_32x16(lane_addr + p.bt + c0, rb);
                    float old[16];
                    if (MODE == ACCUM_F32) {
                        // the sixteen reads of the residual are in flight together
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = t0 + c0 + c;
                            old[c] = (n_ok && t < p.T) ? reinterpret_cast<const float*>(p.out)[(size_t)t * p.ldo + n] : 0.0f;
                        }
                    }
                    tmem_load_wait();
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int t = t0 + c0 + c;
                        if (!(n_ok && t < p.T)) continue;
                        const float a = __uint_as_float(ra[c]);
                        if (MODE == STORE_BF16)
                            reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(a + bias_v);
                        else if (MODE == STORE_F32)
                            reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = a + bias_v;
                        else if (MODE == ACCUM_F32)
                            reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = old[c] + (a + bias_v);
                        else
                            reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] =
                                __float2bfloat16_rn(silu_mul(a, __uint_as_float(rb[c])));
                    }
                }
            }
        } else if (p.cluster) {
            // partials of this split go to this CTA's shared memory, [accumulator][token][weight row]
            float* part = reinterpret_cast<float*>(smem + (size_t)p.stages * stage_bytes);
            for (int c0 = half * 16; c0 < p.bt; c0 += 32) {
                uint32_t ra[16], rb[16];
                if (have) {
                    tmem_load_32x16(lane_addr + c0, ra);
                    if (ACCS == 2) tmem_load_32x16(lane_addr + p.bt + c0, rb);
                    tmem_load_wait();
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    part[(c0 + c) * BLOCK_N + quarter * 32 + lane] = have ? __uint_as_float(ra[c]) : 0.0f;
                    if (ACCS == 2)
                        part[(p.bt + c0 + c) * BLOCK_N + quarter * 32 + lane] = have ? __uint_as_float(rb[c]) : 0.0f;
                }
            }
        } else {
            // partials of this split: scratch[((split * ACCS + a) * T + t) * N + n]
            for (int c0 = half * 16; c0 < p.bt; c0 += 32) {
                if (t0 + c0 >= p.T) break;
                uint32_t ra[16], rb[16];
                if (have) {
                    tmem_load_32x16(lane_addr + c0, ra);
                    if (ACCS == 2) tmem_load_32x16(lane_addr + p.bt + c0, rb);
                    tmem_load_wait();
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int t = t0 + c0 + c;
                    if (n_ok && t < p.T) {
                        p.scratch[((size_t)(split * ACCS) * p.T + t) * p.N + n] = have ? __uint_as_float(ra[c]) : 0.0f;
                        if (ACCS == 2)
                            p.scratch[((size_t)(split * ACCS + 1) * p.T + t) * p.N + n] = have ? __uint_as_float(rb[c]) : 0.0f;
                    }
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (threadIdx.x == 64) {
                const int tile = blockIdx.y * gridDim.x + blockIdx.x;
                const int old = atomicAdd(&p.counters[tile], 1);
                is_last = old == p.splits - 1;
                if (is_last) p.counters[tile] = 0;  // ready for the next launch
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (is_last) {
                __threadfence();
                // the last CTA adds the partials in split order; the two warps of a lane quarter take
                // tokens in turn, four at a time, with the reads of up to eight splits of each in flight
                const int t_end = min(t0 + p.bt, p.T);
                if (n_ok) {
                    for (int tb = t0 + 4 * half; tb < t_end; tb += 8) {
                        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f}, b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        for (int s0 = 0; s0 < p.splits; s0 += 8) {
                            float va[4][8], vb[4][8];
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const int sp = s0 + j, t = tb + q;
                                    const bool ok = sp < p.splits && t < t_end;
                                    va[q][j] = ok ? __ldcg(&p.scratch[((size_t)(sp * ACCS) * p.T + t) * p.N + n]) : 0.0f;
                                    if (ACCS == 2)
                                        vb[q][j] = ok ? __ldcg(&p.scratch[((size_t)(sp * ACCS + 1) * p.T + t) * p.N + n]) : 0.0f;
                                }
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    a[q] += va[q][j];
                                    if (ACCS == 2) b[q] += vb[q][j];
                                }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (tb + q < t_end) write_out<MODE>(p, tb + q, n, a[q], b[q], bias_v);
                    }
                }
            }
        }
    }
    if (p.cluster && p.splits > 1) {
        // every CTA of the cluster has its partial in shared memory: CTA r adds up the tokens r, r + splits, ...
        // of all of them (in split order, so the sum does not depend on timing) and writes those rows out
        FERRIS_TL_MARK(tl_mark, 2);  // partial in shared memory
        cluster_sync();
        FERRIS_TL_MARK(tl_mark, 3);  // all partials of the cluster in place
        const bool by_four = (p.ldo & 3) == 0 && (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        if (warp >= 2 && by_four) {
            // A warp takes a token (the tokens rank, rank + splits, ... of the tile, the eight warps in turn), a lane
            // four weight rows of it: a quarter of the requests to the peers' shared memory, 16-byte reads and writes of
            // the output rows.
            const int e = warp - 2, rank = (int)cluster_ctarank();
            const int n4 = n0 + lane * 4;
            const uint32_t part = smem_u32(smem + (size_t)p.stages * stage_bytes);
            float bias4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (p.bias && n4 < p.N) {
#pragma unroll
                for (int c = 0; c < 4; ++c) bias4[c] = p.bias[n4 + c];
            }
            for (int tl = rank + e * p.splits; tl < p.bt; tl += 8 * p.splits) {
                const int t = t0 + tl;
                if (t >= p.T) break;
                if (n4 >= p.N) continue;
                float4 old = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (MODE == ACCUM_F32) old = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.out) + (size_t)t * p.ldo + n4);
                const uint32_t addr = part + (uint32_t)((tl * BLOCK_N + lane * 4) * 4);
                float a[4] = {0.0f, 0.0f, 0.0f, 0.0f}, b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int s0 = 0; s0 < (WIDE ? 16 : 8); s0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp)
                        v[sp] = s0 + sp < p.splits ? ld_peer_shared_f32x4(addr, s0 + sp) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int sp = 0; sp < 8; ++sp) a[0] += v[sp].x, a[1] += v[sp].y, a[2] += v[sp].z, a[3] += v[sp].w;
                    if (ACCS == 2) {
#pragma unroll
                        for (int sp = 0; sp < 8; ++sp)
                            v[sp] = s0 + sp < p.splits ? ld_peer_shared_f32x4(addr + (uint32_t)(p.bt * BLOCK_N * 4), s0 + sp)
                                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                        for (int sp = 0; sp < 8; ++sp) b[0] += v[sp].x, b[1] += v[sp].y, b[2] += v[sp].z, b[3] += v[sp].w;
                    }
                }
                if (MODE == ACCUM_F32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)t * p.ldo + n4) =
                        make_float4(old.x + (a[0] + bias4[0]), old.y + (a[1] + bias4[1]), old.z + (a[2] + bias4[2]),
                                    old.w + (a[3] + bias4[3]));
                } else if (MODE == STORE_F32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)t * p.ldo + n4) =
                        make_float4(a[0] + bias4[0], a[1] + bias4[1], a[2] + bias4[2], a[3] + bias4[3]);
                } else {
                    float y[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) y[c] = MODE == SWIGLU_BF16 ? silu_mul(a[c], b[c]) : a[c] + bias4[c];
                    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (size_t)t * p.ldo + n4) =
                        make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
                }
            }
        } else if (warp >= 2) {
            const int quarter = warp & 3, half = (warp - 2) >> 2;
            const int n = n0 + quarter * 32 + lane;
            const float bias_v = (p.bias && n < p.N) ? p.bias[n] : 0.0f;
            const uint32_t part = smem_u32(smem + (size_t)p.stages * stage_bytes);
            const int rank = (int)cluster_ctarank();
            // A thread's tokens are rank + half * splits, then every 2 * splits further.  The old value that an
            // accumulating product adds to is requested before the peers' values, so that its trip to L2 overlaps
            // theirs (a decode step of 64 rows at the 0.5B sizes: 1.699 against 1.723 ms).  TOK tokens' reads are in
            // flight together; more than one gains nothing (two: 1.702 ms) or loses (four: 1.794 ms): the peers'
            // shared memory answers no faster when it is asked for more at once.
            constexpr int TOK = 1;
            const int stride = 2 * p.splits;
            const bool n_ok = n < p.N;
            for (int tl0 = rank + half * p.splits; tl0 < p.bt; tl0 += TOK * stride) {
                float a[TOK], b[TOK], old[TOK];
                bool ok[TOK];
#pragma unroll
                for (int q = 0; q < TOK; ++q) {
                    const int tl = tl0 + q * stride;
                    ok[q] = n_ok && tl < p.bt && t0 + tl < p.T;
                    a[q] = b[q] = old[q] = 0.0f;
                    if (MODE == ACCUM_F32 && ok[q]) old[q] = reinterpret_cast<const float*>(p.out)[(size_t)(t0 + tl) * p.ldo + n];
                }
#pragma unroll
                for (int s0 = 0; s0 < (WIDE ? 16 : 8); s0 += 8) {
                    float va[TOK][8], vb[TOK][8];
#pragma unroll
                    for (int q = 0; q < TOK; ++q) {
                        const uint32_t addr = part + (uint32_t)(((tl0 + q * stride) * BLOCK_N + quarter * 32 + lane) * 4);
#pragma unroll
                        for (int s = 0; s < 8; ++s) {
                            const bool live = ok[q] && s0 + s < p.splits;
                            va[q][s] = live ? ld_peer_shared_f32(addr, s0 + s) : 0.0f;
                            if (ACCS == 2) vb[q][s] = live ? ld_peer_shared_f32(addr + (uint32_t)(p.bt * BLOCK_N * 4), s0 + s) : 0.0f;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < TOK; ++q)
#pragma unroll
                        for (int s = 0; s < 8; ++s) {  // in split order: the sum does not depend on timing
                            a[q] += va[q][s];
                            if (ACCS == 2) b[q] += vb[q][s];
                        }
                }
#pragma unroll
                for (int q = 0; q < TOK; ++q) {
                    if (!ok[q]) continue;
                    const int t = t0 + tl0 + q * stride;
                    if (MODE == ACCUM_F32)
                        reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = old[q] + (a[q] + bias_v);
                    else
                        write_out<MODE>(p, t, n, a[q], b[q], bias_v);
                }
            }
        }
        FERRIS_TL_MARK(tl_mark, 4);  // rows summed and written
        cluster_sync();  // nobody leaves while a peer may still read its shared memory
        FERRIS_TL_MARK(tl_mark, 5);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem, tmem_cols);
    }
    FERRIS_TL_END(MODE == ARGMAX_F32 ? 21 : 10 + MODE + (p.norm_h ? 4 : 0) + (p.merge_o ? 8 : 0));
}

// The tiles' entries of mode ARGMAX_F32, [tiles][T] of (key high, key low, maximum, sum), merged per token: one CTA a
// token, its threads over the tiles.
constexpr int AM_THREADS = 256;
__global__ void __launch_bounds__(AM_THREADS)
    argmax_merge_kernel(const float4* part, int tiles, int T, int* __restrict__ out_token,
                        float* __restrict__ out_prob) {
    __shared__ uint32_t s_hi[AM_THREADS / 32], s_lo[AM_THREADS / 32];
    __shared__ float s_m[AM_THREADS / 32], s_sum[AM_THREADS / 32];
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t bh = 0u, bl = 0u;
    float m = -INFINITY, sum = 0.0f;
    for (int i0 = threadIdx.x; i0 < tiles; i0 += 4 * AM_THREADS) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // four loads in flight
            const int i = i0 + j * AM_THREADS;
            v[j] = i < tiles ? part[(size_t)i * T + t] : make_float4(0.0f, 0.0f, -INFINITY, 0.0f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t h = __float_as_uint(v[j].x), l = __float_as_uint(v[j].y);
            if (h > bh || (h == bh && l > bl)) bh = h, bl = l;
            if (v[j].z > m) {
                sum *= expf(m - v[j].z);  // exp(-inf) = 0 the first time
                m = v[j].z;
            }
            sum += v[j].z == -INFINITY ? 0.0f : v[j].w * expf(v[j].z - m);
        }
    }
    // warp, then CTA: the greatest key, the maximum, the sums brought to that maximum
    const uint32_t wh = __reduce_max_sync(0xffffffffu, bh);
    const uint32_t wl = __reduce_max_sync(0xffffffffu, bh == wh ? bl : 0u);
    const float wm = warp_max(m);
    const float ws = warp_sum(m == -INFINITY ? 0.0f : sum * expf(m - wm));
    if (lane == 0) s_hi[warp] = wh, s_lo[warp] = wl, s_m[warp] = wm, s_sum[warp] = ws;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t h = 0u, l = 0u;
        float mm = -INFINITY;
        for (int w = 0; w < AM_THREADS / 32; ++w) {
            if (s_hi[w] > h || (s_hi[w] == h && s_lo[w] > l)) h = s_hi[w], l = s_lo[w];
            mm = fmaxf(mm, s_m[w]);
        }
        float denom = 0.0f;
        for (int w = 0; w < AM_THREADS / 32; ++w) denom += s_m[w] == -INFINITY ? 0.0f : s_sum[w] * expf(s_m[w] - mm);
        out_token[t] = (int)(0xFFFFFFFFu - l);
        if (out_prob) out_prob[t] = 1.0f / denom;
    }
#ifdef FERRIS_TIMELINE
    __syncthreads();
#endif
    FERRIS_TL_END(27);
}

// =============================================================================================
// Long steps (prefill): a PERSISTENT kernel with the TOKENS on the M side of the MMA (128 per tile,
// lane = token) and the weight rows on its N side (256 per tile; 2 x 128 gate / up in SwiGLU mode).
// Each CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the accumulators are double-buffered
// in tensor memory, so the epilogue of one tile (tcgen05.ld, bias / SiLU / residual, 16-byte
// stores along the output row) runs while the MMA warp works on the next.
// =============================================================================================
constexpr int PT_BLOCK_M = 128;     // tokens per tile
constexpr int PT_STAGES = 4;
constexpr int PT_EPI_WARPS = 8;
constexpr int PT_THREADS = (2 + PT_EPI_WARPS) * 32;

struct PTParams {
    void* out;
    const float* bias;
    int T, N, K, ldo;
    int bn;             // weight rows per accumulator and tile: 256, or 128 in SwiGLU mode
    int kblocks;
    int m_tiles, n_tiles;
    int up_row_offset;
    int* status;
    RopeEpilogue rope;  // mode QKV_ROPE_BF16 only
};

// The epilogue of one q/k/v tile for one warp: its 32 tokens (lane = token t) and every second item of 64
// accumulator columns.  An item is a low and a high chunk of 32 columns of ONE head, d/2 apart, so that a thread
// holds both members of 32 rotation pairs: with d = 64 item w is head w of the tile, with d = 128 it is head
// w / 2, pairs i in [32 (w % 2), 32 (w % 2) + 32).  Bias, rotation and rounding happen once, in fp32, on the
// accumulator.
__device__ __forceinline__ void pt_epilogue_qkv_rope(const PTParams& p, uint32_t d0, int n0, int half, int t) {
    const RopeEpilogue& r = p.rope;
    const int d = r.d, hd = d >> 1;
    const int items = p.bn >> 6;
    const bool live = t < p.T;
    int slot = -1;
    if (live && r.slots) slot = __ldg(r.slots + t);
    const int page = slot >= 0 ? slot / r.page_size : 0, in_page = slot >= 0 ? slot % r.page_size : 0;
    for (int w = half; w < items; w += 2) {
        const int head_col = d == 64 ? w * 64 : (w >> 1) * 128;
        const int i0 = d == 64 ? 0 : (w & 1) * 32;
        uint32_t lo[32], hi[32];
        tmem_load_32x32(d0 + head_col + i0, lo);
        tmem_load_32x32(d0 + head_col + i0 + hd, hi);
        tmem_load_wait();
        const int n = n0 + head_col;  // the head's first output column; N is a multiple of d
        const int head = n / d;
        bf16* dst = nullptr;
        if (live && n < p.N) {
            if (head < r.nh)
                dst = reinterpret_cast<bf16*>(p.out) + (size_t)t * p.ldo + n;
            else if (slot >= 0 && head < r.nh + r.nkv)
                dst = r.k_cache + (((size_t)page * r.nkv + (head - r.nh)) * r.page_size + in_page) * d;
            else if (slot >= 0)
                dst = r.v_cache + (((size_t)page * r.nkv + (head - r.nh - r.nkv)) * r.page_size + in_page) * d;
        }
        if (dst) {
            const bool rotate = head < r.nh + r.nkv;
            const float* bl = p.bias ? p.bias + n + i0 : nullptr;
            const float4* ang = reinterpret_cast<const float4*>(r.angles + (size_t)t * hd + i0);
            uint32_t plo[16], phi[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                float l0 = __uint_as_float(lo[c]), l1 = __uint_as_float(lo[c + 1]);
                float h0 = __uint_as_float(hi[c]), h1 = __uint_as_float(hi[c + 1]);
                if (bl) {
                    l0 += __ldg(bl + c);
                    l1 += __ldg(bl + c + 1);
                    h0 += __ldg(bl + hd + c);
                    h1 += __ldg(bl + hd + c + 1);
                }
                if (rotate) {
                    const float4 cs = __ldg(ang + (c >> 1));  // (cos, sin) of pair i0 + c and of pair i0 + c + 1
                    const float a0 = l0 * cs.x - h0 * cs.y, b0 = h0 * cs.x + l0 * cs.y;
                    const float a1 = l1 * cs.z - h1 * cs.w, b1 = h1 * cs.z + l1 * cs.w;
                    l0 = a0, h0 = b0, l1 = a1, h1 = b1;
                }
                plo[c >> 1] = pack_bf16(l0, l1);
                phi[c >> 1] = pack_bf16(h0, h1);
            }
            uint4* olo = reinterpret_cast<uint4*>(dst + i0);
            uint4* ohi = reinterpret_cast<uint4*>(dst + i0 + hd);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                olo[v] = make_uint4(plo[4 * v], plo[4 * v + 1], plo[4 * v + 2], plo[4 * v + 3]);
                ohi[v] = make_uint4(phi[4 * v], phi[4 * v + 1], phi[4 * v + 2], phi[4 * v + 3]);
            }
        }
        __syncwarp();
    }
}

// The epilogue of one token-major tile for one warp: its 32 tokens (TMEM lanes, lane = token t) and every second
// 32-column chunk of the accumulator buffer at d0 (gate columns first, up columns p.bn further in SwiGLU mode).
template <int MODE>
__device__ __forceinline__ void pt_epilogue_tile(const PTParams& p, const CUtensorMap& map_out, uint32_t d0, int m0, int n0,
                                                 int quarter, int half, int lane, int t, uint8_t* out_stage) {
    constexpr int ACCS = MODE == SWIGLU_BF16 ? 2 : 1;
    const int cols = p.bn;  // output columns of this tile
    for (int c0 = half * 32; c0 < cols; c0 += 64) {
        uint32_t ra[32], rb[32];
        tmem_load_32x32(d0 + c0, ra);
        if (ACCS == 2) tmem_load_32x32(d0 + p.bn + c0, rb);
        tmem_load_wait();
        const int n = n0 + c0;
        if (MODE == STORE_F32 || MODE == ACCUM_F32) {
            // the warp's 32 x 32 block goes to shared memory (lane = row, 16-byte chunks swizzled as the
            // tensor map expects) and from there to global memory by one TMA store / add-reduction,
            // which also clips rows >= T and columns >= N
            if (n >= p.N || m0 + quarter * 32 >= p.T) continue;  // warp-uniform
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                float4 r;
                r.x = __uint_as_float(ra[4 * v]) + ((p.bias && n + 4 * v < p.N) ? __ldg(p.bias + n + 4 * v) : 0.0f);
                r.y = __uint_as_float(ra[4 * v + 1]) + ((p.bias && n + 4 * v + 1 < p.N) ? __ldg(p.bias + n + 4 * v + 1) : 0.0f);
                r.z = __uint_as_float(ra[4 * v + 2]) + ((p.bias && n + 4 * v + 2 < p.N) ? __ldg(p.bias + n + 4 * v + 2) : 0.0f);
                r.w = __uint_as_float(ra[4 * v + 3]) + ((p.bias && n + 4 * v + 3 < p.N) ? __ldg(p.bias + n + 4 * v + 3) : 0.0f);
                *reinterpret_cast<float4*>(out_stage + swizzle128(lane, v)) = r;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                if (MODE == ACCUM_F32)
                    tma_reduce_add_2d(&map_out, out_stage, n, m0 + quarter * 32);
                else
                    tma_store_2d(&map_out, out_stage, n, m0 + quarter * 32);
                tma_store_commit();
            }
            continue;
        }
        if (t >= p.T || n >= p.N) continue;
        const bool whole = n + 32 <= p.N;
        if (MODE == STORE_BF16 || MODE == SWIGLU_BF16) {
            bf16* o = reinterpret_cast<bf16*>(p.out) + (size_t)t * p.ldo + n;
            uint32_t packed[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                float v0, v1;
                if (MODE == SWIGLU_BF16) {
                    v0 = silu_mul(__uint_as_float(ra[c]), __uint_as_float(rb[c]));
                    v1 = silu_mul(__uint_as_float(ra[c + 1]), __uint_as_float(rb[c + 1]));
                } else {
                    v0 = __uint_as_float(ra[c]) + ((p.bias && n + c < p.N) ? __ldg(p.bias + n + c) : 0.0f);
                    v1 = __uint_as_float(ra[c + 1]) + ((p.bias && n + c + 1 < p.N) ? __ldg(p.bias + n + c + 1) : 0.0f);
                }
                packed[c >> 1] = pack_bf16(v0, v1);
            }
            if (whole) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    reinterpret_cast<uint4*>(o)[v] = make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c)
                    if (n + c < p.N)
                        o[c] = __ushort_as_bfloat16(
                            (unsigned short)((c & 1) ? (packed[c >> 1] >> 16) : (packed[c >> 1] & 0xffffu)));
            }
        }
    }
}

template <int MODE>
__global__ void __launch_bounds__(PT_THREADS)
    gemm_tokens_m_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_out, const PTParams p) {
    constexpr int ACCS = MODE == SWIGLU_BF16 ? 2 : 1;
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[PT_STAGES], empty[PT_STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_base;
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a_bytes = PT_BLOCK_M * BLOCK_K * 2, b_bytes = p.bn * BLOCK_K * 2;
    const int stage_bytes = a_bytes + ACCS * b_bytes;
    const int acc_cols = 256;  // columns of one accumulator buffer (ACCS * bn of them used)
    const int tiles = p.m_tiles * p.n_tiles;
    // fp32 outputs leave through shared memory and TMA: 4 KB (32 tokens x 32 floats, swizzled) per epilogue warp
    uint8_t* out_stage = smem + (size_t)PT_STAGES * stage_bytes + (size_t)(warp >= 2 ? warp - 2 : 0) * 4096;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_w);
        for (int s = 0; s < PT_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], PT_EPI_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base, 512);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = tmem_base;
    pdl_launch_dependents();
    pdl_wait();
    FERRIS_TL_BEGIN();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * PT_BLOCK_M, n0 = (tile / p.m_tiles) * p.bn;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % PT_STAGES;
                    if (it >= PT_STAGES && !mbar_wait(&empty[s], ((it / PT_STAGES) - 1) & 1, p.status, 20)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + (size_t)s * stage_bytes;
                    mbar_expect_tx(&full[s], stage_bytes);
                    tma_load_2d(st, &map_x, kb * BLOCK_K, m0, &full[s]);
                    tma_load_2d(st + a_bytes, &map_w, kb * BLOCK_K, n0, &full[s]);
                    if (ACCS == 2) tma_load_2d(st + a_bytes + b_bytes, &map_w, kb * BLOCK_K, p.up_row_offset + n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(PT_BLOCK_M, p.bn);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                // the epilogue must have drained this accumulator buffer (two tiles ago)
                if (local >= 2 && !mbar_wait(&tmem_empty[buf], ((local >> 1) - 1) & 1, p.status, 21)) break;
                tcgen05_fence_after();
                const uint32_t d0 = tmem + buf * acc_cols;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % PT_STAGES;
                    if (!mbar_wait(&full[s], (it / PT_STAGES) & 1, p.status, 22)) {
                        ok = false;
                        break;
                    }
                    tcgen05_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
                    const uint64_t a_desc = umma_desc_k_major_sw128(st);
                    const uint64_t b_desc = umma_desc_k_major_sw128(st + a_bytes);
                    const uint64_t b2_desc = umma_desc_k_major_sw128(st + a_bytes + b_bytes);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        tcgen05_mma_bf16(d0, a_desc + adv, b_desc + adv, idesc, acc);
                        if (ACCS == 2) tcgen05_mma_bf16(d0 + p.bn, a_desc + adv, b2_desc + adv, idesc, acc);
                    }
                    tcgen05_commit(&empty[s]);
                }
                if (ok) tcgen05_commit(&tmem_full[buf]);
            }
        }
    } else {
        // epilogue: warp e owns TMEM lane quarter (warp % 4) = 32 tokens, and one half of the columns
        const int e = warp - 2;
        const int quarter = warp & 3, half = e >> 2;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % p.m_tiles) * PT_BLOCK_M, n0 = (tile / p.m_tiles) * p.bn;
            const int t = m0 + quarter * 32 + lane;
            if (!mbar_wait(&tmem_full[buf], (local >> 1) & 1, p.status, 23)) break;
            tcgen05_fence_after();
            const uint32_t d0 = lane_addr + buf * acc_cols;
            if constexpr (MODE == QKV_ROPE_BF16)
                pt_epilogue_qkv_rope(p, d0, n0, half, t);
            else
                pt_epilogue_tile<MODE>(p, map_out, d0, m0, n0, quarter, half, lane, t, out_stage);
            // this warp has read its part of the buffer: the MMA warp may overwrite it
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    }
    if ((MODE == STORE_F32 || MODE == ACCUM_F32) && warp >= 2 && lane == 0) tma_store_wait_all();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem, 512);
    }
    FERRIS_TL_END(22 + MODE);
}

// =============================================================================================
// The same for CTA PAIRS (cta_group::2): a cluster of two CTAs on one TPC takes tiles of 256 tokens (128 per
// CTA) x 256 or 128 weight rows with ONE MMA over both.  Each CTA loads its own token rows and only HALF of the
// weight rows of the tile, so a pair moves two thirds of the bytes that two single CTAs move from L2 for the same
// work, and L2-to-SM traffic is what bounds the single-CTA kernel at these sizes.  The even CTA issues the MMAs;
// both CTAs' TMA loads count on its `full` barrier; tcgen05.commit arrives on `empty` / `tmem_full` of both;
// the epilogue warps of both arrive on its `tmem_empty`.  In SwiGLU mode CTA 0 holds the gate rows and CTA 1 the
// up rows of the tile: accumulator columns [0, 128) are gate, [128, 256) up, as in the single-CTA kernel.
// =============================================================================================
constexpr int PP_STAGES = 6;

template <int MODE>
__global__ void __launch_bounds__(PT_THREADS)
    gemm_tokens_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                            const __grid_constant__ CUtensorMap map_out, const PTParams p) {
    constexpr int ACCS = MODE == SWIGLU_BF16 ? 2 : 1;
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[PP_STAGES], empty[PP_STAGES], tmem_full[2], tmem_empty[2];
    __shared__ uint32_t tmem_base;
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: the leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int n_mma = ACCS * p.bn;            // columns of the pair's MMA and of one accumulator buffer
    const int half_rows = n_mma / 2;          // weight rows this CTA holds per K slice
    const int a_bytes = PT_BLOCK_M * BLOCK_K * 2, b_bytes = half_rows * BLOCK_K * 2;
    const int stage_bytes = a_bytes + b_bytes;
    const int tiles = p.m_tiles * p.n_tiles;  // m_tiles counts pairs of token tiles here
    uint8_t* out_stage = smem + (size_t)PP_STAGES * stage_bytes + (size_t)(warp >= 2 ? warp - 2 : 0) * 4096;

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_w);
        for (int s = 0; s < PP_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 2 * PT_EPI_WARPS);  // the epilogue warps of both CTAs (used in the leader only)
        }
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(&tmem_base, 512);
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers exist before anything arrives on them
    tcgen05_fence_after();
    const uint32_t tmem = tmem_base;
    pdl_launch_dependents();
    pdl_wait();
    FERRIS_TL_BEGIN();

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full = map_to_cta(smem_u32(&full[0]), 0);
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs) {
                const int m0 = (tile % p.m_tiles) * (2 * PT_BLOCK_M) + (int)rank * PT_BLOCK_M;
                const int n0 = (tile / p.m_tiles) * p.bn;
                // SwiGLU: the leader holds the gate rows, its peer the up rows; else each holds one half of the rows
                const int w_row = ACCS == 2 ? (rank == 0 ? n0 : p.up_row_offset + n0) : n0 + (int)rank * half_rows;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % PP_STAGES;
                    if (it >= PP_STAGES && !mbar_wait(&empty[s], ((it / PP_STAGES) - 1) & 1, p.status, 30)) {
                        ok = false;
                        break;
                    }
                    uint8_t* st = smem + (size_t)s * stage_bytes;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * stage_bytes);  // both CTAs' bytes
                    tma_load_2d_pair(st, &map_x, kb * BLOCK_K, m0, leader_full + 8u * s);
                    tma_load_2d_pair(st + a_bytes, &map_w, kb * BLOCK_K, w_row, leader_full + 8u * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_bf16(2 * PT_BLOCK_M, n_mma);
            int it = 0, local = 0;
            bool ok = true;
            long long wait_load = 0, wait_drain = 0, c0 = FERRIS_TL_CLOCK();  // timeline build: where the MMA thread waits
            [[maybe_unused]] const long long began = c0;
            for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
                const int buf = local & 1;
                c0 = FERRIS_TL_CLOCK();
                if (local >= 2 && !mbar_wait(&tmem_empty[buf], ((local >> 1) - 1) & 1, p.status, 31)) break;
                wait_drain += FERRIS_TL_CLOCK() - c0;
                tcgen05_fence_after();
                const uint32_t d0 = tmem + buf * n_mma;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int s = it % PP_STAGES;
                    c0 = FERRIS_TL_CLOCK();
                    if (!mbar_wait(&full[s], (it / PP_STAGES) & 1, p.status, 32)) {
                        ok = false;
                        break;
                    }
                    wait_load += FERRIS_TL_CLOCK() - c0;
                    tcgen05_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
                    const uint64_t a_desc = umma_desc_k_major_sw128(st);
                    const uint64_t b_desc = umma_desc_k_major_sw128(st + a_bytes);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                        tcgen05_mma_bf16_pair(d0, a_desc + adv, b_desc + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit_pair(&empty[s], 3);  // the stage is free in both CTAs
                }
                if (ok) tcgen05_commit_pair(&tmem_full[buf], 3);
            }
            FERRIS_TL_VALUE(pair == 0, 0, (unsigned long long)wait_load);
            FERRIS_TL_VALUE(pair == 0, 1, (unsigned long long)wait_drain);
            FERRIS_TL_VALUE(pair == 0, 2, (unsigned long long)(FERRIS_TL_CLOCK() - began));
            FERRIS_TL_VALUE(pair == 0, 3, (unsigned long long)local);
        }
    } else {
        const int e = warp - 2;
        const int quarter = warp & 3, half = e >> 2;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        int local = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++local) {
            const int buf = local & 1;
            const int m0 = (tile % p.m_tiles) * (2 * PT_BLOCK_M) + (int)rank * PT_BLOCK_M;
            const int n0 = (tile / p.m_tiles) * p.bn;
            const int t = m0 + quarter * 32 + lane;
            if (!mbar_wait(&tmem_full[buf], (local >> 1) & 1, p.status, 33)) break;
            tcgen05_fence_after();
            const uint32_t d0 = lane_addr + buf * n_mma;
            pt_epilogue_tile<MODE>(p, map_out, d0, m0, n0, quarter, half, lane, t, out_stage);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[buf]), 0));
        }
    }
    if ((MODE == STORE_F32 || MODE == ACCUM_F32) && warp >= 2 && lane == 0) tma_store_wait_all();
    tcgen05_fence_before();
    __syncthreads();
    FERRIS_TL_END(30 + MODE);
    cluster_sync();  // neither CTA frees tensor memory or leaves while the pair's MMAs or arrivals may still come
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem, 512);
    }
}

struct WeightMap {
    const void* base;
    uint64_t rows, cols, ld;
    CUtensorMap map;
};
constexpr int WEIGHT_MAPS = 1024;
WeightMap g_weight_maps[WEIGHT_MAPS];
int g_weight_map_count = 0;

int weight_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, CUtensorMap* out) {
    for (int i = 0; i < g_weight_map_count; ++i) {
        const WeightMap& m = g_weight_maps[i];
        if (m.base == base && m.rows == rows && m.cols == cols && m.ld == ld) {
            *out = m.map;
            return FERRIS_OK;
        }
    }
    CUtensorMap m;
    int rc = ferris_make_tensor_map_2d(&m, base, rows, cols, ld, BLOCK_N, BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    const int slot = g_weight_map_count < WEIGHT_MAPS ? g_weight_map_count++ : 0;
    g_weight_maps[slot] = {base, rows, cols, ld, m};
    *out = m;
    return FERRIS_OK;
}

// Weight maps of the token-major kernel: boxes of bn rows.
WeightMap g_pt_maps[WEIGHT_MAPS];
uint32_t g_pt_box[WEIGHT_MAPS];
int g_pt_map_count = 0;

int pt_weight_map(const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, CUtensorMap* out) {
    for (int i = 0; i < g_pt_map_count; ++i) {
        const WeightMap& m = g_pt_maps[i];
        if (m.base == base && m.rows == rows && m.cols == cols && m.ld == ld && g_pt_box[i] == box_rows) {
            *out = m.map;
            return FERRIS_OK;
        }
    }
    CUtensorMap m;
    int rc = ferris_make_tensor_map_2d(&m, base, rows, cols, ld, box_rows, BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    const int slot = g_pt_map_count < WEIGHT_MAPS ? g_pt_map_count++ : 0;
    g_pt_maps[slot] = {base, rows, cols, ld, m};
    g_pt_box[slot] = box_rows;
    *out = m;
    return FERRIS_OK;
}

int g_sms = 0;

// The device's SM count, asked once.
static int sm_count() {
    if (g_sms <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sms <= 0)
            g_sms = 148;
    }
    return g_sms;
}
int g_cluster = -1;

// The K splits reduce through a cluster's shared memory unless the environment says FERRIS_GEMM_CLUSTER=0
// (then: partials in global scratch, added by the CTA that finishes last).
bool ferris_gemm_cluster_enabled() {
    if (g_cluster < 0) {
        const char* v = getenv("FERRIS_GEMM_CLUSTER");
        g_cluster = (v && v[0] == '0') ? 0 : 1;
    }
    return g_cluster != 0;
}

// Which long-step products run on CTA pairs: FERRIS_GEMM_PAIR / ferris_set_gemm_pair = 0 none, 1 all, 2 (the
// default) the gate / up product only.  Measured inside the prefill step of 2,048 tokens, per launch: gate / up
// 38.4 us on pairs against 41.6 us, the products with one accumulator 20.5 us against 19.3 us (same number of
// CTAs either way, and the pair's barriers cost more than the halved weight traffic saves).  Prefill with the
// default against no pairs: 0.5B sizes 3.49-3.58 against 3.51-3.59 ms, 1.5B sizes 8.13-8.20 against 8.47-8.51 ms.
// The gate / up product alone, pairs against single CTAs: 256 tokens 13.8 / 14.2 us, 512 tokens 18.5 / 19.8 us,
// 1,024 tokens 25.1 / 27.0 us (0.5B sizes); 512 tokens 106 / 119 us, 2,048 tokens 377 / 434 us (7B sizes).
// Which of the two kernels a step of T >= 128 tokens runs: the token-major one (tokens on the MMA's M side,
// persistent CTAs, one CTA per tile of 128 x 128) or the weight-major one (K split over a cluster, so that a product
// with few tiles still uses every SM).  Both move the same bytes from L2, 32 KB per tile and K slice; what differs is
// over how many SMs.  Measured on B200: one SM takes in about 107 GB/s, all together about 6.3 TB/s, and the
// cluster's sum costs the weight-major kernel about 3 us.  Down projection of the 0.5B sizes (K = 4864, N = 896),
// token-major / weight-major: 256 tokens 27.2 / 15.2 us, 512 tokens 27.8 / 18.8 us, 768 tokens 28.7 / 24.5 us,
// 1,024 tokens 29.0 / 33.1 us; the estimate below reproduces these within 10 %.
// FERRIS_GEMM_LONG_MIN / ferris_set_gemm_long_min: a fixed number of tokens instead of the estimate.
int g_long_min = -1;
FERRIS_API int ferris_gemm_tcgen05_plan(int T, int N, int K, int accumulators, int* bt_out, int* splits_out,
                                        long long* scratch_floats, int* counters);
static bool token_major_pays(int mode, int T, int N, int K) {
    if (g_long_min < 0) {
        const char* v = getenv("FERRIS_GEMM_LONG_MIN");
        g_long_min = v ? atoi(v) : 0;
        if (g_long_min < 0) g_long_min = 0;
    }
    if (T < PT_BLOCK_M) return false;
    if (g_long_min > 0) return T >= g_long_min;
    const int sms = sm_count();
    const int accs = mode == SWIGLU_BF16 ? 2 : 1;
    const long long tiles = (long long)((T + PT_BLOCK_M - 1) / PT_BLOCK_M) * ((N + 127) / 128);
    if (tiles >= sms / 2) return true;
    int bt, splits, n_counters;
    long long scratch_floats;
    ferris_gemm_tcgen05_plan(T, N, K, accs, &bt, &splits, &scratch_floats, &n_counters);
    if (splits < 2 || !ferris_gemm_cluster_enabled()) return true;
    const double per_sm = 107e3, all_sms = 6.3e6, cluster_sum_us = 3.0;  // bytes per microsecond
    const double kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    const double bytes = (double)tiles * kblocks * (accs + 1) * 128 * BLOCK_K * 2;
    const double wm_ctas = (double)((N + BLOCK_N - 1) / BLOCK_N) * ((T + bt - 1) / bt) * splits;
    const double t_tm = bytes / (tiles * per_sm < all_sms ? tiles * per_sm : all_sms);
    const double t_wm = bytes / (wm_ctas * per_sm < all_sms ? wm_ctas * per_sm : all_sms) + cluster_sum_us;
    // the estimate is within 10 % of what was measured: the kernel with the cluster sum has to win by more
    return t_tm <= 1.15 * t_wm;
}

int g_pair = -1;  // 0: no product on pairs, 1: every long-step product, 2: the SwiGLU product only
bool ferris_gemm_pair_enabled(int mode, int T) {
    if (g_pair < 0) {
        const char* v = getenv("FERRIS_GEMM_PAIR");
        g_pair = (v && v[0] >= '0' && v[0] <= '2') ? v[0] - '0' : 2;
    }
    if (g_pair == 1) return true;
    // A pair's tile has 256 tokens: with an odd number of 128-token tiles the last pair is half empty, which costs
    // more than pairs save while the tiles are few (384 tokens at the 0.5B sizes: 18.3 us on pairs, 14.1 us without).
    const int m128 = (T + PT_BLOCK_M - 1) / PT_BLOCK_M;
    return g_pair == 2 && mode == SWIGLU_BF16 && (m128 % 2 == 0 || m128 >= 9);
}

template <int MODE>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const PTParams& p, int pairs,
                size_t smem, cudaStream_t s) {
    int rc = ferris_allow_dynamic_smem((const void*)gemm_tokens_pair_kernel<MODE>, smem);
    if (rc != FERRIS_OK) return rc;
    cudaError_t e = cudaSuccess;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(PT_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ferris_pdl_enabled() ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, gemm_tokens_pair_kernel<MODE>, mx, mw, mo, p);
    }
    if (e != cudaSuccess) {
        ferris_set_error("gemm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

// How many clusters of `size` CTAs of the short-step kernel (one CTA per SM) the GPU holds at once: the CTAs of a
// cluster share a GPC, so the answer is less than SMs / size where the size does not divide a GPC's SMs.
int g_max_split = -1;
static int max_split() {
    if (g_max_split < 0) {
        const char* v = getenv("FERRIS_GEMM_MAX_SPLIT");
        const int n = v ? atoi(v) : 16;
        g_max_split = (n >= 1 && n <= 16) ? n : 16;
    }
    return g_max_split;
}
int g_active_clusters[17] = {};
int active_clusters(int size) {
    if (size < 1 || size > 16) return 0;
    if (size == 1) return g_sms;
    // no answer: perfect packing is assumed up to the portable size, and no cluster at all beyond it
    const int unknown = size > 8 ? 0 : g_sms / size;
    if (g_active_clusters[size] != 0) return g_active_clusters[size] > 0 ? g_active_clusters[size] : unknown;
    g_active_clusters[size] = -1;
    auto kernel = gemm_tcgen05_kernel<ACCUM_F32, true>;
    const int smem = 200 * 1024;
    if (ferris_allow_dynamic_smem((const void*)kernel, smem) != FERRIS_OK) {  // only ever raises the allowance
        cudaGetLastError();
        return unknown;
    }
    if (size > 8 && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return unknown;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, size);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = size;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        return unknown;
    }
    g_active_clusters[size] = clusters;
    return clusters;
}

template <int MODE>
int launch_pt(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const PTParams& p, int ctas,
              size_t smem, cudaStream_t s) {
    int rc = ferris_allow_dynamic_smem((const void*)gemm_tokens_m_kernel<MODE>, smem);
    if (rc != FERRIS_OK) return rc;
    cudaError_t e = ferris_launch(gemm_tokens_m_kernel<MODE>, dim3(ctas), dim3(PT_THREADS), smem, s, mx, mw, mo, p);
    if (e != cudaSuccess) {
        ferris_set_error("gemm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

template <int MODE>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, dim3 grid, size_t smem, unsigned cluster_z,
           cudaStream_t s) {
    int rc = ferris_allow_dynamic_smem((const void*)gemm_tcgen05_kernel<MODE>, smem);
    if (rc != FERRIS_OK) return rc;
    cudaError_t e = cudaSuccess;
    if (cluster_z > 8) {
        // beyond the portable size: the kernel that sums sixteen peers (one accumulator only), allowed once
        if constexpr (MODE == STORE_BF16 || MODE == STORE_F32 || MODE == ACCUM_F32) {
            rc = ferris_allow_dynamic_smem((const void*)gemm_tcgen05_kernel<MODE, true>, smem);
            if (rc != FERRIS_OK) return rc;
            static bool allowed = false;
            if (!allowed) {
                if (cudaFuncSetAttribute(gemm_tcgen05_kernel<MODE, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) !=
                    cudaSuccess) {
                    cudaGetLastError();
                    FERRIS_REFUSE("gemm: clusters of %u CTAs are not allowed here", cluster_z);
                }
                allowed = true;
            }
            e = ferris_launch_cluster(gemm_tcgen05_kernel<MODE, true>, grid, dim3(THREADS), smem, s, cluster_z, mw, mx, p);
        } else {
            FERRIS_REFUSE("gemm: a K split of %u in mode %d", cluster_z, MODE);
        }
    } else if (cluster_z > 1)
        e = ferris_launch_cluster(gemm_tcgen05_kernel<MODE>, grid, dim3(THREADS), smem, s, cluster_z, mw, mx, p);
    else
        e = ferris_launch(gemm_tcgen05_kernel<MODE>, grid, dim3(THREADS), smem, s, mw, mx, p);
    if (e != cudaSuccess) {
        ferris_set_error("gemm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// 1 if the K splits of the short-step kernel add up through a cluster's shared memory (then no product needs the
// scratch and counters that ferris_gemm_tcgen05_plan speaks of), 0 if through global scratch.
FERRIS_API int ferris_gemm_uses_clusters() { return ferris_gemm_cluster_enabled() ? 1 : 0; }

// From how many tokens on a step runs the token-major kernel (at least 128; 0 selects the default).
FERRIS_API int ferris_set_gemm_long_min(int tokens) {
    g_long_min = tokens > 0 ? tokens : -1;
    return FERRIS_OK;
}

// Long steps on CTA pairs (cta_group::2) instead of single CTAs: 0 none, 1 every product, 2 the gate / up product
// only (the default); any other value selects the default.
FERRIS_API int ferris_set_gemm_pair(int on) {
    g_pair = (on >= 0 && on <= 2) ? on : 2;
    return FERRIS_OK;
}

// How the launcher would cut a product: token tile, K splits, and the fp32 scratch / counters it needs.
// accumulators: 2 for SwiGLU, else 1.
FERRIS_API int ferris_gemm_tcgen05_plan(int T, int N, int K, int accumulators, int* bt_out, int* splits_out,
                                        long long* scratch_floats, int* counters) {
    sm_count();
    // Steps of up to 128 tokens are one tile; longer ones start from the widest tile and narrow it (down to 64)
    // while the SMs would lack CTAs even with the deepest K split.
    const int n_tiles = (N + BLOCK_N - 1) / BLOCK_N;
    const int kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    // a cluster has at most 16 CTAs (8 is the portable size; active_clusters tells whether more are to be had)
    const int widest = (ferris_gemm_cluster_enabled() && accumulators != 2) ? max_split() : 8;
    const int most = kblocks >= 4 ? (kblocks / 2 < widest ? kblocks / 2 : widest) : 1;
    int bt;
    if (T <= 128) {
        // One token tile: a tcgen05.mma costs about the same ~100 cycles for any width up to 128 (measured), so a
        // narrower tile would only multiply the instructions and stream the weights once per tile.
        bt = (T + 15) / 16 * 16;
    } else {
        bt = 16;
        while (bt < T && bt < 256) bt <<= 1;
        while (bt > 64 && n_tiles * ((T + bt - 1) / bt) * (bt <= 128 ? most : 1) < g_sms) bt >>= 1;
    }
    const int t_tiles = (T + bt - 1) / bt;
    // K split: where tiles are fewer than SMs; the CTAs of a tile form a cluster and add their partials
    // through distributed shared memory
    int splits = 1;
    const int tiles = n_tiles * t_tiles;
    if (tiles < g_sms && most > 1 && bt <= 128) {
        splits = g_sms / tiles;  // rounded down: a few CTAs more than SMs would cost a second round
        if (splits > most) splits = most;
        if (splits < 1) splits = 1;
        // the clusters of all tiles must be resident at once (a cluster that waits for SMs of one GPC costs a second
        // round): fewer, longer splits where the cluster size packs badly into the GPCs
        while (splits > 1 && ferris_gemm_cluster_enabled() && tiles > active_clusters(splits)) --splits;
        // no split may be empty
        const int per = (kblocks + splits - 1) / splits;
        splits = (kblocks + per - 1) / per;
    }
    *bt_out = bt;
    *splits_out = splits;
    const bool cluster = ferris_gemm_cluster_enabled();
    *scratch_floats = (splits > 1 && !cluster) ? (long long)splits * accumulators * T * N : 0;
    *counters = (splits > 1 && !cluster) ? tiles : 0;
    return FERRIS_OK;
}

// Stages of the weight / token ring of the short-step kernel: what shared memory holds beside the K-split partials,
// at most MAX_STAGES, and no more than a CTA has K slices.
static int ring_stages(int accs, int bt, bool cluster, int per_split) {
    const int stage_bytes = accs * BLOCK_N * BLOCK_K * 2 + bt * BLOCK_K * 2;
    const int part_bytes = cluster ? accs * bt * BLOCK_N * 4 : 0;
    int stages = (227 * 1024 - 2048 - part_bytes) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > per_split) stages = per_split;
    return stages < 1 ? 1 : stages;
}

// Whether the short-step kernel can form its token operand itself (fused RMSNorm or merge) for this product: at most
// 16 tokens (beyond that every CTA repeating the norm of all rows costs more than a norm kernel saves: measured at
// 32 and 64), a K split that sums through the cluster (or none), and all K slices of a CTA resident at once.
FERRIS_API int ferris_gemm_tcgen05_builds_tokens(int T, int N, int K, int accumulators) {
    if (T <= 0 || T > 16 || (K & 7)) return 0;
    int bt, splits, n_counters;
    long long scratch_floats;
    ferris_gemm_tcgen05_plan(T, N, K, accumulators, &bt, &splits, &scratch_floats, &n_counters);
    const bool cluster = splits > 1 && ferris_gemm_cluster_enabled();
    if (bt > 16 || (splits > 1 && !cluster)) return 0;
    const int per_split = ((K + BLOCK_K - 1) / BLOCK_K + splits - 1) / splits;
    return per_split <= ring_stages(accumulators, bt, cluster, per_split) ? 1 : 0;
}

// x: bf16 [T, K] rows ldx apart; w: bf16 [rows_w, K] rows ldw apart (rows_w = N, or for SwiGLU at
// least up_row_offset + N); out: [T, N] rows ldo apart in the mode's type.
// mode: 0 bf16 = acc + bias; 1 fp32 = acc + bias; 2 fp32 += acc + bias; 3 bf16 = silu(gate) * up.
// scratch / counters: as ferris_gemm_tcgen05_plan says (counters must be zero; they are left zero).
// A token operand that the kernel forms itself instead of loading x: an RMSNorm of fp32 rows, or the merge of the
// partial results of split-KV attention.
struct TokenSource {
    const float* norm_h = nullptr;
    const float* norm_w = nullptr;
    float norm_eps = 0.0f;
    const float* merge_o = nullptr;
    const float* merge_ml = nullptr;
    int merge_splits = 0, merge_heads = 0, merge_d = 0;
};

static int gemm_tcgen05_impl(const void* x, const void* w, const float* bias, void* out, int mode, int T, int N, int K,
                             int ldx, int ldw, int ldo, int rows_w, int up_row_offset, float* scratch, int* counters,
                             void* stream, const TokenSource& src);

FERRIS_API int ferris_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int mode, int T, int N,
                                   int K, int ldx, int ldw, int ldo, int rows_w, int up_row_offset, float* scratch,
                                   int* counters, void* stream) {
    return gemm_tcgen05_impl(x, w, bias, out, mode, T, N, K, ldx, ldw, ldo, rows_w, up_row_offset, scratch, counters,
                             stream, TokenSource());
}

// The same product with RMSNorm fused in front: x = bf16((h * rstd(h)) * norm_w) is formed inside the kernel from the
// fp32 rows h [T, K] (contiguous).  For steps of at most 16 tokens whose K split leaves each CTA no more slices of
// 64 than its shared memory has stages (ferris_gemm_tcgen05_builds_tokens tells); anything else is refused.
FERRIS_API int ferris_norm_gemm_tcgen05(const float* h, const float* norm_w, float norm_eps, const void* w,
                                        const float* bias, void* out, int mode, int T, int N, int K, int ldw, int ldo,
                                        int rows_w, int up_row_offset, void* stream) {
    if (!h || !norm_w) FERRIS_REFUSE("norm + gemm: no rows or no norm weight");
    if (T > 16) FERRIS_REFUSE("norm + gemm: %d tokens (at most 16)", T);
    if (((uintptr_t)h & 15) || ((uintptr_t)norm_w & 15)) FERRIS_REFUSE("norm + gemm: operands must be 16-byte aligned");
    TokenSource src;
    src.norm_h = h;
    src.norm_w = norm_w;
    src.norm_eps = norm_eps;
    return gemm_tcgen05_impl(w, w, bias, out, mode, T, N, K, K, ldw, ldo, rows_w, up_row_offset, nullptr, nullptr, stream,
                             src);
}

// The same product with the merge of split-KV attention fused in front: the token operand x [T, heads * d] is formed
// inside the kernel from the partial results that ferris_decode_attention* leaves when it is told not to merge
// (scratch: fp32 [T, heads, splits, d] followed by [T, heads, splits, 2]).  Same limits as the fused norm.
FERRIS_API int ferris_merge_gemm_tcgen05(const float* scratch_parts, int heads, int d, int attn_splits, const void* w,
                                         const float* bias, void* out, int mode, int T, int N, int ldw, int ldo,
                                         int rows_w, void* stream) {
    if (!scratch_parts) FERRIS_REFUSE("merge + gemm: no partial results");
    if (T > 16) FERRIS_REFUSE("merge + gemm: %d tokens (at most 16)", T);
    if (heads <= 0 || (d != 64 && d != 128) || attn_splits < 1)
        FERRIS_REFUSE("merge + gemm: %d heads of %d over %d key ranges", heads, d, attn_splits);
    if ((uintptr_t)scratch_parts & 15) FERRIS_REFUSE("merge + gemm: operands must be 16-byte aligned");
    if (mode == SWIGLU_BF16) FERRIS_REFUSE("merge + gemm: no SwiGLU mode");
    TokenSource src;
    src.merge_o = scratch_parts;
    src.merge_ml = scratch_parts + (size_t)T * heads * attn_splits * d;
    src.merge_splits = attn_splits;
    src.merge_heads = heads;
    src.merge_d = d;
    const int K = heads * d;
    return gemm_tcgen05_impl(w, w, bias, out, mode, T, N, K, K, ldw, ldo, rows_w, 0, nullptr, nullptr, stream, src);
}

// The persistent token-major kernel for a long step (T >= 128 tokens; output rows aligned for 16-byte stores).
static int run_tokens_m(const void* x, const void* w, const float* bias, void* out, int mode, int T, int N, int K,
                        int ldx, int ldw, int ldo, int rows_w, int up_row_offset, const RopeEpilogue* rope,
                        cudaStream_t s) {
    const int accs = mode == SWIGLU_BF16 ? 2 : 1;
    const int elt = (mode == STORE_F32 || mode == ACCUM_F32) ? 4 : 2;
    sm_count();
    PTParams q;
    q.out = out;
    q.bias = bias;
    q.T = T;
    q.N = N;
    q.K = K;
    q.ldo = ldo;
    q.m_tiles = (T + PT_BLOCK_M - 1) / PT_BLOCK_M;
    // Weight rows per tile.  SwiGLU: 128 + 128.  Otherwise the width among 128 .. 256 that costs least: a CTA takes in (128 + bn) rows per K
    // slice, and the CTAs go through ceil(tiles / SMs) rounds; 192 or 224 rows often fit in one round what 128 rows
    // need two for (2,048 tokens x 1,536 outputs: 192 tiles of 128 in two rounds, 128 tiles of 192 in one).
    if (accs == 2) {
        q.bn = 128;
    } else {
        // the q/k/v mode takes whole heads (and pairs of 32-column chunks): steps of 64 or 128 rows
        const int step = rope ? (rope->d == 64 ? 64 : 128) : 32;
        long long best = -1;
        q.bn = 128;
        for (int bn = 256; bn >= 128; bn -= step) {
            const long long tiles = (long long)q.m_tiles * ((N + bn - 1) / bn);
            const long long cost = ((tiles + g_sms - 1) / g_sms) * (PT_BLOCK_M + bn);
            if (best < 0 || cost < best) {
                best = cost;
                q.bn = bn;
            }
        }
    }
    q.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    q.n_tiles = (N + q.bn - 1) / q.bn;
    q.up_row_offset = up_row_offset;
    q.status = ferris_status_ptr();
    q.rope = rope ? *rope : RopeEpilogue{};
    CUtensorMap mx, mw;
    int rc = ferris_make_tensor_map_2d(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, PT_BLOCK_M, BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    rc = pt_weight_map(w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw, (uint32_t)q.bn, &mw);
    if (rc != FERRIS_OK) return rc;
    CUtensorMap mo = mx;  // unused by the bf16 modes
    if (elt == 4) {
        rc = ferris_make_tensor_map_2d_f32(&mo, out, (uint64_t)T, (uint64_t)N, (uint64_t)ldo, 32);
        if (rc != FERRIS_OK) return rc;
    }
    const int stage_bytes = PT_BLOCK_M * BLOCK_K * 2 + accs * q.bn * BLOCK_K * 2;
    const size_t smem = (size_t)PT_STAGES * stage_bytes + (size_t)PT_EPI_WARPS * 4096 + 1024;
    int ctas = q.m_tiles * q.n_tiles;
    if (ctas > g_sms) ctas = g_sms;
    switch (mode) {
        case STORE_BF16: return launch_pt<STORE_BF16>(mx, mw, mo, q, ctas, smem, s);
        case STORE_F32: return launch_pt<STORE_F32>(mx, mw, mo, q, ctas, smem, s);
        case ACCUM_F32: return launch_pt<ACCUM_F32>(mx, mw, mo, q, ctas, smem, s);
        case SWIGLU_BF16: return launch_pt<SWIGLU_BF16>(mx, mw, mo, q, ctas, smem, s);
        default: return launch_pt<QKV_ROPE_BF16>(mx, mw, mo, q, ctas, smem, s);
    }
}

static int gemm_tcgen05_impl(const void* x, const void* w, const float* bias, void* out, int mode, int T, int N, int K,
                             int ldx, int ldw, int ldo, int rows_w, int up_row_offset, float* scratch, int* counters,
                             void* stream, const TokenSource& src) {
    const bool built = src.norm_h || src.merge_o;
    if (T <= 0 || N <= 0) return FERRIS_OK;
    if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K)
        FERRIS_REFUSE("tensor-core gemm: K=%d and row strides %d, %d must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) FERRIS_REFUSE("tensor-core gemm: operands must be 16-byte aligned");
    if (mode < 0 || mode > 3) FERRIS_REFUSE("tensor-core gemm: unknown mode %d", mode);
    if (mode == SWIGLU_BF16 && (bias || up_row_offset + N > rows_w)) FERRIS_REFUSE("tensor-core gemm: bad SwiGLU operands");
    if (mode != SWIGLU_BF16 && N > rows_w) FERRIS_REFUSE("tensor-core gemm: %d outputs from %d weight rows", N, rows_w);
    if (ldo < N) FERRIS_REFUSE("tensor-core gemm: output row stride %d < %d", ldo, N);
    const int accs = mode == SWIGLU_BF16 ? 2 : 1;
    int bt, splits, n_counters;
    long long scratch_floats;
    ferris_gemm_tcgen05_plan(T, N, K, accs, &bt, &splits, &scratch_floats, &n_counters);
    const bool cluster = splits > 1 && ferris_gemm_cluster_enabled();
    if (splits > 1 && !cluster && (!scratch || !counters))
        FERRIS_REFUSE("tensor-core gemm: a K split needs scratch and counters");

    cudaStream_t s = (cudaStream_t)stream;
    // long steps: the persistent token-major kernel (its 16-byte stores need aligned output rows)
    const int elt = (mode == STORE_BF16 || mode == SWIGLU_BF16) ? 2 : 4;
    const bool long_step = !built && token_major_pays(mode, T, N, K) && ((size_t)ldo * elt) % 16 == 0 && ((uintptr_t)out & 15) == 0;
    if (long_step && T > PT_BLOCK_M && ferris_gemm_pair_enabled(mode, T)) {
        // CTA pairs: tiles of 256 tokens x 256 weight rows (128 + 128 in SwiGLU mode), or x 128 where the
        // wider tile would leave pairs of SMs without work
        PTParams q;
        q.out = out;
        q.bias = bias;
        q.T = T;
        q.N = N;
        q.K = K;
        q.ldo = ldo;
        q.m_tiles = (T + 2 * PT_BLOCK_M - 1) / (2 * PT_BLOCK_M);
        const int pairs_all = g_sms / 2;
        q.bn = (accs == 2 || q.m_tiles * ((N + 255) / 256) < pairs_all) ? 128 : 256;
        q.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
        q.n_tiles = (N + q.bn - 1) / q.bn;
        q.up_row_offset = up_row_offset;
        q.status = ferris_status_ptr();
        const int half_rows = accs * q.bn / 2;
        CUtensorMap mx, mw;
        int rc = ferris_make_tensor_map_2d(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, PT_BLOCK_M, BLOCK_K);
        if (rc != FERRIS_OK) return rc;
        rc = pt_weight_map(w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw, (uint32_t)half_rows, &mw);
        if (rc != FERRIS_OK) return rc;
        CUtensorMap mo = mx;  // unused by the bf16 modes
        if (elt == 4) {
            rc = ferris_make_tensor_map_2d_f32(&mo, out, (uint64_t)T, (uint64_t)N, (uint64_t)ldo, 32);
            if (rc != FERRIS_OK) return rc;
        }
        const int stage_bytes = PT_BLOCK_M * BLOCK_K * 2 + half_rows * BLOCK_K * 2;
        const size_t smem = (size_t)PP_STAGES * stage_bytes + (size_t)PT_EPI_WARPS * 4096 + 1024;
        int pairs = q.m_tiles * q.n_tiles;
        if (pairs > pairs_all) pairs = pairs_all;
        switch (mode) {
            case STORE_BF16: return launch_pair<STORE_BF16>(mx, mw, mo, q, pairs, smem, s);
            case STORE_F32: return launch_pair<STORE_F32>(mx, mw, mo, q, pairs, smem, s);
            case ACCUM_F32: return launch_pair<ACCUM_F32>(mx, mw, mo, q, pairs, smem, s);
            default: return launch_pair<SWIGLU_BF16>(mx, mw, mo, q, pairs, smem, s);
        }
    }
    if (long_step)
        return run_tokens_m(x, w, bias, out, mode, T, N, K, ldx, ldw, ldo, rows_w, up_row_offset, nullptr, s);

    CUtensorMap mw, mx;
    int rc = weight_map(w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw, &mw);
    if (rc != FERRIS_OK) return rc;
    if (built) {
        mx = mw;  // unused: the kernel builds the token tiles itself
    } else {
        rc = ferris_make_tensor_map_2d(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bt, BLOCK_K);
        if (rc != FERRIS_OK) return rc;
    }

    Params p;
    p.out = out;
    p.bias = bias;
    p.scratch = scratch;
    p.counters = counters;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.bt = bt;
    p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    p.splits = splits;
    p.up_row_offset = up_row_offset;
    p.cluster = cluster ? 1 : 0;
    p.norm_h = src.norm_h;
    p.norm_w = src.norm_w;
    p.norm_eps = src.norm_eps;
    p.merge_o = src.merge_o;
    p.merge_ml = src.merge_ml;
    p.merge_splits = src.merge_splits;
    p.merge_heads = src.merge_heads;
    p.merge_d = src.merge_d;
    p.status = ferris_status_ptr();
    const int stage_bytes = accs * BLOCK_N * BLOCK_K * 2 + bt * BLOCK_K * 2;
    const int part_bytes = cluster ? accs * bt * BLOCK_N * 4 : 0;
    const int per_split = (p.kblocks + splits - 1) / splits;
    int stages = ring_stages(accs, bt, cluster, per_split);
    // Many tiles and no K split (the output head over the vocabulary): shallower rings, so that two CTAs share an
    // SM and one streams weights while the other's epilogue and set-up run.
    const long long tiles_all = (long long)((N + BLOCK_N - 1) / BLOCK_N) * ((T + bt - 1) / bt);
    if (splits == 1 && !built && tiles_all >= 4LL * g_sms) {
        const int fit = (227 * 1024 / 2 - 3072) / stage_bytes;
        if (fit >= 4 && stages > fit) stages = fit;
    }
    p.stages = stages;
    if (built && (bt > 16 || per_split > stages || (splits > 1 && !cluster)))
        FERRIS_REFUSE("norm / merge + gemm: this shape (token tile %d, %d K slices per CTA, %d stages) is not taken", bt, per_split,
                      stages);
    const size_t smem = (size_t)stages * stage_bytes + part_bytes + 1024;
    dim3 grid((N + BLOCK_N - 1) / BLOCK_N, (T + bt - 1) / bt, splits);
    if (grid.y > 65535) FERRIS_REFUSE("tensor-core gemm: %d rows are more than one launch takes", T);
    const unsigned cz = cluster ? (unsigned)splits : 1u;
    switch (mode) {
        case STORE_BF16: return launch<STORE_BF16>(mw, mx, p, grid, smem, cz, s);
        case STORE_F32: return launch<STORE_F32>(mw, mx, p, grid, smem, cz, s);
        case ACCUM_F32: return launch<ACCUM_F32>(mw, mx, p, grid, smem, cz, s);
        default: return launch<SWIGLU_BF16>(mw, mx, p, grid, smem, cz, s);
    }
}

// Floats of scratch that ferris_gemm_argmax_tcgen05 needs: one entry of 4 per tile of 128 outputs and token.
FERRIS_API long long ferris_gemm_argmax_scratch_floats(int T, int N) {
    return (long long)((N + BLOCK_N - 1) / BLOCK_N) * T * 4;
}

// The output head of rows that all take their greatest logit: out_token[t] = the lowest index among the greatest of
// sum_k x[t, k] w[n, k], n < N; out_prob[t] = 1 / sum_n exp(l[n] - max) (may be null).  No logits are stored.
// At most 128 rows; scratch: ferris_gemm_argmax_scratch_floats floats, 16-byte aligned.
FERRIS_API int ferris_gemm_argmax_tcgen05(const void* x, const void* w, int* out_token, float* out_prob, int T, int N, int K,
                                          int ldx, int ldw, int rows_w, float* scratch, void* stream) {
    if (T <= 0) return FERRIS_OK;
    if (N <= 0 || T > 128) FERRIS_REFUSE("product + argmax: %d rows (at most 128) over %d outputs", T, N);
    if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K)
        FERRIS_REFUSE("product + argmax: K=%d and row strides %d, %d must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)scratch & 15) || !scratch || !out_token)
        FERRIS_REFUSE("product + argmax: operands must be there and 16-byte aligned");
    if (N > rows_w) FERRIS_REFUSE("product + argmax: %d outputs from %d weight rows", N, rows_w);
    sm_count();
    cudaStream_t s = (cudaStream_t)stream;
    const int bt = (T + 15) / 16 * 16;
    CUtensorMap mw, mx;
    int rc = weight_map(w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw, &mw);
    if (rc != FERRIS_OK) return rc;
    rc = ferris_make_tensor_map_2d(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bt, BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    Params p = {};
    p.out = out_token;
    p.out_prob = out_prob;
    p.scratch = scratch;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = N;
    p.bt = bt;
    p.kblocks = (K + BLOCK_K - 1) / BLOCK_K;
    p.splits = 1;
    p.status = ferris_status_ptr();
    const int stage_bytes = BLOCK_N * BLOCK_K * 2 + bt * BLOCK_K * 2;
    int stages = (227 * 1024 - 2048 - 8192) / stage_bytes;  // 8 KB of the kernel's own for the lane quarters' entries
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > p.kblocks) stages = p.kblocks;
    const int tiles = (N + BLOCK_N - 1) / BLOCK_N;
    if (tiles >= 4 * g_sms) {
        // Many tiles and no K split: shallow rings, so that CTAs share an SM and one streams weights while another's
        // set-up or epilogue runs.  Three to an SM here (three stages of 18 KB at 16 rows; the step of 8 rows at the
        // 0.5B sizes: 0.732-0.734 ms against 0.739 with two and 0.735 with four), where the product that stores the
        // logits is best with two (1.742 / 1.745 / 1.752 ms at 64 rows with two / three / four).
        const int fit = (227 * 1024 / 3 - 3072 - 8192) / stage_bytes;
        if (fit >= 2 && stages > fit) stages = fit;
    }
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    rc = launch<ARGMAX_F32>(mw, mx, p, dim3(tiles, 1, 1), smem, 1u, s);
    if (rc != FERRIS_OK) return rc;
    ferris_launch(argmax_merge_kernel, dim3(T), dim3(AM_THREADS), 0, s, (const float4*)scratch, tiles, T, out_token, out_prob);
    FERRIS_LAUNCH_CHECK();
}

// The q/k/v product of a long step with its rotation and cache write in the epilogue: out[:, :nh d] gets the rotated
// queries (the key and value columns of `out` are NOT written), the paged cache gets the rotated keys and the
// values of the tokens whose slot is >= 0.  Whole-head rotation of heads of 64 or 128, T >= 128 tokens, bf16.
FERRIS_API int ferris_qkv_rope_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int T, int K, int ldx,
                                            int ldw, int ldo, int rows_w, const float* angles, const int* slots,
                                            void* k_cache, void* v_cache, int nh, int nkv, int d, int page_size,
                                            void* stream) {
    if (T <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || page_size <= 0 || (d != 64 && d != 128))
        FERRIS_REFUSE("q/k/v product with rotation: %d + 2 x %d heads of %d, pages of %d", nh, nkv, d, page_size);
    const int N = (nh + 2 * nkv) * d;
    if (T < PT_BLOCK_M) FERRIS_REFUSE("q/k/v product with rotation: %d tokens are fewer than the %d it takes", T, PT_BLOCK_M);
    if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || ldx < K || ldw < K)
        FERRIS_REFUSE("q/k/v product with rotation: K=%d and row strides %d, %d must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || ((uintptr_t)angles & 15) || (ldo & 7) ||
        ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        FERRIS_REFUSE("q/k/v product with rotation: operands must be 16-byte aligned");
    if (N > rows_w || ldo < nh * d) FERRIS_REFUSE("q/k/v product with rotation: %d outputs from %d weight rows, output stride %d", N, rows_w, ldo);
    if (!angles || (slots && (!k_cache || !v_cache))) FERRIS_REFUSE("q/k/v product with rotation: angles or cache missing");
    RopeEpilogue r;
    r.angles = reinterpret_cast<const float2*>(angles);
    r.slots = slots;
    r.k_cache = (bf16*)k_cache;
    r.v_cache = (bf16*)v_cache;
    r.nh = nh;
    r.nkv = nkv;
    r.d = d;
    r.page_size = page_size;
    return run_tokens_m(x, w, bias, out, QKV_ROPE_BF16, T, N, K, ldx, ldw, ldo, rows_w, 0, &r, (cudaStream_t)stream);
}

FERRIS_TIMELINE_TU(gemm_tcgen05)
