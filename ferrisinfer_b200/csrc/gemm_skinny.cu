// Matrix products of steps of at most 16 tokens (decoding):  out[t, n] = sum_k x[t, k] * w[n, k]  (+ bias[n]).
//
// Such a step is a chain of launches, each of which moves a few megabytes of weights and computes next to
// nothing; what it costs is the serial path of every launch after the launch before it has ended.  This kernel keeps
// that path short:
//   * The weight ROWS are divided among the CTAs (one slab of R rows per CTA, R = rows / SMs), never the K
//     dimension: a CTA owns its outputs, so no partial sums cross CTAs, there is no cluster and no barrier but the
//     CTA's own.
//   * A CTA's whole slab ([R, K] bf16; 14 KB to 143 KB per SM at the 0.5B sizes) is requested by TMA
//     (cp.async.bulk.tensor, 128-byte swizzle, one box of R rows x 64 columns per K block) BEFORE the
//     programmatic-launch wait: the weights do not depend on the launch before, and a slab per SM of two
//     consecutive launches fits into shared memory side by side, so the weights of launch N + 1 arrive while
//     launch N runs.  A slab that does not fit goes through the same stages as a ring.
//   * After the wait: the step's rows come into shared memory whole, in the same swizzled boxes of 8 or 16 rows x
//     64 columns: by TMA when they exist as bf16, or formed by the CTA's warps (one row each) as the RMSNorm of
//     the fp32 residual rows (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41).  Then eight warps take the
//     K blocks in turn with mma.sync m16n8k16 (both operands by ldmatrix from shared memory; no load from
//     global memory stands in the loop), and their eight partial tiles are added in warp order through shared
//     memory.
//   * Where the slab does not fit beside the step's rows (long rows: the down projection of the larger sizes), the
//     rows are not held whole: each stage of the ring carries the box of the step's rows for its K blocks behind
//     its box of weights (requested after the wait, counted on the same barrier), so that all of shared memory is
//     weights in flight and nothing has to arrive before the first multiplication.
// The tensor pipe is idle either way at these sizes; tcgen05.mma costs ~100 cycles an instruction whatever its
// width, which caps an SM at ~80 GB/s of weights with 16 tokens, and one thread issues them all.  Eight warps of
// mma.sync take in weights at the rate shared memory delivers them.  Steps of more than 16 tokens run the tcgen05
// kernels of gemm_tcgen05.cu.
//
// Formula of the product: crates/ferrisinfer-kernel/src/cpu/matmul.rs:46-118; bias:
// crates/ferrisinfer-runtime/src/reference.rs:1132-1191; SwiGLU: crates/ferrisinfer-runtime/src/reference.rs:346-360.
#include <stdlib.h>

#include "common.cuh"
#include "sm100.cuh"

namespace {

constexpr int SK_WARPS = 8;                       // warps that multiply
constexpr int SK_THREADS = (SK_WARPS + 1) * 32;   // and one that requests the weights
constexpr int SK_BLOCK_K = 64;                    // one 128-byte swizzle row of bf16
constexpr int SK_MAX_MT = 4;                      // 16-row tiles of a slab (per accumulator set)
constexpr int SK_MAX_ROWS = 16 * SK_MAX_MT;
constexpr int SK_MAX_STAGES = 96;
constexpr int SK_MAX_TOKENS = 16;

enum SkMode { SK_STORE_BF16 = 0, SK_STORE_F32 = 1, SK_ACCUM_F32 = 2, SK_SWIGLU_BF16 = 3 };

struct SkParams {
    const float* norm_h;  // [T, K] fp32 residual rows (contiguous), or null when the rows come by TMA (map_x)
    const float* norm_w;  // [K]
    float norm_eps;
    void* out;
    const float* bias;
    int T, N, K, ldo;
    int rows;      // weight rows per CTA and accumulator set (R)
    int box_rows;  // R rounded up to a multiple of 8: rows of one TMA box of weights
    int x_rows;    // rows of a box of the step's tokens: 8 or 16
    int mt;        // 16-row tiles of the slab
    int kblocks;   // K blocks of 64 columns
    int nb;        // K blocks that one TMA copy brings (a group); odd, or 1
    unsigned nb_magic;  // 2^32 / nb rounded up: kb / nb == umulhi(kb, nb_magic) for kb < 2^16
    int groups;    // ceil(kblocks / nb)
    int stages;    // groups of weights that shared memory holds at once
    int boxes_3d;  // the copies use the 3-D maps (K a multiple of 64); else nb == 1 and the 2-D maps
    int x_in_stages;  // the step's rows travel with the weights, a box per stage, instead of standing whole beside them
    int up_row_offset;
    int mode;
    int* status;
};

__device__ __forceinline__ float sk_silu_mul(float g, float u) { return u * (g * (1.0f / (1.0f + expf(-g)))); }

// a: the product (the gate's in SwiGLU mode), b: the up product, bias_v: bias[n] or 0, old: what out[t, n] held.
__device__ __forceinline__ void sk_write(const SkParams& p, int t, int n, float a, float b, float bias_v, float old) {
    if (p.mode == SK_STORE_BF16) {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(a + bias_v);
    } else if (p.mode == SK_STORE_F32) {
        reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = a + bias_v;
    } else if (p.mode == SK_ACCUM_F32) {
        reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = old + (a + bias_v);
    } else {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(sk_silu_mul(a, b));
    }
}

// ACCS: 2 in SwiGLU mode (gate rows and up rows of the same outputs), else 1.  NT: 8-token tiles (1 or 2).
// Shared memory: the weight stages (a ring when the slab does not fit), then the step's rows, one box per K block.
template <int ACCS, int NT>
__global__ void __launch_bounds__(SK_THREADS, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                       const SkParams p) {
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[SK_MAX_STAGES], empty[SK_MAX_STAGES], full_x;
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * p.rows;
    // A group of nb K blocks is one TMA box: box_rows x nb lines of 128 bytes, line (row * nb + block), swizzled by the
    // line's number (with nb == 1 that is the plain 2-D box of one block).
    const int box_bytes = p.box_rows * p.nb * 128;
    const int x_box_bytes = p.x_rows * p.nb * 128;
    const int stage_bytes = ACCS * box_bytes + (p.x_in_stages ? x_box_bytes : 0);
    uint8_t* x_smem = smem + (size_t)p.stages * stage_bytes;
    const bool ring = p.groups > p.stages;  // the slab does not fit: stages are used again

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_w);
        if (!p.norm_h) tma_prefetch_descriptor(&map_x);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);  // the warp that takes the group
        }
        mbar_init(&full_x, 1);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == SK_WARPS) {
        // The weights depend on no earlier launch: everything the stages hold is requested before any wait.
        // the box of the step's rows for group g, into its stage (counted on the stage's barrier)
        auto request_rows = [&](int g) {
            const int s = g % p.stages;
            uint8_t* at = smem + (size_t)s * stage_bytes + ACCS * box_bytes;
            if (p.boxes_3d)
                tma_load_3d(at, &map_x, 0, g * p.nb, 0, &full[s]);
            else
                tma_load_2d(at, &map_x, g * SK_BLOCK_K, 0, &full[s]);
        };
        auto request = [&](int g, bool with_rows) {
            const int s = g % p.stages;
            uint8_t* st = smem + (size_t)s * stage_bytes;
            mbar_expect_tx(&full[s], stage_bytes);
            if (p.boxes_3d) {
                tma_load_3d(st, &map_w, 0, g * p.nb, n0, &full[s]);
                if (ACCS == 2) tma_load_3d(st + box_bytes, &map_w, 0, g * p.nb, p.up_row_offset + n0, &full[s]);
            } else {
                tma_load_2d(st, &map_w, g * SK_BLOCK_K, n0, &full[s]);
                if (ACCS == 2) tma_load_2d(st + box_bytes, &map_w, g * SK_BLOCK_K, p.up_row_offset + n0, &full[s]);
            }
            if (with_rows) request_rows(g);
        };
        const int first = min(p.groups, p.stages);
        if (lane == 0)
            for (int g = 0; g < first; ++g) request(g, false);
        if (p.x_in_stages) {
            // the rows of the first stages follow their weights after the wait; later stages get both at once
            pdl_wait();
            if (lane == 0)
                for (int g = 0; g < first; ++g) request_rows(g);
        } else if (!p.norm_h) {
            // the step's rows were written by the launch before: requested after the wait, one box per group, the
            // lanes taking the boxes in turn
            pdl_wait();
            if (lane == 0) mbar_expect_tx(&full_x, p.groups * x_box_bytes);
            __syncwarp();
            for (int g = lane; g < p.groups; g += 32) {
                if (p.boxes_3d)
                    tma_load_3d(x_smem + (size_t)g * x_box_bytes, &map_x, 0, g * p.nb, 0, &full_x);
                else
                    tma_load_2d(x_smem + (size_t)g * x_box_bytes, &map_x, g * SK_BLOCK_K, 0, &full_x);
            }
        }
        if (lane == 0)
            for (int g = first; g < p.groups; ++g) {
                if (!mbar_wait(&empty[g % p.stages], ((g / p.stages) - 1) & 1, p.status, 40)) break;
                request(g, p.x_in_stages != 0);
            }
        return;
    }

    // What does not depend on the launch before is read BEFORE the wait, so that no trip to HBM stands on the step's
    // critical path after it: the bias of this thread's outputs and the norm's weight (each layer has its own: they
    // are never in L2 when the step comes to them).  The old values of the outputs (the residual that an accumulating
    // product adds to) are requested right after the wait and used at the very end.
    constexpr int OUTS = SK_MAX_MT * NT / 2;  // outputs of one thread: element tid + 256 i of the accumulator tiles
    const int per_acc = p.mt * NT * 4;
    int out_t[OUTS], out_n[OUTS];
    float bias_r[OUTS], old_r[OUTS];
#pragma unroll
    for (int i = 0; i < OUTS; ++i) {
        const int q = threadIdx.x + SK_WARPS * 32 * i;
        const int ln = q & 31, e = q >> 5;
        const int j = e & 3, nt = (e >> 2) % NT, m = (e >> 2) / NT;
        const int row = m * 16 + (ln >> 2) + ((j & 2) ? 8 : 0);
        const int t = nt * 8 + (ln & 3) * 2 + (j & 1);
        const int n = n0 + row;
        const bool valid = q < per_acc * 32 && row < p.rows && n < p.N && t < p.T;
        out_t[i] = valid ? t : -1;
        out_n[i] = n;
        bias_r[i] = (valid && p.bias) ? p.bias[n] : 0.0f;
        old_r[i] = 0.0f;
    }
    const int n4 = p.K / 4, tile4 = p.kblocks * 16;
    const float4* w4 = reinterpret_cast<const float4*>(p.norm_w);
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 wv[8];
    if (p.norm_h && tile4 <= 256) {
#pragma unroll
        for (int j = 0; j < 8; ++j) wv[j] = j * 32 + lane < n4 ? w4[j * 32 + lane] : zero4;
    } else if (p.norm_h) {
        for (int i = threadIdx.x; i * 32 < p.K; i += SK_WARPS * 32)  // one 128-byte line of the weight per thread
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.norm_w + i * 32));
    }

    pdl_wait();
    FERRIS_TL_BEGIN();
    [[maybe_unused]] const bool tl_mark = threadIdx.x == 0 && blockIdx.x == 0;
    FERRIS_TL_MARK(tl_mark, 9);
    if (p.mode == SK_ACCUM_F32) {
#pragma unroll
        for (int i = 0; i < OUTS; ++i)
            if (out_t[i] >= 0) old_r[i] = reinterpret_cast<const float*>(p.out)[(size_t)out_t[i] * p.ldo + out_n[i]];
    }
    if (p.norm_h) {
        // One warp per row: ms = sum(x^2) / K;  r = 1 / sqrt(ms + eps);  y = (x r) w, rounded to bf16 and written where
        // TMA would have put it (rows of 128 bytes, 16-byte chunks swizzled); rows beyond T and columns beyond K are
        // zero.  A lane takes every 32nd group of four columns, eight groups at a time with all their loads in flight
        // together; a row of up to 1,024 columns is read once and stays in registers between the two passes.
        for (int t = warp; t < p.x_rows; t += SK_WARPS) {
            const float4* row = reinterpret_cast<const float4*>(p.norm_h + (size_t)(t < p.T ? t : 0) * p.K);
            const bool live = t < p.T;
            auto put = [&](int idx, float4 h, float4 w, float r) {  // columns 4 idx .. 4 idx + 3 of row t
                uint2 v = make_uint2(0u, 0u);
                if (live && idx < n4) {
                    v.x = pack_bf16((h.x * r) * w.x, (h.y * r) * w.y);
                    v.y = pack_bf16((h.z * r) * w.z, (h.w * r) * w.w);
                }
                const int kb = idx >> 4;  // K block of these columns; group kb / nb, line t * nb + kb % nb of its box
                const int grp = p.nb == 1 ? kb : (int)__umulhi((unsigned)kb, p.nb_magic);  // kb / nb, exact for small kb
                *reinterpret_cast<uint2*>(x_smem + (size_t)grp * x_box_bytes +
                                          swizzle128(t * p.nb + (kb - grp * p.nb), (idx >> 1) & 7) + (idx & 1) * 8) = v;
            };
            float ss = 0.0f;
            if (tile4 <= 256) {
                float4 hv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) hv[j] = (live && j * 32 + lane < n4) ? row[j * 32 + lane] : zero4;
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += (hv[j].x * hv[j].x + hv[j].y * hv[j].y) + (hv[j].z * hv[j].z + hv[j].w * hv[j].w);
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss / (float)p.K + p.norm_eps);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j * 32 + lane < tile4) put(j * 32 + lane, hv[j], wv[j], r);
            } else {
                for (int base = 0; base < n4 && live; base += 256) {
                    float4 hv[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) hv[j] = base + j * 32 + lane < n4 ? row[base + j * 32 + lane] : zero4;
#pragma unroll
                    for (int j = 0; j < 8; ++j) ss += (hv[j].x * hv[j].x + hv[j].y * hv[j].y) + (hv[j].z * hv[j].z + hv[j].w * hv[j].w);
                }
                ss = warp_sum(ss);
                const float r = 1.0f / sqrtf(ss / (float)p.K + p.norm_eps);
                for (int base = 0; base < tile4; base += 256) {
                    float4 hv[8], wl[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int idx = base + j * 32 + lane;
                        hv[j] = (live && idx < n4) ? row[idx] : zero4;
                        wl[j] = idx < n4 ? w4[idx] : zero4;
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (base + j * 32 + lane < tile4) put(base + j * 32 + lane, hv[j], wl[j], r);
                }
            }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
    } else if (!p.x_in_stages) {
        mbar_wait(&full_x, 0, p.status, 42);
    }
    FERRIS_TL_MARK(tl_mark, 0);

    // Warp w takes the groups w, w + 8, ...; of each of a group's K blocks the four K steps, their fragments loaded
    // together.
    const int mine = p.groups > warp ? (p.groups - warp + SK_WARPS - 1) / SK_WARPS : 0;
    float acc[ACCS][SK_MAX_MT][NT][4];
#pragma unroll
    for (int a = 0; a < ACCS; ++a)
#pragma unroll
        for (int m = 0; m < SK_MAX_MT; ++m)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[a][m][nt][j] = 0.0f;

    const int mi = lane >> 3, r8 = lane & 7;
    const uint32_t x_base = smem_u32(x_smem);
    // stage and phase of this warp's next group, kept without a division in the loop
    int s = warp % p.stages, phase = (warp / p.stages) & 1;
    const int s_step = SK_WARPS % p.stages, phase_step = (SK_WARPS / p.stages) & 1;
    [[maybe_unused]] long long waited = 0, began = FERRIS_TL_CLOCK();  // timeline build: cycles this warp waits for weights
    for (int i = 0; i < mine; ++i) {
        const int g = warp + SK_WARPS * i;
        const long long c0 = FERRIS_TL_CLOCK();
        if (!mbar_wait(&full[s], phase, p.status, 41)) break;
        waited += FERRIS_TL_CLOCK() - c0;
        FERRIS_TL_MARK(tl_mark && i == 0, 1);
        const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
        const uint32_t xg = p.x_in_stages ? st + ACCS * box_bytes : x_base + g * x_box_bytes;
        const int blocks = min(p.nb, p.kblocks - g * p.nb);
        for (int kbi = 0; kbi < blocks; ++kbi) {
            // B fragments of the four K steps: tokens are the rows of the box; matrices (tokens 0-7 | 8-15) x
            // (columns 0-7 | 8-15 of the K step)
            uint32_t b[4][NT][2];
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                if (NT == 2) {
                    uint32_t r[4];
                    ldmatrix_x4(r, xg + swizzle128(((mi >> 1) * 8 + r8) * p.nb + kbi, ks * 2 + (mi & 1)));
                    b[ks][0][0] = r[0], b[ks][0][1] = r[1], b[ks][NT - 1][0] = r[2], b[ks][NT - 1][1] = r[3];
                } else {
                    uint32_t r[2];
                    ldmatrix_x2(r, xg + swizzle128(r8 * p.nb + kbi, ks * 2 + (mi & 1)));
                    b[ks][0][0] = r[0], b[ks][0][1] = r[1];
                }
            }
#pragma unroll
            for (int a = 0; a < ACCS; ++a) {
#pragma unroll
                for (int m = 0; m < SK_MAX_MT; ++m) {
                    if (m >= p.mt) continue;
                    // rows beyond the box (the last tile of a slab whose rows are no multiple of 16) read its last
                    // row again; their outputs are never written
                    const int line = min(m * 16 + (mi & 1) * 8 + r8, p.box_rows - 1) * p.nb + kbi;
                    uint32_t af[4][4];
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) ldmatrix_x4(af[ks], st + a * box_bytes + swizzle128(line, ks * 2 + (mi >> 1)));
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[a][m][nt], af[ks], b[ks][nt][0], b[ks][nt][1]);
                }
            }
        }
        if (ring) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        s += s_step;
        phase ^= phase_step;
        if (s >= p.stages) {
            s -= p.stages;
            phase ^= 1;
        }
    }
    FERRIS_TL_MARK(tl_mark, 2);
    FERRIS_TL_VALUE(tl_mark, 5, (unsigned long long)waited);
    FERRIS_TL_VALUE(tl_mark, 6, (unsigned long long)(FERRIS_TL_CLOCK() - began));
    FERRIS_TL_VALUE(tl_mark, 7, (unsigned long long)mine);

    // The eight warps' partial tiles, added in warp order: [warp][accumulator, tile, token tile, element][lane].
    asm volatile("bar.sync 1, 256;" ::: "memory");  // nobody reads the stages any more
    float* red = reinterpret_cast<float*>(smem);
    const int per_warp = ACCS * per_acc;
#pragma unroll
    for (int a = 0; a < ACCS; ++a)
#pragma unroll
        for (int m = 0; m < SK_MAX_MT; ++m) {
            if (m >= p.mt) continue;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    red[(size_t)(warp * per_warp + a * per_acc + (m * NT + nt) * 4 + j) * 32 + lane] = acc[a][m][nt][j];
        }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    FERRIS_TL_MARK(tl_mark, 3);
#pragma unroll
    for (int i = 0; i < OUTS; ++i) {
        if (out_t[i] < 0) continue;
        const int q = threadIdx.x + SK_WARPS * 32 * i;
        const int ln = q & 31, e = q >> 5;
        float va = 0.0f, vb = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
            va += red[(size_t)(w * per_warp + e) * 32 + ln];
            if (ACCS == 2) vb += red[(size_t)(w * per_warp + per_acc + e) * 32 + ln];
        }
        sk_write(p, out_t[i], out_n[i], va, vb, bias_r[i], old_r[i]);
    }
    FERRIS_TL_MARK(tl_mark, 4);
    FERRIS_TL_END(40 + p.mode + (p.norm_h ? 4 : 0));
}

int g_sk_sms = 0;
int g_sk_enabled = -1;

int sk_sm_count() {
    if (g_sk_sms <= 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&g_sk_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sk_sms <= 0)
            g_sk_sms = 148;
    }
    return g_sk_sms;
}

// How a product is cut: rows per CTA, K blocks per copy, stages, shared memory.
struct SkPlan {
    int rows, box_rows, x_rows, mt, ctas, kblocks, nb, groups, stages;
    size_t smem;
    int x_in_stages;
};

// Shared memory of one CTA: the step's rows whole, the weight stages beside them; a slab that does not fit streams
// through its stages as a ring.  Measured in the decode step of 8 tokens at the 0.5B sizes (24 layers, context
// 4,096): 108 KB a CTA, so that two launches that follow each other always share an SM and the second one's weights
// arrive while the first runs, 1.09 ms a step; 150 KB 1.01 ms; 190 KB 0.95 ms.  A whole slab in place when the wait
// ends is worth more than an early start of the next launch's copies: a ring's later groups are requested only as
// the earlier ones are consumed, one more trip to memory on the step's critical path, while a launch that has to wait
// for the SM still has the ~2 us between the end of the launch before and its own wait for its copies.
// Beyond 190 KB nothing changes at those sizes; the rings of the larger sizes gain from every KB, because more of it
// lets a copy bring more K blocks of a row, and longer runs of a weight row come faster out of HBM: down projection
// of the 7B sizes (rows of 37 KB) 35.4 us with copies of 3 blocks (190 KB), 26.3 us with 5 (200 KB and more); of the
// 1.5B sizes 9.8 us at 190 KB, 9.3 us at 220 KB.  So the default is 220 KB.
// FERRIS_SKINNY_SMEM_KB in the environment overrides (16 to 220).
int g_sk_budget = 0;
int sk_smem_budget() {
    if (g_sk_budget <= 0) {
        const char* v = getenv("FERRIS_SKINNY_SMEM_KB");
        g_sk_budget = (v ? atoi(v) : 220) * 1024;
        if (g_sk_budget < 16 * 1024 || g_sk_budget > 220 * 1024) g_sk_budget = 220 * 1024;
    }
    return g_sk_budget;
}

// rows_by_tma: the step's rows exist as bf16 (not formed by the kernel as a norm), so they may travel with the weights.
bool sk_plan(int T, int N, int K, int accs, bool rows_by_tma, SkPlan* out) {
    if (T < 1 || T > SK_MAX_TOKENS || N < 1 || K < 8 || (K & 7)) return false;
    const int sms = sk_sm_count();
    int rows = (N + sms - 1) / sms;
    if (rows > SK_MAX_ROWS) rows = SK_MAX_ROWS;
    const int ctas = (N + rows - 1) / rows;
    if (ctas > 2 * sms) return false;  // a product this tall (the output head) streams better through the tcgen05 kernel
    const int box_rows = (rows + 7) / 8 * 8;
    const int x_rows = T > 8 ? 16 : 8;
    const int kblocks = (K + SK_BLOCK_K - 1) / SK_BLOCK_K;
    // K blocks per copy.  A copy costs the TMA unit ~30 ns whatever it brings, so boxes of one block of 8 rows (1 KB)
    // arrive at a third of the rate of large ones; a group is also what one warp takes at a time, so the groups should
    // be about as many as the warps, or many more.  Odd sizes only: the eight rows of a block then lie in eight
    // different swizzle phases of the box, and ldmatrix reads them without bank conflicts.  Without whole blocks
    // (K no multiple of 64) the 2-D map brings one block per copy.
    int best_nb = 1, best_stages = 0, best_in_stages = 0;
    double best_cost = 1e30;
    for (int variant = 0; variant < (rows_by_tma ? 2 : 1); ++variant)
    for (int nb = 1; nb <= 15; nb += 2) {
        if (nb > 1 && (K & 63)) break;
        if (nb > kblocks) break;
        const int groups = (kblocks + nb - 1) / nb;
        // variant 1: the rows travel with the weights (only where the slab is a ring anyway)
        const int stage_bytes = (accs * box_rows + (variant ? x_rows : 0)) * nb * 128;
        const int x_bytes = variant ? 0 : groups * x_rows * nb * 128;
        if (x_bytes >= sk_smem_budget()) continue;
        int stages = (sk_smem_budget() - x_bytes) / stage_bytes;
        if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
        if (stages >= groups) {
            if (variant) continue;  // everything fits: the rows stand whole, as one request
            stages = groups;
        } else {
            // A ring: the groups of a stage must all go to one warp, which then sees the stage's fills in order
            // (a wait names a fill by its parity only, so a warp that skipped a fill would take the older one for
            // it).  Warp g % 8 takes group g, which is constant per stage when the stages are a multiple of eight.
            stages = stages / SK_WARPS * SK_WARPS;
            if (stages <= 0) continue;
            // More than 8 tokens beside long rows leave the weights a small ring, and the tcgen05 kernel is then the
            // faster one (down projection of the 0.5B sizes at 16 tokens: 9.4 us here, 7.1 us there).
            if (!variant && x_rows > 8 && stages * 2 < groups) continue;
        }
        // blocks on the busiest warp, the copies it waits for, and what a ring adds: the groups that are not in
        // shared memory when the wait ends, each a trip to memory behind the one before it in its stage
        const double cost = (double)((groups + SK_WARPS - 1) / SK_WARPS) * nb + 0.4 * groups +
                            1.0 * (groups - stages) * (variant ? 0.5 : 1.0);
        if (cost < best_cost) best_cost = cost, best_nb = nb, best_stages = stages, best_in_stages = variant;
    }
    if (best_stages == 0) return false;  // rows too long to stand beside their weights: the tcgen05 kernel's
    const int nb = best_nb, groups = (kblocks + nb - 1) / nb, stages = best_stages;
    const int nt = T > 8 ? 2 : 1;
    const int mt = (rows + 15) / 16;
    const size_t red_bytes = (size_t)SK_WARPS * accs * mt * nt * 4 * 32 * sizeof(float);
    // the warps' partial tiles reuse the stages (and, if they need more, the rows behind them, which nobody reads then)
    size_t smem = best_in_stages ? (size_t)stages * (accs * box_rows + x_rows) * nb * 128
                                 : (size_t)stages * accs * box_rows * nb * 128 + (size_t)groups * x_rows * nb * 128;
    if (smem < red_bytes) smem = red_bytes;
    *out = {rows, box_rows, x_rows, mt, ctas, kblocks, nb, groups, stages, smem + 1024, best_in_stages};
    return true;
}

template <int ACCS, int NT>
int sk_launch(const CUtensorMap& mw, const CUtensorMap& mx, const SkParams& p, int ctas, size_t smem, cudaStream_t s) {
    int rc = ferris_allow_dynamic_smem((const void*)gemm_skinny_kernel<ACCS, NT>, smem);
    if (rc != FERRIS_OK) return rc;
    cudaError_t e = ferris_launch(gemm_skinny_kernel<ACCS, NT>, dim3(ctas), dim3(SK_THREADS), smem, s, mw, mx, p);
    if (e != cudaSuccess) {
        ferris_set_error("skinny gemm: %s", cudaGetErrorString(e));
        return (int)e;
    }
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// Whether steps of at most 16 tokens run this kernel (the default) or the tcgen05 kernels with their K split over a
// cluster: FERRIS_GEMM_SKINNY=0 in the environment, or ferris_set_gemm_skinny(0), selects the latter.
FERRIS_API int ferris_gemm_skinny_enabled() {
    if (g_sk_enabled < 0) {
        const char* v = getenv("FERRIS_GEMM_SKINNY");
        g_sk_enabled = (v && v[0] == '0') ? 0 : 1;
    }
    return g_sk_enabled;
}

FERRIS_API int ferris_set_gemm_skinny(int on) {
    g_sk_enabled = on ? 1 : 0;
    return FERRIS_OK;
}

// 1 if ferris_gemm_skinny takes a product of these sizes (accumulators: 2 for SwiGLU, else 1; rows_by_tma: the step's
// rows exist as bf16, 0 if the kernel is to form them as a norm).
FERRIS_API int ferris_gemm_skinny_takes(int T, int N, int K, int accumulators, int rows_by_tma) {
    SkPlan plan;
    return (ferris_gemm_skinny_enabled() && sk_plan(T, N, K, accumulators == 2 ? 2 : 1, rows_by_tma != 0, &plan)) ? 1 : 0;
}

// x: bf16 [T, K] rows ldx apart (16-byte aligned rows), or null with norm_h / norm_w / norm_eps: the rows are the RMSNorm of the fp32 rows
// norm_h [T, K] (contiguous).  w: bf16 [rows_w, K] rows ldw apart.  out: [T, N] rows ldo apart in the mode's type.
// mode: 0 bf16 = acc + bias; 1 fp32 = acc + bias; 2 fp32 += acc + bias; 3 bf16 = silu(x w[:N]^T) * (x w[up:up+N]^T).
FERRIS_API int ferris_gemm_skinny(const void* x, int ldx, const float* norm_h, const float* norm_w, float norm_eps,
                                  const void* w, const float* bias, void* out, int mode, int T, int N, int K, int ldw,
                                  int ldo, int rows_w, int up_row_offset, void* stream) {
    if (T <= 0 || N <= 0) return FERRIS_OK;
    if (mode < 0 || mode > 3) FERRIS_REFUSE("skinny gemm: unknown mode %d", mode);
    const int accs = mode == SK_SWIGLU_BF16 ? 2 : 1;
    SkPlan plan;
    if (!sk_plan(T, N, K, accs, norm_h == nullptr, &plan))
        FERRIS_REFUSE("skinny gemm: %d tokens x %d outputs x K=%d is not a shape it takes (at most %d tokens, K a "
                      "multiple of 8, at most %d rows)", T, N, K, SK_MAX_TOKENS, 2 * SK_MAX_ROWS * sk_sm_count());
    if ((ldw & 7) || ldw < K || ((uintptr_t)w & 15)) FERRIS_REFUSE("skinny gemm: weight rows must be 16-byte aligned");
    if (norm_h) {
        if (!norm_w || ((uintptr_t)norm_h & 15) || ((uintptr_t)norm_w & 15))
            FERRIS_REFUSE("skinny gemm: the rows to normalise and the norm's weight must be 16-byte aligned");
    } else {
        if (!x || (ldx & 7) || ldx < K || ((uintptr_t)x & 15)) FERRIS_REFUSE("skinny gemm: token rows must be 16-byte aligned");
    }
    if (mode == SK_SWIGLU_BF16 && (bias || up_row_offset + N > rows_w)) FERRIS_REFUSE("skinny gemm: bad SwiGLU operands");
    if (mode != SK_SWIGLU_BF16 && N > rows_w) FERRIS_REFUSE("skinny gemm: %d outputs from %d weight rows", N, rows_w);
    if (ldo < N) FERRIS_REFUSE("skinny gemm: output row stride %d < %d", ldo, N);
    const bool boxes_3d = (K & 63) == 0;
    CUtensorMap mw;
    int rc = boxes_3d ? ferris_make_tensor_map_kblocks(&mw, w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw,
                                                       (uint32_t)plan.box_rows, (uint32_t)plan.nb)
                      : ferris_make_tensor_map_2d(&mw, w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw,
                                                  (uint32_t)plan.box_rows, SK_BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    CUtensorMap mx = mw;  // unused when the rows are formed in the kernel
    if (!norm_h) {
        rc = boxes_3d ? ferris_make_tensor_map_kblocks(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx,
                                                       (uint32_t)plan.x_rows, (uint32_t)plan.nb)
                      : ferris_make_tensor_map_2d(&mx, x, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)plan.x_rows,
                                                  SK_BLOCK_K);
        if (rc != FERRIS_OK) return rc;
    }
    SkParams p;
    p.norm_h = norm_h;
    p.norm_w = norm_w;
    p.norm_eps = norm_eps;
    p.out = out;
    p.bias = bias;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.rows = plan.rows;
    p.box_rows = plan.box_rows;
    p.x_rows = plan.x_rows;
    p.mt = plan.mt;
    p.kblocks = plan.kblocks;
    p.nb = plan.nb;
    p.nb_magic = (unsigned)((0x100000000ull + plan.nb - 1) / plan.nb);
    p.groups = plan.groups;
    p.stages = plan.stages;
    p.boxes_3d = boxes_3d ? 1 : 0;
    p.x_in_stages = plan.x_in_stages;
    p.up_row_offset = up_row_offset;
    p.mode = mode;
    p.status = ferris_status_ptr();
    cudaStream_t s = (cudaStream_t)stream;
    if (accs == 2)
        return T > 8 ? sk_launch<2, 2>(mw, mx, p, plan.ctas, plan.smem, s) : sk_launch<2, 1>(mw, mx, p, plan.ctas, plan.smem, s);
    return T > 8 ? sk_launch<1, 2>(mw, mx, p, plan.ctas, plan.smem, s) : sk_launch<1, 1>(mw, mx, p, plan.ctas, plan.smem, s);
}

FERRIS_TIMELINE_TU(gemm_skinny)
