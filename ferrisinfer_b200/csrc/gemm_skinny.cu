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
//   * After the wait: the step's rows are read straight from global memory (they are a few KB, the same for all
//     CTAs, and come from L2) as the B fragments of mma.sync m16n8k16; eight warps take the 16-column K steps in
//     turn (A fragments by ldmatrix from the swizzled boxes), and their eight partial tiles are added in warp
//     order through shared memory.  With `norm_h` the rows are formed on the way as the RMSNorm of the fp32
//     residual rows (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41).
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
constexpr int SK_PREFETCH = 4;                    // K steps whose token fragments a warp holds ahead

enum SkMode { SK_STORE_BF16 = 0, SK_STORE_F32 = 1, SK_ACCUM_F32 = 2, SK_SWIGLU_BF16 = 3 };

struct SkParams {
    const bf16* x;        // [T, K] rows ldx apart, or null when the rows are formed from norm_h
    const float* norm_h;  // [T, K] fp32 residual rows (contiguous)
    const float* norm_w;  // [K]
    float norm_eps;
    void* out;
    const float* bias;
    int ldx, T, N, K, ldo;
    int rows;      // weight rows per CTA and accumulator set (R)
    int box_rows;  // R rounded up to a multiple of 8: rows of one TMA box
    int mt;        // 16-row tiles of the slab
    int kblocks, stages;
    int up_row_offset;
    int mode;
    int* status;
};

__device__ __forceinline__ float sk_silu_mul(float g, float u) { return u * (g * (1.0f / (1.0f + expf(-g)))); }

__device__ __forceinline__ void sk_write(const SkParams& p, int t, int n, float a, float b) {
    const float bias_v = p.bias ? p.bias[n] : 0.0f;
    if (p.mode == SK_STORE_BF16) {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(a + bias_v);
    } else if (p.mode == SK_STORE_F32) {
        reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = a + bias_v;
    } else if (p.mode == SK_ACCUM_F32) {
        float* o = reinterpret_cast<float*>(p.out) + (size_t)t * p.ldo + n;
        *o = *o + (a + bias_v);
    } else {
        reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16_rn(sk_silu_mul(a, b));
    }
}

// ACCS: 2 in SwiGLU mode (gate rows and up rows of the same outputs), else 1.  NT: 8-token tiles (1 or 2).
template <int ACCS, int NT>
__global__ void __launch_bounds__(SK_THREADS, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const SkParams p) {
    FERRIS_TL_ENTRY();
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full[SK_MAX_STAGES], empty[SK_MAX_STAGES];
    __shared__ float rstd_s[SK_MAX_TOKENS];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * p.rows;
    const int box_bytes = p.box_rows * 128;
    const int stage_bytes = ACCS * box_bytes;
    const bool ring = p.kblocks > p.stages;  // the slab does not fit: stages are used again

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&map_w);
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4);  // the four warps that share a K block
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == SK_WARPS) {
        // The weights depend on no earlier launch: everything the stages hold is requested before any wait.
        if (lane == 0) {
            auto request = [&](int kb) {
                const int s = kb % p.stages;
                uint8_t* st = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(&full[s], stage_bytes);
                tma_load_2d(st, &map_w, kb * SK_BLOCK_K, n0, &full[s]);
                if (ACCS == 2) tma_load_2d(st + box_bytes, &map_w, kb * SK_BLOCK_K, p.up_row_offset + n0, &full[s]);
            };
            const int first = min(p.kblocks, p.stages);
            for (int kb = 0; kb < first; ++kb) request(kb);
            for (int kb = first; kb < p.kblocks; ++kb) {
                if (!mbar_wait(&empty[kb % p.stages], ((kb / p.stages) - 1) & 1, p.status, 40)) break;
                request(kb);
            }
        }
        return;
    }

    pdl_wait();
    FERRIS_TL_BEGIN();
    const bool tl_mark = threadIdx.x == 0 && blockIdx.x == 0;
    FERRIS_TL_MARK(tl_mark, 9);
    if (p.norm_h) {
        // ms = sum(x^2) / K;  r = 1 / sqrt(ms + eps): one warp per row
        for (int t = warp; t < p.T; t += SK_WARPS) {
            const float4* row = reinterpret_cast<const float4*>(p.norm_h + (size_t)t * p.K);
            float ss = 0.0f;
            for (int i = lane; i < p.K / 4; i += 32) {
                const float4 v = row[i];
                ss = fmaf(v.x, v.x, ss);
                ss = fmaf(v.y, v.y, ss);
                ss = fmaf(v.z, v.z, ss);
                ss = fmaf(v.w, v.w, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) rstd_s[t] = 1.0f / sqrtf(ss / (float)p.K + p.norm_eps);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    FERRIS_TL_MARK(tl_mark, 0);

    // Warp w takes K step (w % 4) of the K blocks w / 4, w / 4 + 2, ...: unit u = w + 8 i is K step u % 4 of block u / 4.
    const int units = p.kblocks * 4;
    const int mine = units > warp ? (units - warp + SK_WARPS - 1) / SK_WARPS : 0;
    const int g = lane >> 2, c = lane & 3;
    float acc[ACCS][SK_MAX_MT][NT][4];
#pragma unroll
    for (int a = 0; a < ACCS; ++a)
#pragma unroll
        for (int m = 0; m < SK_MAX_MT; ++m)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[a][m][nt][j] = 0.0f;

    // B fragments of one K step: tokens 8 nt + g, columns k0 + 2c, +1 and k0 + 2c + 8, +9
    auto load_b = [&](int u, uint32_t (&b)[NT][2]) {
        const int k0 = (u >> 2) * SK_BLOCK_K + (u & 3) * 16 + 2 * c;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int t = nt * 8 + g;
#pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                const int k = k0 + 8 * hb;
                uint32_t v = 0u;
                if (t < p.T && k < p.K) {  // K is a multiple of 8: a pair lies inside or outside as a whole
                    if (p.norm_h) {
                        const float2 h2 = *reinterpret_cast<const float2*>(p.norm_h + (size_t)t * p.K + k);
                        const float2 w2 = *reinterpret_cast<const float2*>(p.norm_w + k);
                        const float r = rstd_s[t];
                        v = pack_bf16((h2.x * r) * w2.x, (h2.y * r) * w2.y);
                    } else {
                        v = *reinterpret_cast<const uint32_t*>(p.x + (size_t)t * p.ldx + k);
                    }
                }
                b[nt][hb] = v;
            }
        }
    };

    uint32_t breg[SK_PREFETCH][NT][2];
#pragma unroll
    for (int j = 0; j < SK_PREFETCH; ++j)
        if (j < mine) load_b(warp + SK_WARPS * j, breg[j]);

    const int mi = lane >> 3, r8 = lane & 7;
    bool ok = true;
    for (int i0 = 0; i0 < mine && ok; i0 += SK_PREFETCH) {
#pragma unroll
        for (int j = 0; j < SK_PREFETCH; ++j) {
            const int i = i0 + j;
            if (i >= mine || !ok) continue;
            const int u = warp + SK_WARPS * i;
            const int kb = u >> 2, ks = u & 3, s = kb % p.stages;
            if (!mbar_wait(&full[s], (kb / p.stages) & 1, p.status, 41)) {
                ok = false;
                continue;
            }
            FERRIS_TL_MARK(tl_mark && i == 0, 1);
            const uint32_t st = smem_u32(smem + (size_t)s * stage_bytes);
#pragma unroll
            for (int a = 0; a < ACCS; ++a) {
#pragma unroll
                for (int m = 0; m < SK_MAX_MT; ++m) {
                    if (m >= p.mt) continue;
                    // rows beyond the box (the last tile of a slab whose rows are no multiple of 16) read its last
                    // row again; their outputs are never written
                    const int row = min(m * 16 + (mi & 1) * 8 + r8, p.box_rows - 1);
                    uint32_t af[4];
                    ldmatrix_x4(af, st + a * box_bytes + swizzle128(row, ks * 2 + (mi >> 1)));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma_bf16_16816(acc[a][m][nt], af, breg[j][nt][0], breg[j][nt][1]);
                }
            }
            if (ring) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }
            if (i + SK_PREFETCH < mine) load_b(warp + SK_WARPS * (i + SK_PREFETCH), breg[j]);
        }
    }
    FERRIS_TL_MARK(tl_mark, 2);

    // The eight warps' partial tiles, added in warp order: [warp][accumulator, tile, token tile, element][lane].
    asm volatile("bar.sync 1, 256;" ::: "memory");  // nobody reads the stages any more
    float* red = reinterpret_cast<float*>(smem);
    const int per_acc = p.mt * NT * 4, per_warp = ACCS * per_acc;
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
    for (int q = threadIdx.x; q < per_acc * 32; q += SK_WARPS * 32) {
        const int ln = q & 31, e = q >> 5;
        const int j = e & 3, nt = (e >> 2) % NT, m = (e >> 2) / NT;
        const int row = m * 16 + (ln >> 2) + ((j & 2) ? 8 : 0);
        const int t = nt * 8 + (ln & 3) * 2 + (j & 1);
        const int n = n0 + row;
        if (row >= p.rows || n >= p.N || t >= p.T) continue;
        float va = 0.0f, vb = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
            va += red[(size_t)(w * per_warp + e) * 32 + ln];
            if (ACCS == 2) vb += red[(size_t)(w * per_warp + per_acc + e) * 32 + ln];
        }
        sk_write(p, t, n, va, vb);
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

// How a product is cut: rows per CTA, stages, shared memory.
struct SkPlan {
    int rows, box_rows, mt, ctas, kblocks, stages;
    size_t smem;
};

bool sk_plan(int T, int N, int K, int accs, SkPlan* out) {
    if (T < 1 || T > SK_MAX_TOKENS || N < 1 || K < 8 || (K & 7)) return false;
    const int sms = sk_sm_count();
    int rows = (N + sms - 1) / sms;
    if (rows > SK_MAX_ROWS) rows = SK_MAX_ROWS;
    const int ctas = (N + rows - 1) / rows;
    if (ctas > 2 * sms) return false;  // a product this tall (the output head) streams better through the tcgen05 kernel
    const int box_rows = (rows + 7) / 8 * 8;
    const int kblocks = (K + SK_BLOCK_K - 1) / SK_BLOCK_K;
    const int stage_bytes = accs * box_rows * 128;
    // One CTA per SM may take most of the shared memory, and still leave room for the slab of the next launch
    // where both are small; more CTAs than SMs keep to less than half, so that two share an SM.
    const int budget = ctas > sms ? 100 * 1024 : 176 * 1024;
    int stages = budget / stage_bytes;
    if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
    if (stages > kblocks) stages = kblocks;
    if (stages < 2 && kblocks > 1) return false;
    const int nt = T > 8 ? 2 : 1;
    const int mt = (rows + 15) / 16;
    const size_t red_bytes = (size_t)SK_WARPS * accs * mt * nt * 4 * 32 * sizeof(float);
    size_t smem = (size_t)stages * stage_bytes;
    if (smem < red_bytes) smem = red_bytes;
    *out = {rows, box_rows, mt, ctas, kblocks, stages, smem + 1024};
    return true;
}

template <int ACCS, int NT>
int sk_launch(const CUtensorMap& mw, const SkParams& p, int ctas, size_t smem, cudaStream_t s) {
    int rc = ferris_allow_dynamic_smem((const void*)gemm_skinny_kernel<ACCS, NT>, smem);
    if (rc != FERRIS_OK) return rc;
    cudaError_t e = ferris_launch(gemm_skinny_kernel<ACCS, NT>, dim3(ctas), dim3(SK_THREADS), smem, s, mw, p);
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

// 1 if ferris_gemm_skinny takes a product of these sizes (accumulators: 2 for SwiGLU, else 1).
FERRIS_API int ferris_gemm_skinny_takes(int T, int N, int K, int accumulators) {
    SkPlan plan;
    return (ferris_gemm_skinny_enabled() && sk_plan(T, N, K, accumulators == 2 ? 2 : 1, &plan)) ? 1 : 0;
}

// x: bf16 [T, K] rows ldx apart, or null with norm_h / norm_w / norm_eps: the rows are the RMSNorm of the fp32 rows
// norm_h [T, K] (contiguous).  w: bf16 [rows_w, K] rows ldw apart.  out: [T, N] rows ldo apart in the mode's type.
// mode: 0 bf16 = acc + bias; 1 fp32 = acc + bias; 2 fp32 += acc + bias; 3 bf16 = silu(x w[:N]^T) * (x w[up:up+N]^T).
FERRIS_API int ferris_gemm_skinny(const void* x, int ldx, const float* norm_h, const float* norm_w, float norm_eps,
                                  const void* w, const float* bias, void* out, int mode, int T, int N, int K, int ldw,
                                  int ldo, int rows_w, int up_row_offset, void* stream) {
    if (T <= 0 || N <= 0) return FERRIS_OK;
    if (mode < 0 || mode > 3) FERRIS_REFUSE("skinny gemm: unknown mode %d", mode);
    const int accs = mode == SK_SWIGLU_BF16 ? 2 : 1;
    SkPlan plan;
    if (!sk_plan(T, N, K, accs, &plan))
        FERRIS_REFUSE("skinny gemm: %d tokens x %d outputs x K=%d is not a shape it takes (at most %d tokens, K a "
                      "multiple of 8, at most %d rows)", T, N, K, SK_MAX_TOKENS, 2 * SK_MAX_ROWS * sk_sm_count());
    if ((ldw & 7) || ldw < K || ((uintptr_t)w & 15)) FERRIS_REFUSE("skinny gemm: weight rows must be 16-byte aligned");
    if (norm_h) {
        if (!norm_w || ((uintptr_t)norm_h & 15) || ((uintptr_t)norm_w & 15))
            FERRIS_REFUSE("skinny gemm: the rows to normalise and the norm's weight must be 16-byte aligned");
    } else {
        if (!x || (ldx & 1) || ldx < K || ((uintptr_t)x & 3)) FERRIS_REFUSE("skinny gemm: token rows must be 4-byte aligned");
    }
    if (mode == SK_SWIGLU_BF16 && (bias || up_row_offset + N > rows_w)) FERRIS_REFUSE("skinny gemm: bad SwiGLU operands");
    if (mode != SK_SWIGLU_BF16 && N > rows_w) FERRIS_REFUSE("skinny gemm: %d outputs from %d weight rows", N, rows_w);
    if (ldo < N) FERRIS_REFUSE("skinny gemm: output row stride %d < %d", ldo, N);
    CUtensorMap mw;
    int rc = ferris_make_tensor_map_2d(&mw, w, (uint64_t)rows_w, (uint64_t)K, (uint64_t)ldw, (uint32_t)plan.box_rows,
                                       SK_BLOCK_K);
    if (rc != FERRIS_OK) return rc;
    SkParams p;
    p.x = (const bf16*)x;
    p.norm_h = norm_h;
    p.norm_w = norm_w;
    p.norm_eps = norm_eps;
    p.out = out;
    p.bias = bias;
    p.ldx = ldx;
    p.T = T;
    p.N = N;
    p.K = K;
    p.ldo = ldo;
    p.rows = plan.rows;
    p.box_rows = plan.box_rows;
    p.mt = plan.mt;
    p.kblocks = plan.kblocks;
    p.stages = plan.stages;
    p.up_row_offset = up_row_offset;
    p.mode = mode;
    p.status = ferris_status_ptr();
    cudaStream_t s = (cudaStream_t)stream;
    if (accs == 2)
        return T > 8 ? sk_launch<2, 2>(mw, p, plan.ctas, plan.smem, s) : sk_launch<2, 1>(mw, p, plan.ctas, plan.smem, s);
    return T > 8 ? sk_launch<1, 2>(mw, p, plan.ctas, plan.smem, s) : sk_launch<1, 1>(mw, p, plan.ctas, plan.smem, s);
}

FERRIS_TIMELINE_TU(gemm_skinny)
