// Row-wise and element-wise kernels: token embedding gather, RMSNorm, SwiGLU, and the
// fused rotary-position + cache-write kernel.  All statistics, angles and products are fp32.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :], into the fp32 residual stream.
// Formula: crates/ferrisinfer-kernel/src/cpu/attention.rs:3-99 (a row copy; an id >= vocab is an error).
// An id outside [0, vocab) writes zeros and sets *status to 1 + the offending token index.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* ids,
                                    float* __restrict__ out, int hidden, int vocab, int* status) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * hidden;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, t + 1);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.0f;
    } else {
        const T* row = table + (size_t)id * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
    }
    FERRIS_TL_END(1);
}

FERRIS_API int ferris_embed_gather(const void* table, int dtype, const int* ids, float* out, int tokens,
                                   int hidden, int vocab, int* status, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (hidden <= 0 || vocab <= 0) FERRIS_REFUSE("embed_gather: hidden=%d vocab=%d", hidden, vocab);
    const int threads = hidden >= 1024 ? 256 : 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(embed_gather_kernel<float>, dim3(tokens), dim3(threads), 0, s, (const float*)table, ids, out, hidden, vocab, status);
    else if (dtype == FERRIS_BF16)
        ferris_launch(embed_gather_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (const bf16*)table, ids, out, hidden, vocab, status);
    else
        FERRIS_REFUSE("embed_gather: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm over rows of the fp32 residual stream:
//   ms = sum(x^2) / H;  r = 1 / sqrt(ms + eps);  y_j = (x_j * r) * w_j
// (crates/ferrisinfer-kernel/src/cpu/reduction.rs:35-41: eps inside the root, plain weight).
// With row_index, output row i is the norm of input row row_index[i] (used to norm only the
// rows whose logits are wanted).
// ---------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void rmsnorm_kernel(const float* x, const float* __restrict__ w,
                               const int* __restrict__ row_index, TOut* __restrict__ out, int hidden,
                               float eps) {
    __shared__ float scratch[33];
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int r = blockIdx.x;
    const int src = row_index ? row_index[r] : r;
    const float* xr = x + (size_t)src * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TOut* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<TOut>((xr[i] * inv) * w[i]);
    FERRIS_TL_END(2);
}

__device__ __forceinline__ void store4(float* o, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(o) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store4(bf16* o, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<uint32_t*>(&lo);
    v.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(o) = v;
}

// The same norm, one WARP per row: the row (up to 4096 floats, a multiple of 4) is read once with 16-byte loads
// and stays in registers between the sum of squares and the scaling.  For long steps.
template <typename TOut, int VEC>  // VEC float4 per lane: hidden <= 128 * VEC
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* x, const float* __restrict__ w,
                                                           const int* __restrict__ row_index, TOut* __restrict__ out,
                                                           int rows, int hidden, float eps) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;  // never the block's first thread, which ends the timeline record below
    const int src = row_index ? row_index[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
    const int n4 = hidden >> 2;
    float4 v[VEC];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < n4 ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TOut* o = out + (size_t)r * hidden;
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int i = lane + 32 * j;
        if (i < n4) {
            const float4 g = w4[i];
            store4(o + 4 * i, (v[j].x * inv) * g.x, (v[j].y * inv) * g.y, (v[j].z * inv) * g.z, (v[j].w * inv) * g.w);
        }
    }
    FERRIS_TL_END(6);
}

template <typename TOut>
static void launch_rmsnorm_rows(const float* x, const float* w, const int* row_index, TOut* out, int rows, int hidden,
                                float eps, cudaStream_t s) {
    const dim3 grid((rows + 7) / 8), block(256);
    if (hidden <= 1024)
        ferris_launch(rmsnorm_rows_kernel<TOut, 8>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
    else if (hidden <= 2048)
        ferris_launch(rmsnorm_rows_kernel<TOut, 16>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
    else
        ferris_launch(rmsnorm_rows_kernel<TOut, 32>, grid, block, 0, s, x, w, row_index, out, rows, hidden, eps);
}

FERRIS_API int ferris_rmsnorm(const float* x, const float* w, const int* row_index, void* out, int out_dtype,
                              int rows, int hidden, float eps, void* stream) {
    if (rows <= 0) return FERRIS_OK;
    if (hidden <= 0) FERRIS_REFUSE("rmsnorm: hidden=%d", hidden);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype != FERRIS_F32 && out_dtype != FERRIS_BF16) FERRIS_REFUSE("rmsnorm: unknown dtype %d", out_dtype);
    // A warp per row with the row in registers (16-byte loads, all of a row's in flight) wherever the row is aligned
    // and short enough; a block per row otherwise.  A warp per row also for few rows: the block's two barriers cost
    // more than seven more warps bring (decode step of 24 / 32 / 48 requests at the 0.5B sizes, two norm launches a
    // layer: 1.34 / 1.43 / 1.70 ms with a block per row below 64 rows, 1.28 / 1.37 / 1.65 ms with a warp per row).
    const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0;
    if (hidden % 4 == 0 && hidden <= 4096 && aligned) {
        if (out_dtype == FERRIS_F32)
            launch_rmsnorm_rows<float>(x, w, row_index, (float*)out, rows, hidden, eps, s);
        else
            launch_rmsnorm_rows<bf16>(x, w, row_index, (bf16*)out, rows, hidden, eps, s);
        FERRIS_LAUNCH_CHECK();
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (out_dtype == FERRIS_F32)
        ferris_launch(rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, s, x, w, row_index, (float*)out, hidden, eps);
    else
        ferris_launch(rmsnorm_kernel<bf16>, dim3(rows), dim3(threads), 0, s, x, w, row_index, (bf16*)out, hidden, eps);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: out[t, j] = silu(gate[t, j]) * up[t, j], silu(g) = g * 1 / (1 + exp(-g))
// (crates/ferrisinfer-kernel/src/cpu/elementwise.rs:189-190; crates/ferrisinfer-runtime/src/reference.rs:359-360).
// gate_up holds gate in columns [0, I) and up in [I, 2I) of each row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* gate_up, T* __restrict__ out, int tokens, int inter) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t n = (size_t)tokens * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter, j = i % inter;
        const float g = to_float(gate_up[t * 2 * inter + j]);
        const float u = to_float(gate_up[t * 2 * inter + inter + j]);
        const float sg = g * (1.0f / (1.0f + expf(-g)));
        out[i] = from_float<T>(u * sg);
    }
}

FERRIS_API int ferris_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (inter <= 0) FERRIS_REFUSE("swiglu: intermediate=%d", inter);
    const size_t n = (size_t)tokens * inter;
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, tokens, inter);
    else if (dtype == FERRIS_BF16)
        ferris_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(threads), 0, s, (const bf16*)gate_up, (bf16*)out, tokens, inter);
    else
        FERRIS_REFUSE("swiglu: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Rotary positions on q and k, and the write of k and v into the paged cache.
//   angle = float(pos) * inv_freq[i];  pairs (i, i + R/2), i < R/2 (rotate-half):
//   x_i' = x_i cos - x_{i+R/2} sin;  x_{i+R/2}' = x_{i+R/2} cos + x_i sin; dims >= R untouched
// (crates/ferrisinfer-kernel/src/cpu/attention.rs:1242-1292).  inv_freq is given by the host
// so that the engine and its plain reference agree on how the frequencies are formed.
//
// qkv: [T, (nh + 2 nkv) d] rows; q heads are rotated in place; k heads are rotated and stored
// to k_cache, v heads copied to v_cache, both laid out [page, kv head, slot in page, d].
// slot_mapping[t] = page * page_size + slot, or < 0 to write nothing for that token.
// With write_kv == 0 only q is rotated (a layer that reads another layer's cache).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const float* __restrict__ inv_freq, const int* __restrict__ slot_mapping,
                                        T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv, int d,
                                        int rotary, int page_size, int write_kv) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const int t = blockIdx.x;
    const int half = rotary / 2;
    const float pos = (float)positions[t];
    T* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0;
    const int in_page = slot >= 0 ? slot % page_size : 0;

    // rotate q and k heads: a thread takes a pair index and walks the heads, so that the sine and cosine of a
    // (token, pair) are formed once; with more threads than pairs, groups of threads share the heads
    const int rot_heads = nh + nkv;
    const int groups = half > 0 ? max(1, (int)blockDim.x / half) : 1;
    if (half > 0 && (int)threadIdx.x < groups * half) {
        const int i = threadIdx.x % half, g0 = threadIdx.x / half;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        for (int h = g0; h < rot_heads; h += groups) {
            T* x = row + (size_t)h * d;
            const float lo = to_float(x[i]), hi = to_float(x[i + half]);
            const T nlo = from_float<T>(lo * cs - hi * sn);
            const T nhi = from_float<T>(hi * cs + lo * sn);
            if (h < nh) {
                x[i] = nlo;
                x[i + half] = nhi;
            } else if (slot >= 0) {
                T* kc = k_cache + (((size_t)page * nkv + (h - nh)) * page_size + in_page) * d;
                kc[i] = nlo;
                kc[i + half] = nhi;
            }
        }
    }
    if (slot < 0) {
        FERRIS_TL_END(3);
        return;
    }
    // unrotated tail of k, and all of v
    const int tail = d - rotary;
    for (int w = threadIdx.x; w < nkv * tail; w += blockDim.x) {
        const int h = w / tail, i = rotary + w % tail;
        k_cache[(((size_t)page * nkv + h) * page_size + in_page) * d + i] = row[(size_t)(nh + h) * d + i];
    }
    for (int w = threadIdx.x; w < nkv * d; w += blockDim.x) {
        const int h = w / d, i = w % d;
        v_cache[(((size_t)page * nkv + h) * page_size + in_page) * d + i] = row[(size_t)(nh + nkv + h) * d + i];
    }
    FERRIS_TL_END(3);
}

FERRIS_API int ferris_rope_cache_write(void* qkv, int dtype, const int* positions, const float* inv_freq,
                                       const int* slot_mapping, void* k_cache, void* v_cache, int tokens, int nh,
                                       int nkv, int d, int rotary, int page_size, int write_kv, void* stream) {
    if (tokens <= 0) return FERRIS_OK;
    if (nh <= 0 || nkv <= 0 || d <= 0 || page_size <= 0)
        FERRIS_REFUSE("rope_cache_write: nh=%d nkv=%d d=%d page_size=%d", nh, nkv, d, page_size);
    if (rotary < 0 || rotary > d || (rotary & 1)) FERRIS_REFUSE("rope_cache_write: rotary dims %d of %d", rotary, d);
    if (rotary > 0 && !inv_freq) FERRIS_REFUSE("rope_cache_write: no frequency table");
    if (write_kv && (!slot_mapping || !k_cache || !v_cache)) FERRIS_REFUSE("rope_cache_write: no cache to write");
    const int threads = 128;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == FERRIS_F32)
        ferris_launch(rope_cache_write_kernel<float>, dim3(tokens), dim3(threads), 0, s, (float*)qkv, positions, inv_freq, slot_mapping,
                                                                  (float*)k_cache, (float*)v_cache, nh, nkv, d, rotary,
                                                                  page_size, write_kv);
    else if (dtype == FERRIS_BF16)
        ferris_launch(rope_cache_write_kernel<bf16>, dim3(tokens), dim3(threads), 0, s, (bf16*)qkv, positions, inv_freq, slot_mapping,
                                                                 (bf16*)k_cache, (bf16*)v_cache, nh, nkv, d, rotary,
                                                                 page_size, write_kv);
    else
        FERRIS_REFUSE("rope_cache_write: unknown dtype %d", dtype);
    FERRIS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// The rotation angles of a step, once for all layers that share the frequencies:
// out[t][i] = (cos, sin)(float(position[t]) * inv_freq[i]), the same fp32 expression as the kernel above.
// ---------------------------------------------------------------------------------------------
__global__ void rotary_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     float2* __restrict__ out, int tokens, int half) {
    FERRIS_TL_ENTRY();
    pdl_wait();
    pdl_launch_dependents();
    FERRIS_TL_BEGIN();
    const long long total = (long long)tokens * half;
    for (long long w = (long long)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(w / half), i = (int)(w % half);
        float sn, cs;
        sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
        out[w] = make_float2(cs, sn);
    }
    FERRIS_TL_END(9);
}

FERRIS_API int ferris_rotary_angles(const int* positions, const float* inv_freq, float* out, int tokens, int half,
                                    void* stream) {
    if (tokens <= 0 || half <= 0) return FERRIS_OK;
    const long long total = (long long)tokens * half;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 4096 ? (total + threads - 1) / threads : 4096);
    ferris_launch(rotary_angles_kernel, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, positions, inv_freq,
                  reinterpret_cast<float2*>(out), tokens, half);
    FERRIS_LAUNCH_CHECK();
}

FERRIS_TIMELINE_TU(elementwise)
