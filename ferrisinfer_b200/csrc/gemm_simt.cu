// Plain matrix product on the CUDA cores: out[t, n] = sum_k x[t, k] * w[n, k] (+ bias[n]).
// Every product and sum is an fp32 FMA (no tensor cores, no TF32, no reduced-precision staging),
// and each output accumulates over k in ascending order whatever the number of rows, so a row's
// result does not depend on what else is in the batch.  This is the matrix product of the 32-bit
// path, and the checked fallback for shapes the tensor-core kernel refuses.
//
// The weight keeps the layout of the model folder, [out features, in features]; the reference
// transposes at load and computes out[n] += x[k] * W[k, n] over ascending k
// (crates/ferrisinfer-kernel/src/cpu/matmul.rs:437-446), which is the same sum.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// MODE 0: out = acc (+bias), stored as TOut.  MODE 1: out(float) += acc (+bias).
template <typename TIn, typename TOut, int MODE>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TIn* x, const TIn* __restrict__ w,
                                                        const float* __restrict__ bias, TOut* __restrict__ out,
                                                        int M, int N, int K, int ldx, int ldw, int ldo) {
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = tid / 16, tc = tid % 16;  // this thread's 4x4 patch: rows tr*4.., cols tc*4..
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int m = m0 + lrow, n = n0 + lrow;
            xs[lk + q][lrow] = (m < M && k < K) ? to_float(x[(size_t)m * ldx + k]) : 0.0f;
            ws[lk + q][lrow] = (n < N && k < K) ? to_float(w[(size_t)n * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + tr * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tc * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            TOut* o = out + (size_t)m * ldo + n;
            if (MODE == 1)
                *o = from_float<TOut>(to_float(*o) + v);
            else
                *o = from_float<TOut>(v);
        }
    }
}

template <typename TIn, typename TOut>
int launch(const void* x, const void* w, const float* bias, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
           int accumulate, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (accumulate)
        ferris_launch(gemm_simt_kernel<TIn, TOut, 1>, grid, dim3(256), 0, s, (const TIn*)x, (const TIn*)w, bias, (TOut*)out, M, N, K,
                                                           ldx, ldw, ldo);
    else
        ferris_launch(gemm_simt_kernel<TIn, TOut, 0>, grid, dim3(256), 0, s, (const TIn*)x, (const TIn*)w, bias, (TOut*)out, M, N, K,
                                                           ldx, ldw, ldo);
    FERRIS_LAUNCH_CHECK();
}

}  // namespace

// x: [M, K] rows ldx apart; w: [N, K] rows ldw apart; out: [M, N] rows ldo apart.
// in_dtype is the type of x and w; out_dtype that of out; accumulate != 0 needs an fp32 out.
FERRIS_API int ferris_gemm_simt(const void* x, const void* w, const float* bias, void* out, int in_dtype,
                                int out_dtype, int M, int N, int K, int ldx, int ldw, int ldo, int accumulate,
                                void* stream) {
    if (M <= 0 || N <= 0) return FERRIS_OK;
    if (K <= 0) FERRIS_REFUSE("gemm: K=%d", K);
    if (ldx < K || ldw < K || ldo < N) FERRIS_REFUSE("gemm: row strides %d %d %d too small", ldx, ldw, ldo);
    if (accumulate && out_dtype != FERRIS_F32) FERRIS_REFUSE("gemm: accumulation needs an fp32 output");
    if ((M + BM - 1) / BM > 65535) FERRIS_REFUSE("gemm: %d rows are more than one launch takes", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == FERRIS_F32 && out_dtype == FERRIS_F32)
        return launch<float, float>(x, w, bias, out, M, N, K, ldx, ldw, ldo, accumulate, s);
    if (in_dtype == FERRIS_BF16 && out_dtype == FERRIS_F32)
        return launch<bf16, float>(x, w, bias, out, M, N, K, ldx, ldw, ldo, accumulate, s);
    if (in_dtype == FERRIS_BF16 && out_dtype == FERRIS_BF16)
        return launch<bf16, bf16>(x, w, bias, out, M, N, K, ldx, ldw, ldo, accumulate, s);
    FERRIS_REFUSE("gemm: dtypes in=%d out=%d not supported", in_dtype, out_dtype);
}
