// C = act(A W^T + bias) + res1 + res2 on the CUDA cores, accumulating in true
// 32-bit (FFMA; no tensor-core or reduced-precision matrix mode).
//
// This is the matrix product of the float32 engine, and the product for operand
// type pairs the tensor-core kernel does not take (a matrix stored in 32-bit used
// with bfloat16 activations).  A: [M, K] row-major (row stride lda), W: [N, K]
// row-major, weight rows = outputs, QStream's matvec convention
// (include/qsf/kernels.h:53-58).  Each output element sums its K products in
// ascending k inside one thread, so a row's result does not depend on M or on
// which other rows are in the batch.  The sum is taken in two levels: runs of 256
// products in one accumulator, the runs' sums in a second one, so that the rounding
// error grows with sqrt(256) + sqrt(K / 256) instead of sqrt(K) (at K = 16384 a
// fifth of the single accumulator's error).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 each
constexpr int RUN_TILES = 16;                              // k-tiles per first-level run: 256 products

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
linear_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W,
                   const void* __restrict__ bias, int bias_dtype, int act,
                   const TA* __restrict__ res1, const TA* __restrict__ res2,
                   int M, int N, int K, size_t lda, size_t ldc, size_t ldr) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN], total[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) { acc[i][j] = 0.f; total[i][j] = 0.f; }

    int in_run = 0;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
        }
#pragma unroll
        for (int e = tid; e < BN * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gn = n0 + r, gk = k0 + c;
            Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        if (++in_run == RUN_TILES) {                         // a run is complete: on to the second level
            in_run = 0;
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) { total[i][j] += acc[i][j]; acc[i][j] = 0.f; }
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn >= N) continue;
            float v = total[i][j] + acc[i][j];
            if (bias) v += load_as_f32(bias, bias_dtype, gn);
            v = apply_activation(v, act);
            if (res1) v += to_f32(res1[(size_t)gm * ldr + gn]);
            if (res2) v += to_f32(res2[(size_t)gm * ldr + gn]);
            C[(size_t)gm * ldc + gn] = from_f32<TC>(v);
        }
    }
}

template <typename TA, typename TW, typename TC>
int launch(void* C, const void* A, const void* W, const void* bias, int bias_dtype, int act,
           const void* res1, const void* res2, int M, int N, int K, long long lda, long long ldc,
           long long ldr, cudaStream_t stream) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    linear_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>(
        (TC*)C, (const TA*)A, (const TW*)W, bias, bias_dtype, act, (const TA*)res1, (const TA*)res2,
        M, N, K, (size_t)lda, (size_t)ldc, (size_t)ldr);
    return qs_check_launch("linear_simt");
}

}  // namespace

// a_dtype: type of A, res1, res2.  c_dtype: type of C (a_dtype, or float32 for logits).
QS_API int qs_linear_simt(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype,
                          const void* bias, int bias_dtype, int act, const void* res1, const void* res2,
                          int M, int N, int K, long long lda, long long ldc, long long ldr,
                          cudaStream_t stream) {
    if (M == 0 || N == 0) return QS_OK;
    QS_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    QS_REQUIRE(lda >= K && ldc >= N, "linear: row strides lda=%lld ldc=%lld below K=%d N=%d", lda, ldc, K, N);
    QS_REQUIRE((M + BM - 1) / BM <= 65535, "linear: M=%d exceeds the grid", M);
#define GO(TA, TW, TC) return launch<TA, TW, TC>(C, A, W, bias, bias_dtype, act, res1, res2, M, N, K, lda, ldc, ldr, stream)
    typedef __nv_bfloat16 bf16;
    if (a_dtype == QS_F32 && w_dtype == QS_F32 && c_dtype == QS_F32) GO(float, float, float);
    if (a_dtype == QS_F32 && w_dtype == QS_BF16 && c_dtype == QS_F32) GO(float, bf16, float);
    if (a_dtype == QS_BF16 && w_dtype == QS_BF16 && c_dtype == QS_BF16) GO(bf16, bf16, bf16);
    if (a_dtype == QS_BF16 && w_dtype == QS_BF16 && c_dtype == QS_F32) GO(bf16, bf16, float);
    if (a_dtype == QS_BF16 && w_dtype == QS_F32 && c_dtype == QS_BF16) GO(bf16, float, bf16);
    if (a_dtype == QS_BF16 && w_dtype == QS_F32 && c_dtype == QS_F32) GO(bf16, float, float);
#undef GO
    return qs_fail(QS_ERR_INVALID_INPUT, "linear: unsupported types A=%d W=%d C=%d", a_dtype, w_dtype, c_dtype);
}
