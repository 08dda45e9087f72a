// Plain matrix product C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the ordinary
// float32 units: no tensor cores, no reduced-precision mode.
//
// It is the linear layer of the true 32-bit path and the oracle for the
// tensor-core product.  Weights are [out, in] row-major and applied as x * W^T,
// as in the reference (crates/prelude-core/src/models/commons/linear.rs:48-77).
//
// Each output element is accumulated by one thread over k = 0 .. K-1 in
// ascending order with fused multiply-adds, so a row's result does not depend
// on the number of rows, on the row's place in the batch or on the tile it
// falls in.
#include "common.cuh"

#define GR_BM 64
#define GR_BN 64
#define GR_BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_ref_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                       const float* __restrict__ bias, TC* __restrict__ C, int M,
                                                       int N, int K, long long lda, long long ldw, long long ldc) {
    pb_grid_dep_launch();
    pb_grid_dep_wait();
    __shared__ float As[GR_BK][GR_BM + 1];
    __shared__ float Ws[GR_BK][GR_BN + 1];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * GR_BM, n0 = blockIdx.x * GR_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GR_BK) {
        // 64 x 16 elements per operand, 256 threads: 4 each
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            int idx = tid + r * 256;
            int row = idx / GR_BK, kk = idx % GR_BK;
            int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? pb_ld(A + (size_t)gm * lda + gk) : 0.f;
            Ws[kk][row] = (gn < N && gk < K) ? pb_ld(W + (size_t)gn * ldw + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GR_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += bias[gn];
            pb_st(C + (size_t)gm * ldc + gn, v);
        }
    }
}

// in_dtype: type of A and W; out_dtype: type of C; bias float32 or null.
// lda/ldw/ldc are row strides in elements.
PB_API int pb_gemm_ref(const void* A, const void* W, const float* bias, void* C, int in_dtype, int out_dtype, int M,
                       int N, int K, long long lda, long long ldw, long long ldc, cudaStream_t stream) {
    PB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_ref: bad sizes M=%d N=%d K=%d", M, N, K);
    PB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_ref: a row stride is shorter than its row");
    PB_REQUIRE(A && W && C, "gemm_ref: null pointer");
    if (M == 0) return 0;
    dim3 grid((N + GR_BN - 1) / GR_BN, (M + GR_BM - 1) / GR_BM);
    PB_REQUIRE(grid.y < 65536, "gemm_ref: M=%d too large", M);
    if (in_dtype == PB_F32 && out_dtype == PB_F32)
        pb_launch(gemm_ref_kernel<float, float, float>, dim3(grid), dim3(256), 0, stream, (const float*)A, (const float*)W, bias,
                                                                      (float*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == PB_BF16 && out_dtype == PB_BF16)
        pb_launch(gemm_ref_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, dim3(grid), dim3(256), 0, stream, 
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (__nv_bfloat16*)C, M, N, K, lda, ldw, ldc);
    else if (in_dtype == PB_BF16 && out_dtype == PB_F32)
        pb_launch(gemm_ref_kernel<__nv_bfloat16, __nv_bfloat16, float>, dim3(grid), dim3(256), 0, stream, 
            (const __nv_bfloat16*)A, (const __nv_bfloat16*)W, bias, (float*)C, M, N, K, lda, ldw, ldc);
    else
        return pb_fail("gemm_ref: unsupported types in=%d out=%d", in_dtype, out_dtype);
    PB_CHECK_LAUNCH("gemm_ref");
    return 0;
}
