// Plain matrix product on CUDA cores: C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]),
// float32 accumulation with plain FFMA (no tensor-core mode of any precision).
//
// It is the matrix product of the 32-bit path, the LM head of the bfloat16 path
// when many rows are wanted at an odd shape, and the plain kernel beside the
// tensor-core products.  Every output element is the sum over k = 0..K-1 in that
// order, so a row of C does not depend on M, on N or on where the row sits in the
// batch.  Any M, N, K >= 1 and any leading dimensions are taken.
//
// Reference analogue: F.linear on [out, in] weights (servelab/parallel/
// tp_model.py:48-53,67-68,115-119).
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_tn_simt_kernel(
    const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw, TC* __restrict__ C,
    int ldc, const float* __restrict__ bias, int M, int N, int K) {
    __shared__ __align__(16) float As[GS_BK][GS_BM + 4];
    pdl_wait();
    __shared__ __align__(16) float Ws[GS_BK][GS_BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid >> 4, tx = tid & 15;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int row = idx >> 4, kk = idx & 15;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][row] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            C[(size_t)gm * ldc + gn] = from_float<TC>(acc[i][j] + (bias ? bias[gn] : 0.f));
        }
    }
}

template <typename TA, typename TW, typename TC>
static int launch_gemm(const TA* A, int lda, const TW* W, int ldw, TC* C, int ldc,
                       const float* bias, int M, int N, int K, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K || ldw < K || ldc < N) return SLB_ERR_BAD_ARG;
    const int gy = (M + GS_BM - 1) / GS_BM;
    if (gy > 65535) return SLB_ERR_TOO_LARGE;
    return slb_launch(gemm_tn_simt_kernel<TA, TW, TC>, dim3((N + GS_BN - 1) / GS_BN, gy), dim3(256),
                      0, st, A, lda, W, ldw, C, ldc, bias, M, N, K);
}

extern "C" {
int slb_gemm_simt_f32(const float* A, int lda, const float* W, int ldw, float* C, int ldc,
                      const float* bias, int M, int N, int K, cudaStream_t st) {
    return launch_gemm<float, float, float>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
}
int slb_gemm_simt_bf16(const bf16* A, int lda, const bf16* W, int ldw, bf16* C, int ldc,
                       const float* bias, int M, int N, int K, cudaStream_t st) {
    return launch_gemm<bf16, bf16, bf16>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
}
int slb_gemm_simt_bf16_f32out(const bf16* A, int lda, const bf16* W, int ldw, float* C, int ldc,
                              const float* bias, int M, int N, int K, cudaStream_t st) {
    return launch_gemm<bf16, bf16, float>(A, lda, W, ldw, C, ldc, bias, M, N, K, st);
}
}
