// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores with float32 multiply-adds
// (never a reduced-precision tensor mode).  This is the matrix product of the
// 32-bit path and the plain twin of the tensor-core kernels of the bfloat16
// path.  Each output is one dot product accumulated along K in index order, so
// a row's result depends neither on the other rows nor on M.
//
// GATED: W holds 2N rows, gate rows first and up rows after them; the output is
// silu(A*gate^T) * (A*up^T)  (wick src/model.rs:493-501, src/kernels.rs:374-378).
#include "common.cuh"

namespace wick {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename T, typename TOut, bool GATED>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const T* __restrict__ A, const T* __restrict__ W, TOut* __restrict__ C, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Us[GATED ? BK : 1][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid / 4, lk = (tid % 4) * 4;

    float acc[TM][TN] = {};
    float accu[GATED ? TM : 1][TN] = {};

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int m = m0 + lrow, n = n0 + lrow;
            As[lk + i][lrow] = (m < M && k < K) ? ld(A + (int64_t)m * K + k) : 0.f;
            Ws[lk + i][lrow] = (n < N && k < K) ? ld(W + (int64_t)n * K + k) : 0.f;
            if (GATED) Us[lk + i][lrow] = (n < N && k < K) ? ld(W + ((int64_t)N + n) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN], u[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
            if (GATED) {
#pragma unroll
                for (int j = 0; j < TN; ++j) u[j] = Us[kk][tx * TN + j];
            }
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (GATED) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * accu[i][j];
            st(C + (int64_t)m * N + n, v);
        }
    }
}

template <typename T, typename TOut, bool GATED>
int gemm_nt(const void* A, const void* W, void* C, int M, int N, int K, cudaStream_t s) {
    WICK_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return 0;
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
    WICK_REQUIRE(grid.y <= 65535, "gemm: M=%d is beyond the grid limit", M);
    gemm_nt_kernel<T, TOut, GATED><<<grid, 256, 0, s>>>((const T*)A, (const T*)W, (TOut*)C, M, N, K);
    return check_launch("gemm_simt");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// Names: wick_gemm_simt_<in>_<out>[_gated].  A [M,K], W [N,K] ([2N,K] gated), C [M,N].
WICK_API int wick_gemm_simt_bf16_bf16(const void* A, const void* W, void* C, int M, int N, int K, void* s) {
    return gemm_nt<bf16, bf16, false>(A, W, C, M, N, K, (cudaStream_t)s);
}
WICK_API int wick_gemm_simt_bf16_f32(const void* A, const void* W, void* C, int M, int N, int K, void* s) {
    return gemm_nt<bf16, float, false>(A, W, C, M, N, K, (cudaStream_t)s);
}
WICK_API int wick_gemm_simt_f32_f32(const void* A, const void* W, void* C, int M, int N, int K, void* s) {
    return gemm_nt<float, float, false>(A, W, C, M, N, K, (cudaStream_t)s);
}
WICK_API int wick_gemm_simt_bf16_bf16_gated(const void* A, const void* W, void* C, int M, int N, int K, void* s) {
    return gemm_nt<bf16, bf16, true>(A, W, C, M, N, K, (cudaStream_t)s);
}
WICK_API int wick_gemm_simt_f32_f32_gated(const void* A, const void* W, void* C, int M, int N, int K, void* s) {
    return gemm_nt<float, float, true>(A, W, C, M, N, K, (cudaStream_t)s);
}
