// The plain matrix product of the model:  C[M,N] (=|+=) A[M,K] * W[N,K]^T, both
// operands K-major as checkpoints store them, FMA on the CUDA cores in true 32-bit.
//
// It is the product of the 32-bit path of the whole model and the fallback of the
// bfloat16 path for operand types that the tensor-core kernels do not take (a weight
// kept in 32 bits beside 16-bit activations).  Each output element is one chain of
// FMAs over k = 0..K-1 in ascending order, whatever M is and wherever the element lies
// in a tile: a token's result does not depend on what else is in the batch.
// (The reference uses cublasGemmEx for M>1 and a split-K gemv pair for small M,
//  crates/cuda/src/gemm.rs:226-372, crates/cuda/kernels/gemm_m1.cu:63-235.)
#include "common.cuh"

#define RG_BM 64
#define RG_BN 64
#define RG_BK 16

// MODE 0: C = acc (type TO).  MODE 1: C(float) += acc.
template <typename TA, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_ref_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ C,
                int M, int N, int K, long long lda, long long ldw, long long ldc) {
    __shared__ float As[RG_BK][RG_BM + 4];
    __shared__ float Ws[RG_BK][RG_BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * RG_BM, n0 = blockIdx.x * RG_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += RG_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k fastest for coalescing
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int gk = k0 + kk;
            const int gm = m0 + r, gn = n0 + r;
            As[kk][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.0f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RG_BK; ++kk) {
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
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            TO* c = C + (size_t)gm * ldc + gn;
            if (MODE == 0) *c = from_f32<TO>(acc[i][j]);
            else *c = from_f32<TO>(to_f32(*c) + acc[i][j]);
        }
    }
}

template <typename TA, typename TW>
static int gemm_ref_dispatch(const void* A, const void* W, void* C, int c_dtype, int accumulate,
                             int M, int N, int K, long long lda, long long ldw, long long ldc, cudaStream_t s) {
    dim3 grid(rb_ceil_div(N, RG_BN), rb_ceil_div(M, RG_BM));
    if (accumulate) {
        if (c_dtype != RB_F32) RB_REFUSE("gemm: accumulation needs a float destination");
        gemm_ref_kernel<TA, TW, float, 1><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (float*)C, M, N, K, lda, ldw, ldc);
    } else if (c_dtype == RB_F32) {
        gemm_ref_kernel<TA, TW, float, 0><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (float*)C, M, N, K, lda, ldw, ldc);
    } else if (c_dtype == RB_BF16) {
        gemm_ref_kernel<TA, TW, bf16, 0><<<grid, 256, 0, s>>>((const TA*)A, (const TW*)W, (bf16*)C, M, N, K, lda, ldw, ldc);
    } else RB_REFUSE("gemm: destination dtype %d", c_dtype);
    return RB_LAUNCH_RESULT();
}

extern "C" int rb_gemm_ref(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                           int accumulate, int M, int N, int K, long long lda, long long ldw, long long ldc,
                           void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) RB_REFUSE("gemm: K=%d", K);
    if (M > 65535 * RG_BM) RB_REFUSE("gemm: M=%d exceeds the grid", M);
    cudaStream_t s = (cudaStream_t)stream;
    if (a_dtype == RB_F32 && w_dtype == RB_F32) return gemm_ref_dispatch<float, float>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, s);
    if (a_dtype == RB_F32 && w_dtype == RB_BF16) return gemm_ref_dispatch<float, bf16>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, s);
    if (a_dtype == RB_BF16 && w_dtype == RB_F32) return gemm_ref_dispatch<bf16, float>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, s);
    if (a_dtype == RB_BF16 && w_dtype == RB_BF16) return gemm_ref_dispatch<bf16, bf16>(A, W, C, c_dtype, accumulate, M, N, K, lda, ldw, ldc, s);
    RB_REFUSE("gemm: operand dtypes %d, %d", a_dtype, w_dtype);
}
