// True 32-bit matrix product C[M,N] = A[M,K] * W[N,K]^T with plain FFMA: no
// tensor core, no TF32, no library. Each output element is summed over k in
// ascending order by one thread, so the value of C[m,n] depends on row m of A
// and row n of W only, never on M or on the other rows of the batch.
// W may be stored in float32 or in bfloat16 (widened exactly on load).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TW>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const TW* __restrict__ W, float* __restrict__ C, int M,
                int N, int K) {
    pdl_wait();      // nothing of this kernel touches global memory before this
    pdl_trigger();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64x16 tile of each operand, 4 elements a thread, k fastest in memory.
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = threadIdx.x + i * 256;  // 0..1023
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.0f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
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
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j];
        }
    }
}

LUMEN_API int lumen_gemm_f32(const float* A, const void* W, int w_is_bf16, float* C, int M, int N,
                             int K, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return LUMEN_ERR_BAD_ARGUMENT;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return LUMEN_ERR_UNSUPPORTED;
    if (w_is_bf16)
        lumen_launch(gemm_f32_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, A, (const __nv_bfloat16*)W, C, M, N, K);
    else
        lumen_launch(gemm_f32_kernel<float>, dim3(grid), dim3(256), 0, stream, A, (const float*)W, C, M, N, K);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
