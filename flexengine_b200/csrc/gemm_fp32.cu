// C[M,N] = A[M,K] . W[N,K]^T (+ bias[N]) in true float32 on CUDA cores: no tensor cores, no
// reduced-precision mode.  Every output element is one chain of fused multiply-adds over
// k = 0..K-1 in ascending order, so a row's result does not depend on how many rows are in
// the batch.  The reference runs these products through nn.Linear in float32
// (inference/models/qwen2.py:99-101,129-130,135 with dtype float32).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_fp32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                 float* __restrict__ C, int M, int N, int K) {
    fe::griddep_wait();
    fe::griddep_launch_dependents();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; ++i) {
            const int idx = tid + i * 256;
            const int row = idx / BK, col = idx % BK;
            const int gm = m0 + row, gn = n0 + row, gk = k0 + col;
            As[col][row] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.f;
            Ws[col][row] = (gn < N && gk < K) ? W[(size_t)gn * K + gk] : 0.f;
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
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)gm * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
        }
    }
}

}  // namespace

extern "C" int fe_gemm_fp32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                            cudaStream_t stream) {
    FE_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_fp32: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return 0;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    FE_REQUIRE(grid.y <= 65535, "gemm_fp32: too many rows (%d)", M);
    fe::launch(gemm_fp32_kernel, grid, 256, 0, stream, A, W, bias, C, M, N, K);
    return fe_check_launch("gemm_fp32");
}
