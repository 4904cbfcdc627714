// True 32-bit linear layer: y[M, N] = x[M, K] · w[N, K]^T (+ nothing), IEEE fp32 fused
// multiply-adds, no tensor cores, no TF32.
//
// Every output element is the sum over k = 0 .. K-1 in that order, whatever M is and wherever the
// row sits in the batch, so a token's result is bit-identical under every way of cutting the
// work.  This is the matrix product of the whole-model 32-bit path; it is not meant to be fast.
// Reference call site: crates/mrun-engine/src/load.rs:294-306 (`x · Wᵀ`, weights [out, in]).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__global__ void __launch_bounds__(256)
gemm_f32_nt_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M,
                   int N, int K, long ldx, long ldy) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int tr = (tid / 16) * TM, tc = (tid % 16) * TN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, k = e % BK;
            const int gr = row0 + r, gk = k0 + k;
            xs[k][r] = (gr < M && gk < K) ? x[(size_t)gr * ldx + gk] : 0.f;
            const int gc = col0 + r;
            ws[k][r] = (gc < N && gk < K) ? w[(size_t)gc * K + gk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[k][tr + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[k][tc + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gr = row0 + tr + i;
        if (gr >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gc = col0 + tc + j;
            if (gc < N) y[(size_t)gr * ldy + gc] = acc[i][j];
        }
    }
}

}  // namespace

// x rows are ldx floats apart, y rows ldy floats apart; w is dense [N, K].
MRUN_API int mrun_gemm_f32_nt(const float* x, const float* w, float* y, int M, int N, int K, long ldx,
                              long ldy, cudaStream_t stream) {
    MRUN_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32_nt: bad sizes M=%d N=%d K=%d", M, N, K);
    MRUN_REQUIRE(ldx >= K && ldy >= N, "gemm_f32_nt: row strides ldx=%ld ldy=%ld below K=%d N=%d", ldx, ldy,
                 K, N);
    if (M == 0) return 0;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    MRUN_REQUIRE(grid.y <= 65535, "gemm_f32_nt: M=%d exceeds the supported %d rows", M, 65535 * BM);
    gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(x, w, y, M, N, K, ldx, ldy);
    MRUN_CHECK_LAUNCH("gemm_f32_nt");
    return 0;
}
