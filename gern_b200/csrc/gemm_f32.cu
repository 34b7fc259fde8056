// fp32 matrix multiply C (+)= A * B (row-major) on the CUDA cores.
//
// Stands where Gern's emitted "kernel_10" schedule stands (gernels/mm/kernel_10.cu:108-131,
// copy of the emitted code in gernels/mm/bench.cu:10-44): a block tile of C, A and B tiles
// staged through shared memory per K step, a register tile per thread, leaf
// matrix_multiply<k_dim> (gernels/mm/impl/matrix_multiply.h:50-61).  Differences by design:
// the C tile stays in registers for the whole K loop (the emitted kernel writes C back to
// global memory after every K tile, bench.cu:41), each thread owns a TM x TN register tile
// instead of one element, and edges are bounds-checked, so no divisibility is required.
//
// Every C element is accumulated by one thread in ascending k with fused multiply-adds, the
// same order as the reference's CPU leaf (test/library/matrix/impl/cpu-matrix.h:196-212);
// results differ from it only by fma-vs-(mul,add) rounding and K-tile reassociation.
// fp32 inputs stay on the fp32 pipe on purpose: tf32 tensor cores would drop 13 mantissa bits.
#include "common.cuh"

namespace gb200 {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_kernel(const float *__restrict__ A, int64_t lda, const float *__restrict__ B, int64_t ldb,
                float *__restrict__ C, int64_t ldc, int M, int N, int K, int accumulate) {
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];  // stored transposed: As[k][m]
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += NT) {
            const int m = e / BK, k = e % BK;
            const int gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < M && gk < K) ? A[static_cast<int64_t>(gm) * lda + gk] : 0.0f;
        }
        for (int e = tid; e < BK * BN; e += NT) {
            const int k = e / BN, n = e % BN;
            const int gk = k0 + k, gn = n0 + n;
            Bs[k][n] = (gk < K && gn < N) ? B[static_cast<int64_t>(gk) * ldb + gn] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
            float *c = C + static_cast<int64_t>(gm) * ldc + gn;
            *c = accumulate ? (*c + acc[i][j]) : acc[i][j];
        }
    }
}

int check_gemm_args(const void *A, int64_t lda, const void *B, int64_t ldb, void *C,
                           int64_t ldc, int64_t M, int64_t N, int64_t K, bool b_colmajor) {
    GB200_REQUIRE(M >= 0 && N >= 0 && K >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    GB200_REQUIRE(M < (1ll << 30) && N < (1ll << 30) && K < (1ll << 30), GB200_ERR_UNSUPPORTED,
                  "extent beyond 2^30");
    if (M == 0 || N == 0) return 1;
    GB200_REQUIRE(C != nullptr && (K == 0 || (A != nullptr && B != nullptr)),
                  GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(lda >= K && ldc >= N && ldb >= (b_colmajor ? K : N), GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                  (long long)lda, (long long)ldb, (long long)ldc);
    return GB200_OK;
}

int gemm_f32_dispatch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                      float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                      cudaStream_t stream) {
    const int64_t big_tiles = ((M + 127) / 128) * ((N + 127) / 128);
    if (big_tiles >= 2 * (int64_t)ctx->sm_count) {
        dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 127) / 128));
        gemm_f32_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, stream>>>(A, lda, B, ldb, C, ldc, (int)M,
                                                                      (int)N, (int)K, accumulate);
    } else {
        dim3 grid((unsigned)((N + 31) / 32), (unsigned)((M + 31) / 32));
        gemm_f32_kernel<32, 32, 32, 4, 4><<<grid, 64, 0, stream>>>(A, lda, B, ldb, C, ldc, (int)M,
                                                                   (int)N, (int)K, accumulate);
    }
    return after_launch(ctx, "gemm_f32_kernel");
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_gemm_f32(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                   float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                   void *stream) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, false);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_f32_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, accumulate,
                             static_cast<cudaStream_t>(stream));
}

int gb200_gemm_f32_host(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                        float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, false);
    if (rc) return rc < 0 ? rc : GB200_OK;
    rc = stage_reserve(ctx, 0, (size_t)M * K * 4 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 1, (size_t)K * N * 4 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 2, (size_t)M * N * 4);
    if (rc) return rc;
    float *dA = static_cast<float *>(ctx->stage[0]);
    float *dB = static_cast<float *>(ctx->stage[1]);
    float *dC = static_cast<float *>(ctx->stage[2]);
    cudaStream_t s = ctx->copy_stream[0];
    if (K > 0) {
        GB200_CUDA_TRY(cudaMemcpy2DAsync(dA, K * 4, A, lda * 4, K * 4, M, cudaMemcpyHostToDevice, s));
        GB200_CUDA_TRY(cudaMemcpy2DAsync(dB, N * 4, B, ldb * 4, N * 4, K, cudaMemcpyHostToDevice, s));
    }
    if (accumulate)
        GB200_CUDA_TRY(cudaMemcpy2DAsync(dC, N * 4, C, ldc * 4, N * 4, M, cudaMemcpyHostToDevice, s));
    rc = gemm_f32_dispatch(ctx, dA, K, dB, N, dC, N, M, N, K, accumulate, s);
    if (rc) return rc;
    GB200_CUDA_TRY(cudaMemcpy2DAsync(C, ldc * 4, dC, N * 4, N * 4, M, cudaMemcpyDeviceToHost, s));
    GB200_CUDA_TRY(cudaStreamSynchronize(s));
    return GB200_OK;
}

}  // extern "C"
