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
// Every C element is accumulated in ascending k with fused multiply-adds (one chain per K tile;
// the small-problem kernel sums four K slices in a fixed order), the order of the reference's
// tiled CPU path (test/library/matrix/impl/cpu-matrix.h:196-212 under Reduce(k_dim, tk)); results
// differ from it only by fma-vs-(mul,add) rounding and K-tile reassociation.
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

// Kernel for problems too small to fill the machine with 128 x 128 tiles (the 512^3 correctness
// configuration is one): a CTA owns a 32 x 32 tile of C and its four warps each reduce one
// quarter of K on their own -- private shared-memory staging, no block barrier in the main loop,
// the next 16 columns of K prefetched into registers while the current ones are multiplied -- and
// the four partial tiles are summed through shared memory in a fixed order at the end, so the
// result is deterministic.  Per lane: a 4 x 8 register tile, 3 shared loads per 32 FMAs.
__global__ void __launch_bounds__(128)
gemm_f32_warpk_kernel(const float *__restrict__ A, int64_t lda, const float *__restrict__ B,
                      int64_t ldb, float *__restrict__ C, int64_t ldc, int M, int N, int K,
                      int accumulate, int vec_ok) {
    constexpr int BK = 16;
    __shared__ __align__(16) float As[4][BK][32 + 4];   // [warp][k][m]
    __shared__ __align__(16) float Bs[4][BK][32 + 4];   // [warp][k][n]
    __shared__ __align__(16) float Cs[4][32][32 + 4];   // partial tiles
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
    // this warp's slice of K, in whole BK chunks
    const int chunks = (K + BK - 1) / BK;
    const int per = (chunks + 3) / 4;
    const int c_begin = warp * per, c_end = min(chunks, c_begin + per);
    const int ty = lane >> 2, tx = lane & 3;   // 8 x 4 lanes: rows 4*ty.., cols 8*tx..
    const bool interior = vec_ok && m0 + 32 <= M && n0 + 32 <= N;

    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float4 pa[4], pb[4];   // prefetch registers: A row `lane`, 16 k; B row k = lane / 2, 16 n
    auto fetch = [&](int c) {
        const int k0 = c * BK;
        if (interior && k0 + BK <= K) {
            const float4 *ap = reinterpret_cast<const float4 *>(A + static_cast<int64_t>(m0 + lane) * lda + k0);
            const float4 *bp = reinterpret_cast<const float4 *>(
                B + static_cast<int64_t>(k0 + (lane >> 1)) * ldb + n0 + (lane & 1) * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                pa[q] = __ldg(ap + q);
                pb[q] = __ldg(bp + q);
            }
        } else {
            float ta[16], tb[16];
            const int gm = m0 + lane, gk = k0 + (lane >> 1), gn = n0 + (lane & 1) * 16;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                ta[q] = (gm < M && k0 + q < K) ? A[static_cast<int64_t>(gm) * lda + k0 + q] : 0.0f;
                tb[q] = (gk < K && gn + q < N) ? B[static_cast<int64_t>(gk) * ldb + gn + q] : 0.0f;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                pa[q] = make_float4(ta[4 * q], ta[4 * q + 1], ta[4 * q + 2], ta[4 * q + 3]);
                pb[q] = make_float4(tb[4 * q], tb[4 * q + 1], tb[4 * q + 2], tb[4 * q + 3]);
            }
        }
    };
    auto stage = [&]() {
        // A arrives row-wise (lane = m): store transposed so that 4 consecutive m are one LDS.128
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            As[warp][4 * q + 0][lane] = pa[q].x;
            As[warp][4 * q + 1][lane] = pa[q].y;
            As[warp][4 * q + 2][lane] = pa[q].z;
            As[warp][4 * q + 3][lane] = pa[q].w;
            *reinterpret_cast<float4 *>(&Bs[warp][lane >> 1][(lane & 1) * 16 + 4 * q]) = pb[q];
        }
    };

    if (c_begin < c_end) fetch(c_begin);
    for (int c = c_begin; c < c_end; ++c) {
        __syncwarp();   // everyone is done reading the previous chunk
        stage();
        __syncwarp();
        if (c + 1 < c_end) fetch(c + 1);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4 *>(&As[warp][k][4 * ty]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[warp][k][8 * tx]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[warp][k][8 * tx + 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    // partial tiles -> shared memory, then a fixed-order sum of the four K slices
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        *reinterpret_cast<float4 *>(&Cs[warp][4 * ty + i][8 * tx]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4 *>(&Cs[warp][4 * ty + i][8 * tx + 4]) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * 32; e += 128) {
        const int r = e >> 5, cidx = e & 31;
        const int gm = m0 + r, gn = n0 + cidx;
        if (gm < M && gn < N) {
            const float sum = ((Cs[0][r][cidx] + Cs[1][r][cidx]) + Cs[2][r][cidx]) + Cs[3][r][cidx];
            float *dst = C + static_cast<int64_t>(gm) * ldc + gn;
            *dst = accumulate ? (*dst + sum) : sum;
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

int gemm_f32_tc_dispatch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                         float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                         cudaStream_t stream);

#ifndef GB200_GEMM_F32_TC_MIN_FLOP
#define GB200_GEMM_F32_TC_MIN_FLOP 6.0e8   // pre-pass path against the CUDA cores: 512^3 19.0 vs 24.8 us, 768^3 43.6 vs 34.7 us
#endif

int gemm_f32_fused_launch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                          int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate, cudaStream_t stream,
                          int cluster_hint = 0);

// The single-launch tensor-core kernel (gemm_f32_fused.cu) takes the middle: from cold L2 it measures
// 14.8 / 21.2 / 22.7 / 40.0 us at 512^3 / 640^3 / 768^3 / 1024^3 against 21.6 / 33.0 / 47.6 / 110 us
// for the CUDA-core kernels, 30 / 34 / 41 / 48 us for the three-launch tensor-core path and 20.1 /
// 25.1 / 28.0 / 51.2 us for cuBLAS with tf32 off; at 256^3 / 384^3 the CUDA-core kernel is faster
// (12.1 / 13.9 against 14.6 / 16.5 us), and from about 3 GFLOP (more than one round of its 128 x 64
// tiles, whose eight converting warps are bound by the fp32 -> bf16 conversions) the pre-passes pay.
#ifndef GB200_GEMM_F32_FUSED_MIN_FLOP
#define GB200_GEMM_F32_FUSED_MIN_FLOP 2.0e8
#endif
#ifndef GB200_GEMM_F32_FUSED_MAX_FLOP
#define GB200_GEMM_F32_FUSED_MAX_FLOP 3.0e9
#endif

// kernel_choice: 0 = pick, 1 = CUDA cores, 2 = tensor cores with split pre-passes (three launches),
// 3 = tensor cores with the split inside the kernel (one launch; a cluster per tile shares its K
// range when there are few tiles), 5 = the same without clusters.
int gemm_f32_dispatch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                      float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                      cudaStream_t stream, int kernel_choice = 0) {
    const bool tc_ok = ctx->encode_tiled != nullptr && K > 0;
    const double flop = 2.0 * (double)M * (double)N * (double)K;
    const bool tc_pays = flop >= GB200_GEMM_F32_TC_MIN_FLOP;
    // one round of 128 x 64 tiles at most, and not so few K chunks that the prologue dominates
    const int64_t fused_tiles = ((M + 127) / 128) * ((N + 63) / 64);
    const bool fused_pays = tc_ok && flop >= GB200_GEMM_F32_FUSED_MIN_FLOP && flop < GB200_GEMM_F32_FUSED_MAX_FLOP &&
                            fused_tiles <= ctx->sm_count && K >= 256;
    if (tc_ok && (kernel_choice == 2 || (kernel_choice == 0 && tc_pays && !fused_pays)))
        return gemm_f32_tc_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, accumulate, stream);
    if (K > 0 && (kernel_choice == 3 || kernel_choice == 5 || (kernel_choice == 0 && fused_pays)))
        return gemm_f32_fused_launch(ctx, A, lda, B, ldb, C, ldc, M, N, K, accumulate, stream,
                                     kernel_choice == 5 ? 1 : 0);
    const int64_t big_tiles = ((M + 127) / 128) * ((N + 127) / 128);
    const bool big = big_tiles >= 2 * (int64_t)ctx->sm_count;
    const int bm = big ? 128 : 32;
    const int vec_ok = (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(B) & 15) == 0 && lda % 4 == 0 && ldb % 4 == 0;
    // Row blocks sit in grid.y (at most 65535): a taller problem goes out as several launches over
    // consecutive row panels, which are independent.
    const int64_t panel = (int64_t)kMaxGridY * bm;
    for (int64_t m0 = 0; m0 < M; m0 += panel) {
        const int64_t mp = M - m0 < panel ? M - m0 : panel;
        const float *Ap = A + m0 * lda;
        float *Cp = C + m0 * ldc;
        if (big) {
            dim3 grid((unsigned)((N + 127) / 128), (unsigned)((mp + 127) / 128));
            gemm_f32_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, stream>>>(Ap, lda, B, ldb, Cp, ldc, (int)mp,
                                                                          (int)N, (int)K, accumulate);
        } else {
            dim3 grid((unsigned)((N + 31) / 32), (unsigned)((mp + 31) / 32));
            gemm_f32_warpk_kernel<<<grid, 128, 0, stream>>>(Ap, lda, B, ldb, Cp, ldc, (int)mp, (int)N,
                                                           (int)K, accumulate, vec_ok);
        }
        int rc = after_launch(ctx, "gemm_f32_kernel");
        if (rc) return rc;
    }
    return GB200_OK;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_gemm_f32(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                   float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                   void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, false);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_f32_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, accumulate,
                             static_cast<cudaStream_t>(stream));
}

// Test / benchmark hook: kernel chosen by the caller (1 = CUDA cores, 2 = tensor cores).
int gb200_gemm_f32_variant(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                           float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                           void *stream, int variant) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, false);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_f32_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, accumulate,
                             static_cast<cudaStream_t>(stream), variant);
}

int gb200_gemm_f32_host(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                        float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
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
    return host_finish(ctx, s, nullptr);
}

}  // extern "C"
