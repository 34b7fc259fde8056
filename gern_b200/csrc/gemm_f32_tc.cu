// fp32 matrix multiply on the tensor cores without giving up fp32 accuracy.
//
// The reference's matmul is fp32 (gernels/mm/impl/matrix_multiply.h:50-61; CPU twin
// test/library/matrix/impl/cpu-matrix.h:196-212).  tcgen05 has no fp32 input type, and its tf32
// kind keeps 10 mantissa bits, which misses the 1e-5 parity bar.  Instead every operand is written
// as a sum of three bf16 numbers, a = a1 + a2 + a3 with a1 = bf16(a), a2 = bf16(a - a1),
// a3 = bf16(a - a1 - a2), which together hold 24 mantissa bits, and the product is accumulated in
// fp32 in TMEM from the six partial products whose magnitude can matter,
//     a3 b1 + a2 b2 + a1 b3 + a2 b1 + a1 b2 + a1 b1          (smallest first),
// each of which is exact in fp32.  What is dropped (a2 b3, a3 b2, a3 b3) is below 2^-24 of the
// result.  One pre-pass per operand does the split (and turns the row-major B into the
// K-contiguous layout the MMA reads); the GEMM itself is the bf16 kernel of gemm_bf16.cu walking
// six segment pairs in its K loop and storing fp32.
#include "common.cuh"

namespace gb200 {

int gemm_f32x3_launch(gb200_ctx *ctx, const void *A3, const void *B3, float *C, int64_t ldc,
                      int64_t M, int64_t N, int64_t Kp, int accumulate, cudaStream_t stream);

__device__ __forceinline__ void split3(float v, __nv_bfloat16 &h1, __nv_bfloat16 &h2, __nv_bfloat16 &h3) {
    h1 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h1);       // exact
    h2 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h2);      // exact
    h3 = __float2bfloat16_rn(r2);
}

// A [rows][cols] fp32 (ld) -> out [rows][3 * Kp] bf16: segment s of a row holds term s + 1 of the
// row's elements, columns cols..Kp-1 of every segment are zero.  A thread converts 8 adjacent
// elements (two 128-bit loads when the row allows, three 128-bit stores).
__global__ void __launch_bounds__(256)
split_rows_kernel(const float *__restrict__ A, int64_t ld, int rows, int cols, int Kp,
                  __nv_bfloat16 *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = Kp / 8;
    const int64_t total = static_cast<int64_t>(rows) * groups;
    const bool vec = (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / groups;
        const int c = static_cast<int>(i - r * groups) * 8;
        float v[8];
        const float *src = A + r * ld + c;
        if (vec && c + 8 <= cols) {
            const float4 lo = __ldg(reinterpret_cast<const float4 *>(src));
            const float4 hi = __ldg(reinterpret_cast<const float4 *>(src + 4));
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
            v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = (c + k < cols) ? src[k] : 0.0f;
        }
        uint32_t w[3][4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __nv_bfloat16 a1, a2, a3, b1, b2, b3;
            split3(v[2 * k], a1, a2, a3);
            split3(v[2 * k + 1], b1, b2, b3);
            w[0][k] = __bfloat16_as_ushort(a1) | (static_cast<uint32_t>(__bfloat16_as_ushort(b1)) << 16);
            w[1][k] = __bfloat16_as_ushort(a2) | (static_cast<uint32_t>(__bfloat16_as_ushort(b2)) << 16);
            w[2][k] = __bfloat16_as_ushort(a3) | (static_cast<uint32_t>(__bfloat16_as_ushort(b3)) << 16);
        }
        __nv_bfloat16 *o = out + r * (3ll * Kp) + c;   // 16-byte aligned: Kp % 64 == 0, c % 8 == 0
#pragma unroll
        for (int sgm = 0; sgm < 3; ++sgm)
            *reinterpret_cast<uint4 *>(o + static_cast<int64_t>(sgm) * Kp) =
                make_uint4(w[sgm][0], w[sgm][1], w[sgm][2], w[sgm][3]);
    }
}

// B [K][N] fp32 row-major (ld) -> out [N][3 * Kp] bf16 (transposed, so that K is contiguous),
// through a 64 (k) x 32 (n) shared-memory tile: rows of B are read 128 bytes per warp, and each
// thread writes 8 adjacent k of one n as three 16-byte stores.  Rows K..Kp-1 of B count as zero.
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float *__restrict__ B, int64_t ld, int K, int N, int Kp,
                       __nv_bfloat16 *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float tile[64][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 32;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int k = k0 + ty + 8 * i, n = n0 + tx;
        tile[ty + 8 * i][tx] = (k < K && n < N) ? B[static_cast<int64_t>(k) * ld + n] : 0.0f;
    }
    __syncthreads();
    const int nl = threadIdx.x >> 3, kg = (threadIdx.x & 7) * 8;   // this thread: row n0 + nl, k0 + kg ..+7
    const int n = n0 + nl;
    if (n < N) {
        uint32_t w[3][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __nv_bfloat16 a1, a2, a3, b1, b2, b3;
            split3(tile[kg + 2 * j][nl], a1, a2, a3);
            split3(tile[kg + 2 * j + 1][nl], b1, b2, b3);
            w[0][j] = __bfloat16_as_ushort(a1) | (static_cast<uint32_t>(__bfloat16_as_ushort(b1)) << 16);
            w[1][j] = __bfloat16_as_ushort(a2) | (static_cast<uint32_t>(__bfloat16_as_ushort(b2)) << 16);
            w[2][j] = __bfloat16_as_ushort(a3) | (static_cast<uint32_t>(__bfloat16_as_ushort(b3)) << 16);
        }
        __nv_bfloat16 *o = out + static_cast<int64_t>(n) * (3ll * Kp) + k0 + kg;   // 16-byte aligned
#pragma unroll
        for (int sgm = 0; sgm < 3; ++sgm)
            *reinterpret_cast<uint4 *>(o + static_cast<int64_t>(sgm) * Kp) =
                make_uint4(w[sgm][0], w[sgm][1], w[sgm][2], w[sgm][3]);
    }
}

// C (+)= A B, fp32 row-major operands, on the tensor cores (see the head of this file).
int gemm_f32_tc_dispatch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                         float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                         cudaStream_t stream) {
    const int64_t Kp = (K + 63) / 64 * 64;
    GB200_REQUIRE(6 * Kp < (1ll << 31) && M < (1ll << 31) && N < (1ll << 31), GB200_ERR_UNSUPPORTED,
                  "fp32 matmul on the tensor cores: extent beyond 2^31 / 6");
    const size_t a_bytes = (size_t)M * 3 * Kp * 2, b_bytes = (size_t)N * 3 * Kp * 2;
    const size_t a_off = 0, b_off = (a_bytes + 255) / 256 * 256;
    int rc = workspace_reserve(ctx, b_off + b_bytes);
    if (rc) return rc;
    __nv_bfloat16 *A3 = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(ctx->workspace) + a_off);
    __nv_bfloat16 *B3 = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(ctx->workspace) + b_off);
    int64_t blocks = (M * (Kp / 8) + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 32) blocks = (int64_t)ctx->sm_count * 32;
    GB200_CUDA_TRY(launch_pdl(split_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, A, lda, (int)M,
                              (int)K, (int)Kp, A3));
    rc = after_launch(ctx, "split_rows_kernel");
    if (rc) return rc;
    dim3 grid((unsigned)((N + 31) / 32), (unsigned)(Kp / 64));
    GB200_CUDA_TRY(launch_pdl(split_transpose_kernel, grid, dim3(256), 0, stream, B, ldb, (int)K, (int)N,
                              (int)Kp, B3));
    rc = after_launch(ctx, "split_transpose_kernel");
    if (rc) return rc;
    return gemm_f32x3_launch(ctx, A3, B3, C, ldc, M, N, Kp, accumulate, stream);
}

}  // namespace gb200
