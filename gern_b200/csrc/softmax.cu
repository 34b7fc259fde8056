// One-pass row softmax for sm_100a:  out(i,:) = exp(x - max) / sum(exp(x - max)).
//
// Fuses the five separately annotated Gern ops MaxRow, SubstractVec, ExpMatrix, SumRow and
// DivideVec (apps/common/annot/functions.h:9-173; device leaves apps/common/impl/impl.h:7-188,
// CPU twins test/library/matrix/impl/cpu-matrix.h:134-194) into a single read and a single
// write of the matrix.  The reference's leaves reduce a row across `stride` threads through
// shared memory with two block barriers per reduction (impl.h:80-188); here one warp owns one
// row, keeps it in registers as 128-bit vectors, and reduces with five xor-shuffles, so no
// barrier or shared memory is involved.  Rows longer than 1024 columns switch to a CTA per row
// (softmax_cta_kernel) so that a thread holds at most 8 vectors and many warps stay resident.
//
// Numerics: expf (not __expf), one correctly rounded reciprocal of the row sum and a multiply per
// element (within 2 ulp of the true quotient), fp32 throughout.  The reference's pieces as
// written are not a usable definition (its CPU subtract_vec computes max - x,
// cpu-matrix.h:178; max is seeded with FLT_MIN / 0, cpu-matrix.h:161, impl.h:144), so the
// mathematically stated form above is what is implemented.
#include <float.h>

#include "common.cuh"

namespace gb200 {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Warp-per-row kernel.  NV = float4 vectors per lane; covers cols <= 128 * NV, cols % 4 == 0,
// 16-byte aligned rows.  Rows are dealt to warps round-robin over a persistent grid.
template <int NV>
__global__ void __launch_bounds__(128)
softmax_warp_kernel(const float *__restrict__ in, int64_t ld_in, float *__restrict__ out,
                    int64_t ld_out, int64_t rows, int cols) {
    pdl_launch_dependents();   // launched with launch_pdl: see common.cuh
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int nvec = cols >> 2;  // vectors in a row

    for (int64_t row = warp; row < rows; row += n_warps) {
        const float4 *src = reinterpret_cast<const float4 *>(in + row * ld_in);
        float4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec)
                v[i] = __ldcs(src + idx);
            else
                v[i] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        }
        float m = -FLT_MAX;
#pragma unroll
        for (int i = 0; i < NV; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        m = warp_max(m);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec) {
                v[i].x = expf(v[i].x - m);
                v[i].y = expf(v[i].y - m);
                v[i].z = expf(v[i].z - m);
                v[i].w = expf(v[i].w - m);
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        }
        s = warp_sum(s);
        // one correctly rounded reciprocal per row, then multiplies: within 2 ulp of the quotient
        const float inv = 1.0f / s;
        float4 *dst = reinterpret_cast<float4 *>(out + row * ld_out);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + 32 * i;
            if (idx < nvec)
                __stcs(dst + idx, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
        }
    }
}

// CTA-per-row kernel for long rows: THREADS threads keep NV float4 each (cols <= 4*NV*THREADS),
// so a thread needs few registers and many warps are resident to cover HBM latency.  Row max
// and row sum go warp-shuffle -> shared memory -> every thread re-reduces the per-warp values
// (one block barrier per reduction; the scratch is double-buffered by row parity so no third
// barrier is needed).  Rows are dealt round-robin over a persistent grid.
template <int NV, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_cta_kernel(const float *__restrict__ in, int64_t ld_in, float *__restrict__ out,
                   int64_t ld_out, int64_t rows, int cols) {
    constexpr int NW = THREADS / 32;
    __shared__ float red_max[2][NW];
    __shared__ float red_sum[2][NW];
    pdl_launch_dependents();   // launched with launch_pdl: see common.cuh
    pdl_wait();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nvec = cols >> 2;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, parity ^= 1) {
        const float4 *src = reinterpret_cast<const float4 *>(in + row * ld_in);
        float4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + THREADS * i;
            if (idx < nvec)
                v[i] = __ldcs(src + idx);
            else
                v[i] = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        }
        float m = -FLT_MAX;
#pragma unroll
        for (int i = 0; i < NV; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        m = warp_max(m);
        if (lane == 0) red_max[parity][wid] = m;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < NW; ++w) m = fmaxf(m, red_max[parity][w]);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + THREADS * i;
            if (idx < nvec) {
                v[i].x = expf(v[i].x - m);
                v[i].y = expf(v[i].y - m);
                v[i].z = expf(v[i].z - m);
                v[i].w = expf(v[i].w - m);
                s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            }
        }
        s = warp_sum(s);
        if (lane == 0) red_sum[parity][wid] = s;
        __syncthreads();
        s = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; ++w) s += red_sum[parity][w];
        const float inv = 1.0f / s;   // see the warp kernel
        float4 *dst = reinterpret_cast<float4 *>(out + row * ld_out);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = threadIdx.x + THREADS * i;
            if (idx < nvec)
                __stcs(dst + idx, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
        }
    }
}

// Block-per-row kernel for everything else (any cols, any alignment): pass 1 finds the max,
// pass 2 the sum, pass 3 writes; passes 2 and 3 re-read the row (from L2 for rows that fit).
__global__ void __launch_bounds__(256)
softmax_block_kernel(const float *__restrict__ in, int64_t ld_in, float *__restrict__ out,
                     int64_t ld_out, int64_t rows, int64_t cols) {
    __shared__ float red[8];
    __shared__ float bcast;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float *src = in + row * ld_in;
        float *dst = out + row * ld_out;
        float m = -FLT_MAX;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, src[j]);
        m = warp_max(m);
        if (lane == 0) red[wid] = m;
        __syncthreads();
        if (wid == 0) {
            float t = lane < 8 ? red[lane] : -FLT_MAX;
            t = warp_max(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        m = bcast;
        float s = 0.0f;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) s += expf(src[j] - m);
        s = warp_sum(s);
        __syncthreads();
        if (lane == 0) red[wid] = s;
        __syncthreads();
        if (wid == 0) {
            float t = lane < 8 ? red[lane] : 0.0f;
            t = warp_sum(t);
            if (lane == 0) bcast = t;
        }
        __syncthreads();
        s = bcast;
        for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) dst[j] = expf(src[j] - m) / s;
        __syncthreads();
    }
}

template <int NV>
static int launch_warp(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out, int64_t ld_out,
                       int64_t rows, int64_t cols, cudaStream_t stream) {
    // 4 rows per CTA (one per warp), one CTA per 4 rows: see launch_cta for why not persistent.
    int64_t blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffll) blocks = 0x7fffffffll;
    GB200_CUDA_TRY(launch_pdl(softmax_warp_kernel<NV>, dim3((unsigned)blocks), dim3(128), 0, stream, in,
                              ld_in, out, ld_out, rows, (int)cols));
    return after_launch(ctx, "softmax_warp_kernel");
}

template <int NV, int THREADS>
static int launch_cta(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out, int64_t ld_out,
                      int64_t rows, int64_t cols, cudaStream_t stream) {
    // One row per CTA, not a persistent grid: the block scheduler refills an SM as soon as a row
    // is done, which keeps more loads in flight than CTAs that loop over rows (measured at
    // 65536 x 4096 with 16 / 32 / 64 / 128 looping CTAs per SM and with one CTA per row:
    // 6169 / 6435 / 6612 / 6722 / 6858 GB/s).  The loop in the kernel covers grids capped below.
    int64_t blocks = rows;
    if (blocks > 0x7fffffffll) blocks = 0x7fffffffll;
    if (blocks > rows) blocks = rows;
    GB200_CUDA_TRY(launch_pdl(softmax_cta_kernel<NV, THREADS>, dim3((unsigned)blocks), dim3(THREADS), 0,
                              stream, in, ld_in, out, ld_out, rows, (int)cols));
    return after_launch(ctx, "softmax_cta_kernel");
}

static int softmax_dispatch(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                            int64_t ld_out, int64_t rows, int64_t cols, cudaStream_t stream,
                            int variant = 0) {
    const bool vec = (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ld_in % 4 == 0 &&
                     ld_out % 4 == 0 && cols % 4 == 0 && cols <= 4096;
    const bool vec_ptr = (reinterpret_cast<uintptr_t>(in) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ld_in % 4 == 0 &&
                         ld_out % 4 == 0 && cols % 4 == 0;
    // variant 0 picks; 1 forces the warp-per-row kernel (cols <= 4096), 2..4 force a CTA shape.
    if (vec_ptr && variant == 2 && cols <= 4096)
        return launch_cta<4, 256>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
    if (vec_ptr && variant == 3 && cols <= 4096)
        return launch_cta<2, 512>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
    if (vec_ptr && variant != 1 && cols > 1024) {
        if (cols <= 4096) return launch_cta<8, 128>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 8192) return launch_cta<8, 256>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 16384) return launch_cta<8, 512>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 32768) return launch_cta<8, 1024>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
    }
    if (vec) {
        if (cols <= 128) return launch_warp<1>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 256) return launch_warp<2>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 512) return launch_warp<4>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 1024) return launch_warp<8>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        if (cols <= 2048) return launch_warp<16>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
        return launch_warp<32>(ctx, in, ld_in, out, ld_out, rows, cols, stream);
    }
    int64_t blocks = rows;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    softmax_block_kernel<<<(unsigned)blocks, 256, 0, stream>>>(in, ld_in, out, ld_out, rows, cols);
    return after_launch(ctx, "softmax_block_kernel");
}

static int check_softmax_args(const float *in, int64_t ld_in, float *out, int64_t ld_out,
                              int64_t rows, int64_t cols) {
    GB200_REQUIRE(rows >= 0 && cols >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    if (rows == 0 || cols == 0) return 1;
    GB200_REQUIRE(in != nullptr && out != nullptr, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(ld_in >= cols && ld_out >= cols, GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row");
    return GB200_OK;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_softmax_rows_f32(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                           int64_t ld_out, int64_t rows, int64_t cols, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_softmax_args(in, ld_in, out, ld_out, rows, cols);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return softmax_dispatch(ctx, in, ld_in, out, ld_out, rows, cols,
                            static_cast<cudaStream_t>(stream));
}

// Test / benchmark hook: same contract, kernel variant chosen by the caller.
int gb200_softmax_rows_f32_variant(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                                   int64_t ld_out, int64_t rows, int64_t cols, void *stream,
                                   int variant) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_softmax_args(in, ld_in, out, ld_out, rows, cols);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return softmax_dispatch(ctx, in, ld_in, out, ld_out, rows, cols,
                            static_cast<cudaStream_t>(stream), variant);
}

int gb200_softmax_rows_f32_host(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                                int64_t ld_out, int64_t rows, int64_t cols) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_softmax_args(in, ld_in, out, ld_out, rows, cols);
    if (rc) return rc < 0 ? rc : GB200_OK;
    const int64_t dld = (cols + 3) / 4 * 4;
    rc = stage_reserve(ctx, 0, (size_t)rows * dld * 4);
    if (rc) return rc;
    rc = stage_reserve(ctx, 1, (size_t)rows * dld * 4);
    if (rc) return rc;
    float *d_in = static_cast<float *>(ctx->stage[0]);
    float *d_out = static_cast<float *>(ctx->stage[1]);
    // Row chunks pipeline upload, kernel and download on two streams.
    const int n_chunks = rows >= 4096 ? 8 : 1;
    const int64_t per = (rows + n_chunks - 1) / n_chunks;
    cudaStream_t up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    for (int c = 0; c < n_chunks; ++c) {
        const int64_t r0 = c * per, r1 = (r0 + per < rows) ? r0 + per : rows;
        if (r0 >= r1) break;
        GB200_CUDA_TRY(cudaMemcpy2DAsync(d_in + r0 * dld, dld * 4, in + r0 * ld_in, ld_in * 4,
                                         cols * 4, r1 - r0, cudaMemcpyHostToDevice, up));
        GB200_CUDA_TRY(cudaEventRecord(ctx->ev[0], up));
        GB200_CUDA_TRY(cudaStreamWaitEvent(down, ctx->ev[0], 0));
        rc = softmax_dispatch(ctx, d_in + r0 * dld, dld, d_out + r0 * dld, dld, r1 - r0, cols,
                              down);
        if (rc) return rc;
        GB200_CUDA_TRY(cudaMemcpy2DAsync(out + r0 * ld_out, ld_out * 4, d_out + r0 * dld, dld * 4,
                                         cols * 4, r1 - r0, cudaMemcpyDeviceToHost, down));
    }
    return host_finish(ctx, down, up);
}

}  // extern "C"
