// Fused two-stage 3-tap box blur for sm_100a.
//
//   t(i,j)   = (in(i,j) + in(i,j+1) + in(i,j+2)) / 3        (apps/common/impl/impl.h:190-214)
//   out(i,j) = (t(i,j)  + t(i+1,j)  + t(i+2,j))  / 3        (apps/common/impl/impl.h:216-250)
//
// Both stages run in one kernel and the intermediate `t` lives in registers only.  The
// reference's emitted kernel (apps/blur/blur.cu:19-45) gathers a 6x12 patch per thread
// straight from global memory; here a CTA owns a column strip of the image, walks down it, and
// receives the input through a ring of TMA tiles in shared memory, so every input element is
// fetched from HBM once per strip and read from shared memory once.
//
// Arithmetic: the association (a+b+c) and a correctly rounded division by 3 are kept, so the
// result equals the reference's CPU loops (apps/blur/blur.cpp:11-25) under `==` for every finite
// input.  The division is done as q = x*(1/3); r = fma(-3,q,x); q' = fma(r,1/3,q), which is the
// correctly rounded x/3 for all finite floats (checked exhaustively on the host against `/`);
// the one difference is the sign of zero when x is -0.
#include "common.cuh"

namespace gb200 {

__device__ __forceinline__ float div3(float x) {
    const float rc = 0x1.555556p-2f;  // RN(1/3)
    float q = x * rc;
    float r = fmaf(-3.0f, q, x);
    return fmaf(r, rc, q);
}

// ---------------------------------------------------------------------------------------
// TMA kernel: strip width TW output columns, NT = TW/4 threads, ring of S stages of RS rows.
// ---------------------------------------------------------------------------------------
template <int TW, int RS, int S>
struct BlurTmaCfg {
    static_assert(TW % 256 == 0, "strip width is a whole number of 256-column TMA boxes");
    static constexpr int NT = TW / 4;
    static constexpr int NBOX = TW / 256;                 // a TMA box is at most 256 elements wide
    static constexpr int BOX_F = RS * 256;                // floats per main box
    static constexpr int PAD_F = RS * 4;                  // the 4 columns right of the strip
    static constexpr int TX_BYTES = (NBOX * BOX_F + PAD_F) * 4;   // bytes TMA delivers per stage
    static constexpr int STAGE_F = (NBOX * BOX_F + PAD_F + 31) / 32 * 32;  // 128-byte aligned stages
    static constexpr int STAGE_BYTES = STAGE_F * 4;
    static constexpr int SMEM_BYTES = S * STAGE_BYTES + S * 8 + 128;
};

template <int TW, int RS, int S>
__global__ void __launch_bounds__(TW / 4)
blur3x3_tma_kernel(const __grid_constant__ CUtensorMap in_map,
                   const __grid_constant__ CUtensorMap pad_map, float *__restrict__ out,
                   int64_t out_ld, int out_rows, int out_cols, int rows_per_band, int n_strips,
                   int out_vec, int *status) {
    using Cfg = BlurTmaCfg<TW, RS, S>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // The dynamic shared window is only guaranteed 16-byte aligned; TMA wants 128.
    unsigned char *base = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    float *stage = reinterpret_cast<float *>(base);
    uint64_t *full = reinterpret_cast<uint64_t *>(base + S * Cfg::STAGE_BYTES);

    const int tid = threadIdx.x;
    const int strip = blockIdx.x % n_strips;
    const int band = blockIdx.x / n_strips;
    const int x0 = strip * TW;
    const int r_begin = band * rows_per_band;                     // first output row
    const int r_end = min(r_begin + rows_per_band, out_rows);     // one past last output row
    if (r_begin >= r_end) return;                                 // uniform over the CTA
    const int in_rows_needed = r_end - r_begin + 2;
    const int n_chunks = (in_rows_needed + RS - 1) / RS;

    auto issue = [&](int chunk, int s) {
        float *dst = stage + s * Cfg::STAGE_F;
        const int y = r_begin + chunk * RS;
        mbar_expect_tx(&full[s], Cfg::TX_BYTES);
#pragma unroll
        for (int b = 0; b < Cfg::NBOX; ++b)
            tma_load_2d(dst + b * Cfg::BOX_F, &in_map, x0 + b * 256, y, &full[s]);
        tma_load_2d(dst + Cfg::NBOX * Cfg::BOX_F, &pad_map, x0 + TW, y, &full[s]);
    };

    if (tid == 0) {
        prefetch_tmap(&in_map);
        prefetch_tmap(&pad_map);
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
        const int pre = n_chunks < S ? n_chunks : S;
        for (int c = 0; c < pre; ++c) issue(c, c);
    }

    // Where this thread's 4 + 2 input columns sit inside a stage.
    const int box = tid / 64, lane64 = tid % 64;
    const int a_off = box * Cfg::BOX_F + lane64 * 4;      // row stride 256
    int b_off, b_stride;
    if (lane64 < 63) {
        b_off = a_off + 4;
        b_stride = 256;
    } else if (box + 1 < Cfg::NBOX) {
        b_off = (box + 1) * Cfg::BOX_F;
        b_stride = 256;
    } else {
        b_off = Cfg::NBOX * Cfg::BOX_F;
        b_stride = 4;
    }

    const int c0 = x0 + tid * 4;                 // first output column of this thread
    const int ncol = min(4, out_cols - c0);      // <= 0: nothing to store
    const bool vec_ok = (ncol == 4) && out_vec;  // 16-byte stores need an aligned output row
    float h0[4] = {0.f, 0.f, 0.f, 0.f}, h1[4] = {0.f, 0.f, 0.f, 0.f};
    bool alive = true;

    for (int c = 0; c < n_chunks; ++c) {
        const int s = c % S;
        const uint32_t parity = (c / S) & 1;
        if (alive && !mbar_wait(&full[s], parity, status, 101)) alive = false;
        const float *st = stage + s * Cfg::STAGE_F;
        const int rows_here = min(RS, in_rows_needed - c * RS);
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            if (r < rows_here) {
                const float4 a = *reinterpret_cast<const float4 *>(st + a_off + r * 256);
                const float2 b = *reinterpret_cast<const float2 *>(st + b_off + r * b_stride);
                float h[4];
                h[0] = div3(a.x + a.y + a.z);
                h[1] = div3(a.y + a.z + a.w);
                h[2] = div3(a.z + a.w + b.x);
                h[3] = div3(a.w + b.x + b.y);
                const int in_r = c * RS + r;     // row index inside this band's input window
                if (in_r >= 2 && ncol > 0) {
                    float o[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = div3(h0[k] + h1[k] + h[k]);
                    float *dst = out + static_cast<int64_t>(r_begin + in_r - 2) * out_ld + c0;
                    if (vec_ok) {
                        __stcs(reinterpret_cast<float4 *>(dst), make_float4(o[0], o[1], o[2], o[3]));
                    } else {
                        for (int k = 0; k < ncol; ++k) dst[k] = o[k];
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    h0[k] = h1[k];
                    h1[k] = h[k];
                }
            }
        }
        __syncthreads();  // every thread is done with stage s
        if (tid == 0 && c + S < n_chunks) issue(c + S, s);
    }
}

// ---------------------------------------------------------------------------------------
// Direct kernel: any shape, any alignment, and the row-band form whose last two input rows
// come from a separate `halo` pointer (possibly a peer GPU's memory; plain loads only).
// One thread owns VEC adjacent output columns and walks down `rows_per_thread` output rows
// with the two previous horizontal sums in registers.
// ---------------------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(128)
blur3x3_direct_kernel(const float *__restrict__ in, int64_t in_ld, int in_rows_local,
                      const float *__restrict__ halo, int64_t halo_ld, int in_cols,
                      float *__restrict__ out, int64_t out_ld, int out_row_begin, int out_row_end,
                      int rows_per_thread) {
    const int out_cols = in_cols - 2;
    const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c0 >= out_cols) return;
    const int r_begin = out_row_begin + blockIdx.y * rows_per_thread;
    const int r_end = min(r_begin + rows_per_thread, out_row_end);
    if (r_begin >= r_end) return;
    const int ncol = min(VEC, out_cols - c0);
    const bool full_vec = (VEC == 4) && (c0 + 6 <= in_cols);

    auto row_ptr = [&](int r) -> const float * {
        return r < in_rows_local ? in + static_cast<int64_t>(r) * in_ld
                                 : halo + static_cast<int64_t>(r - in_rows_local) * halo_ld;
    };
    auto hsum = [&](int r, float (&h)[VEC]) {
        const float *p = row_ptr(r) + c0;
        float v[VEC + 2];
        if (full_vec) {
            const float4 a = *reinterpret_cast<const float4 *>(p);
            const float2 b = *reinterpret_cast<const float2 *>(p + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            if (VEC == 4) { v[VEC] = b.x; v[VEC + 1] = b.y; }
        } else {
#pragma unroll
            for (int k = 0; k < VEC + 2; ++k) v[k] = (c0 + k < in_cols) ? p[k] : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) h[k] = div3(v[k] + v[k + 1] + v[k + 2]);
    };

    float h0[VEC], h1[VEC], h2[VEC];
    hsum(r_begin, h0);
    hsum(r_begin + 1, h1);
    for (int r = r_begin; r < r_end; ++r) {
        hsum(r + 2, h2);
        float o[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = div3(h0[k] + h1[k] + h2[k]);
        float *dst = out + static_cast<int64_t>(r) * out_ld + c0;
        if (VEC == 4 && ncol == 4) {
            *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[VEC - 1]);
        } else {
            for (int k = 0; k < ncol; ++k) dst[k] = o[k];
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            h0[k] = h1[k];
            h1[k] = h2[k];
        }
    }
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Launches the direct kernel over output rows [row_begin, row_end).
static int launch_direct(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows_local,
                         const float *halo, int64_t halo_ld, int64_t in_cols, float *out,
                         int64_t out_ld, int64_t row_begin, int64_t row_end, cudaStream_t stream) {
    if (row_end <= row_begin) return GB200_OK;
    const int64_t out_cols = in_cols - 2;
    const bool vec = aligned16(in) && aligned16(out) && in_ld % 4 == 0 && out_ld % 4 == 0 &&
                     (halo == nullptr || (aligned16(halo) && halo_ld % 4 == 0));
    const int rows_per_thread = 32;
    const int vecw = vec ? 4 : 1;
    dim3 block(128);
    dim3 grid((unsigned)((out_cols + vecw * 128 - 1) / (vecw * 128)),
              (unsigned)((row_end - row_begin + rows_per_thread - 1) / rows_per_thread));
    if (vec)
        blur3x3_direct_kernel<4><<<grid, block, 0, stream>>>(
            in, in_ld, (int)in_rows_local, halo, halo_ld, (int)in_cols, out, out_ld,
            (int)row_begin, (int)row_end, rows_per_thread);
    else
        blur3x3_direct_kernel<1><<<grid, block, 0, stream>>>(
            in, in_ld, (int)in_rows_local, halo, halo_ld, (int)in_cols, out, out_ld,
            (int)row_begin, (int)row_end, rows_per_thread);
    return after_launch(ctx, "blur3x3_direct_kernel");
}

template <int TW, int RS, int S>
static int launch_tma(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                      int64_t in_cols, float *out, int64_t out_ld, cudaStream_t stream) {
    using Cfg = BlurTmaCfg<TW, RS, S>;
    const int64_t out_rows = in_rows - 2, out_cols = in_cols - 2;
    CUtensorMap tm, tm_pad;
    int rc = get_tmap_2d(ctx, in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)in_cols,
                         (uint64_t)in_rows, (uint64_t)in_ld * 4, 256, RS,
                         CU_TENSOR_MAP_SWIZZLE_NONE, &tm);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)in_cols,
                     (uint64_t)in_rows, (uint64_t)in_ld * 4, 4, RS, CU_TENSOR_MAP_SWIZZLE_NONE,
                     &tm_pad);
    if (rc) return rc;
    const int n_strips = (int)((out_cols + TW - 1) / TW);
    // One wave of CTAs: as many row bands as fit the resident-CTA budget of the device.
    const int ctas_per_sm = (int)((ctx->smem_optin + 1024) / (Cfg::SMEM_BYTES + 1024));
    int64_t target = (int64_t)ctx->sm_count * (ctas_per_sm < 1 ? 1 : ctas_per_sm);
    int64_t bands = target / n_strips;
    if (bands < 1) bands = 1;
    int64_t rows_per_band = (out_rows + bands - 1) / bands;
    if (rows_per_band < 8) rows_per_band = 8;
    bands = (out_rows + rows_per_band - 1) / rows_per_band;
    auto kern = blur3x3_tma_kernel<TW, RS, S>;
    GB200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::SMEM_BYTES));
    kern<<<(unsigned)(bands * n_strips), Cfg::NT, Cfg::SMEM_BYTES, stream>>>(
        tm, tm_pad, out, out_ld, (int)out_rows, (int)out_cols, (int)rows_per_band, n_strips,
        (aligned16(out) && out_ld % 4 == 0) ? 1 : 0, ctx->d_status);
    return after_launch(ctx, "blur3x3_tma_kernel");
}

static int check_blur_args(const float *in, int64_t in_ld, int64_t in_rows, int64_t in_cols,
                           float *out, int64_t out_ld) {
    GB200_REQUIRE(in_rows >= 0 && in_cols >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    GB200_REQUIRE(in_rows < (1ll << 30) && in_cols < (1ll << 30), GB200_ERR_UNSUPPORTED,
                  "extent beyond 2^30");
    if (in_rows <= 2 || in_cols <= 2) return 1;  // empty output: nothing to do
    GB200_REQUIRE(in != nullptr && out != nullptr, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(in_ld >= in_cols && out_ld >= in_cols - 2, GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row (in_ld=%lld out_ld=%lld cols=%lld)",
                  (long long)in_ld, (long long)out_ld, (long long)in_cols);
    return GB200_OK;
}

// variant: 0 = pick (TMA when aligned), 1 = direct kernel only, 2.. = other TMA tilings.
// Exposed for benchmarking and for the parity tests of the non-default kernels.
int blur_dispatch(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows, int64_t in_cols,
                  float *out, int64_t out_ld, cudaStream_t stream, int variant) {
    const bool tma_ok = variant != 1 && ctx->encode_tiled && aligned16(in) && in_ld % 4 == 0 &&
                        in_cols >= 64 && in_rows >= 16;
    if (tma_ok) {
        switch (variant) {
            case 2: return launch_tma<512, 8, 3>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
            case 3: return launch_tma<256, 4, 8>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
            case 4: return launch_tma<256, 16, 3>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
            case 5: return launch_tma<512, 4, 6>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
            default: return launch_tma<256, 8, 4>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
        }
    }
    return launch_direct(ctx, in, in_ld, in_rows, nullptr, 0, in_cols, out, out_ld, 0, in_rows - 2,
                         stream);
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_blur3x3_f32(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                      int64_t in_cols, float *out, int64_t out_ld, void *stream) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_blur_args(in, in_ld, in_rows, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return blur_dispatch(ctx, in, in_ld, in_rows, in_cols, out, out_ld,
                         static_cast<cudaStream_t>(stream), 0);
}

// Test / benchmark hook: same contract, kernel variant chosen by the caller.
int gb200_blur3x3_f32_variant(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                              int64_t in_cols, float *out, int64_t out_ld, void *stream,
                              int variant) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_blur_args(in, in_ld, in_rows, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return blur_dispatch(ctx, in, in_ld, in_rows, in_cols, out, out_ld,
                         static_cast<cudaStream_t>(stream), variant);
}

int gb200_blur3x3_f32_band(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t band_rows,
                           int64_t in_cols, const float *halo, int64_t halo_ld, float *out,
                           int64_t out_ld, void *stream_) {
    int rc = enter(ctx);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (halo == nullptr)
        return gb200_blur3x3_f32(ctx, in, in_ld, band_rows, in_cols, out, out_ld, stream_);
    rc = check_blur_args(in, in_ld, band_rows + 2, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    GB200_REQUIRE(halo_ld >= in_cols, GB200_ERR_INVALID_ARG, "halo_ld smaller than the row");
    // Rows that need only this GPU's band go through the normal path; the last two output
    // rows read the halo and are produced by the direct kernel.
    const int64_t body_rows = band_rows - 2;  // output rows computable without the halo
    if (body_rows > 0) {
        rc = blur_dispatch(ctx, in, in_ld, band_rows, in_cols, out, out_ld, stream, 0);
        if (rc) return rc;
    }
    const int64_t tail_begin = body_rows > 0 ? body_rows : 0;
    return launch_direct(ctx, in, in_ld, band_rows, halo, halo_ld, in_cols, out, out_ld, tail_begin,
                         band_rows, stream);
}

int gb200_blur3x3_f32_host(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                           int64_t in_cols, float *out, int64_t out_ld) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_blur_args(in, in_ld, in_rows, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    const int64_t out_rows = in_rows - 2, out_cols = in_cols - 2;
    // Device images are packed with a pitch rounded up to 4 floats so that the TMA path applies.
    const int64_t d_in_ld = (in_cols + 3) / 4 * 4, d_out_ld = (out_cols + 3) / 4 * 4;
    rc = stage_reserve(ctx, 0, (size_t)in_rows * d_in_ld * 4);
    if (rc) return rc;
    rc = stage_reserve(ctx, 1, (size_t)out_rows * d_out_ld * 4);
    if (rc) return rc;
    float *d_in = static_cast<float *>(ctx->stage[0]);
    float *d_out = static_cast<float *>(ctx->stage[1]);
    // Row bands pipeline the three legs: band b's upload, kernel and download overlap with
    // its neighbours' on two streams (PCIe is full duplex).
    const int n_bands = out_rows >= 1024 ? 8 : 1;
    const int64_t rows_per = (out_rows + n_bands - 1) / n_bands;
    cudaStream_t up = ctx->copy_stream[0], down = ctx->copy_stream[1];
    int64_t uploaded = 0;  // input rows already enqueued for upload
    for (int b = 0; b < n_bands; ++b) {
        const int64_t r0 = b * rows_per;
        const int64_t r1 = (r0 + rows_per < out_rows) ? r0 + rows_per : out_rows;
        if (r0 >= r1) break;
        const int64_t need = r1 + 2;
        if (need > uploaded) {
            GB200_CUDA_TRY(cudaMemcpy2DAsync(d_in + uploaded * d_in_ld, d_in_ld * 4,
                                             in + uploaded * in_ld, in_ld * 4, in_cols * 4,
                                             need - uploaded, cudaMemcpyHostToDevice, up));
            uploaded = need;
        }
        GB200_CUDA_TRY(cudaEventRecord(ctx->ev[0], up));
        GB200_CUDA_TRY(cudaStreamWaitEvent(down, ctx->ev[0], 0));
        rc = blur_dispatch(ctx, d_in + r0 * d_in_ld, d_in_ld, r1 - r0 + 2, in_cols,
                           d_out + r0 * d_out_ld, d_out_ld, down, 0);
        if (rc) return rc;
        GB200_CUDA_TRY(cudaMemcpy2DAsync(out + r0 * out_ld, out_ld * 4, d_out + r0 * d_out_ld,
                                         d_out_ld * 4, out_cols * 4, r1 - r0,
                                         cudaMemcpyDeviceToHost, down));
    }
    GB200_CUDA_TRY(cudaStreamSynchronize(up));
    GB200_CUDA_TRY(cudaStreamSynchronize(down));
    return GB200_OK;
}

}  // extern "C"
