// Fused two-stage 3-tap box blur for sm_100a.
//
//   t(i,j)   = (in(i,j) + in(i,j+1) + in(i,j+2)) / 3        (apps/common/impl/impl.h:190-214)
//   out(i,j) = (t(i,j)  + t(i+1,j)  + t(i+2,j))  / 3        (apps/common/impl/impl.h:216-250)
//
// Both stages run in one kernel and the intermediate `t` never reaches memory.  The reference's
// emitted kernel (apps/blur/blur.cu:19-45) gathers a 6x12 patch per thread straight from global
// memory.  Three kernels here:
//   blur3x3_reg_kernel    (default) short-lived blocks of 512 columns x ROWS output rows; a thread
//                         loads its patch with 128-bit and 64-bit loads and keeps both passes in
//                         registers; the 2-row overlap between vertical neighbours is an L2 hit;
//                         its band form reads two halo rows through a second pointer.
//   blur3x3_tma_kernel    (variant) a warp owns a column strip, walks down it and receives the
//                         input through a ring of TMA tiles in shared memory.
//   blur3x3_direct_kernel (generic) any alignment and leading dimension.
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

__device__ __forceinline__ uint64_t div3_2(uint64_t x) {
    const uint64_t rc = pk2(0x1.555556p-2f, 0x1.555556p-2f);
    const uint64_t m3 = pk2(-3.0f, -3.0f);
    const uint64_t q = mul2(x, rc);
    const uint64_t r = fma2(m3, q, x);
    return fma2(r, rc, q);
}
// Horizontal pass on 4 adjacent outputs: inputs a = in[c..c+3], b = in[c+4..c+5].
// h[k] = ((in[c+k] + in[c+k+1]) + in[c+k+2]) / 3, returned as two packed pairs.
__device__ __forceinline__ void hpass4(const float4 a, const float2 b, uint64_t &h01, uint64_t &h23) {
    const uint64_t a01 = pk2(a.x, a.y), a12 = pk2(a.y, a.z), a23 = pk2(a.z, a.w);
    const uint64_t a3b = pk2(a.w, b.x), b01 = pk2(b.x, b.y);
    h01 = div3_2(add2(add2(a01, a12), a23));
    h23 = div3_2(add2(add2(a23, a3b), b01));
}
// Vertical pass: ((t0 + t1) + t2) / 3 on a packed pair.
__device__ __forceinline__ uint64_t vpass2(uint64_t t0, uint64_t t1, uint64_t t2) {
    return div3_2(add2(add2(t0, t1), t2));
}
__device__ __forceinline__ void store4(float *dst, uint64_t o01, uint64_t o23, int ncol, bool vec) {
    if (vec) {
        *reinterpret_cast<ulonglong2 *>(dst) = make_ulonglong2(o01, o23);
    } else {
        float o[4];
        asm("mov.b64 {%0, %1}, %2;" : "=f"(o[0]), "=f"(o[1]) : "l"(o01));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(o[2]), "=f"(o[3]) : "l"(o23));
        for (int k = 0; k < ncol; ++k) dst[k] = o[k];
    }
}

// ---------------------------------------------------------------------------------------
// TMA-staged kernel: every warp owns a 128-column strip of a row band and runs its own ring of
// S stages of RS rows x 132 columns (one TMA box: the strip plus the 4 columns to its right)
// with private mbarriers, so no block-level barrier exists and warps drift freely.  The stencil
// runs on fp32x2 pairs, the output pointer is carried instead of recomputed, and whole chunks
// of interior lanes take a branch-free path.  With one wave of long-lived strips it is clearly
// slower on B200 than the register-staged kernel below (the strips spread the DRAM accesses over
// the whole image: 105 against 79 us at 8192^2); cut into 16 waves of strips about 10 rows tall it
// comes within 1.4 % (80.0 us).  It stays an alternative, not the default.
// ---------------------------------------------------------------------------------------
template <int RS, int S>
struct BlurWarpCfg {
    static constexpr int WARPS = 4;
    static constexpr int ROW_F = 132;                                 // 528 bytes per staged row
    static constexpr int TX_BYTES = RS * ROW_F * 4;
    static constexpr int STAGE_F = (RS * ROW_F + 31) / 32 * 32;      // stages start 128-byte aligned
    static constexpr int WARP_F = S * STAGE_F;
    static constexpr int SMEM_BYTES = WARPS * WARP_F * 4 + WARPS * S * 8 + 128;
};

template <int RS, int S>
__global__ void __launch_bounds__(128)
blur3x3_tma_kernel(const __grid_constant__ CUtensorMap in_map, float *__restrict__ out,
                         int64_t out_ld, int out_rows, int out_cols, int rows_per_band,
                         int n_strips, int n_items, int out_vec, int *status) {
    using Cfg = BlurWarpCfg<RS, S>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *base = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~static_cast<uintptr_t>(127));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *stage = reinterpret_cast<float *>(base) + warp * Cfg::WARP_F;
    uint64_t *full = reinterpret_cast<uint64_t *>(base + Cfg::WARPS * Cfg::WARP_F * 4) + warp * S;

    // launched with launch_pdl: nothing is read before the previous kernel of the stream is done
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.x * Cfg::WARPS + warp;
    if (item >= n_items) return;
    const int strip = item % n_strips;
    const int band = item / n_strips;
    const int x0 = strip * 128;
    const int r_begin = band * rows_per_band;
    const int r_end = min(r_begin + rows_per_band, out_rows);
    if (r_begin >= r_end) return;
    const int in_rows_needed = r_end - r_begin + 2;
    const int n_chunks = (in_rows_needed + RS - 1) / RS;

    if (lane == 0) {
        prefetch_tmap(&in_map);
        for (int s = 0; s < S; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
        const int pre = n_chunks < S ? n_chunks : S;
        for (int c = 0; c < pre; ++c) {
            mbar_expect_tx(&full[c], Cfg::TX_BYTES);
            tma_load_2d(stage + c * Cfg::STAGE_F, &in_map, x0, r_begin + c * RS, &full[c]);
        }
    }
    __syncwarp();

    const int c0 = x0 + lane * 4;
    const int ncol = min(4, out_cols - c0);
    const bool vec_ok = (ncol == 4) && out_vec;
    float *dst = out + static_cast<int64_t>(r_begin) * out_ld + c0;   // next output row
    uint64_t t0a = 0, t0b = 0, t1a = 0, t1b = 0;                      // two previous rows of t
    bool alive = true;

    for (int c = 0; c < n_chunks; ++c) {
        const int s = c % S;
        const uint32_t parity = (c / S) & 1;
        if (alive && !mbar_wait(&full[s], parity, status, 103)) alive = false;
        const float *st = stage + s * Cfg::STAGE_F + lane * 4;
        const int rows_here = min(RS, in_rows_needed - c * RS);
        if (c > 0 && rows_here == RS && vec_ok) {
            // interior chunk, interior lane: RS outputs, no predicates
#pragma unroll
            for (int r = 0; r < RS; ++r) {
                const float4 a = *reinterpret_cast<const float4 *>(st + r * Cfg::ROW_F);
                const float2 b = *reinterpret_cast<const float2 *>(st + r * Cfg::ROW_F + 4);
                uint64_t ta, tb;
                hpass4(a, b, ta, tb);
                *reinterpret_cast<ulonglong2 *>(dst) =
                    make_ulonglong2(vpass2(t0a, t1a, ta), vpass2(t0b, t1b, tb));
                dst += out_ld;
                t0a = t1a; t0b = t1b; t1a = ta; t1b = tb;
            }
        } else {
            for (int r = 0; r < rows_here; ++r) {
                const float4 a = *reinterpret_cast<const float4 *>(st + r * Cfg::ROW_F);
                const float2 b = *reinterpret_cast<const float2 *>(st + r * Cfg::ROW_F + 4);
                uint64_t ta, tb;
                hpass4(a, b, ta, tb);
                if (c * RS + r >= 2) {
                    if (ncol > 0) store4(dst, vpass2(t0a, t1a, ta), vpass2(t0b, t1b, tb), ncol, vec_ok);
                    dst += out_ld;
                }
                t0a = t1a; t0b = t1b; t1a = ta; t1b = tb;
            }
        }
        __syncwarp();  // every lane is done with stage s
        if (lane == 0 && c + S < n_chunks) {
            mbar_expect_tx(&full[s], Cfg::TX_BYTES);
            tma_load_2d(stage + s * Cfg::STAGE_F, &in_map, x0, r_begin + (c + S) * RS, &full[s]);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Register-staged kernel (the default) for images whose rows are 16-byte aligned: a block
// covers 512 columns x ROWS output rows; a thread loads its 6 x (ROWS+2) input patch with
// 128-bit + 64-bit loads, keeps the horizontal pass in registers and runs the stencil on fp32x2
// pairs.  Blocks are short-lived and scheduled row-major in many waves, so the set of rows in
// flight is a compact window that moves down the image: the 2-row overlap between vertically
// adjacent blocks is served by L2, and DRAM sees long sequential runs.  Same tile shape as the
// reference's emitted kernel (per-thread register patch, apps/blur/blur.cu:19-45), minus its
// redundant read of the output tile and with 4 columns per thread.
// ---------------------------------------------------------------------------------------
#ifndef GB200_BLUR_STCS
#define GB200_BLUR_STCS 0
#endif
#ifdef GB200_BLUR_TRACE
// Debug-only timeline (compiled out of the library), %globaltimer nanoseconds.  Thread 0 of the
// first block of the grid (with a halo: the block row that reads it) fills [0..3]: entry, previous
// kernel complete, loads returned, stores issued; thread 0 of the first block of the next block
// row fills [4..7]; [8] = latest "stores issued" over all blocks, [9] = earliest entry.
__device__ unsigned long long g_blur_trace[16];
__device__ __forceinline__ unsigned long long blur_now() { return global_timer_ns(); }
__device__ __forceinline__ unsigned long long blur_now_after(float v) {
    unsigned long long t;
    asm volatile("{\n\t.reg .f32 z;\n\tmov.f32 z, %1;\n\tmov.u64 %0, %%globaltimer;\n\t}" : "=l"(t) : "f"(v) : "memory");
    return t;
}
#endif
template <int ROWS>
__global__ void __launch_bounds__(128)
blur3x3_reg_kernel(const float *__restrict__ in, int64_t in_ld, int in_cols,
                   float *__restrict__ out, int64_t out_ld, int out_rows, int out_vec,
                   int in_rows_local, const float *__restrict__ halo, int64_t halo_ld,
                   const int *__restrict__ halo_flag, int halo_expect, int *status) {
    // Input rows >= in_rows_local are not in `in`: they are the rows of the next row band and
    // are read from `halo` (which may be a peer GPU's memory; ordinary loads only).  With
    // `halo_flag`, `halo` is a local slot that a copy engine fills: the blocks that read it wait
    // (bounded) until the flag holds `halo_expect`.
    const int out_cols = in_cols - 2;
    // one-dimensional grid (the y extent of a grid stops at 65535 block rows): column blocks
    // fastest, so that blocks in flight walk the image row-major
    const int nbx = (out_cols + 511) / 512;
    const int bx = blockIdx.x % nbx, by_lin = blockIdx.x / nbx, nby = gridDim.x / nbx;
    const int c0 = (bx * 128 + threadIdx.x) * 4;
#ifdef GB200_BLUR_TRACE
    const int trace_slot = (threadIdx.x == 0 && blockIdx.x == 0) ? 0 : (threadIdx.x == 0 && blockIdx.x == nbx) ? 4 : -1;
    const unsigned long long t_entry = blur_now();
    if (trace_slot >= 0) g_blur_trace[trace_slot] = t_entry;
#endif
    // Launched with programmatic stream serialisation: blocks may become resident while the
    // previous kernel of the stream drains; nothing is read before that kernel has completed.
    pdl_launch_dependents();
    pdl_wait();
#ifdef GB200_BLUR_TRACE
    if (trace_slot >= 0) g_blur_trace[trace_slot + 1] = blur_now();
#endif
    if (c0 >= out_cols) return;
    // With a halo the block rows run bottom-up, so that the few blocks that read the (possibly
    // remote, high-latency) halo rows start first and finish under the rest of the kernel.
    const int by = halo != nullptr ? (nby - 1 - by_lin) : by_lin;
    const int r_begin = by * ROWS;
    const int n_out = min(ROWS, out_rows - r_begin);
    const int ncol = min(4, out_cols - c0);
    const float *src = in + static_cast<int64_t>(r_begin) * in_ld + c0;
    float *dst = out + static_cast<int64_t>(r_begin) * out_ld + c0;
    const bool local = r_begin + n_out + 2 <= in_rows_local;   // uniform over the block
    if (!local && halo_flag != nullptr) wait_flag_equals(halo_flag, halo_expect, status, 320);
    // the block row that needs the halo takes the same vector path when the halo rows are
    // 16-byte aligned: all its loads, the remote ones included, are in flight at once
    const bool halo_vec = halo != nullptr && (reinterpret_cast<uintptr_t>(halo) & 15) == 0 && halo_ld % 4 == 0;
    if (n_out == ROWS && c0 + 6 <= in_cols && out_vec && (local || halo_vec)) {
        float4 a[ROWS + 2];
        float2 b[ROWS + 2];
        if (local) {
#pragma unroll
            for (int r = 0; r < ROWS + 2; ++r) {
                a[r] = __ldg(reinterpret_cast<const float4 *>(src + r * in_ld));
                b[r] = __ldg(reinterpret_cast<const float2 *>(src + r * in_ld + 4));
            }
        } else {
#pragma unroll
            for (int r = 0; r < ROWS + 2; ++r) {
                const int gr = r_begin + r;
                // plain loads: the halo may be another GPU's memory
                const float *rp = gr < in_rows_local
                                      ? src + r * in_ld
                                      : halo + static_cast<int64_t>(gr - in_rows_local) * halo_ld + c0;
                a[r] = *reinterpret_cast<const float4 *>(rp);
                b[r] = *reinterpret_cast<const float2 *>(rp + 4);
            }
        }
#ifdef GB200_BLUR_TRACE
        if (trace_slot >= 0) {
            float dep = 0.0f;
#pragma unroll
            for (int r = 0; r < ROWS + 2; ++r) dep += a[r].x + b[r].y;
            g_blur_trace[trace_slot + 2] = blur_now_after(dep);
        }
#endif
        uint64_t ta[ROWS + 2], tb[ROWS + 2];
#pragma unroll
        for (int r = 0; r < ROWS + 2; ++r) hpass4(a[r], b[r], ta[r], tb[r]);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const ulonglong2 o = make_ulonglong2(vpass2(ta[r], ta[r + 1], ta[r + 2]),
                                                 vpass2(tb[r], tb[r + 1], tb[r + 2]));
#if GB200_BLUR_STCS
            // the output is never read again: streaming stores leave L2 to the input rows
            __stcs(reinterpret_cast<float4 *>(dst + r * out_ld),
                   make_float4(__uint_as_float((uint32_t)o.x), __uint_as_float((uint32_t)(o.x >> 32)),
                               __uint_as_float((uint32_t)o.y), __uint_as_float((uint32_t)(o.y >> 32))));
#else
            *reinterpret_cast<ulonglong2 *>(dst + r * out_ld) = o;
#endif
        }
    } else {
        // ragged bottom or right edge, or output rows that are not 16-byte aligned
        uint64_t t0a = 0, t0b = 0, t1a = 0, t1b = 0;
        for (int r = 0; r < n_out + 2; ++r) {
            const int gr = r_begin + r;
            const float *rp = gr < in_rows_local
                                  ? src + r * in_ld
                                  : halo + static_cast<int64_t>(gr - in_rows_local) * halo_ld + c0;
            float v[6];
#pragma unroll
            for (int k = 0; k < 6; ++k) v[k] = (c0 + k < in_cols) ? rp[k] : 0.0f;
#ifdef GB200_BLUR_TRACE
            if (trace_slot >= 0 && r == n_out + 1) g_blur_trace[trace_slot + 2] = blur_now_after(v[0] + v[5]);
#endif
            uint64_t ta, tb;
            hpass4(make_float4(v[0], v[1], v[2], v[3]), make_float2(v[4], v[5]), ta, tb);
            if (r >= 2)
                store4(dst + (r - 2) * out_ld, vpass2(t0a, t1a, ta), vpass2(t0b, t1b, tb), ncol,
                       ncol == 4 && out_vec);
            t0a = t1a; t0b = t1b; t1a = ta; t1b = tb;
        }
    }
#ifdef GB200_BLUR_TRACE
    {
        const unsigned long long t_end = blur_now();
        if (trace_slot >= 0) g_blur_trace[trace_slot + 3] = t_end;
        if (threadIdx.x == 0 && (blockIdx.x & 63) == 0) atomicMax(&g_blur_trace[8], t_end);
    }
#endif
}

// ---------------------------------------------------------------------------------------
// Direct kernel: any shape, any alignment, and the row-band form whose last two input rows
// come from a separate `halo` pointer (possibly a peer GPU's memory; plain loads only).
// One thread owns VEC adjacent output columns and walks down `rows_per_thread` output rows
// with the two previous horizontal sums in registers.
// ---------------------------------------------------------------------------------------
template <int VEC, bool STCS = false>
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
            if (STCS)
                __stcs(reinterpret_cast<float4 *>(dst), make_float4(o[0], o[1], o[2], o[VEC - 1]));
            else
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
                         int64_t out_ld, int64_t row_begin, int64_t row_end, cudaStream_t stream,
                         int rows_per_thread = 32, bool stcs = false) {
    if (row_end <= row_begin) return GB200_OK;
    // row strips sit in grid.y (at most 65535): taller images get taller strips
    while ((row_end - row_begin + rows_per_thread - 1) / rows_per_thread > kMaxGridY) rows_per_thread *= 2;
    const int64_t out_cols = in_cols - 2;
    const bool vec = aligned16(in) && aligned16(out) && in_ld % 4 == 0 && out_ld % 4 == 0 &&
                     (halo == nullptr || (aligned16(halo) && halo_ld % 4 == 0));
    const int vecw = vec ? 4 : 1;
    dim3 block(128);
    dim3 grid((unsigned)((out_cols + vecw * 128 - 1) / (vecw * 128)),
              (unsigned)((row_end - row_begin + rows_per_thread - 1) / rows_per_thread));
    if (vec && stcs)
        blur3x3_direct_kernel<4, true><<<grid, block, 0, stream>>>(
            in, in_ld, (int)in_rows_local, halo, halo_ld, (int)in_cols, out, out_ld,
            (int)row_begin, (int)row_end, rows_per_thread);
    else if (vec)
        blur3x3_direct_kernel<4><<<grid, block, 0, stream>>>(
            in, in_ld, (int)in_rows_local, halo, halo_ld, (int)in_cols, out, out_ld,
            (int)row_begin, (int)row_end, rows_per_thread);
    else
        blur3x3_direct_kernel<1><<<grid, block, 0, stream>>>(
            in, in_ld, (int)in_rows_local, halo, halo_ld, (int)in_cols, out, out_ld,
            (int)row_begin, (int)row_end, rows_per_thread);
    return after_launch(ctx, "blur3x3_direct_kernel");
}

template <int RS, int S>
static int launch_tma(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                            int64_t in_cols, float *out, int64_t out_ld, cudaStream_t stream,
                            int waves = 1) {
    using Cfg = BlurWarpCfg<RS, S>;
    const int64_t out_rows = in_rows - 2, out_cols = in_cols - 2;
    CUtensorMap tm;
    int rc = get_tmap_2d(ctx, in, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)in_cols,
                         (uint64_t)in_rows, (uint64_t)in_ld * 4, Cfg::ROW_F, RS,
                         CU_TENSOR_MAP_SWIZZLE_NONE, &tm);
    if (rc) return rc;
    const int n_strips = (int)((out_cols + 127) / 128);
    int ctas_per_sm = (int)((ctx->smem_optin + 1024) / (Cfg::SMEM_BYTES + 1024));
    if (ctas_per_sm > 16) ctas_per_sm = 16;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    const int64_t target = (int64_t)ctx->sm_count * ctas_per_sm * Cfg::WARPS * waves;
    int64_t bands = target / n_strips;
    if (bands < 1) bands = 1;
    int64_t rows_per_band = (out_rows + bands - 1) / bands;
    if (rows_per_band < 8) rows_per_band = 8;
    bands = (out_rows + rows_per_band - 1) / rows_per_band;
    const int64_t n_items = bands * n_strips;
    auto kern = blur3x3_tma_kernel<RS, S>;
    {
        const int rc_attr = ensure_dynamic_smem(ctx, kern, Cfg::SMEM_BYTES);
        if (rc_attr) return rc_attr;
    }
    GB200_CUDA_TRY(launch_pdl(kern, dim3((unsigned)((n_items + Cfg::WARPS - 1) / Cfg::WARPS)), dim3(128),
                              (size_t)Cfg::SMEM_BYTES, stream, tm, out, out_ld, (int)out_rows, (int)out_cols,
                              (int)rows_per_band, n_strips, (int)n_items,
                              (aligned16(out) && out_ld % 4 == 0) ? 1 : 0, ctx->d_status));
    return after_launch(ctx, "blur3x3_tma_kernel");
}

// `in_rows` counts the halo rows too: in holds in_rows - (halo ? 2 : 0) rows.
// Halo rows on another device: a copy engine brings them into the next slot of the context's ring
// and then sets the slot's flag, on a stream of its own, so that the blur kernel itself reads
// local memory only.  (A grid that has read a peer's memory completes about 3 us later, measured,
// whatever it read; the kernels of a stream of dependent launches would each pay that.)  On return
// *slot_rows is the slot, *flag its flag and *expect the flag's value.
// The device that owns `p` if it is another device's memory, else -1 (this device's memory, or
// memory the driver does not know as device memory).
static int other_device_of(gb200_ctx *ctx, const void *p) {
    if (p == ctx->last_halo) return ctx->last_halo_device;   // a loop of steps asks about the same rows
    cudaPointerAttributes at;
    int dev = -1;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess)
        cudaGetLastError();
    else if (at.type == cudaMemoryTypeDevice && at.device != ctx->device)
        dev = at.device;
    ctx->last_halo = p;
    ctx->last_halo_device = dev;
    return dev;
}
// Whether kernels of the context's device may read device `dev`'s memory (peer access is switched
// on at the first question; memory mapped with its own access rights, such as symmetric memory,
// needs no more than that).
static bool peer_readable(gb200_ctx *ctx, int dev) {
    if (dev < 0 || dev >= 64) return false;
    if (ctx->peer_state[dev] == 0) {
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, ctx->device, dev) != cudaSuccess) cudaGetLastError();
        if (can) {
            const cudaError_t e = cudaDeviceEnablePeerAccess(dev, 0);
            if (e != cudaSuccess) cudaGetLastError();
            can = (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled);
        }
        ctx->peer_state[dev] = can ? 1 : -1;
    }
    return ctx->peer_state[dev] == 1;
}
static int halo_prefetch(gb200_ctx *ctx, const float *halo, int64_t halo_ld, int64_t in_cols,
                         const float **slot_rows, const int **flag, int *expect) {
    *slot_rows = nullptr;
    if (ctx->halo_stream == nullptr) {
        GB200_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->halo_stream, cudaStreamNonBlocking));
        GB200_CUDA_TRY(cudaMalloc(&ctx->halo_flags, kHaloSlots * sizeof(int)));
        GB200_CUDA_TRY(cudaMemset(ctx->halo_flags, 0, kHaloSlots * sizeof(int)));
        GB200_CUDA_TRY(cudaMallocHost(&ctx->halo_flag_values, 256 * sizeof(int)));
        for (int i = 0; i < 256; ++i) ctx->halo_flag_values[i] = i + 1;
        for (int i = 0; i < 4; ++i) GB200_CUDA_TRY(cudaEventCreateWithFlags(&ctx->halo_ev[i], cudaEventDisableTiming));
    }
    const size_t need = 2 * (size_t)in_cols;
    if (ctx->halo_slot_floats < need) {
        GB200_CUDA_TRY(cudaDeviceSynchronize());   // nothing may still read the old ring
        if (ctx->halo_ring) GB200_CUDA_TRY(cudaFree(ctx->halo_ring));
        ctx->halo_ring = nullptr;
        ctx->halo_slot_floats = 0;
        GB200_CUDA_TRY(cudaMalloc(&ctx->halo_ring, kHaloSlots * need * sizeof(float)));
        ctx->halo_slot_floats = need;
    }
    const unsigned long long k = ctx->halo_step;
    const int slot = (int)(k % kHaloSlots);
    // the launch that read this slot last (32 steps back) must be over before it is overwritten
    if (k >= (unsigned long long)kHaloSlots && k % kHaloEventEvery == 0)
        GB200_CUDA_TRY(cudaStreamWaitEvent(ctx->halo_stream, ctx->halo_ev[(k / kHaloEventEvery) % 4], 0));
    float *dst = ctx->halo_ring + (size_t)slot * ctx->halo_slot_floats;
    GB200_CUDA_TRY(cudaMemcpy2DAsync(dst, (size_t)in_cols * sizeof(float), halo, (size_t)halo_ld * sizeof(float),
                                     (size_t)in_cols * sizeof(float), 2, cudaMemcpyDefault, ctx->halo_stream));
    GB200_CUDA_TRY(cudaMemcpyAsync(ctx->halo_flags + slot, ctx->halo_flag_values + (k & 255), sizeof(int),
                                   cudaMemcpyHostToDevice, ctx->halo_stream));
    *slot_rows = dst;
    *flag = ctx->halo_flags + slot;
    *expect = (int)(k & 255) + 1;
    return GB200_OK;
}
// After the launch that reads the slot handed out by halo_prefetch.
static int halo_prefetch_launched(gb200_ctx *ctx, cudaStream_t stream) {
    const unsigned long long k = ctx->halo_step++;
    if (k % kHaloEventEvery == kHaloEventEvery - 1)
        GB200_CUDA_TRY(cudaEventRecord(ctx->halo_ev[(k / kHaloEventEvery) % 4], stream));
    return GB200_OK;
}

template <int ROWS>
static int launch_reg(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                      int64_t in_cols, float *out, int64_t out_ld, cudaStream_t stream,
                      const float *halo = nullptr, int64_t halo_ld = 0) {
    const int64_t out_rows = in_rows - 2, out_cols = in_cols - 2;
    const int64_t n_blocks = ((out_cols + 511) / 512) * ((out_rows + ROWS - 1) / ROWS);
    GB200_REQUIRE(n_blocks < (1ll << 31), GB200_ERR_UNSUPPORTED, "blur: more than 2^31 blocks");
    dim3 grid((unsigned)n_blocks);
    const float *slot_rows = nullptr;
    const int *flag = nullptr;
    int expect = 0;
    const int halo_dev = halo != nullptr ? other_device_of(ctx, halo) : -1;
    if (halo_dev >= 0) {
        // Large bands: the copy engine (the copy hides under the kernel).  Small ones read the rows
        // themselves, unless this device's kernels cannot read that device's memory at all.
        const bool large = in_rows * in_cols * (int64_t)sizeof(float) >= ctx->halo_prefetch_min_bytes;
        if (large || !peer_readable(ctx, halo_dev)) {
            int rc = halo_prefetch(ctx, halo, halo_ld, in_cols, &slot_rows, &flag, &expect);
            if (rc) return rc;
            halo = slot_rows;
            halo_ld = in_cols;
        }
    }
    GB200_CUDA_TRY(launch_pdl(blur3x3_reg_kernel<ROWS>, grid, dim3(128), 0, stream, in, in_ld, (int)in_cols,
                              out, out_ld, (int)out_rows, (aligned16(out) && out_ld % 4 == 0) ? 1 : 0,
                              (int)(halo ? in_rows - 2 : in_rows), halo, halo_ld, flag, expect, ctx->d_status));
    int rc = after_launch(ctx, "blur3x3_reg_kernel");
    if (rc == GB200_OK && slot_rows != nullptr) rc = halo_prefetch_launched(ctx, stream);
    return rc;
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

// variant 0 picks: the register-staged kernel for 16-byte aligned input rows, else the generic
// kernel.  Other variants exist for the parity tests and for benchmarking:
//   1 = generic direct kernel,  2 = TMA-staged kernel (one wave),  3 = TMA-staged, 4 waves,
//   50 + k = TMA-staged, 4 * 2^k waves of ever shorter strips (52: 16 waves, its best: 80.0 us
//   at 8192^2 against 78.9 us for the register-staged kernel),
//   40 + k = register-staged kernel with 2, 3, 4, 6, 8 output rows per block (k = 0..4).
int blur_dispatch(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows, int64_t in_cols,
                  float *out, int64_t out_ld, cudaStream_t stream, int variant) {
    const bool in_aligned = aligned16(in) && in_ld % 4 == 0;
    const bool tma_ok = ctx->encode_tiled && in_aligned && in_cols >= 64 && in_rows >= 16;
    if (variant == 1 || !in_aligned)
        return launch_direct(ctx, in, in_ld, in_rows, nullptr, 0, in_cols, out, out_ld, 0,
                             in_rows - 2, stream);
    if (variant == 2 && tma_ok)
        return launch_tma<8, 2>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream, 1);
    if (variant == 3 && tma_ok)
        return launch_tma<8, 2>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream, 4);
    if (variant >= 50 && variant < 60 && tma_ok)   // 50 + k: 2^k * 4 waves of ever shorter strips
        return launch_tma<8, 2>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream, 4 << (variant - 50));
    switch (variant) {
        case 40: return launch_reg<2>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
        case 41: return launch_reg<3>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
        case 43: return launch_reg<6>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
        case 44: return launch_reg<8>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
        default: return launch_reg<4>(ctx, in, in_ld, in_rows, in_cols, out, out_ld, stream);
    }
}

}  // namespace gb200

using namespace gb200;

extern "C" {

#ifdef GB200_BLUR_TRACE
// Debug builds only: copies the timeline out and resets it for the next launch.
int gb200_blur_trace_read(unsigned long long *out) {
    cudaError_t e = cudaMemcpyFromSymbol(out, gb200::g_blur_trace, sizeof(unsigned long long) * 16);
    unsigned long long init[16] = {0};
    init[9] = ~0ull;
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(gb200::g_blur_trace, init, sizeof(init));
    return (int)e;
}
#endif

int gb200_blur3x3_f32(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                      int64_t in_cols, float *out, int64_t out_ld, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
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
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_blur_args(in, in_ld, in_rows, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return blur_dispatch(ctx, in, in_ld, in_rows, in_cols, out, out_ld,
                         static_cast<cudaStream_t>(stream), variant);
}

// Test hook: the band size from which a halo on another device is prefetched by a copy engine.
int gb200_ctx_set_halo_prefetch_min_bytes(gb200_ctx *ctx, long long bytes) {
    GB200_REQUIRE(ctx != nullptr && bytes >= 0, GB200_ERR_INVALID_ARG, "bad argument");
    ctx->halo_prefetch_min_bytes = bytes;
    return GB200_OK;
}

int gb200_blur3x3_f32_band(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t band_rows,
                           int64_t in_cols, const float *halo, int64_t halo_ld, float *out,
                           int64_t out_ld, void *stream_) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (halo == nullptr)
        return gb200_blur3x3_f32(ctx, in, in_ld, band_rows, in_cols, out, out_ld, stream_);
    rc = check_blur_args(in, in_ld, band_rows + 2, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    GB200_REQUIRE(halo_ld >= in_cols, GB200_ERR_INVALID_ARG, "halo_ld smaller than the row");
    // Aligned images: one launch of the register-staged kernel; only its last block row reads
    // the halo.  Otherwise the generic kernel does the same with per-row pointer selection.
    if (aligned16(in) && in_ld % 4 == 0)
        return launch_reg<4>(ctx, in, in_ld, band_rows + 2, in_cols, out, out_ld, stream, halo,
                             halo_ld);
    const int halo_dev = other_device_of(ctx, halo);
    GB200_REQUIRE(halo_dev < 0 || peer_readable(ctx, halo_dev), GB200_ERR_UNSUPPORTED,
                  "the halo rows are on device %d, which device %d cannot read, and an unaligned band has no "
                  "copy-engine path", halo_dev, ctx->device);
    return launch_direct(ctx, in, in_ld, band_rows, halo, halo_ld, in_cols, out, out_ld, 0,
                         band_rows, stream);
}

int gb200_blur3x3_f32_host(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                           int64_t in_cols, float *out, int64_t out_ld) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_blur_args(in, in_ld, in_rows, in_cols, out, out_ld);
    if (rc) return rc < 0 ? rc : GB200_OK;
    const int64_t out_rows = in_rows - 2, out_cols = in_cols - 2;
    // Device images are packed with a pitch rounded up to 4 floats so that the TMA path applies.
    // When the host pitch is 16-byte friendly and only slightly wider than the row, the device
    // copy keeps that pitch so that uploads are plain linear copies (a strided 2-D copy of
    // 32 KB rows runs well below PCIe speed); the same for the output.
    const bool lin_in = in_ld % 4 == 0 && in_ld - in_cols <= in_cols / 8;
    const bool lin_out = out_ld == out_cols && out_cols % 4 == 0;   // never write host padding
    const int64_t d_in_ld = lin_in ? in_ld : (in_cols + 3) / 4 * 4;
    const int64_t d_out_ld = lin_out ? out_ld : (out_cols + 3) / 4 * 4;
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
            if (lin_in) {
                // rows [uploaded, need) in one piece; the image's last row ends after in_cols
                const int64_t elems = (need - uploaded - 1) * in_ld + (need == in_rows ? in_cols : in_ld);
                GB200_CUDA_TRY(cudaMemcpyAsync(d_in + uploaded * d_in_ld, in + uploaded * in_ld,
                                               elems * 4, cudaMemcpyHostToDevice, up));
            } else {
                GB200_CUDA_TRY(cudaMemcpy2DAsync(d_in + uploaded * d_in_ld, d_in_ld * 4,
                                                 in + uploaded * in_ld, in_ld * 4, in_cols * 4,
                                                 need - uploaded, cudaMemcpyHostToDevice, up));
            }
            uploaded = need;
        }
        GB200_CUDA_TRY(cudaEventRecord(ctx->ev[0], up));
        GB200_CUDA_TRY(cudaStreamWaitEvent(down, ctx->ev[0], 0));
        rc = blur_dispatch(ctx, d_in + r0 * d_in_ld, d_in_ld, r1 - r0 + 2, in_cols,
                           d_out + r0 * d_out_ld, d_out_ld, down, 0);
        if (rc) return rc;
        if (lin_out) {
            const int64_t elems = (r1 - r0 - 1) * out_ld + (r1 == out_rows ? out_cols : out_ld);
            GB200_CUDA_TRY(cudaMemcpyAsync(out + r0 * out_ld, d_out + r0 * d_out_ld, elems * 4,
                                           cudaMemcpyDeviceToHost, down));
        } else {
            GB200_CUDA_TRY(cudaMemcpy2DAsync(out + r0 * out_ld, out_ld * 4, d_out + r0 * d_out_ld,
                                             d_out_ld * 4, out_cols * 4, r1 - r0,
                                             cudaMemcpyDeviceToHost, down));
        }
    }
    return host_finish(ctx, down, up);
}

}  // extern "C"
