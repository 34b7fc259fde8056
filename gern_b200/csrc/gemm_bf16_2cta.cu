// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 tile of C per pair of SMs.
//
// Same operator and operand layout as gemm_bf16_tc_kernel (gemm_bf16.cu); what changes is the
// mapping onto the machine.  Two CTAs of a cluster share one MMA: CTA r of the pair holds rows
// [128 r, 128 r + 128) of the A tile and columns [128 r, 128 r + 128) of the B tile in its shared
// memory, the leader (rank 0) issues M256 N256 K16 instructions that read both CTAs' operand
// halves, and each CTA's TMEM receives the accumulator rows of its own half of M.  Per CTA and
// MMA that is 4 KiB of A + 4 KiB of B from shared memory instead of 4 + 8 for the 128 x 256
// single-CTA tile, and each B tile is fetched from L2 once per pair, which leaves room for a
// 6-deep ring.  Every CTA loads its own halves with ordinary (non-multicast) TMA tile loads that
// report their bytes to the leader's barrier; ring slots and accumulators are released to both
// CTAs with tcgen05.commit on both CTAs' barriers.  Waits on mbarriers are time-bounded; the
// cluster barriers at start and end are the only unbounded synchronisation and are reached by
// every thread on every path.
#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

#ifndef GB200_GEMM2_STAGES
#define GB200_GEMM2_STAGES 6
#endif
#ifndef GB200_GEMM2_GROUP_M
#define GB200_GEMM2_GROUP_M 8
#endif

namespace gemm2 {
constexpr int BM = 256, BN = 256, BK = 64, STAGES = GB200_GEMM2_STAGES;
constexpr int HALF = 128;                            // rows of A / of B per CTA
constexpr int A_BYTES = HALF * BK * 2;               // 16 KiB
constexpr int B_BYTES = HALF * BK * 2;               // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;       // 32 KiB per CTA
constexpr int NUM_THREADS = smem::Gemm2CtaLayout::kThreads;
constexpr smem::Gemm2CtaLayout kLayout = smem::gemm_2cta_layout(STAGES);
static_assert(kLayout.stage_bytes == STAGE_BYTES && kLayout.stages.offset == 0, "kernel and planner disagree");
constexpr int SMEM_BYTES = kLayout.dynamic_bytes;
constexpr int GROUP_M = GB200_GEMM2_GROUP_M;         // 256-row tile rows per rasterisation group
}  // namespace gemm2

__device__ __forceinline__ void tile_coords2(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
    const int per_group = gemm2::GROUP_M * tiles_n;
    const int g = t / per_group;
    const int first_m = g * gemm2::GROUP_M;
    const int rows_in_group = min(gemm2::GROUP_M, tiles_m - first_m);
    const int r = t - g * per_group;
    tm = first_m + r % rows_in_group;
    tn = r / rows_in_group;
}

// fp32 output from three-way bf16 splits (gemm_f32_tc.cu): when c32 is set the K loop walks six
// (segment of A, segment of B) pairs of seg_kb K blocks each and the epilogue stores fp32.
struct Gemm2F32 {
    float *c32;
    int64_t ldc32;
    int accumulate;
    int seg_kb;
    // consumers fused into the epilogue (MODE 2), as in the single-CTA kernel of gemm_bf16.cu:
    // t = alpha * acc; t -= row_sub[i]; t = exp(t); t /= row_div[i]; then bf16 C, row maxima, row sums
    float alpha;
    const float *row_sub;
    const float *row_div;
    float *row_max;
    float *row_sum;
    int apply_exp;
};

// MODE 0: bf16 C = A B.  MODE 1: fp32 C from three-way bf16 splits.  MODE 2: bf16 C with consumers.
// TN: columns of C per tile, 256 or 224 (each CTA then holds 112 rows of B in its 16 KiB slot; the
// accumulator buffers stay 256 TMEM columns apart).  148 tiles of 224 columns are exactly two
// rounds on 74 CTA pairs where 128 tiles of 256 columns are 1.73: see pick_pair_tile_n.
template <int MODE, int TN = 256>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm2::NUM_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b, __nv_bfloat16 *__restrict__ C,
                      int64_t ldc, int M, int N, int K, int *status, Gemm2F32 f32) {
    using namespace gemm2;
    constexpr bool F32X3 = MODE == 1;
    constexpr bool EPI = MODE == 2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kLayout.full.offset);            // [STAGES] used in the leader only
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + kLayout.empty.offset);          // [STAGES] one per CTA
    uint64_t *acc_full = reinterpret_cast<uint64_t *>(smem + kLayout.acc_full.offset);    // [2] one per CTA
    uint64_t *acc_empty = reinterpret_cast<uint64_t *>(smem + kLayout.acc_empty.offset);  // [2] used in the leader only (8 arrivals)
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(smem + kLayout.tmem_slot.offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    static_assert(TN % 32 == 0 && TN <= BN && (TN / 2) * BK * 2 <= B_BYTES, "tile width");
    constexpr int B_HALF = TN / 2;                          // rows of B per CTA
    constexpr int B_TILE_BYTES = B_HALF * BK * 2;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + TN - 1) / TN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);   // 4 epilogue warps in each of the two CTAs
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_base_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // launched with launch_pdl: the set-up above may overlap the previous kernel's tail
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                int tm, tn;
                tile_coords2(t, tiles_m, tiles_n, tm, tn);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1, status, 221)) { ok = false; break; }
                    unsigned char *sa = smem + s * STAGE_BYTES;
                    // the leader's barrier collects the bytes of all four loads of the pair
                    if (leader) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_TILE_BYTES));
                    const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
                    int xa = kb * BK, xb = kb * BK;
                    if (F32X3) {
                        // a3 b1, a2 b2, a1 b3, a2 b1, a1 b2, a1 b1 (smallest first); segment i of
                        // an operand starts at column i * seg_kb * BK of its rows
                        const int sp = kb / f32.seg_kb, r = kb - sp * f32.seg_kb;
                        const int seg_a = (0x210100 >> (4 * (5 - sp))) & 15;
                        const int seg_b = (0x012010 >> (4 * (5 - sp))) & 15;
                        xa = (seg_a * f32.seg_kb + r) * BK;
                        xb = (seg_b * f32.seg_kb + r) * BK;
                    }
                    tma_load_2d_pair(sa, &tmap_a, xa, tm * BM + (int)rank * HALF, full_leader);
                    tma_load_2d_pair(sa + A_BYTES, &tmap_b, xb, tn * TN + (int)rank * B_HALF, full_leader);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, TN, 0);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs, ++tile_it) {
                const int buf = tile_it & 1;
                const uint32_t acc_ph = (tile_it >> 1) & 1;
                if (!mbar_wait(&acc_empty[buf], acc_ph ^ 1, status, 222)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full[s], ph, status, 223)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = umma_desc_sw128(sa, 16, 1024);
                    const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_f16_ss_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                         (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(&empty[s]);   // frees the slot in both CTAs
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): TMEM -> registers -> bf16 -> global ----------------
        const int lane_group = warp & 3;
        uint32_t tile_it = 0;
        bool ok = true;
        const bool vec_ok = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        const bool vec32_ok = (ldc % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 31) == 0);
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++tile_it) {
            int tm, tn;
            tile_coords2(t, tiles_m, tiles_n, tm, tn);
            const int buf = tile_it & 1;
            const uint32_t acc_ph = (tile_it >> 1) & 1;
            if (!mbar_wait(&acc_full[buf], acc_ph, status, 224)) { ok = false; break; }
            tc_fence_after();
            const int row = tm * BM + (int)rank * HALF + lane_group * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(buf * BN);
            float e_sub = 0.0f, e_inv = 1.0f, e_max = -INFINITY, e_sum = 0.0f;
            if (EPI && row < M) {
                if (f32.row_sub) e_sub = f32.row_sub[row];
                if (f32.row_div) e_inv = 1.0f / f32.row_div[row];
            }
#pragma unroll 1
            for (int ch = 0; ch < TN / 32; ++ch) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + ch * 32, r);
                tmem_ld_wait();
                const int col = tn * TN + ch * 32;
                if (EPI) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float v = fmaf(__uint_as_float(r[j]), f32.alpha, -e_sub);
                        if (f32.apply_exp) v = __expf(v);
                        v *= e_inv;
                        r[j] = __float_as_uint(v);
                        if (col + j < N) {
                            e_max = fmaxf(e_max, v);
                            e_sum += v;
                        }
                    }
                }
                if (EPI && C == nullptr) {
                    // reductions only: the product itself is a temporary that is never stored
                } else if (F32X3) {
                    if (row < M && col < N) {
                        float *dst = f32.c32 + static_cast<int64_t>(row) * f32.ldc32 + col;
                        const bool v4 = (f32.ldc32 % 4 == 0) &&
                                        ((reinterpret_cast<uintptr_t>(f32.c32) & 15) == 0) && col + 32 <= N;
                        if (v4) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float4 o = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                                if (f32.accumulate) {
                                    const float4 c = *reinterpret_cast<const float4 *>(dst + 4 * q);
                                    o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                                }
                                *reinterpret_cast<float4 *>(dst + 4 * q) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < N)
                                    dst[j] = __uint_as_float(r[j]) + (f32.accumulate ? dst[j] : 0.0f);
                        }
                    }
                } else if (row < M && col < N) {
                    __nv_bfloat16 *dst = C + static_cast<int64_t>(row) * ldc + col;
                    if (vec32_ok && col + 32 <= N) {
                        // a thread owns 64 contiguous bytes of its row: two full 32-byte sectors
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                w[i] = pack_bf16(__uint_as_float(r[16 * h + 2 * i]),
                                                 __uint_as_float(r[16 * h + 2 * i + 1]));
                            st_global_256(dst + 16 * h, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
                        }
                    } else if (vec_ok && col + 32 <= N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                            v.y = pack_bf16(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                            v.z = pack_bf16(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                            v.w = pack_bf16(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                            *reinterpret_cast<uint4 *>(dst + 8 * q) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                    }
                }
            }
            if (EPI && row < M) {
                // one atomic per row and 256-column tile; the vectors were initialised by the host side
                if (f32.row_max) atomic_max_f32(f32.row_max + row, e_max);
                if (f32.row_sum) atomicAdd(f32.row_sum + row, e_sum);
            }
            tc_fence_before();
            __syncwarp();
            // the accumulator buffer is free once both CTAs have drained their halves
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // no CTA may leave while its partner can still signal into it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// Tile width of the pair kernel: rounds of tiles over the CTA pairs times the width of a tile; 224
// columns only where that is at least 5 % less than with 256.  1024 x 8192 (an eighth of 8192^2):
// 128 tiles of 256 columns are two rounds of which the second is 0.73 full, 148 tiles of 224 are two
// full ones.  Measured, the narrower MMAs do not run 224/256 as long, so the gain is 3 %, not 12:
// 1024 x 8192 x 8192 90.1-92.7 against 93.8-94.6 us, 2048 x 8192 x 8192 177-178 against 184 us; where
// the rounds come out equal (8192^3, 4096 x 8192 x 8192) 224 columns lose 4-15 % and are not picked.
static int pick_pair_tile_n(int64_t M, int64_t N, int sm_count) {
    const int64_t pairs = sm_count / 2 > 0 ? sm_count / 2 : 1;
    auto cost = [&](int w) {
        const int64_t tiles = ((M + gemm2::BM - 1) / gemm2::BM) * ((N + w - 1) / w);
        return ((tiles + pairs - 1) / pairs) * w;
    };
    return cost(224) * 100 <= cost(256) * 95 ? 224 : 256;
}

// Launches the pair kernel; the caller has checked alignment (same rules as the single-CTA path).
// tile_n_hint: 0 = pick the tile width, 224 / 256 = that width.
int gemm_bf16_2cta_launch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                          void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t stream,
                          int tile_n_hint) {
    using namespace gemm2;
    const int tile_n = tile_n_hint == 224 || tile_n_hint == 256 ? tile_n_hint : pick_pair_tile_n(M, N, ctx->sm_count);
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                         (uint64_t)lda * 2, BK, HALF, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                     (uint64_t)ldb * 2, BK, tile_n / 2, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + tile_n - 1) / tile_n);
    int64_t pairs = ctx->sm_count / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    auto kern = tile_n == 224 ? gemm_bf16_2cta_kernel<0, 224> : gemm_bf16_2cta_kernel<0, 256>;
    rc = ensure_dynamic_smem(ctx, kern, SMEM_BYTES);
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(kern, dim3((unsigned)(2 * pairs)), dim3(NUM_THREADS),
                              (size_t)SMEM_BYTES, stream, ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M,
                              (int)N, (int)K, ctx->d_status, Gemm2F32{}));
    return after_launch(ctx, "gemm_bf16_2cta_kernel");
}

// fp32 C (+)= A B on CTA pairs from operands split into three bf16 terms: A3 [M][3*Kp],
// B3 [N][3*Kp], K-contiguous, Kp a multiple of 64 (see gemm_f32_tc.cu).
int gemm_f32x3_2cta_launch(gb200_ctx *ctx, const void *A3, const void *B3, float *C, int64_t ldc,
                           int64_t M, int64_t N, int64_t Kp, int accumulate, cudaStream_t stream) {
    using namespace gemm2;
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(3 * Kp), (uint64_t)M,
                         (uint64_t)(3 * Kp) * 2, BK, HALF, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(3 * Kp), (uint64_t)N,
                     (uint64_t)(3 * Kp) * 2, BK, HALF, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    int64_t pairs = ctx->sm_count / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    rc = ensure_dynamic_smem(ctx, gemm_bf16_2cta_kernel<1>, SMEM_BYTES);
    if (rc) return rc;
    Gemm2F32 f32{};
    f32.c32 = C;
    f32.ldc32 = ldc;
    f32.accumulate = accumulate;
    f32.seg_kb = (int)(Kp / BK);
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_2cta_kernel<1>, dim3((unsigned)(2 * pairs)), dim3(NUM_THREADS),
                              (size_t)SMEM_BYTES, stream, ta, tb, static_cast<__nv_bfloat16 *>(nullptr),
                              (int64_t)0, (int)M, (int)N, (int)(6 * Kp), ctx->d_status, f32));
    return after_launch(ctx, "gemm_bf16_2cta_kernel<f32x3>");
}

// bf16 GEMM with consumers in the epilogue on CTA pairs; the caller has initialised row_max / row_sum.
int gemm_bf16_2cta_epilogue_launch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                                   void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha,
                                   const float *row_sub, int apply_exp, const float *row_div, float *row_max,
                                   float *row_sum, cudaStream_t stream) {
    using namespace gemm2;
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                         (uint64_t)lda * 2, BK, HALF, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                     (uint64_t)ldb * 2, BK, HALF, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    int64_t pairs = ctx->sm_count / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    rc = ensure_dynamic_smem(ctx, gemm_bf16_2cta_kernel<2>, SMEM_BYTES);
    if (rc) return rc;
    Gemm2F32 e{};
    e.alpha = alpha;
    e.row_sub = row_sub;
    e.row_div = row_div;
    e.row_max = row_max;
    e.row_sum = row_sum;
    e.apply_exp = apply_exp;
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_2cta_kernel<2>, dim3((unsigned)(2 * pairs)), dim3(NUM_THREADS),
                              (size_t)SMEM_BYTES, stream, ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M,
                              (int)N, (int)K, ctx->d_status, e));
    return after_launch(ctx, "gemm_bf16_2cta_kernel<epilogue>");
}

int kernel_regs_gemm_2cta() { return kernel_registers(gemm_bf16_2cta_kernel<0>); }

}  // namespace gb200
