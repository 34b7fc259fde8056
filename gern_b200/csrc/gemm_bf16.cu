// bf16 x bf16 -> fp32 (TMEM) -> bf16 matrix multiply on the sm_100a tensor cores.
//
// C[M,N] = A[M,K] * B[K,N] with A row-major and B column-major (both K-contiguous), the
// operator that annot::MatrixMultiply describes (gernels/mm/gern_annot/functions.h:7-60).  The
// reference's schedule for it (gernels/mm/kernel_10.cu:108-131) stages 32x32 tiles through
// shared memory with cooperative copies and block barriers and computes on the fp32 pipe,
// writing C back every K tile (gernels/mm/bench.cu:18-41).  This kernel keeps the same tile
// structure -- block tile of C, Reduce over K tiles, operands staged in shared memory -- and
// maps it to Blackwell:
//   * a persistent CTA per SM walks 128x256 tiles of C;
//   * warp 0 feeds a 4-deep ring of {A 128x64, B 256x64} bf16 stages with TMA
//     (128-byte swizzle, completion on mbarriers, no multicast);
//   * warp 1 issues tcgen05.mma (M128 N256 K16, cta_group::1) from shared-memory descriptors
//     into one of two 256-column fp32 accumulators in TMEM and releases ring slots with
//     tcgen05.commit;
//   * warps 2-5 drain the finished accumulator with tcgen05.ld, round to bf16 and store C,
//     overlapping the next tile's main loop (the other TMEM accumulator);
//   * problems with at least one 256 x 256 tile per pair of SMs go to the CTA-pair kernel
//     (gemm_bf16_2cta.cu, tcgen05.mma.cta_group::2), measured 3-4 % faster at 8192^3;
//   * problems with too few tiles to fill the SMs are split along K: each (tile, split) item
//     writes an fp32 partial slab to a workspace and a small second kernel sums the slabs.
// Every wait is bounded; a wait that runs out records a code in the context's status word and
// the kernel winds down (TMEM is always freed).
#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

namespace gemm {
using Layout = smem::GemmTcLayout;
constexpr int BM = Layout::kBM, BN = 256, BK = Layout::kBK, STAGES = Layout::kStages;
constexpr int A_BYTES = BM * BK * 2;              // 16 KiB
constexpr int B_BYTES = BN * BK * 2;              // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;    // 48 KiB
constexpr int NUM_THREADS = Layout::kThreads;
// stage ring, barriers, TMEM slot: one planned layout per tile width
template <int TILE_N>
constexpr smem::GemmTcLayout kLayout = smem::gemm_tc_layout(TILE_N);
constexpr int SMEM_BYTES = kLayout<BN>.dynamic_bytes;
#ifndef GB200_GEMM_AUTO_PAIR
#define GB200_GEMM_AUTO_PAIR 1
#endif
#ifndef GB200_GEMM_GROUP_M
#define GB200_GEMM_GROUP_M 16
#endif
constexpr int GROUP_M = GB200_GEMM_GROUP_M;       // tile rows per L2 rasterisation group
}  // namespace gemm

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int &tm, int &tn) {
    // Walk tiles in groups of GROUP_M tile-rows, column by column inside a group, so that the
    // CTAs running at the same time share A panels and B panels in L2.
    const int per_group = gemm::GROUP_M * tiles_n;
    const int g = t / per_group;
    const int first_m = g * gemm::GROUP_M;
    const int rows_in_group = min(gemm::GROUP_M, tiles_m - first_m);
    const int r = t - g * per_group;
    tm = first_m + r % rows_in_group;
    tn = r / rows_in_group;
}

// Consumers fused into the epilogue while the accumulator is still in TMEM / registers: the
// reference's elementwise and row-reduction leaves applied to the product before it is rounded
// (test/library/matrix/impl/cpu-matrix.h:134-194: exp_matrix, subtract_vec, divide_vec, max_row,
// sum_row), in the order  t = alpha * acc;  t -= row_sub[i];  t = exp(t);  t /= row_div[i].
struct GemmEpi {
    float alpha;
    const float *row_sub;
    const float *row_div;
    float *row_max;
    float *row_sum;
    int apply_exp;
    // fp32 product from three-way bf16 splits (gemm_f32_tc.cu): fp32 output instead of bf16, and
    // the K loop walks six (segment of A, segment of B) pairs of seg_kb K blocks each.
    float *c32;
    int64_t ldc32;
    int accumulate;
    int seg_kb;
};


__global__ void epilogue_init_kernel(float *row_max, float *row_sum, int M) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < M) {
        if (row_max) row_max[i] = -INFINITY;
        if (row_sum) row_sum[i] = 0.0f;
    }
}

// TILE_N: columns of C per tile (256 by default; 192 and 128 serve problems whose 256-wide tiles
// would leave SMs idle, see pick_tile_n).
template <bool EPI, int TILE_N = 256>
__global__ void __launch_bounds__(gemm::NUM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, __nv_bfloat16 *__restrict__ C,
                    int64_t ldc, int M, int N, int K, int splits, float *__restrict__ ws,
                    int *status, GemmEpi epi) {
    using namespace gemm;
    constexpr int BN = TILE_N;                        // these shadow the 256-wide defaults
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile width");
    (void)B_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    static_assert(kLayout<BN>.stage_bytes == STAGE_BYTES && kLayout<BN>.stages.offset == 0, "kernel and planner disagree");
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kLayout<BN>.full.offset);            // [STAGES] TMA -> MMA
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + kLayout<BN>.empty.offset);          // [STAGES] MMA -> TMA
    uint64_t *acc_full = reinterpret_cast<uint64_t *>(smem + kLayout<BN>.acc_full.offset);    // [2] MMA -> epilogue
    uint64_t *acc_empty = reinterpret_cast<uint64_t *>(smem + kLayout<BN>.acc_empty.offset);  // [2] epilogue -> MMA
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(smem + kLayout<BN>.tmem_slot.offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int k_blocks = (K + BK - 1) / BK;
    // Split-K: a work item is (tile, split); split s reduces k blocks [s*kb_per, (s+1)*kb_per)
    // into an fp32 slab of the workspace, and a second kernel sums the slabs into C.
    const int kb_per = (k_blocks + splits - 1) / splits;
    const int n_tiles = tiles_m * tiles_n * splits;   // work items

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    // launched with launch_pdl: the set-up above may overlap the previous kernel's tail
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                int tm, tn;
                tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
                const int kb_begin = (t % splits) * kb_per, kb_end = min(k_blocks, kb_begin + kb_per);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty[s], ph ^ 1, status, 201)) { ok = false; break; }
                    unsigned char *sa = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    int xa = kb * BK, xb = kb * BK;
                    if (EPI && epi.seg_kb > 0) {
                        // a = a1 + a2 + a3, b = b1 + b2 + b3 (bf16 each); the six products that
                        // matter, smallest first: a3 b1, a2 b2, a1 b3, a2 b1, a1 b2, a1 b1.
                        // Segment i of an operand starts at column i * seg_kb * BK of its rows.
                        const int pair = kb / epi.seg_kb, r = kb - pair * epi.seg_kb;
                        const int seg_a = (0x210100 >> (4 * (5 - pair))) & 15;   // 2 1 0 1 0 0
                        const int seg_b = (0x012010 >> (4 * (5 - pair))) & 15;   // 0 1 2 0 1 0
                        xa = (seg_a * epi.seg_kb + r) * BK;
                        xb = (seg_b * epi.seg_kb + r) * BK;
                    }
                    tma_load_2d(sa, &tmap_a, xa, tm * BM, &full[s]);
                    tma_load_2d(sa + A_BYTES, &tmap_b, xb, tn * BN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0);
            uint32_t it = 0, tile_it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tile_it) {
                const int buf = tile_it & 1;
                const uint32_t acc_ph = (tile_it >> 1) & 1;
                if (!mbar_wait(&acc_empty[buf], acc_ph ^ 1, status, 202)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int kb_begin = (t % splits) * kb_per, kb_end = min(k_blocks, kb_begin + kb_per);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full[s], ph, status, 203)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t da = umma_desc_sw128(sa, 16, 1024);
                    const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 bf16 = 32 bytes along K inside the 128-byte swizzle row
                        umma_f16_ss(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc,
                                    (kb != kb_begin || k != 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);  // slot is free once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> bf16 -> global ----------------
        const int lane_group = warp & 3;  // TMEM lanes this warp may touch: 32*(warp%4)...
        uint32_t tile_it = 0;
        bool ok = true;
        const bool vec_ok = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        const bool vec32_ok = (ldc % 16 == 0) && ((reinterpret_cast<uintptr_t>(C) & 31) == 0);
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++tile_it) {
            int tm, tn;
            tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
            const int split = t % splits;
            const bool empty_range = split * kb_per >= k_blocks;   // nothing was accumulated
            const int buf = tile_it & 1;
            const uint32_t acc_ph = (tile_it >> 1) & 1;
            if (!mbar_wait(&acc_full[buf], acc_ph, status, 204)) { ok = false; break; }
            tc_fence_after();
            const int row = tm * BM + lane_group * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                                   static_cast<uint32_t>(buf * BN);
            float e_sub = 0.0f, e_inv = 1.0f, e_max = -INFINITY, e_sum = 0.0f;
            if (EPI && row < M) {
                if (epi.row_sub) e_sub = epi.row_sub[row];
                if (epi.row_div) e_inv = 1.0f / epi.row_div[row];
            }
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ++ch) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + ch * 32, r);
                tmem_ld_wait();
                const int col = tn * BN + ch * 32;
                if (EPI) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float v = fmaf(__uint_as_float(r[j]), epi.alpha, -e_sub);
                        if (epi.apply_exp) v = __expf(v);
                        v *= e_inv;
                        r[j] = __float_as_uint(v);
                        if (col + j < N) {
                            e_max = fmaxf(e_max, v);
                            e_sum += v;
                        }
                    }
                }
                if (EPI && epi.c32 != nullptr) {
                    if (row < M && col < N) {
                        float *dst = epi.c32 + static_cast<int64_t>(row) * epi.ldc32 + col;
                        const bool v4 = (epi.ldc32 % 4 == 0) && ((reinterpret_cast<uintptr_t>(epi.c32) & 15) == 0) &&
                                        col + 32 <= N;
                        if (v4) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float4 o = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                                if (epi.accumulate) {
                                    const float4 c = *reinterpret_cast<const float4 *>(dst + 4 * q);
                                    o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                                }
                                *reinterpret_cast<float4 *>(dst + 4 * q) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < N)
                                    dst[j] = __uint_as_float(r[j]) + (epi.accumulate ? dst[j] : 0.0f);
                        }
                    }
                } else if (EPI && C == nullptr) {
                    // reductions only: the product itself is a temporary that is never stored
                } else if (splits > 1) {
                    // fp32 partial sums into slab `split` of the workspace ([splits][M][N])
                    if (row < M && col < N) {
                        float *dst = ws + (static_cast<int64_t>(split) * M + row) * N + col;
                        if ((N & 3) == 0 && col + 32 <= N) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                *reinterpret_cast<uint4 *>(dst + 4 * q) =
                                    empty_range ? make_uint4(0, 0, 0, 0)
                                                : make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < N) dst[j] = empty_range ? 0.0f : __uint_as_float(r[j]);
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
            if (EPI && row < M) {
                // one atomic per row and tile: the tiles of a row meet in the output vectors
                if (epi.row_max) atomic_max_f32(epi.row_max + row, e_max);
                if (epi.row_sum) atomicAdd(epi.row_sum + row, e_sum);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Second step of split-K: C = bf16(sum over slabs), one thread per 4 adjacent columns.
__global__ void __launch_bounds__(256)
gemm_splitk_reduce_kernel(const float *__restrict__ ws, int splits, __nv_bfloat16 *__restrict__ C,
                          int64_t ldc, int M, int N) {
    pdl_launch_dependents();   // launched with launch_pdl right behind the GEMM kernel: its blocks
    pdl_wait();                // are resident and waiting when the last slab is written
    const int64_t groups_per_row = (N + 3) / 4;
    const int64_t total = static_cast<int64_t>(M) * groups_per_row;
    const int64_t slab = static_cast<int64_t>(M) * N;
    const bool vec = (N & 3) == 0 && (ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 7) == 0;
    for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < total;
         g += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t row = g / groups_per_row;
        const int col = static_cast<int>(g % groups_per_row) * 4;
        const float *src = ws + row * N + col;
        if (vec) {
            float4 acc = *reinterpret_cast<const float4 *>(src);
            for (int s = 1; s < splits; ++s) {
                const float4 v = *reinterpret_cast<const float4 *>(src + s * slab);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            uint2 out;
            out.x = pack_bf16(acc.x, acc.y);
            out.y = pack_bf16(acc.z, acc.w);
            *reinterpret_cast<uint2 *>(C + row * ldc + col) = out;
        } else {
            for (int j = 0; j < 4 && col + j < N; ++j) {
                float acc = src[j];
                for (int s = 1; s < splits; ++s) acc += src[j + s * slab];
                C[row * ldc + col + j] = __float2bfloat16_rn(acc);
            }
        }
    }
}

// Fallback for operands the TMA path cannot take (pitch or base not 16-byte aligned):
// plain CUDA-core kernel, fp32 accumulate in ascending k.
__global__ void __launch_bounds__(256)
gemm_bf16_simple_kernel(const __nv_bfloat16 *__restrict__ A, int64_t lda,
                        const __nv_bfloat16 *__restrict__ B, int64_t ldb,
                        __nv_bfloat16 *__restrict__ C, int64_t ldc, int M, int N, int K) {
    __shared__ float As[16][17], Bs[16][17];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m = blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        const int ka = k0 + tx;
        As[ty][tx] = (m < M && ka < K) ? __bfloat162float(A[static_cast<int64_t>(m) * lda + ka]) : 0.f;
        const int nb = blockIdx.x * 16 + ty;
        Bs[ty][tx] = (nb < N && ka < K) ? __bfloat162float(B[static_cast<int64_t>(nb) * ldb + ka]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(As[ty][k], Bs[tx][k], acc);
        __syncthreads();
    }
    if (m < M && n < N) C[static_cast<int64_t>(m) * ldc + n] = __float2bfloat16_rn(acc);
}

int check_gemm_args(const void *A, int64_t lda, const void *B, int64_t ldb, void *C, int64_t ldc,
                    int64_t M, int64_t N, int64_t K, bool b_colmajor);

// How many K splits to use: only when the tiles alone leave most SMs idle and K is long enough
// (>= 2048) to pay for the second launch (measured: 512x512x8192 44 -> 19 us, 1024^3 13 -> 17 us);
// never fewer than 8 k-blocks (512 columns of K) per split, at most 16.
int pick_splits(int64_t n_tiles, int64_t k_blocks, int sm_count) {
    if (n_tiles * 2 > sm_count || k_blocks < 32) return 1;
    int64_t s = sm_count / n_tiles;
    if (s > k_blocks / 8) s = k_blocks / 8;
    if (s > 16) s = 16;
    return s < 2 ? 1 : (int)s;
}

int gemm_bf16_2cta_launch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                          void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t stream,
                          int tile_n_hint = 0);

// Tile width for the single-CTA kernel: rounds of tiles over the SMs times the time of one tile
// (tensor-bound at 256 and 192 columns, shared-memory-bound and a little slower per flop at 128).
// 1000 x 3000: 96 tiles of 256 columns leave a third of the SMs idle, 128 tiles of 192 columns
// fill one round with tiles that take three quarters of the time.
static int pick_tile_n(int64_t M, int64_t N, int sm_count) {
    const int64_t tiles_m = (M + gemm::BM - 1) / gemm::BM;
    const int widths[3] = {256, 192, 128};
    const int cost_per_tile[3] = {128, 96, 72};
    int best = 256;
    int64_t best_cost = -1;
    for (int i = 0; i < 3; ++i) {
        const int64_t tiles = tiles_m * ((N + widths[i] - 1) / widths[i]);
        const int64_t cost = ((tiles + sm_count - 1) / sm_count) * cost_per_tile[i];
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = widths[i];
        }
    }
    return best;
}

template <int TILE_N>
static int launch_tc_plain(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                           void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
    using namespace gemm;
    constexpr int smem_bytes = gemm::kLayout<TILE_N>.dynamic_bytes;
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                         (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                     (uint64_t)ldb * 2, BK, TILE_N, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + TILE_N - 1) / TILE_N);
    const int grid = (int)(n_tiles < ctx->sm_count ? n_tiles : ctx->sm_count);
    rc = ensure_dynamic_smem(ctx, gemm_bf16_tc_kernel<false, TILE_N>, smem_bytes);
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_tc_kernel<false, TILE_N>, dim3(grid), dim3(NUM_THREADS),
                              (size_t)smem_bytes, stream, ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M,
                              (int)N, (int)K, 1, static_cast<float *>(nullptr), ctx->d_status, GemmEpi{}));
    return after_launch(ctx, "gemm_bf16_tc_kernel");
}

template <int TILE_N>
static int launch_tc_f32x3(gb200_ctx *ctx, const void *A3, const void *B3, float *C, int64_t ldc,
                           int64_t M, int64_t N, int64_t Kp, int accumulate, cudaStream_t stream) {
    using namespace gemm;
    constexpr int smem_bytes = gemm::kLayout<TILE_N>.dynamic_bytes;
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(3 * Kp), (uint64_t)M,
                         (uint64_t)(3 * Kp) * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)(3 * Kp), (uint64_t)N,
                     (uint64_t)(3 * Kp) * 2, BK, TILE_N, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + TILE_N - 1) / TILE_N);
    const int grid = (int)(n_tiles < ctx->sm_count ? n_tiles : ctx->sm_count);
    rc = ensure_dynamic_smem(ctx, gemm_bf16_tc_kernel<true, TILE_N>, smem_bytes);
    if (rc) return rc;
    GemmEpi epi{};
    epi.alpha = 1.0f;
    epi.c32 = C;
    epi.ldc32 = ldc;
    epi.accumulate = accumulate;
    epi.seg_kb = (int)(Kp / BK);
    // the kernel sees one K loop of 6 * Kp: six segment pairs of Kp each
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_tc_kernel<true, TILE_N>, dim3(grid), dim3(NUM_THREADS),
                              (size_t)smem_bytes, stream, ta, tb, static_cast<__nv_bfloat16 *>(nullptr),
                              (int64_t)0, (int)M, (int)N, (int)(6 * Kp), 1, static_cast<float *>(nullptr),
                              ctx->d_status, epi));
    return after_launch(ctx, "gemm_bf16_tc_kernel<f32x3>");
}

// fp32 C (+)= A B from operands already split into three bf16 terms each: A3 is [M][3*Kp], B3 is
// [N][3*Kp] (both K-contiguous, Kp a multiple of 64, zero-padded).  Used by gemm_f32_tc.cu.
int gemm_f32x3_2cta_launch(gb200_ctx *ctx, const void *A3, const void *B3, float *C, int64_t ldc,
                           int64_t M, int64_t N, int64_t Kp, int accumulate, cudaStream_t stream);

int gemm_f32x3_launch(gb200_ctx *ctx, const void *A3, const void *B3, float *C, int64_t ldc,
                      int64_t M, int64_t N, int64_t Kp, int accumulate, cudaStream_t stream) {
    GB200_REQUIRE(ctx->encode_tiled != nullptr, GB200_ERR_NO_DEVICE, "TMA descriptors unavailable");
    // CTA-pair tiles when there are enough of them to fill the SM pairs, as for bf16 operands
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    if (GB200_GEMM_AUTO_PAIR && pair_tiles >= ctx->sm_count / 2)
        return gemm_f32x3_2cta_launch(ctx, A3, B3, C, ldc, M, N, Kp, accumulate, stream);
    const int tile_n = pick_tile_n(M, N, ctx->sm_count);
    if (tile_n == 192) return launch_tc_f32x3<192>(ctx, A3, B3, C, ldc, M, N, Kp, accumulate, stream);
    if (tile_n == 128) return launch_tc_f32x3<128>(ctx, A3, B3, C, ldc, M, N, Kp, accumulate, stream);
    return launch_tc_f32x3<256>(ctx, A3, B3, C, ldc, M, N, Kp, accumulate, stream);
}

// kernel_choice: 0 = pick, 1 = single-CTA 128 x 256 tiles, 2 = CTA-pair tiles (width picked), 3 / 4 =
// single-CTA tiles of 192 / 128 columns, 5 / 6 = CTA-pair tiles of 224 / 256 columns.
int gemm_bf16_dispatch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                       void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t stream,
                       int forced_splits = 0, int kernel_choice = 0) {
    using namespace gemm;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool tc_ok = ctx->encode_tiled && al16(A) && al16(B) && lda % 8 == 0 && ldb % 8 == 0 &&
                       K > 0;
    if (!tc_ok) {
        // row blocks sit in grid.y (at most 65535): taller problems go out as several row panels
        const int64_t panel = (int64_t)kMaxGridY * 16;
        for (int64_t m0 = 0; m0 < M; m0 += panel) {
            const int64_t mp = M - m0 < panel ? M - m0 : panel;
            dim3 grid((unsigned)((N + 15) / 16), (unsigned)((mp + 15) / 16));
            gemm_bf16_simple_kernel<<<grid, 256, 0, stream>>>(
                static_cast<const __nv_bfloat16 *>(A) + m0 * lda, lda, static_cast<const __nv_bfloat16 *>(B), ldb,
                static_cast<__nv_bfloat16 *>(C) + m0 * ldc, ldc, (int)mp, (int)N, (int)K);
            int rc0 = after_launch(ctx, "gemm_bf16_simple_kernel");
            if (rc0) return rc0;
        }
        return GB200_OK;
    }
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                         (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                     (uint64_t)ldb * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int splits = forced_splits > 0 ? forced_splits : pick_splits(n_tiles, (K + BK - 1) / BK, ctx->sm_count);
    // CTA-pair tiles (256 x 256) when there are enough of them to fill the SM pairs
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const bool want_pair = kernel_choice == 2 || kernel_choice == 5 || kernel_choice == 6 ||
                           (kernel_choice == 0 && GB200_GEMM_AUTO_PAIR && pair_tiles >= ctx->sm_count / 2);
    if (want_pair && splits == 1 && forced_splits <= 1)
        return gemm_bf16_2cta_launch(ctx, A, lda, B, ldb, C, ldc, M, N, K, stream,
                                     kernel_choice == 5 ? 224 : kernel_choice == 6 ? 256 : 0);
    if (splits == 1 && forced_splits <= 1 && kernel_choice != 1) {
        const int tile_n = kernel_choice == 3 ? 192 : kernel_choice == 4 ? 128
                                                                        : pick_tile_n(M, N, ctx->sm_count);
        if (tile_n == 192) return launch_tc_plain<192>(ctx, A, lda, B, ldb, C, ldc, M, N, K, stream);
        if (tile_n == 128) return launch_tc_plain<128>(ctx, A, lda, B, ldb, C, ldc, M, N, K, stream);
    }
    float *ws = nullptr;
    if (splits > 1) {
        rc = workspace_reserve(ctx, (size_t)splits * M * N * sizeof(float));
        if (rc) return rc;
        ws = static_cast<float *>(ctx->workspace);
    }
    const int64_t items = n_tiles * splits;
    const int grid = (int)(items < ctx->sm_count ? items : ctx->sm_count);
    rc = ensure_dynamic_smem(ctx, gemm_bf16_tc_kernel<false>, SMEM_BYTES);
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_tc_kernel<false>, dim3(grid), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                              stream, ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M, (int)N, (int)K,
                              splits, ws, ctx->d_status, GemmEpi{}));
    rc = after_launch(ctx, "gemm_bf16_tc_kernel");
    if (rc || splits == 1) return rc;
    const int64_t groups = M * ((N + 3) / 4);
    int64_t blocks = (groups + 255) / 256;
    if (blocks > (int64_t)ctx->sm_count * 8) blocks = (int64_t)ctx->sm_count * 8;
    GB200_CUDA_TRY(launch_pdl(gemm_splitk_reduce_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
                              static_cast<const float *>(ws), splits, static_cast<__nv_bfloat16 *>(C), ldc,
                              (int)M, (int)N));
    return after_launch(ctx, "gemm_splitk_reduce_kernel");
}

// GEMM with consumers fused into the epilogue (single-CTA tiles, no split-K: the reductions and
// the exponential need the complete dot product).
int gemm_bf16_2cta_epilogue_launch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                                   void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha,
                                   const float *row_sub, int apply_exp, const float *row_div, float *row_max,
                                   float *row_sum, cudaStream_t stream);

int gemm_bf16_epilogue_dispatch(gb200_ctx *ctx, const void *A, int64_t lda, const void *B,
                                int64_t ldb, void *C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                const GemmEpi &epi, cudaStream_t stream, int kernel_choice = 0) {
    using namespace gemm;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    GB200_REQUIRE(ctx->encode_tiled != nullptr, GB200_ERR_NO_DEVICE, "TMA descriptors unavailable");
    GB200_REQUIRE(al16(A) && al16(B) && lda % 8 == 0 && ldb % 8 == 0, GB200_ERR_UNSUPPORTED,
                  "gemm epilogue: A and B need 16-byte aligned rows (base and leading dimension)");
    if (epi.row_max || epi.row_sum) {
        epilogue_init_kernel<<<(unsigned)((M + 255) / 256), 256, 0, stream>>>(epi.row_max, epi.row_sum, (int)M);
        int rc0 = after_launch(ctx, "epilogue_init_kernel");
        if (rc0) return rc0;
    }
    // CTA-pair tiles when there are enough of them to fill the SM pairs, as for the plain GEMM
    // (kernel_choice: 0 = pick, 1 = single-CTA tiles, 2 = CTA pairs)
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    if (kernel_choice == 2 || (kernel_choice == 0 && GB200_GEMM_AUTO_PAIR && pair_tiles >= ctx->sm_count / 2))
        return gemm_bf16_2cta_epilogue_launch(ctx, A, lda, B, ldb, C, ldc, M, N, K, epi.alpha, epi.row_sub,
                                              epi.apply_exp, epi.row_div, epi.row_max, epi.row_sum, stream);
    CUtensorMap ta, tb;
    int rc = get_tmap_2d(ctx, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)M,
                         (uint64_t)lda * 2, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B, &ta);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                     (uint64_t)ldb * 2, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B, &tb);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = (int)(n_tiles < ctx->sm_count ? n_tiles : ctx->sm_count);
    rc = ensure_dynamic_smem(ctx, gemm_bf16_tc_kernel<true>, SMEM_BYTES);
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(gemm_bf16_tc_kernel<true>, dim3(grid), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                              stream, ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M, (int)N, (int)K, 1,
                              static_cast<float *>(nullptr), ctx->d_status, epi));
    return after_launch(ctx, "gemm_bf16_tc_kernel<epilogue>");
}

int kernel_regs_gemm_tc() { return kernel_registers(gemm_bf16_tc_kernel<false>); }

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_gemm_bf16_epilogue(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                             void *C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                             const gb200_gemm_epilogue *e, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(e != nullptr, GB200_ERR_INVALID_ARG, "epilogue description is NULL");
    GB200_REQUIRE(C != nullptr || e->row_max != nullptr || e->row_sum != nullptr, GB200_ERR_INVALID_ARG,
                  "nothing to produce: C, row_max and row_sum are all NULL");
    GB200_REQUIRE(M >= 0 && N >= 0 && K >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    GB200_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), GB200_ERR_UNSUPPORTED,
                  "extent beyond 2^31");
    if (M == 0 || N == 0) return GB200_OK;
    GB200_REQUIRE(K > 0, GB200_ERR_UNSUPPORTED, "gemm epilogue: K must be positive");
    GB200_REQUIRE(A != nullptr && B != nullptr, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(lda >= K && ldb >= K && (C == nullptr || ldc >= N), GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row");
    GemmEpi epi{};
    epi.alpha = e->alpha;
    epi.row_sub = e->row_sub;
    epi.row_div = e->row_div;
    epi.row_max = e->row_max;
    epi.row_sum = e->row_sum;
    epi.apply_exp = e->apply_exp;
    return gemm_bf16_epilogue_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, epi,
                                       static_cast<cudaStream_t>(stream));
}

// Test / benchmark hook: kernel chosen by the caller (1 = single-CTA tiles, 2 = CTA pairs).
int gb200_gemm_bf16_epilogue_variant(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                                     void *C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                     const gb200_gemm_epilogue *e, void *stream, int variant) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(e != nullptr, GB200_ERR_INVALID_ARG, "epilogue description is NULL");
    GB200_REQUIRE(C != nullptr || e->row_max != nullptr || e->row_sum != nullptr, GB200_ERR_INVALID_ARG,
                  "nothing to produce: C, row_max and row_sum are all NULL");
    GB200_REQUIRE(M >= 0 && N >= 0 && K >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    GB200_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), GB200_ERR_UNSUPPORTED,
                  "extent beyond 2^31");
    if (M == 0 || N == 0) return GB200_OK;
    GB200_REQUIRE(K > 0, GB200_ERR_UNSUPPORTED, "gemm epilogue: K must be positive");
    GB200_REQUIRE(A != nullptr && B != nullptr, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(lda >= K && ldb >= K && (C == nullptr || ldc >= N), GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row");
    GemmEpi epi{};
    epi.alpha = e->alpha;
    epi.row_sub = e->row_sub;
    epi.row_div = e->row_div;
    epi.row_max = e->row_max;
    epi.row_sum = e->row_sum;
    epi.apply_exp = e->apply_exp;
    return gemm_bf16_epilogue_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, epi,
                                       static_cast<cudaStream_t>(stream), variant);
}

int gb200_gemm_bf16(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                    void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_bf16_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K,
                              static_cast<cudaStream_t>(stream));
}

int gb200_gemm_bf16_cluster(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                            void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int cluster_x,
                            void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(cluster_x == 1 || cluster_x == 2, GB200_ERR_UNSUPPORTED,
                  "the bf16 GEMM has kernels for clusters of 1 and 2 thread blocks (asked for %d)", cluster_x);
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_bf16_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K, static_cast<cudaStream_t>(stream), 1,
                              cluster_x);
}

// Test / benchmark hook: same contract with the number of K splits chosen by the caller
// (0 = let the library pick, 1 = no split).
int gb200_gemm_bf16_splitk(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                           void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, void *stream,
                           int splits) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    GB200_REQUIRE(splits >= 0 && splits <= 64, GB200_ERR_INVALID_ARG, "splits out of range");
    return gemm_bf16_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K,
                              static_cast<cudaStream_t>(stream), splits);
}

// ---- split-K GEMM for callers that must not allocate --------------------------------------
//
// Same kernels as gb200_gemm_bf16 with K splits, but the fp32 slab workspace and the status word
// live in the two file-scope device arrays below instead of memory owned by a gb200_ctx, and no
// context is needed at all.  It serves host code that is not allowed to reach the CUDA allocator
// at the point where it needs a GEMM: a latency-critical serving loop (cudaMalloc and cudaFree
// synchronise the whole device), a process whose device memory has been handed in full to
// another allocator so that cudaMalloc would fail, or a callback that runs where allocation
// calls are forbidden.  The price is a fixed capacity: kStaticWsFloats floats (16 MiB), which
// every GPU that loads this library keeps reserved until the process exits.
constexpr size_t kStaticWsFloats = 4u * 1024u * 1024u;
static __device__ __align__(256) float g_static_ws[kStaticWsFloats];
static __device__ __align__(256) int g_static_status[64];

namespace {
struct StaticDeviceState {
    bool ready = false;
    float *ws = nullptr;        // device address of g_static_ws on this device
    int *status = nullptr;      // device address of g_static_status on this device
    int sm_count = 0;
    gb200::EncodeTiledFn encode = nullptr;
};
constexpr int kMaxDevices = 64;
StaticDeviceState g_static_state[kMaxDevices];
std::mutex g_static_mu;

// In host code `g_static_ws` names a host-side shadow of the array, not device memory; the
// device address has to be asked for, per device, with that device current.
int static_setup(int device, StaticDeviceState **out) {
    GB200_REQUIRE(device >= 0 && device < kMaxDevices, GB200_ERR_UNSUPPORTED,
                  "device ordinal %d beyond the %d this entry point tracks", device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDeviceState &st = g_static_state[device];
    if (!st.ready) {
        void *p = nullptr;
        GB200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_ws));
        st.ws = static_cast<float *>(p);
        GB200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_status));
        st.status = static_cast<int *>(p);
        int major = 0;
        GB200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        GB200_REQUIRE(major == 10, GB200_ERR_NO_DEVICE, "device %d is not sm_100", device);
        GB200_CUDA_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, device));
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        GB200_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        GB200_REQUIRE(q == cudaDriverEntryPointSuccess && fn != nullptr, GB200_ERR_NO_DEVICE,
                      "cuTensorMapEncodeTiled is not available from this driver");
        st.encode = reinterpret_cast<gb200::EncodeTiledFn>(fn);
        GB200_CUDA_TRY(cudaFuncSetAttribute(gemm_bf16_tc_kernel<false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            gemm::SMEM_BYTES));
        st.ready = true;
    }
    *out = &st;
    return GB200_OK;
}

int encode_bf16_map(const StaticDeviceState &st, const void *ptr, uint64_t inner, uint64_t rows,
                    uint64_t pitch_bytes, uint32_t box_rows, CUtensorMap *tm) {
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {(cuuint32_t)gemm::BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult rc = st.encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims,
                            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    GB200_REQUIRE(rc == CUDA_SUCCESS, GB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)rc);
    return GB200_OK;
}
}  // namespace

int gb200_gemm_bf16_splitk_static(const void *A, int64_t lda, const void *B, int64_t ldb, void *C,
                                  int64_t ldc, int64_t M, int64_t N, int64_t K, int splits,
                                  void *stream_) {
    using namespace gemm;
    int rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    GB200_REQUIRE(K > 0, GB200_ERR_INVALID_ARG, "K must be positive");
    GB200_REQUIRE(splits >= 0 && splits <= 16, GB200_ERR_INVALID_ARG, "splits must be 0 (choose) .. 16");
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    GB200_REQUIRE(al16(A) && al16(B) && lda % 8 == 0 && ldb % 8 == 0, GB200_ERR_UNSUPPORTED,
                  "operands need 16-byte aligned bases and pitches (TMA)");
    int device = 0;
    GB200_CUDA_TRY(cudaGetDevice(&device));
    // The kernels run on the current device: operands in host memory or on another GPU would be
    // read through addresses that mean nothing there.  The query is host-only and allocates nothing.
    const void *operands[3] = {A, B, C};
    for (int i = 0; i < 3; ++i) {
        cudaPointerAttributes attr;
        GB200_CUDA_TRY(cudaPointerGetAttributes(&attr, operands[i]));
        GB200_REQUIRE((attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) &&
                          (attr.type == cudaMemoryTypeManaged || attr.device == device),
                      GB200_ERR_INVALID_ARG,
                      "operand %c is not device memory of the current device %d (memory type %d, device %d)",
                      "ABC"[i], device, (int)attr.type, attr.device);
    }
    StaticDeviceState *st = nullptr;
    rc = static_setup(device, &st);
    if (rc) return rc;
    const int64_t n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int64_t k_blocks = (K + BK - 1) / BK;
    if (splits == 0) splits = pick_splits(n_tiles, k_blocks, st->sm_count);
    const size_t need = splits > 1 ? (size_t)splits * (size_t)M * (size_t)N : 0;
    GB200_REQUIRE(need <= kStaticWsFloats, GB200_ERR_TOO_LARGE,
                  "splits * M * N = %llu floats exceeds the fixed workspace of %llu floats (16 MiB); "
                  "use fewer splits or gb200_gemm_bf16 with a context",
                  (unsigned long long)need, (unsigned long long)kStaticWsFloats);
    CUtensorMap ta, tb;
    rc = encode_bf16_map(*st, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BM, &ta);
    if (rc) return rc;
    rc = encode_bf16_map(*st, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BN, &tb);
    if (rc) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t items = n_tiles * splits;
    const int grid = (int)(items < st->sm_count ? items : st->sm_count);
    // Every (tile, split) item overwrites its whole region of the slabs, so nothing left in the
    // array by an earlier call is ever read; the status word is only ever set, never relied on.
    gemm_bf16_tc_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(
        ta, tb, static_cast<__nv_bfloat16 *>(C), ldc, (int)M, (int)N, (int)K, splits,
        splits > 1 ? st->ws : nullptr, st->status, GemmEpi{});
    cudaError_t err = cudaPeekAtLastError();
    GB200_REQUIRE(err == cudaSuccess, GB200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(err));
    if (splits > 1) {
        const int64_t groups = M * ((N + 3) / 4);
        int64_t blocks = (groups + 255) / 256;
        if (blocks > (int64_t)st->sm_count * 8) blocks = (int64_t)st->sm_count * 8;
        gemm_splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
            st->ws, splits, static_cast<__nv_bfloat16 *>(C), ldc, (int)M, (int)N);
        err = cudaPeekAtLastError();
        GB200_REQUIRE(err == cudaSuccess, GB200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(err));
    }
    return GB200_OK;
}

// Reports whether a kernel of gb200_gemm_bf16_splitk_static gave up a bounded wait on the current
// device since the last query.  Synchronises the device (the word is read after everything
// enqueued so far), clears the word, allocates nothing.
int gb200_static_status(int *code) {
    if (code) *code = 0;
    int device = 0;
    GB200_CUDA_TRY(cudaGetDevice(&device));
    StaticDeviceState *st = nullptr;
    int rc = static_setup(device, &st);
    if (rc) return rc;
    GB200_CUDA_TRY(cudaDeviceSynchronize());
    int word = 0;
    GB200_CUDA_TRY(cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (word == 0) return GB200_OK;
    GB200_CUDA_TRY(cudaMemset(st->status, 0, sizeof(int)));
    if (code) *code = word;
    set_error("a kernel of gb200_gemm_bf16_splitk_static gave up a bounded wait (status code %d); "
              "products computed since the last query are not valid", word);
    return GB200_ERR_TIMEOUT;
}

// Test / benchmark hook: kernel chosen by the caller (1 = single-CTA tiles, 2 = CTA-pair tiles).
int gb200_gemm_bf16_variant(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                            void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, void *stream,
                            int variant) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return gemm_bf16_dispatch(ctx, A, lda, B, ldb, C, ldc, M, N, K,
                              static_cast<cudaStream_t>(stream), 1, variant);
}

int gb200_gemm_bf16_host(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                         void *C, int64_t ldc, int64_t M, int64_t N, int64_t K) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_gemm_args(A, lda, B, ldb, C, ldc, M, N, K, true);
    if (rc) return rc < 0 ? rc : GB200_OK;
    const int64_t dk = (K + 7) / 8 * 8, dn = (N + 7) / 8 * 8;
    rc = stage_reserve(ctx, 0, (size_t)M * dk * 2 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 1, (size_t)N * dk * 2 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 2, (size_t)M * dn * 2 + 16);
    if (rc) return rc;
    cudaStream_t s = ctx->copy_stream[0];
    if (K > 0) {
        GB200_CUDA_TRY(cudaMemcpy2DAsync(ctx->stage[0], dk * 2, A, lda * 2, K * 2, M,
                                         cudaMemcpyHostToDevice, s));
        GB200_CUDA_TRY(cudaMemcpy2DAsync(ctx->stage[1], dk * 2, B, ldb * 2, K * 2, N,
                                         cudaMemcpyHostToDevice, s));
    }
    rc = gemm_bf16_dispatch(ctx, ctx->stage[0], dk, ctx->stage[1], dk, ctx->stage[2], dn, M, N, K, s);
    if (rc) return rc;
    GB200_CUDA_TRY(cudaMemcpy2DAsync(C, ldc * 2, ctx->stage[2], dn * 2, N * 2, M,
                                     cudaMemcpyDeviceToHost, s));
    return host_finish(ctx, s, nullptr);
}

}  // extern "C"
