// fp32 matrix multiply on the tensor cores in ONE launch, for problems too small to pay for the
// two split pre-passes of gemm_f32_tc.cu (the reference's 512^3 case,
// gernels/mm/kernel_10.cu:108-131 / test/test-cpu-mm.cpp:13-83).
//
// Same arithmetic as gemm_f32_tc.cu: every fp32 operand is written as a sum of three bf16 numbers
// (24 mantissa bits in all, each residual exact in fp32), and the six partial products whose
// magnitude can matter are accumulated in fp32 in TMEM, smallest first.  Here the split happens
// inside the kernel: eight warps read a 64-wide K chunk of the CTA's A rows (128 x 64 fp32) and of
// B (64 x 64 fp32, row-major) straight from global memory, split each value, and write the three
// bf16 terms of A and of B^T into shared memory in exactly the layout TMA would have produced with
// 128-byte swizzle (rows of 64 bf16; the 16-byte chunk index of a row XORed with row mod 8; groups
// of 8 rows 1024 bytes apart), which is the layout the K-major shared-memory descriptors of
// tcgen05.mma read.  One thread of a ninth warp issues 6 x 4 MMAs of 128 x 64 x 16 per chunk.  Two
// chunk buffers: the conversion of chunk c+1 runs under the MMAs of chunk c.  No workspace, no
// pre-pass, one tile of 128 x 64 per CTA.
#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

namespace f32f {
constexpr int BM = 128, BN = 64, BK = 64;
constexpr int CONVERT_WARPS = 8;
constexpr int NUM_THREADS = (CONVERT_WARPS + 1) * 32;     // 8 converting warps + the MMA warp
constexpr int A_TERM_BYTES = BM * BK * 2;                 // 16 KiB: one bf16 term of the A chunk
constexpr int B_TERM_BYTES = BN * BK * 2;                 //  8 KiB: one bf16 term of the B^T chunk
constexpr int STAGE_BYTES = 3 * (A_TERM_BYTES + B_TERM_BYTES);   // 72 KiB
constexpr int STAGES = 2;
constexpr uint32_t TMEM_COLS = 64;

struct Layout {
    smem::Region stages, full, empty, acc_full, tmem_slot;
    int dynamic_bytes = 0;
};
constexpr Layout plan() {
    Layout l;
    smem::Planner p;
    l.stages = p.tiles(STAGES, STAGE_BYTES);
    l.full = p.barriers(STAGES);
    l.empty = p.barriers(STAGES);
    l.acc_full = p.barriers(1);
    l.tmem_slot = p.words(1);
    l.dynamic_bytes = p.dynamic_bytes();
    return l;
}
constexpr Layout kLayout = plan();
static_assert(kLayout.dynamic_bytes <= smem::kMaxDynamicBytes, "layout exceeds a block's shared memory");
}  // namespace f32f

__device__ __forceinline__ void split3_bits(float v, uint32_t &h1, uint32_t &h2, uint32_t &h3) {
    const __nv_bfloat16 b1 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(b1);       // exact
    const __nv_bfloat16 b2 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(b2);      // exact
    const __nv_bfloat16 b3 = __float2bfloat16_rn(r2);
    h1 = __bfloat16_as_ushort(b1);
    h2 = __bfloat16_as_ushort(b2);
    h3 = __bfloat16_as_ushort(b3);
}

// Byte offset of element (row, k) in a K-major tile of 64 bf16 per row laid out as TMA's
// SWIZZLE_128B does: 16-byte chunk index XOR (row mod 8); 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint32_t sw128_offset(int row, int k) {
    const uint32_t chunk = static_cast<uint32_t>(k >> 3) ^ static_cast<uint32_t>(row & 7);
    return static_cast<uint32_t>(row >> 3) * 1024u + static_cast<uint32_t>(row & 7) * 128u + chunk * 16u +
           static_cast<uint32_t>(k & 7) * 2u;
}

__global__ void __launch_bounds__(f32f::NUM_THREADS, 1)
gemm_f32_fused_kernel(const float *__restrict__ A, int64_t lda, const float *__restrict__ B, int64_t ldb,
                      float *__restrict__ C, int64_t ldc, int M, int N, int K, int accumulate, int vec_ok,
                      int *status) {
    using namespace f32f;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kLayout.full.offset);       // [2] converters -> MMA
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + kLayout.empty.offset);     // [2] MMA -> converters
    uint64_t *acc_full = reinterpret_cast<uint64_t *>(smem + kLayout.acc_full.offset);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kLayout.tmem_slot.offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN;
    const int m0 = (blockIdx.x / tiles_n) * BM, n0 = (blockIdx.x % tiles_n) * BN;
    const int k_chunks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], CONVERT_WARPS);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        mbar_fence_init();
    }
    if (warp == CONVERT_WARPS) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp == CONVERT_WARPS) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, 0);   // A and B^T both K-major
            bool ok = true;
            for (int c = 0; c < k_chunks && ok; ++c) {
                const int s = c % STAGES;
                if (!mbar_wait(&full[s], (c / STAGES) & 1, status, 361)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES);
                const uint32_t b_base = a_base + 3 * A_TERM_BYTES;
                // per 16-wide K step: a3 b1, a2 b2, a1 b3, a2 b1, a1 b2, a1 b1 (smallest first)
                constexpr int ta[6] = {2, 1, 0, 1, 0, 0};
                constexpr int tb[6] = {0, 1, 2, 0, 1, 0};
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) {
#pragma unroll
                    for (int p = 0; p < 6; ++p) {
                        const uint64_t da = umma_desc_sw128(a_base + ta[p] * A_TERM_BYTES + ks * 32, 16, 1024);
                        const uint64_t db = umma_desc_sw128(b_base + tb[p] * B_TERM_BYTES + ks * 32, 16, 1024);
                        umma_f16_ss(tmem_base, da, db, idesc, (c | ks | p) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(&empty[s]);                 // the chunk buffer may be rewritten
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        // ---------------- load, split, lay out (8 warps) ----------------
        // A chunk: 128 rows x 64 k = 2048 groups of 4 consecutive k; thread t takes groups t, t+256, ...
        // (8 per chunk): a warp covers 2 rows of 64 k, 16-byte loads, coalesced.
        // B chunk: 64 k x 64 n = 1024 groups of 4 consecutive n (4 per thread): each value goes to
        // row n of the B^T tile at column k.
        const int t = threadIdx.x;
        bool ok = true;
        float4 ra[8], rb[4];
        auto load_chunk = [&](int c) {
            const int k0 = c * BK;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int g = t + i * 256;
                const int row = m0 + (g >> 4), k = k0 + (g & 15) * 4;
                const float *src = A + static_cast<int64_t>(row) * lda + k;
                if (vec_ok && row < M && k + 4 <= K) {
                    ra[i] = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    ra[i].x = (row < M && k + 0 < K) ? src[0] : 0.0f;
                    ra[i].y = (row < M && k + 1 < K) ? src[1] : 0.0f;
                    ra[i].z = (row < M && k + 2 < K) ? src[2] : 0.0f;
                    ra[i].w = (row < M && k + 3 < K) ? src[3] : 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int g = t + i * 256;
                const int k = k0 + (g >> 4), n = n0 + (g & 15) * 4;
                const float *src = B + static_cast<int64_t>(k) * ldb + n;
                if (vec_ok && k < K && n + 4 <= N) {
                    rb[i] = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    rb[i].x = (k < K && n + 0 < N) ? src[0] : 0.0f;
                    rb[i].y = (k < K && n + 1 < N) ? src[1] : 0.0f;
                    rb[i].z = (k < K && n + 2 < N) ? src[2] : 0.0f;
                    rb[i].w = (k < K && n + 3 < N) ? src[3] : 0.0f;
                }
            }
        };
        if (k_chunks > 0) load_chunk(0);
        for (int c = 0; c < k_chunks; ++c) {
            const int s = c % STAGES;
            if (ok && c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) - 1) & 1, status, 362)) ok = false;
            if (!ok) break;
            unsigned char *a_tile = smem + s * STAGE_BYTES;
            unsigned char *b_tile = a_tile + 3 * A_TERM_BYTES;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int g = t + i * 256;
                const int row = g >> 4, k = (g & 15) * 4;
                uint32_t h[3][4];
                split3_bits(ra[i].x, h[0][0], h[1][0], h[2][0]);
                split3_bits(ra[i].y, h[0][1], h[1][1], h[2][1]);
                split3_bits(ra[i].z, h[0][2], h[1][2], h[2][2]);
                split3_bits(ra[i].w, h[0][3], h[1][3], h[2][3]);
                const uint32_t off = sw128_offset(row, k);        // 4 consecutive k: one 8-byte store
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    uint2 v;
                    v.x = h[term][0] | (h[term][1] << 16);
                    v.y = h[term][2] | (h[term][3] << 16);
                    *reinterpret_cast<uint2 *>(a_tile + term * A_TERM_BYTES + off) = v;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int g = t + i * 256;
                const int k = g >> 4, n = (g & 15) * 4;
                const float vals[4] = {rb[i].x, rb[i].y, rb[i].z, rb[i].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint32_t h1, h2, h3;
                    split3_bits(vals[e], h1, h2, h3);
                    const uint32_t off = sw128_offset(n + e, k);  // transposed: row = n, column = k
                    *reinterpret_cast<uint16_t *>(b_tile + 0 * B_TERM_BYTES + off) = static_cast<uint16_t>(h1);
                    *reinterpret_cast<uint16_t *>(b_tile + 1 * B_TERM_BYTES + off) = static_cast<uint16_t>(h2);
                    *reinterpret_cast<uint16_t *>(b_tile + 2 * B_TERM_BYTES + off) = static_cast<uint16_t>(h3);
                }
            }
            // next chunk's global loads are in flight while the MMA warp works on this one
            if (c + 1 < k_chunks) load_chunk(c + 1);
            fence_proxy_async_smem();       // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }

        // ---------------- epilogue (warps 0-3): TMEM -> fp32 C ----------------
        if (warp < 4 && k_chunks > 0) {
            if (ok) ok = mbar_wait(acc_full, 0, status, 363);
            if (ok) {
                tc_fence_after();
                const int row = m0 + warp * 32 + lane;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ++ch) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + ch * 32, r);
                    tmem_ld_wait();
                    const int col = n0 + ch * 32;
                    if (row < M && col < N) {
                        float *dst = C + static_cast<int64_t>(row) * ldc + col;
                        const bool v4 = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && col + 32 <= N;
                        if (v4) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float4 o = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                                if (accumulate) {
                                    const float4 cc = *reinterpret_cast<const float4 *>(dst + 4 * q);
                                    o.x += cc.x; o.y += cc.y; o.z += cc.z; o.w += cc.w;
                                }
                                *reinterpret_cast<float4 *>(dst + 4 * q) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < N) dst[j] = __uint_as_float(r[j]) + (accumulate ? dst[j] : 0.0f);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == f32f::CONVERT_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, f32f::TMEM_COLS);
    }
}

// fp32 C (+)= A B, all row-major, one launch (K > 0).
int gemm_f32_fused_launch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                          int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate, cudaStream_t stream) {
    using namespace f32f;
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    GB200_REQUIRE(tiles < (1ll << 31), GB200_ERR_UNSUPPORTED, "too many tiles for one launch");
    int rc = ensure_dynamic_smem(ctx, gemm_f32_fused_kernel, kLayout.dynamic_bytes);
    if (rc) return rc;
    const int vec_ok = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0 &&
                       lda % 4 == 0 && ldb % 4 == 0;
    GB200_CUDA_TRY(launch_pdl(gemm_f32_fused_kernel, dim3((unsigned)tiles), dim3(NUM_THREADS),
                              (size_t)kLayout.dynamic_bytes, stream, A, lda, B, ldb, C, ldc, (int)M, (int)N, (int)K,
                              accumulate, vec_ok, ctx->d_status));
    return after_launch(ctx, "gemm_f32_fused_kernel");
}

}  // namespace gb200
