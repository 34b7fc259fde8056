// fp32 matrix multiply on the tensor cores in ONE launch, for problems too small to pay for the
// two split pre-passes of gemm_f32_tc.cu (the reference's 512^3 case,
// gernels/mm/kernel_10.cu:108-131 / test/test-cpu-mm.cpp:13-83).
//
// Same arithmetic as gemm_f32_tc.cu: every fp32 operand is written as a sum of three bf16 numbers
// (24 mantissa bits in all, each residual exact in fp32), and the six partial products whose
// magnitude can matter are accumulated in fp32 in TMEM.  Here the split happens inside the kernel:
// eight warps read a 64-wide K chunk of the CTA's A rows (128 x 64 fp32) and of B (64 x 64 fp32,
// row-major) straight from global memory, two chunks ahead, split each pair of values with packed
// conversions, and write the three bf16 terms of A and of B^T into shared memory in exactly the
// layout TMA would have produced with 128-byte swizzle (rows of 64 bf16; the 16-byte chunk index of
// a row XORed with row mod 8; groups of 8 rows 1024 bytes apart), which is the layout the K-major
// shared-memory descriptors of tcgen05.mma read.  One thread of a ninth warp issues 6 x 4 MMAs of
// 128 x 64 x 16 per chunk into two accumulators: a1 b1 has its own, because the tensor core
// truncates when it adds into the accumulator and the five small products lose less among
// themselves.  Two chunk buffers: the conversion of chunk c+1 runs under the MMAs of chunk c.
//
// One tile of 128 x 64 per CTA, or, when the tiles are few, per cluster of 2 or 4 CTAs: each CTA
// takes a range of the K chunks (the conversions, which bound the kernel, spread over four times
// the SMs), leaves its partial tile in its shared memory, and after a cluster barrier adds up its
// share of the tile's rows out of all the CTAs' shared memories in the order of their rank.  No
// workspace, no pre-pass.
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
constexpr uint32_t TMEM_COLS = 128;   // two accumulators of 64 columns: a1 b1, and the five smaller products

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

// v = b1 + b2 + b3 with bf16 terms (each residual exact in fp32), for two values at once: each
// term comes out as a bf16 pair (v0 in the low half) from one cvt.rn.bf16x2.f32; the conversion
// instructions are what bounds this kernel's eight converting warps, and the packed form halves
// their number.
__device__ __forceinline__ void split3_pair(float v0, float v1, uint32_t &p1, uint32_t &p2, uint32_t &p3) {
    p1 = pack_bf16(v0, v1);
    float r0 = v0 - __uint_as_float(p1 << 16), r1 = v1 - __uint_as_float(p1 & 0xffff0000u);   // exact
    p2 = pack_bf16(r0, r1);
    r0 -= __uint_as_float(p2 << 16);                                                            // exact
    r1 -= __uint_as_float(p2 & 0xffff0000u);
    p3 = pack_bf16(r0, r1);
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
    // A cluster of csize CTAs shares one tile: CTA r takes the K chunks [c_begin, c_end) and the
    // partial tiles are added up through distributed shared memory at the end (csize = 1: no
    // cluster, the tile goes from TMEM to C).  The host sizes the cluster so that no range is empty.
    const int csize = static_cast<int>(cluster_nctarank()), crank = static_cast<int>(cluster_ctarank());
    const int tile = static_cast<int>(blockIdx.x) / csize;
    const int tiles_n = (N + BN - 1) / BN;
    const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
    const int all_chunks = (K + BK - 1) / BK;
    const int per_rank = (all_chunks + csize - 1) / csize;
    const int c_begin = crank * per_rank;
    const int k_chunks = max(0, min(per_rank, all_chunks - c_begin));   // this CTA's, counted from c_begin

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
                        // a1 b1 has an accumulator of its own: the tensor core truncates when it
                        // adds into the accumulator, and five small products added into a large
                        // sum per step lose six times as much as they do among themselves
                        // (measured at K = 1024: 6.8e-6 relative against 1.1e-6)
                        if (p == 5)
                            umma_f16_ss(tmem_base, da, db, idesc, (c | ks) != 0 ? 1u : 0u);   // c counts this CTA's chunks
                        else
                            umma_f16_ss(tmem_base + BN, da, db, idesc, (c | ks | p) != 0 ? 1u : 0u);
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
        // B chunk: 64 k x 64 n, wanted as B^T (row n, 64 k): thread t takes column n = t mod 64 and
        // the groups of 8 consecutive k  t / 64  and  t / 64 + 4  (a warp's load of one k is 32
        // consecutive n of one B row, coalesced), so that the 8 bf16 of a term are one 16-byte
        // store, which the swizzle spreads over the banks.
        const int t = threadIdx.x;
        bool ok = true;
        // two chunks of operands in registers: from a cold L2 a chunk's loads take longer than its
        // conversion, so the loads of chunk c + 2 are issued as soon as chunk c has been converted
        float4 ra[2][8];
        float rb[2][2][8];
        auto load_chunk = [&](int c, float4(&qa)[8], float(&qb)[2][8]) {
            const int k0 = (c_begin + c) * BK;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int g = t + i * 256;
                const int row = m0 + (g >> 4), k = k0 + (g & 15) * 4;
                const float *src = A + static_cast<int64_t>(row) * lda + k;
                if (vec_ok && row < M && k + 4 <= K) {
                    qa[i] = __ldg(reinterpret_cast<const float4 *>(src));
                } else {
                    qa[i].x = (row < M && k + 0 < K) ? src[0] : 0.0f;
                    qa[i].y = (row < M && k + 1 < K) ? src[1] : 0.0f;
                    qa[i].z = (row < M && k + 2 < K) ? src[2] : 0.0f;
                    qa[i].w = (row < M && k + 3 < K) ? src[3] : 0.0f;
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int n = n0 + (t & 63), kg = (t >> 6) + 4 * i;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int k = k0 + kg * 8 + e;
                    qb[i][e] = (k < K && n < N) ? __ldg(B + static_cast<int64_t>(k) * ldb + n) : 0.0f;
                }
            }
        };
        // split chunk c (in qa / qb) into its stage, then refill the registers with chunk c + 2
        auto convert_chunk = [&](int c, float4(&qa)[8], float(&qb)[2][8]) -> bool {
            const int s = c % STAGES;
            if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) - 1) & 1, status, 362)) return false;
            unsigned char *a_tile = smem + s * STAGE_BYTES;
            unsigned char *b_tile = a_tile + 3 * A_TERM_BYTES;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int g = t + i * 256;
                const int row = g >> 4, k = (g & 15) * 4;
                uint32_t h[3][2];
                split3_pair(qa[i].x, qa[i].y, h[0][0], h[1][0], h[2][0]);
                split3_pair(qa[i].z, qa[i].w, h[0][1], h[1][1], h[2][1]);
                const uint32_t off = sw128_offset(row, k);        // 4 consecutive k: one 8-byte store
#pragma unroll
                for (int term = 0; term < 3; ++term)
                    *reinterpret_cast<uint2 *>(a_tile + term * A_TERM_BYTES + off) = make_uint2(h[term][0], h[term][1]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int n = t & 63, kg = (t >> 6) + 4 * i;
                uint32_t h[3][4];
#pragma unroll
                for (int e = 0; e < 4; ++e) split3_pair(qb[i][2 * e], qb[i][2 * e + 1], h[0][e], h[1][e], h[2][e]);
                const uint32_t off = sw128_offset(n, kg * 8);     // transposed: row = n, 8 consecutive k
#pragma unroll
                for (int term = 0; term < 3; ++term)
                    *reinterpret_cast<uint4 *>(b_tile + term * B_TERM_BYTES + off) =
                        make_uint4(h[term][0], h[term][1], h[term][2], h[term][3]);
            }
            if (c + 2 < k_chunks) load_chunk(c + 2, qa, qb);
            fence_proxy_async_smem();       // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
            return true;
        };
        if (k_chunks > 0) load_chunk(0, ra[0], rb[0]);
        if (k_chunks > 1) load_chunk(1, ra[1], rb[1]);
        for (int c = 0; c < k_chunks && ok; c += 2) {
            ok = convert_chunk(c, ra[0], rb[0]);
            if (ok && c + 1 < k_chunks) ok = convert_chunk(c + 1, ra[1], rb[1]);
        }

        // ---------------- epilogue (warps 0-3): TMEM -> fp32 C ----------------
        if (warp < 4 && k_chunks > 0 && csize > 1) {
            // partial tile -> this CTA's shared memory (over the chunk buffers, which the MMAs have
            // left): row-major 128 x 64 floats, the 16-byte pieces of a row rotated by the row so
            // that a warp's stores (32 rows, the same piece) spread over the banks
            if (ok) ok = mbar_wait(acc_full, 0, status, 363);
            if (ok) {
                tc_fence_after();
                const int r = warp * 32 + lane;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
                float *part = reinterpret_cast<float *>(smem);
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ++ch) {
                    uint32_t v[32], w[32];
                    tmem_ld_32x32(taddr + ch * 32, v);
                    tmem_ld_32x32(taddr + BN + ch * 32, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(w[i]));
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<float4 *>(part + (r * 16 + ((ch * 8 + q) ^ (r & 15))) * 4) =
                            make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                        __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                }
            }
        } else if (warp < 4 && k_chunks > 0) {
            if (ok) ok = mbar_wait(acc_full, 0, status, 363);
            if (ok) {
                tc_fence_after();
                const int row = m0 + warp * 32 + lane;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ++ch) {
                    uint32_t r[32], w[32];
                    tmem_ld_32x32(taddr + ch * 32, r);
                    tmem_ld_32x32(taddr + BN + ch * 32, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(w[i]));
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

    if (csize > 1) {
        // CTA r adds up rows [r * share, (r + 1) * share) of the tile out of all the CTAs' shared
        // memories, in the order of their rank
        cluster_sync_all();
        const int share = (BM + csize - 1) / csize;
        const float *part = reinterpret_cast<const float *>(smem);
        const bool v4 = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
        if (warp < CONVERT_WARPS) {
            for (int idx = threadIdx.x; idx < share * 16; idx += CONVERT_WARPS * 32) {
                const int r = crank * share + (idx >> 4), piece = idx & 15;
                const int row = m0 + r, col = n0 + piece * 4;
                if (r >= BM || row >= M || col >= N) continue;
                const uint32_t addr = smem_u32(part + (r * 16 + (piece ^ (r & 15))) * 4);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int k = 0; k < csize; ++k) {
                    const float4 v = ld_dsmem_f4(map_to_cta(addr, k));
                    acc.x += v.x;
                    acc.y += v.y;
                    acc.z += v.z;
                    acc.w += v.w;
                }
                float *dst = C + static_cast<int64_t>(row) * ldc + col;
                if (v4 && col + 4 <= N) {
                    if (accumulate) {
                        const float4 cc = *reinterpret_cast<const float4 *>(dst);
                        acc.x += cc.x; acc.y += cc.y; acc.z += cc.z; acc.w += cc.w;
                    }
                    *reinterpret_cast<float4 *>(dst) = acc;
                } else {
                    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
                    for (int j = 0; j < 4; ++j)
                        if (col + j < N) dst[j] = a4[j] + (accumulate ? dst[j] : 0.0f);
                }
            }
        }
        cluster_sync_all();   // no CTA leaves while another still reads its shared memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == f32f::CONVERT_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, f32f::TMEM_COLS);
    }
}

// fp32 C (+)= A B, all row-major, one launch (K > 0).
// cluster_hint: 0 = pick the cluster size, n = that many CTAs per tile (1: no cluster).
int gemm_f32_fused_launch(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                          int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate, cudaStream_t stream,
                          int cluster_hint) {
    using namespace f32f;
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    GB200_REQUIRE(tiles < (1ll << 31), GB200_ERR_UNSUPPORTED, "too many tiles for one launch");
    int rc = ensure_dynamic_smem(ctx, gemm_f32_fused_kernel, kLayout.dynamic_bytes);
    if (rc) return rc;
    const int vec_ok = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0 &&
                       lda % 4 == 0 && ldb % 4 == 0;
    // Few tiles: the K chunks of a tile are dealt out to a cluster of 2 or 4 CTAs (every CTA at
    // least two chunks), as many as keep the CTA count within the SMs.  (Larger clusters of CTAs
    // that each need most of an SM's shared memory are not all resident at once.)
    const int chunks = (int)((K + BK - 1) / BK);
    int csize = 1;
    while (csize * 2 <= 4 && tiles * (csize * 2) <= ctx->sm_count && chunks >= 2 * (csize * 2)) csize *= 2;
    if (cluster_hint > 0) csize = cluster_hint > 8 ? 8 : cluster_hint;
    if (csize > 1) {
        const int per = (chunks + csize - 1) / csize;
        csize = (chunks + per - 1) / per;               // no empty range
    }
    if (csize > 1) {
        GB200_CUDA_TRY(launch_pdl_cluster(gemm_f32_fused_kernel, dim3((unsigned)(tiles * csize)), dim3(NUM_THREADS),
                                          (size_t)kLayout.dynamic_bytes, stream, (unsigned)csize, A, lda, B, ldb, C, ldc,
                                          (int)M, (int)N, (int)K, accumulate, vec_ok, ctx->d_status));
    } else {
        GB200_CUDA_TRY(launch_pdl(gemm_f32_fused_kernel, dim3((unsigned)tiles), dim3(NUM_THREADS),
                                  (size_t)kLayout.dynamic_bytes, stream, A, lda, B, ldb, C, ldc, (int)M, (int)N, (int)K,
                                  accumulate, vec_ok, ctx->d_status));
    }
    return after_launch(ctx, "gemm_f32_fused_kernel");
}

}  // namespace gb200
