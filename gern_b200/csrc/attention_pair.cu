// GEMM -> row softmax -> GEMM chain on CTA pairs with two Q tiles per CTA.
//
// The softmax, the TMEM layout (S_t and O_t in TMEM, P_t written back over S_t and read from there
// as the A operand of P V) and the order of work are those of attention_bf16_kernel (attention.cu).
// What changes is who multiplies: the two CTAs of a cluster share every MMA.  The leader issues
// M256 N128 K16 instructions (tcgen05 cta_group::2) whose A operand is tile t of BOTH CTAs and
// whose B operand is split across the pair -- CTA r holds kv rows [64 r, 64 r + 64) of K_j and
// head-dimension columns [64 r, 64 r + 64) of V_j.  Consequences, against one CTA per two tiles:
//   * Q K^T reads 4 KiB of Q and 2 KiB of K per SM and MMA from shared memory instead of 4 + 4; with
//     both operands in shared memory a 128 x 128 x 16 MMA needs the whole 128 bytes per clock of
//     the shared-memory port, and the single-CTA kernel's MMAs measured 77 cycles on average
//     where the tensor pipe needs 64;
//   * each CTA fetches half of every K/V block, so the L2 traffic per Q row halves and the same
//     shared memory holds a ring of ten half blocks (five K/V pairs in flight instead of two and a
//     half);
//   * one thread issues the MMAs of four tiles.
// Barriers that gather both CTAs (Q and K/V data arrived, P_t written) live in the leader and are
// signalled across the pair; barriers that release (S_t ready, O_t final, ring slot free) exist in
// both CTAs and are signalled in both by tcgen05.commit.  mbarrier waits are time-bounded; the
// cluster barriers at start and end are reached by every thread on every path.
#include <float.h>

#include <type_traits>

#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

namespace attn2 {
using Layout = smem::AttentionPairLayout;
constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILES = Layout::kTiles;          // Q tiles (of BM rows) per CTA
constexpr int TILE_BYTES = Layout::kTileBytes; // 32 KiB: a 128 x 128 bf16 tile (2 swizzle chunks)
constexpr int CHUNK_BYTES = 128 * 128;         // 16 KiB: 128 rows x 64 bf16
constexpr int HALF_BYTES = Layout::kHalfBytes; // this CTA's half of a K or V block
constexpr int KV_SLOTS = Layout::kKvSlots;     // ring of halves: K_0 V_0 K_1 V_1 ...
constexpr int NUM_THREADS = Layout::kThreads;  // 8 softmax warps + MMA warp + TMA warp
constexpr smem::AttentionPairLayout kLayout = smem::attention_pair_layout();
static_assert(kLayout.q.offset == 0 && kLayout.kv.offset == TILES * TILE_BYTES, "kernel and planner disagree");
constexpr int SMEM_BYTES = kLayout.dynamic_bytes;
constexpr uint32_t TMEM_COLS = 512;            // S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512)
constexpr float RESCALE_THRESHOLD = 8.0f;      // log2 units
}  // namespace attn2

// The helpers below are the single-CTA kernel's (attention.cu), under names of their own.
__device__ __forceinline__ float pr_fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float pr_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint64_t pr_expr_pair(uint64_t x2) {
    float x0, x1;
    unpk2(x2, x0, x1);
    return pk2(pr_fast_exp2(x0), pr_fast_exp2(x1));
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(attn2::NUM_THREADS, 1)
attention_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16 *__restrict__ O,
                      int64_t ldo, int nq, int nkv, float scale_log2, int *status) {
    using namespace attn2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *sQ = smem;                               // [TILES] tiles
    unsigned char *sKV = smem + kLayout.kv.offset;          // [KV_SLOTS] half blocks of 16 KiB
    auto bar_at = [&](int offset) { return reinterpret_cast<uint64_t *>(smem + offset); };
    uint64_t *q_full = bar_at(kLayout.q_full.offset);        // [1]
    uint64_t *kv_full = bar_at(kLayout.kv_full.offset);      // [KV_SLOTS]
    uint64_t *kv_empty = bar_at(kLayout.kv_empty.offset);    // [KV_SLOTS]
    uint64_t *s_full = bar_at(kLayout.s_full.offset);        // [2] MMA -> softmax t: S_t holds block j
    uint64_t *sp_ready = bar_at(kLayout.sp_ready.offset);    // [2] softmax t -> MMA: P_t written over S_t
    uint64_t *o_full = bar_at(kLayout.o_full.offset);        // [2] MMA -> softmax t: O_t final
    uint64_t *p_half = bar_at(kLayout.p_half.offset);        // [2] softmax t -> MMA: kv 0-63 of P_t written
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kLayout.tmem_slot.offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    // a cluster owns four consecutive Q tiles; CTA `rank` owns the two at rank * 2 and rank * 2 + 1
    const int q0 = (blockIdx.x >> 1) * (2 * BM * TILES) + (int)rank * (BM * TILES);
    const int n_blocks = (nkv + BN - 1) / BN;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_SLOTS; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < TILES; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&sp_ready[t], 8);   // 4 softmax warps of tile t in each of the two CTAs
            mbar_init(&o_full[t], 1);
            mbar_init(&p_half[t], 8);
        }
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc_pair(tmem_slot, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched with launch_pdl: barrier set-up and the TMEM allocation above may overlap the tail
    // of the previous kernel of the stream; no global memory is touched before it has completed.
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 9) {
        // ---------------- TMA producer (both CTAs: own Q tiles, own halves of K_j and V_j) ----------------
        if (lane == 0) {
            const uint32_t q_full_leader = map_to_cta(smem_u32(q_full), 0);
            if (leader) mbar_expect_tx(q_full, 2 * TILES * TILE_BYTES);
            for (int t = 0; t < TILES; ++t) {
                tma_load_2d_pair(sQ + t * TILE_BYTES, &tmap_q, 0, q0 + t * BM, q_full_leader);
                tma_load_2d_pair(sQ + t * TILE_BYTES + CHUNK_BYTES, &tmap_q, 64, q0 + t * BM, q_full_leader);
            }
            // ring order: K_0 V_0 K_1 V_1 ...; the byte count of both CTAs' halves lands on the leader's barrier
            for (int u = 0; u < 2 * n_blocks; ++u) {
                const int slot = u % KV_SLOTS;
                const uint32_t ph = (u / KV_SLOTS) & 1;
                if (!mbar_wait(&kv_empty[slot], ph ^ 1, status, 341)) break;
                unsigned char *dst = sKV + slot * HALF_BYTES;
                const uint32_t full_leader = map_to_cta(smem_u32(&kv_full[slot]), 0);
                if (leader) mbar_expect_tx(&kv_full[slot], 2 * HALF_BYTES);
                const int j = u >> 1;
                if ((u & 1) == 0) {
                    // K_j: kv rows [64 rank, 64 rank + 64), both 64-column chunks of d
                    tma_load_2d_pair(dst, &tmap_k, 0, j * BN + (int)rank * 64, full_leader);
                    tma_load_2d_pair(dst + 8192, &tmap_k, 64, j * BN + (int)rank * 64, full_leader);
                } else {
                    // V_j: all 128 kv rows, d columns [64 rank, 64 rank + 64)
                    tma_load_2d_pair(dst, &tmap_v, (int)rank * 64, j * BN, full_leader);
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- MMA issuer (leader only: every MMA spans both CTAs) ----------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(2 * BM, BN, 0);  // A, B both K-major
            constexpr uint32_t idesc_pv = umma_idesc_bf16(2 * BM, D, 1);   // B (= V) is MN-major
            bool ok = mbar_wait(q_full, 0, status, 343);

            auto wait_kv = [&](int u) -> bool {
                return mbar_wait(&kv_full[u % KV_SLOTS], (u / KV_SLOTS) & 1, status, 344);
            };
            // S_t = Q_t K_j^T for tile t of both CTAs: A = each CTA's own Q tile (same offset in both),
            // B = K_j, of which each CTA holds 64 kv rows
            auto issue_qk = [&](int t, int j) {
                const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
                const uint32_t k_addr = smem_u32(sKV + ((2 * j) % KV_SLOTS) * HALF_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t a_off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;   // Q: 128-row chunks
                    const uint32_t b_off = (ks / 4) * 8192 + (ks % 4) * 32;          // K half: 64-row chunks
                    umma_f16_ss_pair(tmem_base + t * BN, umma_desc_sw128(q_addr + a_off, 16, 1024),
                                     umma_desc_sw128(k_addr + b_off, 16, 1024), idesc_qk, ks != 0);
                }
                umma_commit_pair(&s_full[t]);
            };
            // O_t += P_t V_j: A = P_t from each CTA's own TMEM, B = V_j, of which each CTA holds 64 of
            // the 128 head-dimension columns (MN-major, one swizzle chunk; 16 kv rows = 2048 bytes)
            auto issue_pv = [&](int t, int j, int half) {
                const uint32_t v_addr = smem_u32(sKV + ((2 * j + 1) % KV_SLOTS) * HALF_BYTES);
#pragma unroll
                for (int ks = half * 4; ks < half * 4 + 4; ++ks) {
                    const uint32_t b_off = ks * 16 * 128;
                    umma_f16_ts_pair(tmem_base + 256 + t * D, tmem_base + t * BN + ks * 8,
                                     umma_desc_sw128(v_addr + b_off, CHUNK_BYTES, 1024), idesc_pv,
                                     (j | ks) != 0);
                }
            };

            if (ok && n_blocks > 0) ok = wait_kv(0);
            if (ok && n_blocks > 0) {
                tc_fence_after();
                issue_qk(0, 0);
                issue_qk(1, 0);
                umma_commit_pair(&kv_empty[0]);
            }
            for (int j = 0; j < n_blocks && ok; ++j) {
                if (!wait_kv(2 * j + 1)) { ok = false; break; }
                const bool more = j + 1 < n_blocks;
                if (more && !wait_kv(2 * j + 2)) { ok = false; break; }
                for (int t = 0; t < TILES; ++t) {
                    if (!mbar_wait(&p_half[t], j & 1, status, 346)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(t, j, 0);
                    if (!mbar_wait(&sp_ready[t], j & 1, status, 347)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(t, j, 1);
                    if (more)
                        issue_qk(t, j + 1);   // completes after PV(t, j): the tensor pipe is in order
                    else
                        umma_commit_pair(&o_full[t]);
                }
                if (!ok) break;
                umma_commit_pair(&kv_empty[(2 * j + 1) % KV_SLOTS]);
                if (more) umma_commit_pair(&kv_empty[(2 * j + 2) % KV_SLOTS]);
            }
        }
    } else {
        // ---------------- softmax / correction / epilogue ----------------
        // warps 0-3 own Q tile 0, warps 4-7 own Q tile 1; one row per thread.
        const int t = warp >> 2;
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        const uint32_t t_s = t_row + t * BN;
        const uint32_t t_o = t_row + 256 + t * D;
        float m_used = -FLT_MAX;  // maximum the exponentials are taken against (log2 domain)
        float l = 0.0f;           // running row sum
        bool ok = true;
        // P_t of both CTAs feeds one MMA: both report to the leader's barriers
        const uint32_t p_half_leader = map_to_cta(smem_u32(&p_half[t]), 0);
        const uint32_t sp_ready_leader = map_to_cta(smem_u32(&sp_ready[t]), 0);

        for (int j = 0; j < n_blocks && ok; ++j) {
            // s_full(j) also tells that P_t V_{j-1} has finished: the tensor pipe runs in order.
            if (!mbar_wait(&s_full[t], j & 1, status, 348)) { ok = false; break; }
            tc_fence_after();
            const int valid = min(BN, nkv - j * BN);

            // pass 1: row maximum of the block.  All four TMEM loads are in flight at once (a TMEM
            // round trip costs a few hundred cycles); the 128 values are dropped again so that the
            // exponential pass below has registers left for instruction-level parallelism.
            float m_blk = -FLT_MAX;
            {
            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sr[c]);
            tmem_ld_wait();
            if (valid == BN) {
                float m0 = -FLT_MAX, m1 = -FLT_MAX;
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        m0 = pr_max3(m0, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
                        m1 = pr_max3(m1, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
                    }
                m_blk = fmaxf(m0, m1);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i < valid) m_blk = fmaxf(m_blk, __uint_as_float(sr[c][i]));
            }
            }
            // pass 2's first load: in flight during the bookkeeping below
            uint32_t buf[2][32];
            tmem_ld_32x32(t_s, buf[0]);
            m_blk *= scale_log2;  // scale > 0: the maximum commutes with the scaling
            // Lazy rescale: keep the old reference maximum unless it has fallen behind by more
            // than the threshold, so that O is touched rarely.
            const bool grow = (m_blk - m_used) > RESCALE_THRESHOLD;
            if (j == 0) {
                m_used = m_blk;
            } else if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = pr_fast_exp2(m_used - m_blk);
                    m_used = m_blk;
                    l *= alpha;
                }
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32(t_o + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x32(t_o + c * 32, o);
                }
                tmem_st_wait();
            }
            const uint64_t scale2 = pk2(scale_log2, scale_log2);
            const uint64_t negm2 = pk2(-m_used, -m_used);

            // pass 2: p = 2^(s * scale_log2 - m) on fp32x2 pairs, row sum, and bf16 P back into
            // TMEM, two kv values per 32-bit column (the lower kv index in the low half).
            uint64_t sum2 = pk2(0.0f, 0.0f);
            auto exp_chunk = [&](auto masked, int c, const uint32_t(&sr)[32]) {
                uint32_t pb[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const uint64_t x2 =
                        fma2(pk2(__uint_as_float(sr[2 * k]), __uint_as_float(sr[2 * k + 1])), scale2, negm2);
                    uint64_t e2 = pr_expr_pair(x2);
                    float e0, e1;
                    unpk2(e2, e0, e1);
                    if (decltype(masked)::value) {
                        if (c * 32 + 2 * k >= valid) e0 = 0.0f;
                        if (c * 32 + 2 * k + 1 >= valid) e1 = 0.0f;
                        e2 = pk2(e0, e1);
                    }
                    sum2 = add2(sum2, e2);
                    pb[k] = pack_bf16(e0, e1);
                }
                if (c == 2) {
                    // chunks 0 and 1 were stored a whole chunk ago: this wait does not stall
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(p_half_leader);
                }
                // P chunk c lands on columns [16c, 16c+16) of S_t, which chunk c's own load (columns
                // [32c, 32c+32)) and every earlier one have already left.
                tmem_st_32x16(t_s + c * 16, pb);
            };
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                tmem_ld_wait();
                if (c < 3) tmem_ld_32x32(t_s + (c + 1) * 32, buf[(c + 1) & 1]);
                if (valid == BN)
                    exp_chunk(std::false_type{}, c, buf[c & 1]);
                else
                    exp_chunk(std::true_type{}, c, buf[c & 1]);
            }
            float sum_lo, sum_hi;
            unpk2(sum2, sum_lo, sum_hi);
            const float sum = sum_lo + sum_hi;
            l += sum;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(sp_ready_leader);
        }

        // ---- epilogue: O / l -> bf16 -> global ----
        if (ok && n_blocks > 0) ok = mbar_wait(&o_full[t], 0, status, 350);
        if (ok && n_blocks > 0) {
            tc_fence_after();
            const float inv = 1.0f / l;
            const int row = q0 + t * BM + row_in_tile;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
            const bool vec32_ok = (ldo % 16 == 0) && ((reinterpret_cast<uintptr_t>(O) & 31) == 0);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row < nq) {
                    __nv_bfloat16 *dst = O + static_cast<int64_t>(row) * ldo + c * 32;
                    if (vec32_ok) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                w[i] = pack_bf16(__uint_as_float(o[16 * h + 2 * i]) * inv,
                                                 __uint_as_float(o[16 * h + 2 * i + 1]) * inv);
                            st_global_256(dst + 16 * h, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
                        }
                    } else if (vec_ok) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
                            v.y = pack_bf16(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
                            v.z = pack_bf16(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
                            v.w = pack_bf16(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
                            *reinterpret_cast<uint4 *>(dst + 8 * q) = v;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            dst[i] = __float2bfloat16_rn(__uint_as_float(o[i]) * inv);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // no CTA may leave while its partner can still signal into it
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, attn2::TMEM_COLS);
    }
}


int attention_pair_launch(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                           const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq, int64_t nkv,
                           int64_t d, float scale, cudaStream_t stream) {
    using namespace attn2;
    CUtensorMap tq, tk, tv;
    int rc = get_tmap_2d(ctx, Q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nq,
                         (uint64_t)ldq * 2, 64, BM, CU_TENSOR_MAP_SWIZZLE_128B, &tq);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, K, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nkv,
                     (uint64_t)ldk * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B, &tk);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, V, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nkv,
                     (uint64_t)ldv * 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B, &tv);
    if (rc) return rc;
    rc = ensure_dynamic_smem(ctx, attention_bf16_pair_kernel, SMEM_BYTES);
    if (rc) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    const unsigned clusters = (unsigned)((nq + 2 * BM * TILES - 1) / (2 * BM * TILES));
    GB200_CUDA_TRY(launch_pdl(attention_bf16_pair_kernel, dim3(2 * clusters), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                              stream, tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv,
                              scale_log2, ctx->d_status));
    return after_launch(ctx, "attention_bf16_pair_kernel");
}

int kernel_regs_attention_pair() { return kernel_registers(attention_bf16_pair_kernel); }

}  // namespace gb200
