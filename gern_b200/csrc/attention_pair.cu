// GEMM -> row softmax -> GEMM chain on CTA pairs (tcgen05.mma.cta_group::2).
//
// Same operator as attention_bf16_kernel (attention.cu); the mapping differs.  Two CTAs of a
// cluster each own one 128-row Q tile and share every MMA: the leader issues M256 N128 K16
// instructions whose A operand is the two CTAs' Q (or P) tiles and whose B operand is K_j (or V_j)
// split across the pair -- CTA r holds kv rows [64 r, 64 r + 64) of K_j and head-dimension columns
// [64 r, 64 r + 64) of V_j.  Consequences:
//   * each CTA fetches half of every K/V block, so the L2 traffic per Q row is that of a 256-row
//     tile although every SM works on its own tile;
//   * one tile per SM leaves TMEM room for two S buffers (S_{j+1} is computed while block j is in
//     the softmax) next to O, and shared memory room for two P buffers, so the softmax of a tile
//     runs back to back and the tensor pipe only ever waits for P;
//   * a 128 x 128 x 16 slice of work costs each SM 4 KiB of A + 2 KiB of B from shared memory
//     instead of 4 + 4.
// Warps 0-7 are the softmax (two threads per row, 64 columns each), warp 8 issues the MMAs (leader
// CTA only), warp 9 is the TMA producer.  Barriers that gather both CTAs (data arrived, S buffer
// free, P ready) live in the leader and are signalled across the pair; barriers that release
// (S ready, slot free, P consumed) exist in both CTAs and are signalled by tcgen05.commit on both.
// mbarrier waits are time-bounded; the cluster barriers at start and end and the softmax's named
// barrier are reached by every thread on every path.
//
// Status: correct (same parity tests as the single-CTA kernel) but not the default.  Measured at
// 32768 x 4096 x 128: 94.6 us against 84.3 us.  Its period per 128-column block is the softmax of
// one tile (row maximum 390 cycles, exponentials 1350, barrier hand-offs 700 of 2440 cycles),
// and 256 tiles on 148 SMs take two rounds, while the single-CTA kernel runs its 128 two-tile CTAs
// in one round at 4000 cycles per block.
#include <float.h>

#include <type_traits>

#include "common.cuh"

namespace gb200 {

namespace attn2 {
constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;   // 32 KiB: a 128 x 128 bf16 tile (2 swizzle chunks)
constexpr int CHUNK_BYTES = 128 * 128;      // 16 KiB: 128 rows x 64 bf16
constexpr int HALF_BYTES = 16 * 1024;       // this CTA's half of a K or V block
constexpr int KV_SLOTS = 6;                 // ring of halves: K_0 V_0 K_1 V_1 ...
constexpr int NUM_THREADS = 320;            // 8 softmax warps + MMA warp + TMA warp
// Q, P (2 buffers), K/V ring, barriers, row-maximum exchange
constexpr int PAYLOAD_BYTES = 3 * TILE_BYTES + KV_SLOTS * HALF_BYTES;
constexpr int SMEM_BYTES = PAYLOAD_BYTES + 1024 + 256 + 1024;
constexpr uint32_t TMEM_COLS = 512;         // S0 [0,128) S1 [128,256) O [256,384)
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units
}  // namespace attn2

#ifdef GB200_ATTN_TRACE
__device__ long long g_attn2_trace[16 * 64];
#define ATTN2_TRACE(slot, j)                                                           \
    do {                                                                               \
        if (blockIdx.x == 0 && (j) < 64) g_attn2_trace[(slot) * 64 + (j)] = clock64(); \
    } while (0)
#else
#define ATTN2_TRACE(slot, j) do { } while (0)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two non-negative finite fp32 values -> two bf16 (round half up) in one word, on the integer
// pipe: the F2FP conversion shares the 16-lane unit that the exponentials keep busy.
__device__ __forceinline__ uint32_t pack_bf16_int(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
__device__ __forceinline__ void softmax256_bar_sync() {
    asm volatile("bar.sync 1, 256;" ::: "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(attn2::NUM_THREADS, 1)
attention_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v,
                           __nv_bfloat16 *__restrict__ O, int64_t ldo, int nq, int nkv,
                           float scale_log2, int *status) {
    using namespace attn2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *sQ = smem;
    unsigned char *sP = smem + TILE_BYTES;                   // [2] buffers
    unsigned char *sKV = smem + 3 * TILE_BYTES;              // [KV_SLOTS] halves
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + PAYLOAD_BYTES);
    uint64_t *q_full = bars;             // [1] leader: both Q tiles have landed
    uint64_t *kv_full = bars + 1;        // [6] leader: both halves of a block have landed
    uint64_t *kv_empty = bars + 7;       // [6] each CTA: the slot may be refilled
    uint64_t *s_full = bars + 13;        // [2] each CTA: S[buf] holds a block
    uint64_t *s_free = bars + 15;        // [2] leader: both softmaxes have read S[buf] (16 arrivals)
    uint64_t *p_ready = bars + 17;       // [2] leader: both P[buf] tiles are written (16 arrivals)
    uint64_t *pv_done = bars + 19;       // [2] each CTA: P[buf] V has been accumulated
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 21);
    // Row-maximum exchange between the two threads of a row: [2 parities][2 halves][128 rows] of
    // 16-bit values (upper half of an fp32, rounded up); reused for the fp32 half-row sums.
    uint16_t *xmax = reinterpret_cast<uint16_t *>(bars + 32);
    float *xsum = reinterpret_cast<float *>(bars + 32);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int q0 = (blockIdx.x >> 1) * (2 * BM) + (int)rank * BM;   // this CTA's Q tile
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
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&s_free[b], 16);
            mbar_init(&p_ready[b], 16);
            mbar_init(&pv_done[b], 1);
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

    if (warp == 9) {
        // ---------------- TMA producer (both CTAs: own Q tile, own halves of K_j and V_j) ----------------
        if (lane == 0) {
            const uint32_t q_full_leader = map_to_cta(smem_u32(q_full), 0);
            if (leader) mbar_expect_tx(q_full, 2 * TILE_BYTES);
            tma_load_2d_pair(sQ, &tmap_q, 0, q0, q_full_leader);
            tma_load_2d_pair(sQ + CHUNK_BYTES, &tmap_q, 64, q0, q_full_leader);
            for (int u = 0; u < 2 * n_blocks; ++u) {
                const int slot = u % KV_SLOTS;
                const uint32_t ph = (u / KV_SLOTS) & 1;
                if (!mbar_wait(&kv_empty[slot], ph ^ 1, status, 321)) break;
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
        // ---------------- MMA issuer (leader only) ----------------
        if (leader && lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(2 * BM, BN, 0);  // A, B both K-major
            constexpr uint32_t idesc_pv = umma_idesc_bf16(2 * BM, D, 1);   // B (= V) is MN-major
            const uint32_t q_addr = smem_u32(sQ);
            bool ok = mbar_wait(q_full, 0, status, 323);

            auto wait_kv = [&](int u) -> bool {
                return mbar_wait(&kv_full[u % KV_SLOTS], (u / KV_SLOTS) & 1, status, 324);
            };
            // S[j & 1] = Q K_j^T for both tiles; the buffer was last read by the softmax of block j-2
            auto issue_qk = [&](int j) -> bool {
                const int buf = j & 1;
                if (!wait_kv(2 * j)) return false;
                if (!mbar_wait(&s_free[buf], ((j >> 1) & 1) ^ 1, status, 325)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sKV + ((2 * j) % KV_SLOTS) * HALF_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t a_off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;   // Q: 128-row chunks
                    const uint32_t b_off = (ks / 4) * 8192 + (ks % 4) * 32;          // K half: 64-row chunks
                    umma_f16_ss_pair(tmem_base + buf * BN, umma_desc_sw128(q_addr + a_off, 16, 1024),
                                     umma_desc_sw128(k_addr + b_off, 16, 1024), idesc_qk, ks != 0);
                }
                umma_commit_pair(&kv_empty[(2 * j) % KV_SLOTS]);
                umma_commit_pair(&s_full[buf]);
                return true;
            };

            if (ok && n_blocks > 0) ok = issue_qk(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                ATTN2_TRACE(4, j);
                if (j + 1 < n_blocks && !issue_qk(j + 1)) { ok = false; break; }
                ATTN2_TRACE(5, j);
                const int pb = j & 1;
                if (!wait_kv(2 * j + 1)) { ok = false; break; }
                ATTN2_TRACE(6, j);
                if (!mbar_wait(&p_ready[pb], (j >> 1) & 1, status, 327)) { ok = false; break; }
                ATTN2_TRACE(7, j);
                tc_fence_after();
                const uint32_t p_addr = smem_u32(sP + pb * TILE_BYTES);
                const uint32_t v_addr = smem_u32(sKV + ((2 * j + 1) % KV_SLOTS) * HALF_BYTES);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // A = P: K-major, 16 kv values = 32 bytes inside the swizzle row.
                    const uint32_t a_off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
                    // B = this CTA's 64 d columns of V: MN-major, one swizzle chunk; 16 kv rows
                    // = 2048 bytes, 8-row groups 1024 bytes apart.
                    const uint32_t b_off = ks * 16 * 128;
                    umma_f16_ss_pair(tmem_base + 256, umma_desc_sw128(p_addr + a_off, 16, 1024),
                                     umma_desc_sw128(v_addr + b_off, CHUNK_BYTES, 1024), idesc_pv,
                                     (j | ks) != 0);
                }
                umma_commit_pair(&kv_empty[(2 * j + 1) % KV_SLOTS]);
                umma_commit_pair(&pv_done[pb]);
                ATTN2_TRACE(8, j);
            }
        }
    } else {
        // ---------------- softmax / correction / epilogue (both CTAs, own tile) ----------------
        // Two threads per row: warps 0-3 own kv columns 0-63 of every block (and d columns 0-63
        // of O), warps 4-7 own columns 64-127.  Warp w and warp w+4 touch the same TMEM lanes.
        const int half = warp >> 2;
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        const uint32_t t_o = t_row + 256 + half * 64;
        float m_used = -FLT_MAX;  // maximum the exponentials are taken against (log2 domain)
        float l = 0.0f;           // running sum of this thread's half of the row
        bool ok = true;
        const int sw = row_in_tile & 7;
        const uint32_t s_free_leader0 = map_to_cta(smem_u32(&s_free[0]), 0);
        const uint32_t p_ready_leader0 = map_to_cta(smem_u32(&p_ready[0]), 0);

        // A warp whose bounded wait ran out keeps walking the loop (doing nothing) so that it
        // still meets its partners at the one named barrier of every block.
        for (int j = 0; j < n_blocks; ++j) {
            const int buf = j & 1;
            if (ok && !mbar_wait(&s_full[buf], (j >> 1) & 1, status, 328)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (warp == 0 && lane == 0) ATTN2_TRACE(0, j);
            tc_fence_after();
            const uint32_t t_s = t_row + buf * BN + half * 64;
            const int valid = min(BN, nkv - j * BN) - half * 64;   // valid columns of this half

            // pass 1: maximum of this thread's 64 columns, both TMEM loads in flight at once; the
            // values are dropped again so that pass 2 has registers for instruction-level parallelism
            float m_half = -FLT_MAX;
            {
                uint32_t a0[32], a1[32];
                tmem_ld_32x32(t_s, a0);
                tmem_ld_32x32(t_s + 32, a1);
                tmem_ld_wait();
                if (valid >= 64) {
                    float m0 = -FLT_MAX, m1 = -FLT_MAX;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        m0 = fmaxf(m0, fmaxf(__uint_as_float(a0[i]), __uint_as_float(a0[i + 1])));
                        m1 = fmaxf(m1, fmaxf(__uint_as_float(a1[i]), __uint_as_float(a1[i + 1])));
                    }
                    m_half = fmaxf(m0, m1);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (i < valid) m_half = fmaxf(m_half, __uint_as_float(a0[i]));
                        if (32 + i < valid) m_half = fmaxf(m_half, __uint_as_float(a1[i]));
                    }
                }
            }
            // pass 2's first load: in flight during the exchange below
            uint32_t buf2[2][32];
            tmem_ld_32x32(t_s, buf2[0]);
            // Exchange the half-row maxima (double-buffered by block parity: one barrier per block).
            // Both threads of a row must end up with the same number, so each uses the 16-bit
            // form of both halves: the upper half of the fp32, rounded towards +inf, which is
            // >= the true maximum (exponentials stay <= 1) and is what the partner can see.
            const uint32_t mb = __float_as_uint(m_half);
            const uint32_t m_up = (m_half >= 0.0f ? mb + 0xFFFFu : mb) >> 16;
            xmax[((j & 1) * 2 + half) * 128 + row_in_tile] = static_cast<uint16_t>(m_up);
            softmax256_bar_sync();
            if (!ok) {
                tmem_ld_wait();
                continue;
            }
            const uint32_t m_other = xmax[((j & 1) * 2 + (half ^ 1)) * 128 + row_in_tile];
            float m_blk = fmaxf(__uint_as_float(m_up << 16), __uint_as_float(m_other << 16));
            m_blk *= scale_log2;  // scale > 0: the maximum commutes with the scaling
            if (warp == 0 && lane == 0) ATTN2_TRACE(1, j);
            // Lazy rescale: keep the old reference maximum unless it has fallen behind by more
            // than the threshold, so that O is touched rarely.  Both threads of a row take the
            // same decision from the same numbers.
            const bool grow = (m_blk - m_used) > RESCALE_THRESHOLD;
            if (j == 0) {
                m_used = m_blk;
            } else if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = ex2_approx(m_used - m_blk);
                    m_used = m_blk;
                    l *= alpha;
                }
                tmem_ld_wait();
                // O holds P_0 V_0 + ... + P_{j-1} V_{j-1} only after the last of them has finished
                if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, status, 329))) {
                    ok = false;
                    continue;
                }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32(t_o + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x32(t_o + c * 32, o);
                }
                tmem_st_wait();
            }
            if (warp == 0 && lane == 0) ATTN2_TRACE(3, j);
            const uint64_t scale2 = pk2(scale_log2, scale_log2);
            const uint64_t negm2 = pk2(-m_used, -m_used);
            // P[j & 1] was last read by P_{j-2} V_{j-2}
            if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[buf], ((j >> 1) & 1) ^ 1, status, 331))) {
                tmem_ld_wait();
                ok = false;
                continue;
            }

            if (warp == 0 && lane == 0) ATTN2_TRACE(9, j);
            // pass 2: p = 2^(s * scale_log2 - m) (MUFU), row sum on fp32x2 pairs, bf16 P into shared
            // memory in the 128-byte swizzled K-major layout (16-byte unit u of row r sits at unit
            // u ^ (r % 8)); this thread's 64 kv columns are one 64-column chunk of the P tile.
            unsigned char *p_row = sP + buf * TILE_BYTES + half * CHUNK_BYTES + row_in_tile * 128;
            uint64_t sum2 = pk2(0.0f, 0.0f);
            auto exp_chunk = [&](auto masked, int c, const uint32_t(&sr)[32]) {
                uint32_t pb[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const uint64_t x2 =
                        fma2(pk2(__uint_as_float(sr[2 * k]), __uint_as_float(sr[2 * k + 1])), scale2, negm2);
                    float x0, x1;
                    unpk2(x2, x0, x1);
                    float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
                    if (decltype(masked)::value) {
                        if (c * 32 + 2 * k >= valid) e0 = 0.0f;
                        if (c * 32 + 2 * k + 1 >= valid) e1 = 0.0f;
                    }
                    sum2 = add2(sum2, pk2(e0, e1));
                    pb[k] = pack_bf16_int(e0, e1);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int unit = c * 4 + q;
                    *reinterpret_cast<uint4 *>(p_row + ((unit ^ sw) << 4)) =
                        make_uint4(pb[4 * q], pb[4 * q + 1], pb[4 * q + 2], pb[4 * q + 3]);
                }
            };
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                tmem_ld_wait();
                if (c == 0) {
                    tmem_ld_32x32(t_s + 32, buf2[1]);
                } else {
                    // both halves of this thread's S columns are in registers: release S[buf]
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(s_free_leader0 + buf * 8);
                }
                if (warp == 0 && lane == 0) ATTN2_TRACE(10 + 2 * c, j);
                if (valid >= 64)
                    exp_chunk(std::false_type{}, c, buf2[c]);
                else
                    exp_chunk(std::true_type{}, c, buf2[c]);
                if (warp == 0 && lane == 0) ATTN2_TRACE(11 + 2 * c, j);
            }
            float sum_lo, sum_hi;
            unpk2(sum2, sum_lo, sum_hi);
            l += sum_lo + sum_hi;
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(p_ready_leader0 + buf * 8);
            if (warp == 0 && lane == 0) ATTN2_TRACE(2, j);
        }

        // ---- epilogue: O / l -> bf16 -> global (each thread: 64 of the row's 128 columns) ----
        if (ok && n_blocks > 0)
            ok = mbar_wait(&pv_done[(n_blocks - 1) & 1], ((n_blocks - 1) >> 1) & 1, status, 330);
        ok = __all_sync(0xffffffffu, ok);
        // total row sum = sum of the two halves (the exchange buffer is reused: everybody must be
        // past its last read of the maxima first)
        softmax256_bar_sync();
        xsum[half * 128 + row_in_tile] = l;
        softmax256_bar_sync();
        if (ok && n_blocks > 0) {
            tc_fence_after();
            const float inv = 1.0f / (l + xsum[(half ^ 1) * 128 + row_in_tile]);
            const int row = q0 + row_in_tile;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row < nq) {
                    __nv_bfloat16 *dst = O + static_cast<int64_t>(row) * ldo + half * 64 + c * 32;
                    if (vec_ok) {
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

#ifdef GB200_ATTN_TRACE
extern "C" int gb200_attn2_trace_read(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_attn2_trace, sizeof(long long) * 16 * 64);
}
#endif

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
    const unsigned pairs = (unsigned)((nq + 2 * BM - 1) / (2 * BM));
    attention_bf16_pair_kernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(
        tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv, scale_log2,
        ctx->d_status);
    return after_launch(ctx, "attention_bf16_pair_kernel");
}

}  // namespace gb200
