// Fused GEMM -> row softmax -> GEMM chain on the sm_100a tensor cores:
//     O = softmax_rows(scale * Q K^T) V,   Q [nq,128], K [nkv,128], V [nkv,128], O [nq,128] bf16.
//
// In Gern's terms this is the program  Tile(O.row)( mm(Q,K^T -> S), softmax pieces(S -> P),
// mm(P,V -> O) )  with S and P as per-tile temporaries, the shape of the reference's chained
// matmul fusion (test/test-cpu-mm.cpp:266-408, E = (A*B)*D with C allocated per tile) with the
// five softmax ops (apps/common/annot/functions.h:9-173) between the two multiplies.  Here the
// temporaries never reach HBM: S lives in TMEM, P is re-quantised to bf16 in place (over the first
// half of S's columns) and read from TMEM as the A operand of the second multiply, and the softmax is computed online over 128-wide blocks
// of K/V with a running row maximum and row sum.
//
// One CTA owns two 128-row tiles of Q.  Warp 9 streams K and V blocks through one 5-slot TMA
// ring (K_0 V_0 K_1 V_1 ...); warp 8 issues tcgen05.mma in the order P_t V_j, Q_t K_{j+1}^T for
// tile t = 0, 1, so that while one tile's S is in the softmax the tensor pipe works on the other
// tile; warps 0-3 (tile 0) and 4-7 (tile 1) own one row each: they read S_t from TMEM with all
// loads in flight at once (a TMEM round trip costs a few hundred cycles), update max/sum, write P_t back
// to TMEM (two bf16 per column, so that the second multiply reads only V from shared memory: with
// both operands in shared memory a 128 x 128 x 16 MMA needs the full 128 bytes per clock of the
// shared-memory port and the softmax's own stores starve it), rescale O_t in TMEM when the
// running maximum has grown by more than 2^8, and at the end normalise and store O.  The first half of P_t (kv 0-63) is announced to the
// MMA warp while the second half is still being computed, so that half of P_t V_j runs under the
// softmax.  Every wait is bounded and reports through the status word.
//
// How the pairs of Q tiles and their K/V blocks are dealt out to CTAs is a separate matter (three
// schedules, see the enum below): whole pairs, K/V ranges with a combine kernel when there are few
// Q rows, and equal runs of (pair, K/V block) units when whole pairs would leave SMs idle in their
// last round; all roles walk the same list of segments, and the barrier phases run on across it.
#include <float.h>

#include <type_traits>

#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

namespace attn {
constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILES = 2;                   // Q tiles (of BM rows) per CTA
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KiB: any 128 x 128 bf16 tile (2 swizzle chunks)
constexpr int CHUNK_BYTES = 128 * 128;     // 16 KiB: 128 rows x 64 bf16
constexpr int KV_SLOTS = 5;                // one ring for K_0 V_0 K_1 V_1 ...
constexpr int NUM_THREADS = 320;           // 8 softmax warps + MMA warp + TMA warp
// Q (2 tiles), K/V ring, then barriers and the TMEM slot
constexpr smem::AttentionLayout kLayout = smem::attention_layout(NUM_THREADS);
static_assert(smem::AttentionLayout::kTiles == TILES && smem::AttentionLayout::kKvSlots == KV_SLOTS &&
                  smem::AttentionLayout::kTileBytes == TILE_BYTES && kLayout.q.offset == 0 &&
                  kLayout.kv.offset == TILES * TILE_BYTES,
              "kernel and planner disagree");
constexpr int SMEM_BYTES = kLayout.dynamic_bytes;
// S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t (bf16 pairs) overwrites S_t's first 64
constexpr uint32_t TMEM_COLS = 512;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
}  // namespace attn

// Which fp32x2 pairs take their exponential on the FMA pipe instead of the MUFU: pair k does when
// (k & GB200_POLY_AND) == GB200_POLY_AND (1: every second pair, 3: every fourth, 7: every eighth,
// 255: none).  Measured on B200 at 32768 x 4096 x 128: 89 / 85 / 82.5 / 82.9 us, so the default
// keeps every exponential on the MUFU; the cubic stays available for shapes where it pays.
#ifndef GB200_POLY_AND
#define GB200_POLY_AND 255
#endif
#ifndef GB200_ATTN_PACK_CVT
#define GB200_ATTN_PACK_CVT 1
#endif
#ifndef GB200_ATTN_MAX3
#define GB200_ATTN_MAX3 1
#endif

#ifdef GB200_ATTN_TRACE
#ifndef GB200_ATTN_TRACE_CTA
#define GB200_ATTN_TRACE_CTA 0
#endif
// Debug-only timeline (compiled out of the library): one CTA records clock64() at a few points,
// indexed by the K/V blocks it has done so far.
__device__ long long g_attn_trace[28 * 64];
#define ATTN_TRACE(slot, j)                                                          \
    do {                                                                             \
        if (blockIdx.x == GB200_ATTN_TRACE_CTA && (j) < 64) g_attn_trace[(slot) * 64 + (j)] = clock64(); \
    } while (0)
#else
#define ATTN_TRACE(slot, j) do { } while (0)
#endif

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for a pair on the FMA pipe (no MUFU): round x to the nearest integer n with the
// 1.5*2^23 trick, evaluate a cubic for 2^f on f = x - n in [-0.5, 0.5], and add n into the
// exponent field.  Relative error below 1e-3, under the bf16 rounding P receives next.  x is
// clamped to >= -126 so that the exponent arithmetic cannot wrap.
__device__ __forceinline__ uint64_t poly_exp2_pair(uint64_t x2) {
    float x0, x1;
    unpk2(x2, x0, x1);
    x2 = pk2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t magic = pk2(12582912.0f, 12582912.0f);       // 1.5 * 2^23
    const uint64_t neg_magic = pk2(-12582912.0f, -12582912.0f);
    const uint64_t t = add2(x2, magic);
    const uint64_t n = add2(t, neg_magic);
    const uint64_t f = fma2(n, pk2(-1.0f, -1.0f), x2);
    uint64_t p = fma2(f, pk2(0.0555041087f, 0.0555041087f), pk2(0.2402265069f, 0.2402265069f));
    p = fma2(p, f, pk2(0.6931471806f, 0.6931471806f));
    p = fma2(p, f, pk2(1.0f, 1.0f));
    float p0, p1, t0, t1;
    unpk2(p, p0, p1);
    unpk2(t, t0, t1);
    // p * 2^n: the low mantissa bits of t hold n; one integer multiply-add moves it into the exponent
    p0 = __int_as_float(__float_as_int(t0) * 0x800000 + __float_as_int(p0));
    p1 = __int_as_float(__float_as_int(t1) * 0x800000 + __float_as_int(p1));
    return pk2(p0, p1);
}
// Two non-negative finite fp32 values -> two bf16 (round half up) in one word, on the integer
// pipe (two adds and a byte permute instead of one cvt.rn.bf16x2.f32).  With P in shared memory
// this was the faster form; with P in TMEM the conversion instruction measures 4 % faster
// (71.0 -> 68.0 us at 32768 x 4096 x 128) and is the default (GB200_ATTN_PACK_CVT).
__device__ __forceinline__ uint32_t pack_bf16_alu(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}
// max(a, b, c) in one instruction (three-input form of max.f32, sm_100 and later).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint64_t mufu_exp2_pair(uint64_t x2) {
    float x0, x1;
    unpk2(x2, x0, x1);
    return pk2(fast_exp2(x0), fast_exp2(x1));
}

// The bf16 output and how one thread stores 32 columns of one row of it.
struct OutRows {
    __nv_bfloat16 *O;
    int64_t ldo;
    int nq;
    // 32 fp32 values of row `row`, columns [32c, 32c + 32), times inv -> bf16 -> global
    __device__ __forceinline__ void store_chunk(int row, int c, const uint32_t (&o)[32], float inv) const {
        if (row >= nq) return;
        const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
        const bool vec32_ok = (ldo % 16 == 0) && ((reinterpret_cast<uintptr_t>(O) & 31) == 0);
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
            for (int i = 0; i < 32; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(o[i]) * inv);
        }
    }
};

// What one CTA works on is a list of segments: a pair of Q tiles (256 rows) and a range of K/V
// blocks.  The three schedules differ only in that list.
enum : int {
    WHOLE = 0,     // blockIdx.x = pair; all K/V blocks; bf16 O stored directly
    SPLIT = 1,     // blockIdx.x = pair, blockIdx.y = range of `per` K/V blocks; the CTA stores its
                   // unnormalised fp32 O, reference maximum and row sum, attention_combine_kernel
                   // merges the ranges.  Used when there are too few Q tiles to fill the GPU.
    BALANCED = 2,  // the pairs x blocks units, pair-major, are cut into equal runs of `per` units,
                   // one run per CTA (so a CTA may finish one pair and start the next).  A pair
                   // that several CTAs share is merged by whichever of them finishes last: every
                   // sharer stores its partial result and counts itself in; the one that finds the
                   // count complete reads all of them back and stores O.  Nobody waits.
};
struct Segment {
    int pair, b0, n_blocks, part, parts;
};
template <int MODE>
struct SegmentIter {
    int total_blocks, per, cursor, end;
    bool done = false;
    __device__ SegmentIter(int total_blocks_, int per_, int pairs) : total_blocks(total_blocks_), per(per_) {
        cursor = static_cast<int>(blockIdx.x) * per;
        end = min(cursor + per, pairs * total_blocks);
    }
    __device__ bool next(Segment &s) {
        if (MODE == WHOLE) {
            if (done) return false;
            done = true;
            s = {static_cast<int>(blockIdx.x), 0, total_blocks, 0, 1};
            return total_blocks > 0;
        } else if (MODE == SPLIT) {
            if (done) return false;
            done = true;
            const int b0 = static_cast<int>(blockIdx.y) * per;
            s = {static_cast<int>(blockIdx.x), b0, min(per, total_blocks - b0), static_cast<int>(blockIdx.y),
                 static_cast<int>(gridDim.y)};
            return s.n_blocks > 0;
        } else {
            if (cursor >= end) return false;
            s.pair = cursor / total_blocks;
            s.b0 = cursor - s.pair * total_blocks;
            s.n_blocks = min(total_blocks - s.b0, end - cursor);
            const int first = (s.pair * total_blocks) / per;
            const int last = ((s.pair + 1) * total_blocks - 1) / per;
            s.part = static_cast<int>(blockIdx.x) - first;
            s.parts = last - first + 1;
            cursor += s.n_blocks;
            return true;
        }
    }
};

// `per`: K/V blocks per range (SPLIT) or units per CTA (BALANCED).  part_o / part_ml: partial
// results, [range][nq] rows (SPLIT) or [pair][max_parts][256] rows (BALANCED); `counters`
// (BALANCED): one word per 32-row group of every pair, zero between launches.
template <int MODE>
__global__ void __launch_bounds__(attn::NUM_THREADS, 1)
attention_bf16_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16 *__restrict__ O,
                      int64_t ldo, int nq, int nkv, float scale_log2, int *status,
                      int per, float *__restrict__ part_o, float *__restrict__ part_ml,
                      int max_parts, int *__restrict__ counters) {
    using namespace attn;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *sQ = smem;                               // [TILES] tiles
    unsigned char *sKV = smem + TILES * TILE_BYTES;         // [KV_SLOTS] tiles
    auto bar_at = [&](int offset) { return reinterpret_cast<uint64_t *>(smem + offset); };
    uint64_t *q_full = bar_at(kLayout.q_full.offset);        // [1] TMA -> MMA: the segment's Q tiles
    uint64_t *q_empty = bar_at(kLayout.q_empty.offset);      // [1] MMA -> TMA: last Q K^T of the segment done
    uint64_t *kv_full = bar_at(kLayout.kv_full.offset);      // [KV_SLOTS]
    uint64_t *kv_empty = bar_at(kLayout.kv_empty.offset);    // [KV_SLOTS]
    uint64_t *s_full = bar_at(kLayout.s_full.offset);        // [2] MMA -> softmax t: S_t holds block j
    uint64_t *sp_ready = bar_at(kLayout.sp_ready.offset);    // [2] softmax t -> MMA: P_t written over S_t
    uint64_t *o_full = bar_at(kLayout.o_full.offset);        // [2] MMA -> softmax t: O_t final
    uint64_t *p_half = bar_at(kLayout.p_half.offset);        // [2] softmax t -> MMA: kv 0-63 of P_t written
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kLayout.tmem_slot.offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef GB200_ATTN_TRACE
    if (threadIdx.x == 0 && blockIdx.x == GB200_ATTN_TRACE_CTA) {
        g_attn_trace[24 * 64] = clock64();
        g_attn_trace[25 * 64] = (long long)global_timer_ns();
    }
#endif
    const int total_blocks = (nkv + BN - 1) / BN;
    const int pairs = (nq + BM * TILES - 1) / (BM * TILES);
    // Every role walks the same list of segments; barriers that complete once per K/V block, per
    // ring slot or per segment take their phase from counters that run across segments.

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int s = 0; s < KV_SLOTS; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int t = 0; t < TILES; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&sp_ready[t], 4);
            mbar_init(&o_full[t], 1);
            mbar_init(&p_half[t], 4);
        }
        mbar_fence_init();
    }
    if (warp == 8) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Launched with launch_pdl: barrier set-up and the TMEM allocation above may overlap the tail
    // of the previous kernel of the stream; no global memory is touched before it has completed.
    pdl_launch_dependents();
    pdl_wait();
#ifdef GB200_ATTN_TRACE
    if (threadIdx.x == 0 && blockIdx.x == GB200_ATTN_TRACE_CTA) g_attn_trace[24 * 64 + 1] = clock64();
#endif

    if (warp == 9) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            SegmentIter<MODE> it(total_blocks, per, pairs);
            Segment sg;
            bool ok = true;
            int ring = 0;   // ring units issued so far
            for (int seg = 0; ok && it.next(sg); ++seg) {
                const int q0 = sg.pair * (BM * TILES);
                if (seg > 0 && !mbar_wait(q_empty, (seg - 1) & 1, status, 302)) break;
                ATTN_TRACE(12, seg);
                mbar_expect_tx(q_full, TILES * TILE_BYTES);
                for (int t = 0; t < TILES; ++t) {
                    tma_load_2d(sQ + t * TILE_BYTES, &tmap_q, 0, q0 + t * BM, q_full);
                    tma_load_2d(sQ + t * TILE_BYTES + CHUNK_BYTES, &tmap_q, 64, q0 + t * BM, q_full);
                }
                // ring order: K_0 V_0 K_1 V_1 ...
                for (int u = 0; u < 2 * sg.n_blocks; ++u, ++ring) {
                    const int slot = ring % KV_SLOTS;
                    const uint32_t ph = (ring / KV_SLOTS) & 1;
                    if (!mbar_wait(&kv_empty[slot], ph ^ 1, status, 301)) { ok = false; break; }
                    const CUtensorMap *tm = (u & 1) ? &tmap_v : &tmap_k;
                    unsigned char *dst = sKV + slot * TILE_BYTES;
                    mbar_expect_tx(&kv_full[slot], TILE_BYTES);
                    tma_load_2d(dst, tm, 0, (sg.b0 + (u >> 1)) * BN, &kv_full[slot]);
                    tma_load_2d(dst + CHUNK_BYTES, tm, 64, (sg.b0 + (u >> 1)) * BN, &kv_full[slot]);
                    if (u == 0) ATTN_TRACE(13, seg);
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BN, 0);  // A, B both K-major
            constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, D, 1);   // B (= V) is MN-major
            SegmentIter<MODE> it(total_blocks, per, pairs);
            Segment sg;
            bool ok = true;
            int ring = 0;   // ring units consumed before this segment
            int blk = 0;    // K/V blocks done before this segment (phase of p_half / sp_ready)

            // u, j below count within the segment
            auto wait_kv = [&](int u) -> bool {
                return mbar_wait(&kv_full[(ring + u) % KV_SLOTS], ((ring + u) / KV_SLOTS) & 1, status, 304);
            };
            auto issue_qk = [&](int t, int j) {
                const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
                const uint32_t k_addr = smem_u32(sKV + ((ring + 2 * j) % KV_SLOTS) * TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
                    umma_f16_ss(tmem_base + t * BN, umma_desc_sw128(q_addr + off, 16, 1024),
                                umma_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks != 0);
                }
                umma_commit(&s_full[t]);
            };
            auto issue_pv = [&](int t, int j, int half) {
                const uint32_t v_addr = smem_u32(sKV + ((ring + 2 * j + 1) % KV_SLOTS) * TILE_BYTES);
#pragma unroll
                for (int ks = half * 4; ks < half * 4 + 4; ++ks) {
                    // A = P from TMEM: row = lane, 16 kv values = 8 columns of bf16 pairs.
                    // B = V: MN-major; 16 kv rows = 2048 bytes; the two 64-wide d chunks are
                    // CHUNK_BYTES apart (leading offset), 8-row groups 1024 bytes apart.
                    const uint32_t b_off = ks * 16 * 128;
                    umma_f16_ts(tmem_base + 256 + t * D, tmem_base + t * BN + ks * 8,
                                umma_desc_sw128(v_addr + b_off, CHUNK_BYTES, 1024), idesc_pv,
                                (j | ks) != 0);
                }
            };

            for (int seg = 0; ok && it.next(sg); ++seg) {
                const int n_blocks = sg.n_blocks;
                // The first Q K^T of a segment may run while the softmax warps still read the
                // previous segment's O: S is free (the tensor pipe runs in order), and the first
                // P V waits for p_half, which the softmax warps reach only after their epilogue.
                ATTN_TRACE(14, seg);
                if (!mbar_wait(q_full, seg & 1, status, 303)) { ok = false; break; }
                ATTN_TRACE(15, seg);
                if (!wait_kv(0)) { ok = false; break; }
                ATTN_TRACE(16, seg);
                tc_fence_after();
                issue_qk(0, 0);
                issue_qk(1, 0);
                ATTN_TRACE(17, seg);
                umma_commit(&kv_empty[ring % KV_SLOTS]);
                if (n_blocks == 1) umma_commit(q_empty);
                for (int j = 0; j < n_blocks && ok; ++j) {
                    if (!wait_kv(2 * j + 1)) { ok = false; break; }
                    const bool more = j + 1 < n_blocks;
                    if (more && !wait_kv(2 * j + 2)) { ok = false; break; }
                    const uint32_t ph = (blk + j) & 1;
                    for (int t = 0; t < TILES; ++t) {
                        // the first half of P_t (kv 0-63) is announced while the softmax still works
                        // on the second, so half of P_t V_j leaves the chain softmax -> PV -> QK
                        if (!mbar_wait(&p_half[t], ph, status, 306)) { ok = false; break; }
                        tc_fence_after();
                        issue_pv(t, j, 0);
                        if (!mbar_wait(&sp_ready[t], ph, status, 307)) { ok = false; break; }
                        ATTN_TRACE(8 + 2 * t, blk + j);
                        tc_fence_after();
                        issue_pv(t, j, 1);
                        if (more)
                            issue_qk(t, j + 1);   // completes after PV(t, j): tensor pipe is in order
                        else
                            umma_commit(&o_full[t]);
                        ATTN_TRACE(9 + 2 * t, blk + j);
                    }
                    if (!ok) break;
                    umma_commit(&kv_empty[(ring + 2 * j + 1) % KV_SLOTS]);
                    if (more) umma_commit(&kv_empty[(ring + 2 * j + 2) % KV_SLOTS]);
                    // the segment's last Q K^T has been issued: Q may be replaced once it is done
                    if (j + 2 == n_blocks) umma_commit(q_empty);
                }
                ring += 2 * n_blocks;
                blk += n_blocks;
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
        SegmentIter<MODE> it(total_blocks, per, pairs);
        Segment sg;
        bool ok = true;
        int blk = 0;   // K/V blocks done before this segment (phase of s_full)
        const OutRows out{O, ldo, nq};

        for (int seg = 0; ok && it.next(sg); ++seg) {
        const int n_blocks = sg.n_blocks, b0 = sg.b0;
        float m_used = -FLT_MAX;  // maximum the exponentials are taken against (log2 domain)
        float l = 0.0f;           // running row sum

        for (int j = 0; j < n_blocks && ok; ++j) {
            // s_full(j) also tells that P_t V_{j-1} has finished: the tensor pipe runs in order.
            if (!mbar_wait(&s_full[t], (blk + j) & 1, status, 308)) { ok = false; break; }
            if (lane_group == 0 && lane == 0) ATTN_TRACE(4 * t + 0, blk + j);
            tc_fence_after();
            const int valid = min(BN, nkv - (b0 + j) * BN);

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
#if GB200_ATTN_MAX3
                        m0 = max3(m0, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
                        m1 = max3(m1, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
#else
                        m0 = fmaxf(m0, fmaxf(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])));
                        m1 = fmaxf(m1, fmaxf(__uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3])));
#endif
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
            if (lane_group == 0 && lane == 0) ATTN_TRACE(4 * t + 1, blk + j);
            // Lazy rescale: keep the old reference maximum unless it has fallen behind by more
            // than the threshold, so that O is touched rarely.
            const bool grow = (m_blk - m_used) > RESCALE_THRESHOLD;
            if (j == 0) {
                m_used = m_blk;
            } else if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);
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
                    uint64_t e2 = ((k & GB200_POLY_AND) == GB200_POLY_AND) ? poly_exp2_pair(x2) : mufu_exp2_pair(x2);
                    float e0, e1;
                    unpk2(e2, e0, e1);
                    if (decltype(masked)::value) {
                        if (c * 32 + 2 * k >= valid) e0 = 0.0f;
                        if (c * 32 + 2 * k + 1 >= valid) e1 = 0.0f;
                        e2 = pk2(e0, e1);
                    }
                    sum2 = add2(sum2, e2);
#if GB200_ATTN_PACK_CVT
                    pb[k] = pack_bf16(e0, e1);
#else
                    pb[k] = pack_bf16_alu(e0, e1);
#endif
                }
                if (c == 2) {
                    // chunks 0 and 1 were stored a whole chunk ago: this wait does not stall
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&p_half[t]);
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
            if (lane_group == 0 && lane == 0) ATTN_TRACE(4 * t + 2, blk + j);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sp_ready[t]);
            if (lane_group == 0 && lane == 0) ATTN_TRACE(4 * t + 3, blk + j);
        }

        blk += n_blocks;

        // ---- epilogue: O / l -> bf16 -> global, or the segment's partial result ----
        if (lane_group == 0 && lane == 0) ATTN_TRACE(18 + 3 * t, seg);
        // A pair shared with other CTAs (BALANCED): partial results lie per warp as
        // [part][four columns][lane][4] (a warp's store or load of four columns is 512 contiguous bytes);
        // whichever sharer finds all the others counted in merges them with its own O, which is
        // still in TMEM.  The last segment of a run is usually that sharer (the others were first
        // segments of their CTAs): it looks at the count while its last P V is still running.
        const bool shared = (MODE == BALANCED) && sg.parts > 1;
        const int others = sg.parts - 1;
        const int group = (sg.pair * TILES + t) * 4 + lane_group;          // 32 rows of the pair
        int *counter = counters + group;
        auto ml_at = [&](int k) { return part_ml + 2 * ((static_cast<int64_t>(group) * max_parts + k) * 32 + lane); };
        auto o_at = [&](int k) { return part_o + (static_cast<int64_t>(group) * max_parts + k) * (32 * D) + lane * 4; };
        int seen = -1;
        if (shared && it.cursor >= it.end) {
            if (lane == 0) asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
            seen = __shfl_sync(0xffffffffu, seen, 0);
            __syncwarp();
        }
        if (ok) ok = mbar_wait(&o_full[t], seg & 1, status, 310);
        if (!ok) break;
        if (lane_group == 0 && lane == 0) ATTN_TRACE(19 + 3 * t, seg);
        tc_fence_after();
        const int row = sg.pair * (BM * TILES) + t * BM + row_in_tile;
        if (MODE == WHOLE || (MODE == BALANCED && sg.parts == 1)) {
            const float inv = 1.0f / l;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                out.store_chunk(row, c, o, inv);
            }
        } else if (MODE == SPLIT) {
            // partial result of this K/V range: O as accumulated (relative to m_used), m_used, l
            const int64_t slot = static_cast<int64_t>(sg.part) * nq + row;
            if (row < nq) *reinterpret_cast<float2 *>(part_ml + 2 * slot) = make_float2(m_used, l);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row < nq) {
                    float4 *dst = reinterpret_cast<float4 *>(part_o + slot * D + c * 32);
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        dst[q] = make_float4(__uint_as_float(o[4 * q]), __uint_as_float(o[4 * q + 1]),
                                             __uint_as_float(o[4 * q + 2]), __uint_as_float(o[4 * q + 3]));
                }
            }
        } else {
            if (seen != others) {
                *reinterpret_cast<float2 *>(ml_at(sg.part)) = make_float2(m_used, l);
                float *dst = o_at(sg.part);
#pragma unroll 1
                for (int c = 0; c < 4; c += 2) {
                    uint32_t o[2][32];
                    tmem_ld_32x32(t_o + c * 32, o[0]);
                    tmem_ld_32x32(t_o + c * 32 + 32, o[1]);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 64; i += 4)
                        *reinterpret_cast<float4 *>(dst + (c * 32 + i) * 32) =
                            make_float4(__uint_as_float(o[i >> 5][i & 31]), __uint_as_float(o[i >> 5][(i & 31) + 1]),
                                        __uint_as_float(o[i >> 5][(i & 31) + 2]), __uint_as_float(o[i >> 5][(i & 31) + 3]));
                }
                // the warp's stores, then one release that counts it in
                __syncwarp();
                if (lane == 0)
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(seen) : "l"(counter) : "memory");
                seen = __shfl_sync(0xffffffffu, seen, 0);
                __syncwarp();
            }
            if (seen == others) {
                if (lane == 0) *counter = 0;   // as the next launch expects it
                // reference maximum over all parts
                float m_all = m_used;
#pragma unroll 4
                for (int kk = 0; kk < others; ++kk) m_all = fmaxf(m_all, __ldcg(ml_at(kk + (kk >= sg.part))));
                // This CTA's own part from TMEM first, then steps (column chunk c, other part kk),
                // the loads of a step in flight while the step before it is added up.  (The sums
                // start from the merging sharer's part, so their last bit can depend on which sharer
                // merges: normally the one whose part ends its CTA's run.)
                const float w_own = fast_exp2(m_used - m_all);
                float l_all = w_own * l;
                float inv = 0.0f;
                const int n_steps = 4 * others;                      // even
                float buf[2][32];
                float2 ml_buf[2];
                auto fetch = [&](int step, float(&v)[32], float2 &ml) {
                    const int c = step / others, kk = step - c * others, k = kk + (kk >= sg.part);
                    ml = __ldcg(reinterpret_cast<const float2 *>(ml_at(k)));
                    const float *src = o_at(k) + c * 32 * 32;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 f = __ldcg(reinterpret_cast<const float4 *>(src + i * 32));
                        v[i] = f.x;
                        v[i + 1] = f.y;
                        v[i + 2] = f.z;
                        v[i + 3] = f.w;
                    }
                };
                uint32_t o[32];
                auto add_up = [&](int step, const float(&v)[32], const float2 &ml) {
                    const int c = step / others, kk = step - c * others;
                    const float w = fast_exp2(ml.x - m_all);
                    if (kk == 0) {
                        tmem_ld_32x32(t_o + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * w_own);
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(fmaf(w, v[i], __uint_as_float(o[i])));
                    if (c == 0) l_all = fmaf(w, ml.y, l_all);
                    if (kk == others - 1) {
                        if (c == 0) inv = 1.0f / l_all;
                        out.store_chunk(row, c, o, inv);
                    }
                };
                fetch(0, buf[0], ml_buf[0]);
#pragma unroll 1
                for (int step = 0; step < n_steps; step += 2) {
                    fetch(step + 1, buf[1], ml_buf[1]);
                    add_up(step, buf[0], ml_buf[0]);
                    if (step + 2 < n_steps) fetch(step + 2, buf[0], ml_buf[0]);
                    add_up(step + 1, buf[1], ml_buf[1]);
                }
            }
        }
        if (lane_group == 0 && lane == 0) ATTN_TRACE(20 + 3 * t, seg);
        }   // segments
    }

    tc_fence_before();
    __syncthreads();
#ifdef GB200_ATTN_TRACE
    if (threadIdx.x == 0 && blockIdx.x == GB200_ATTN_TRACE_CTA) {
        g_attn_trace[26 * 64] = clock64();
        g_attn_trace[27 * 64] = (long long)global_timer_ns();
    }
#endif
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, attn::TMEM_COLS);
    }
}

// Merges the partial results of `splits` K/V ranges: with M = max_s m_s,
// O = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s.  One warp per row, four columns per lane.
__global__ void __launch_bounds__(256)
attention_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                         __nv_bfloat16 *__restrict__ O, int64_t ldo, int nq, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= nq) return;
    float m_all = -FLT_MAX;
    for (int s = 0; s < splits; ++s) {
        const float2 ml = *reinterpret_cast<const float2 *>(part_ml + 2 * (static_cast<int64_t>(s) * nq + row));
        if (ml.y > 0.0f) m_all = fmaxf(m_all, ml.x);
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l_all = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const int64_t slot = static_cast<int64_t>(s) * nq + row;
        const float2 ml = *reinterpret_cast<const float2 *>(part_ml + 2 * slot);
        if (!(ml.y > 0.0f)) continue;      // a range that saw no block contributes nothing
        const float w = exp2f(ml.x - m_all);
        const float4 o = *reinterpret_cast<const float4 *>(part_o + slot * attn::D + lane * 4);
        acc.x = fmaf(w, o.x, acc.x);
        acc.y = fmaf(w, o.y, acc.y);
        acc.z = fmaf(w, o.z, acc.z);
        acc.w = fmaf(w, o.w, acc.w);
        l_all = fmaf(w, ml.y, l_all);
    }
    const float inv = 1.0f / l_all;
    __nv_bfloat16 *dst = O + static_cast<int64_t>(row) * ldo + lane * 4;
    if ((ldo % 4 == 0) && ((reinterpret_cast<uintptr_t>(O) & 7) == 0)) {
        uint2 v;
        v.x = pack_bf16(acc.x * inv, acc.y * inv);
        v.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2 *>(dst) = v;
    } else {
        dst[0] = __float2bfloat16_rn(acc.x * inv);
        dst[1] = __float2bfloat16_rn(acc.y * inv);
        dst[2] = __float2bfloat16_rn(acc.z * inv);
        dst[3] = __float2bfloat16_rn(acc.w * inv);
    }
}

int attention_pair_launch(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                          const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq, int64_t nkv,
                          int64_t d, float scale, cudaStream_t stream);


#ifndef GB200_ATTN_AUTO_PAIR
#define GB200_ATTN_AUTO_PAIR 0
#endif
// Equal runs per CTA are chosen when the longest CTA's walk plus this allowance (in K/V blocks)
// comes to at most this share of the whole-pair schedule's.
#ifndef GB200_ATTN_BALANCED_GAIN_PCT
#define GB200_ATTN_BALANCED_GAIN_PCT 95
#endif
#ifndef GB200_ATTN_BALANCED_COST_BLOCKS
#define GB200_ATTN_BALANCED_COST_BLOCKS 4
#endif

// kernel_choice: 0 = pick, 1 = one CTA per two Q tiles, 2 = CTA pairs with two Q tiles per CTA
// (attention_pair.cu).
// kv_splits: 0 = pick, 1 = every CTA walks all K/V blocks of its Q tiles, n > 1 = that many K/V
// ranges merged by a second kernel (fewer if there are not enough blocks), -1 = equal runs of
// (Q tile pair, K/V block) units per CTA, merged inside the kernel.
int attention_dispatch(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                       const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq, int64_t nkv,
                       int64_t d, float scale, cudaStream_t stream, int kernel_choice = 0, int kv_splits = 0) {
    using namespace attn;
    GB200_REQUIRE(d == D, GB200_ERR_UNSUPPORTED, "attention: d must be %d in this build (got %lld)",
                  D, (long long)d);
    GB200_REQUIRE(ctx->encode_tiled != nullptr, GB200_ERR_NO_DEVICE, "TMA descriptors unavailable");
    if (kernel_choice == 2 || (kernel_choice == 0 && GB200_ATTN_AUTO_PAIR))
        return attention_pair_launch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale, stream);
    CUtensorMap tq, tk, tv;
    int rc = get_tmap_2d(ctx, Q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nq,
                         (uint64_t)ldq * 2, 64, BM, CU_TENSOR_MAP_SWIZZLE_128B, &tq);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, K, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nkv,
                     (uint64_t)ldk * 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B, &tk);
    if (rc) return rc;
    rc = get_tmap_2d(ctx, V, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)d, (uint64_t)nkv,
                     (uint64_t)ldv * 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B, &tv);
    if (rc) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    const unsigned grid = (unsigned)((nq + BM * TILES - 1) / (BM * TILES));
    const int total_blocks = (int)((nkv + BN - 1) / BN);
    const int sms = ctx->sm_count;
    int splits = kv_splits;
    if (splits == 0) {
        splits = 1;
        const int64_t units = (int64_t)grid * total_blocks;
        const int64_t whole_time = (int64_t)((grid + sms - 1) / sms) * total_blocks;   // in K/V blocks
        const int64_t balanced_time = (units + sms - 1) / sms;
        if ((int)grid * 2 <= sms && total_blocks >= 4) {
            // Few Q tiles: K/V ranges of at least two blocks go to the idle SMs; the combine pass
            // costs one read of the partials.
            splits = sms / (int)grid;
            if (splits > total_blocks / 2) splits = total_blocks / 2;
        } else if ((balanced_time + GB200_ATTN_BALANCED_COST_BLOCKS) * 100 <= whole_time * GB200_ATTN_BALANCED_GAIN_PCT) {
            // The last wave of whole pairs would leave SMs idle: equal runs.  Handing a pair over
            // inside a CTA and merging the shared pairs at the end (all CTAs at once, bound by the
            // L2) cost nearly four K/V blocks' time: 128 pairs x 32 blocks on 148 SMs gain nothing
            // worth a result that depends on which CTA merges (measured 67.6 against 67.9 us) and
            // stay whole, 157 pairs x 32 blocks take 80 instead of 135 us and 128 pairs x 128
            // blocks 226 instead of 262 us.
            splits = -1;
        }
    }
    if (splits > total_blocks) splits = total_blocks;
    if (splits == -1 && (int64_t)grid * total_blocks > (int64_t)1 << 30) splits = 1;
    // Whole pairs picked by the library for 16 K/V blocks or more go through the segment-walking
    // instantiation with runs of one pair: the same bits, and its block loop measures 2-3 % faster
    // than the WHOLE instantiation's (67.9 against 70.0 us at 32768 x 4096, 133 against 138 us at
    // 65536 x 4096; 22.4 against 22.0 us at 32768 x 1024, hence the threshold).
    if ((splits == 1 || splits == 0) && kv_splits == 0 && total_blocks >= 16 &&
        (int64_t)grid * total_blocks < ((int64_t)1 << 30))
        splits = -9;
    if (splits == 1 || splits == 0) {
        rc = ensure_dynamic_smem(ctx, attention_bf16_kernel<WHOLE>, SMEM_BYTES);
        if (rc) return rc;
        GB200_CUDA_TRY(launch_pdl(attention_bf16_kernel<WHOLE>, dim3(grid), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                                  stream, tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv,
                                  scale_log2, ctx->d_status, 0, static_cast<float *>(nullptr),
                                  static_cast<float *>(nullptr), 0, static_cast<int *>(nullptr)));
        return after_launch(ctx, "attention_bf16_kernel");
    }
    if (splits == -1 || splits == -9) {
        const int64_t units = (int64_t)grid * total_blocks;
        const int per = splits == -9 ? total_blocks : (int)((units + sms - 1) / sms);
        const unsigned ctas = (unsigned)((units + per - 1) / per);
        const int max_parts = (total_blocks + per - 1) / per + 1;
        const size_t rows = (size_t)grid * max_parts * (BM * TILES);
        float *part_o = nullptr, *part_ml = nullptr;
        if (per != total_blocks) {      // runs of whole pairs share nothing
            rc = workspace_reserve(ctx, rows * (D + 2) * sizeof(float));
            if (rc) return rc;
            rc = merge_counters_reserve(ctx, (size_t)grid * TILES * 4);
            if (rc) return rc;
            part_o = static_cast<float *>(ctx->workspace);
            part_ml = part_o + rows * D;
        }
        rc = ensure_dynamic_smem(ctx, attention_bf16_kernel<BALANCED>, SMEM_BYTES);
        if (rc) return rc;
        GB200_CUDA_TRY(launch_pdl(attention_bf16_kernel<BALANCED>, dim3(ctas), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                                  stream, tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv,
                                  scale_log2, ctx->d_status, per, part_o, part_ml, max_parts, ctx->merge_counters));
        return after_launch(ctx, "attention_bf16_kernel<balanced>");
    }
    const int per = (total_blocks + splits - 1) / splits;
    splits = (total_blocks + per - 1) / per;          // every range holds at least one block
    rc = workspace_reserve(ctx, (size_t)splits * (size_t)nq * (D + 2) * sizeof(float));
    if (rc) return rc;
    float *part_o = static_cast<float *>(ctx->workspace);
    float *part_ml = part_o + (size_t)splits * (size_t)nq * D;
    rc = ensure_dynamic_smem(ctx, attention_bf16_kernel<SPLIT>, SMEM_BYTES);
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(attention_bf16_kernel<SPLIT>, dim3(grid, (unsigned)splits), dim3(NUM_THREADS),
                              (size_t)SMEM_BYTES, stream, tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo,
                              (int)nq, (int)nkv, scale_log2, ctx->d_status, per, part_o, part_ml, 0,
                              static_cast<int *>(nullptr)));
    rc = after_launch(ctx, "attention_bf16_kernel<split>");
    if (rc) return rc;
    GB200_CUDA_TRY(launch_pdl(attention_combine_kernel, dim3((unsigned)((nq + 7) / 8)), dim3(256), 0, stream,
                              static_cast<const float *>(part_o), static_cast<const float *>(part_ml),
                              static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, splits));
    return after_launch(ctx, "attention_combine_kernel");
}

static int check_attention_args(const void *Q, int64_t ldq, const void *K, int64_t ldk,
                                const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                                int64_t nkv, int64_t d, float scale) {
    GB200_REQUIRE(nq >= 0 && nkv >= 0 && d >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    // The kernels take the row maximum of the raw scores and scale it afterwards, which is the
    // maximum of the scaled scores only for a positive scale.
    GB200_REQUIRE(scale > 0.0f && scale <= 3.0e38f, GB200_ERR_INVALID_ARG,
                  "scale must be positive and finite (got %g)", (double)scale);
    GB200_REQUIRE(nq < (1ll << 30) && nkv < (1ll << 30), GB200_ERR_UNSUPPORTED, "extent beyond 2^30");
    if (nq == 0 || d == 0) return 1;
    GB200_REQUIRE(nkv > 0, GB200_ERR_INVALID_ARG, "softmax over an empty row (nkv == 0)");
    GB200_REQUIRE(Q && K && V && O, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(ldq >= d && ldk >= d && ldv >= d && ldo >= d, GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row");
    return GB200_OK;
}

// Registers per thread of the widest instantiation (the library picks among them per shape).
int kernel_regs_attention() {
    const int a = kernel_registers(attention_bf16_kernel<WHOLE>), b = kernel_registers(attention_bf16_kernel<SPLIT>),
              c = kernel_registers(attention_bf16_kernel<BALANCED>);
    if (a < 0 || b < 0 || c < 0) return -1;
    return a > b ? (a > c ? a : c) : (b > c ? b : c);
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_attention_bf16(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                         const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                         int64_t nkv, int64_t d, float scale, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return attention_dispatch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale,
                              static_cast<cudaStream_t>(stream));
}

int gb200_attention_bf16_cluster(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                                 const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                                 int64_t nkv, int64_t d, float scale, int cluster_x, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(cluster_x == 1 || cluster_x == 2, GB200_ERR_UNSUPPORTED,
                  "the chain has kernels for clusters of 1 and 2 thread blocks (asked for %d)", cluster_x);
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return attention_dispatch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale,
                              static_cast<cudaStream_t>(stream), cluster_x);
}

#ifdef GB200_ATTN_TRACE
int gb200_attn_trace_read(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(long long) * 28 * 64);
}
#endif

// Test / benchmark hook: kernel chosen by the caller (1 = single CTA, 2 = CTA pair).
int gb200_attention_bf16_variant(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K,
                                 int64_t ldk, const void *V, int64_t ldv, void *O, int64_t ldo,
                                 int64_t nq, int64_t nkv, int64_t d, float scale, void *stream,
                                 int variant) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return attention_dispatch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale,
                              static_cast<cudaStream_t>(stream), variant);
}

// Test / benchmark hook: the single-CTA kernel with the schedule chosen by the caller (0 = let the
// library pick, 1 = whole pairs, n > 1 = that many K/V ranges and a combine pass, -1 = equal runs
// per CTA merged inside the kernel, -9 = whole pairs through the segment-walking instantiation).
int gb200_attention_bf16_splitkv(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                                 const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                                 int64_t nkv, int64_t d, float scale, void *stream, int splits) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE((splits >= -1 || splits == -9) && splits <= 1024, GB200_ERR_INVALID_ARG, "splits out of range");
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return attention_dispatch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale,
                              static_cast<cudaStream_t>(stream), 1, splits);
}

int gb200_attention_bf16_host(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K,
                              int64_t ldk, const void *V, int64_t ldv, void *O, int64_t ldo,
                              int64_t nq, int64_t nkv, int64_t d, float scale) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale);
    if (rc) return rc < 0 ? rc : GB200_OK;
    rc = stage_reserve(ctx, 0, (size_t)nq * d * 2 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 1, (size_t)nkv * d * 2 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 2, (size_t)nkv * d * 2 + 16);
    if (rc) return rc;
    rc = stage_reserve(ctx, 3, (size_t)nq * d * 2 + 16);
    if (rc) return rc;
    cudaStream_t s = ctx->copy_stream[0];
    GB200_CUDA_TRY(cudaMemcpy2DAsync(ctx->stage[0], d * 2, Q, ldq * 2, d * 2, nq, cudaMemcpyHostToDevice, s));
    GB200_CUDA_TRY(cudaMemcpy2DAsync(ctx->stage[1], d * 2, K, ldk * 2, d * 2, nkv, cudaMemcpyHostToDevice, s));
    GB200_CUDA_TRY(cudaMemcpy2DAsync(ctx->stage[2], d * 2, V, ldv * 2, d * 2, nkv, cudaMemcpyHostToDevice, s));
    rc = attention_dispatch(ctx, ctx->stage[0], d, ctx->stage[1], d, ctx->stage[2], d, ctx->stage[3], d,
                            nq, nkv, d, scale, s);
    if (rc) return rc;
    GB200_CUDA_TRY(cudaMemcpy2DAsync(O, ldo * 2, ctx->stage[3], d * 2, d * 2, nq, cudaMemcpyDeviceToHost, s));
    return host_finish(ctx, s, nullptr);
}

}  // extern "C"
