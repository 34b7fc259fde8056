// GEMM -> row softmax -> GEMM chain, two softmax threads per row.
//
// Same operator, tiling, TMA ring and MMA order as attention_bf16_kernel (attention.cu): a CTA owns
// two 128-row Q tiles, S_t and O_t live in TMEM, P_t is written back over S_t as bf16 pairs and
// read from there as the A operand of P V.  What differs is the softmax: a row of S_t is shared by
// two threads, 64 columns each, in two warps that sit on the same scheduler (warps w and w + 4 of
// a tile's eight), so that each scheduler always has a second warp to issue from while the first
// waits for the 16-lane exponential unit or for TMEM.  With one thread per row the exponential
// phase of a block took 1850 cycles against the unit's 1024.
//
// Per 128-column block and tile:
//   both halves  wait S_t, load their 64 columns once (they stay in registers), take the partial
//                row maximum, and merge it into the row's running maximum with one shared-memory
//                atomic max; a 64-thread named barrier per 32-row group then makes the merged value
//                (and the fact that both halves hold their S columns) visible to both
//   both halves  decide on the lazy rescale from the same merged value (same decision in both) and
//                rescale their 64 columns of O_t when it is due
//   half 0       exponentials of kv 0-63 -> P columns [0,32) of S_t -> arrives on p_half[t]
//   half 1       exponentials of kv 64-127 -> P columns [32,64) -> arrives on sp_ready[t]
// P columns [32,64) overwrite S columns 32-63, which half 0 loaded before the named barrier.
// Row sums stay per half and are added once, in the epilogue, where each half normalises and stores
// its 64 columns of O.  Every mbarrier wait is bounded; the named barriers are reached by both
// halves on every path (a half whose wait ran out keeps walking the barriers of the blocks left).
#include <float.h>

#include "common.cuh"
#include "smem_plan.hpp"

namespace gb200 {

namespace attn3 {
constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILES = 2;
constexpr int TILE_BYTES = 128 * 128 * 2;
constexpr int CHUNK_BYTES = 128 * 128;
constexpr int KV_SLOTS = 5;
constexpr int SOFTMAX_WARPS = 16;          // 2 tiles x 2 column halves x 4 lane groups
constexpr int NUM_THREADS = 640;           // 16 softmax warps + MMA warp + TMA warp + 2 spare (warpgroup of 4)
// Q (2 tiles), K/V ring, barriers, the TMEM slot and one running-maximum word per Q row
constexpr smem::AttentionLayout kLayout = smem::attention_layout(NUM_THREADS, 1);
static_assert(smem::AttentionLayout::kTiles == TILES && smem::AttentionLayout::kKvSlots == KV_SLOTS &&
                  smem::AttentionLayout::kTileBytes == TILE_BYTES && kLayout.q.offset == 0 &&
                  kLayout.kv.offset == TILES * TILE_BYTES && kLayout.row_words.bytes == TILES * BM * 4,
              "kernel and planner disagree");
constexpr int SMEM_BYTES = kLayout.dynamic_bytes;
constexpr uint32_t TMEM_COLS = 512;        // S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512)
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
}  // namespace attn3

#ifndef GB200_ATTN3_SETMAXNREG
#define GB200_ATTN3_SETMAXNREG 1
#endif


#ifdef GB200_ATTN_TRACE
// Debug-only timeline (compiled out of the library): CTA 0 records clock64() at a few points.
__device__ long long g_attn3_trace[16 * 64];
#define ATTN3_TRACE(slot, j)                                                           \
    do {                                                                               \
        if (blockIdx.x == 0 && (j) < 64) g_attn3_trace[(slot) * 64 + (j)] = clock64(); \
    } while (0)
#else
#define ATTN3_TRACE(slot, j) do { } while (0)
#endif

__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// Order-preserving map between fp32 and signed integers, so that the row maximum of two threads
// can be merged with one integer atomic max.
__device__ __forceinline__ int float_to_ordered(float f) {
    const int b = __float_as_int(f);
    return b ^ ((b >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ordered_to_float(int k) {
    return __int_as_float(k ^ ((k >> 31) & 0x7fffffff));
}
__device__ __forceinline__ void pair_bar_sync(int id) {
    asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

__global__ void __launch_bounds__(attn3::NUM_THREADS, 1)
attention_bf16_split_kernel(const __grid_constant__ CUtensorMap tmap_q,
                            const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16 *__restrict__ O,
                            int64_t ldo, int nq, int nkv, float scale_log2, int *status) {
    using namespace attn3;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *sQ = smem;
    unsigned char *sKV = smem + TILES * TILE_BYTES;
    auto bar_at = [&](int offset) { return reinterpret_cast<uint64_t *>(smem + offset); };
    uint64_t *q_full = bar_at(kLayout.q_full.offset);        // [1]
    uint64_t *kv_full = bar_at(kLayout.kv_full.offset);      // [KV_SLOTS]
    uint64_t *kv_empty = bar_at(kLayout.kv_empty.offset);    // [KV_SLOTS]
    uint64_t *s_full = bar_at(kLayout.s_full.offset);        // [2] MMA -> softmax t: S_t holds block j
    uint64_t *sp_ready = bar_at(kLayout.sp_ready.offset);    // [2] half 1 of tile t -> MMA: kv 64-127 of P_t written
    uint64_t *o_full = bar_at(kLayout.o_full.offset);        // [2] MMA -> softmax t: O_t final
    uint64_t *p_half = bar_at(kLayout.p_half.offset);        // [2] half 0 of tile t -> MMA: kv 0-63 of P_t written
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kLayout.tmem_slot.offset);
    int *row_max = reinterpret_cast<int *>(smem + kLayout.row_words.offset);   // [TILES][BM]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * (BM * TILES);
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
            mbar_init(&sp_ready[t], 4);
            mbar_init(&o_full[t], 1);
            mbar_init(&p_half[t], 4);
        }
        mbar_fence_init();
    }
    if (threadIdx.x < TILES * BM) row_max[threadIdx.x] = float_to_ordered(-FLT_MAX);
    if (warp == SOFTMAX_WARPS) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();

    if (warp >= SOFTMAX_WARPS) {
#if GB200_ATTN3_SETMAXNREG
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
#endif
        if (warp == SOFTMAX_WARPS + 1) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                mbar_expect_tx(q_full, TILES * TILE_BYTES);
                for (int t = 0; t < TILES; ++t) {
                    tma_load_2d(sQ + t * TILE_BYTES, &tmap_q, 0, q0 + t * BM, q_full);
                    tma_load_2d(sQ + t * TILE_BYTES + CHUNK_BYTES, &tmap_q, 64, q0 + t * BM, q_full);
                }
                for (int u = 0; u < 2 * n_blocks; ++u) {          // ring order: K_0 V_0 K_1 V_1 ...
                    const int slot = u % KV_SLOTS;
                    const uint32_t ph = (u / KV_SLOTS) & 1;
                    if (!mbar_wait(&kv_empty[slot], ph ^ 1, status, 321)) break;
                    const CUtensorMap *tm = (u & 1) ? &tmap_v : &tmap_k;
                    unsigned char *dst = sKV + slot * TILE_BYTES;
                    mbar_expect_tx(&kv_full[slot], TILE_BYTES);
                    tma_load_2d(dst, tm, 0, (u >> 1) * BN, &kv_full[slot]);
                    tma_load_2d(dst + CHUNK_BYTES, tm, 64, (u >> 1) * BN, &kv_full[slot]);
                }
            }
        } else if (warp == SOFTMAX_WARPS) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BN, 0);
                constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, D, 1);
                bool ok = mbar_wait(q_full, 0, status, 323);
                auto wait_kv = [&](int u) -> bool {
                    return mbar_wait(&kv_full[u % KV_SLOTS], (u / KV_SLOTS) & 1, status, 324);
                };
                auto issue_qk = [&](int t, int j) {
                    const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
                    const uint32_t k_addr = smem_u32(sKV + ((2 * j) % KV_SLOTS) * TILE_BYTES);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
                        umma_f16_ss(tmem_base + t * BN, umma_desc_sw128(q_addr + off, 16, 1024),
                                    umma_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks != 0);
                    }
                    umma_commit(&s_full[t]);
                };
                auto issue_pv = [&](int t, int j, int half) {
                    const uint32_t v_addr = smem_u32(sKV + ((2 * j + 1) % KV_SLOTS) * TILE_BYTES);
#pragma unroll
                    for (int ks = half * 4; ks < half * 4 + 4; ++ks) {
                        const uint32_t b_off = ks * 16 * 128;
                        umma_f16_ts(tmem_base + 256 + t * D, tmem_base + t * BN + ks * 8,
                                    umma_desc_sw128(v_addr + b_off, CHUNK_BYTES, 1024), idesc_pv,
                                    (j | ks) != 0);
                    }
                };
                if (ok && n_blocks > 0) ok = wait_kv(0);
                if (ok && n_blocks > 0) {
                    tc_fence_after();
                    issue_qk(0, 0);
                    issue_qk(1, 0);
                    umma_commit(&kv_empty[0]);
                }
                for (int j = 0; j < n_blocks && ok; ++j) {
                    if (!wait_kv(2 * j + 1)) { ok = false; break; }
                    const bool more = j + 1 < n_blocks;
                    if (more && !wait_kv(2 * j + 2)) { ok = false; break; }
                    for (int t = 0; t < TILES; ++t) {
                        if (!mbar_wait(&p_half[t], j & 1, status, 326)) { ok = false; break; }
                        tc_fence_after();
                        issue_pv(t, j, 0);
                        if (!mbar_wait(&sp_ready[t], j & 1, status, 327)) { ok = false; break; }
                        ATTN3_TRACE(8 + 2 * t, j);
                        tc_fence_after();
                        issue_pv(t, j, 1);
                        if (more)
                            issue_qk(t, j + 1);   // completes after PV(t, j): the tensor pipe is in order
                        else
                            umma_commit(&o_full[t]);
                        ATTN3_TRACE(9 + 2 * t, j);
                    }
                    if (!ok) break;
                    umma_commit(&kv_empty[(2 * j + 1) % KV_SLOTS]);
                    if (more) umma_commit(&kv_empty[(2 * j + 2) % KV_SLOTS]);
                }
            }
        }
    } else {
#if GB200_ATTN3_SETMAXNREG
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
#endif
        // ---------------- softmax / correction / epilogue ----------------
        // warps 8t .. 8t+7 own Q tile t; warp 8t + 4h + g holds rows 32g .. 32g+31, columns 64h .. 64h+63
        const int t = warp >> 3;
        const int h = (warp >> 2) & 1;
        const int g = warp & 3;
        const int row_in_tile = g * 32 + lane;
        const int bar_id = 1 + t * 4 + g;                 // named barrier of this 32-row group's two warps
        int *my_max = &row_max[t * BM + row_in_tile];
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(g * 32) << 16);
        const uint32_t t_s = t_row + t * BN + h * 64;     // this half's S columns
        const uint32_t t_p = t_row + t * BN + h * 32;     // where this half's P words go
        const uint32_t t_o = t_row + 256 + t * D + h * 64;
        uint64_t *done_bar = h == 0 ? &p_half[t] : &sp_ready[t];
        float m_used = -FLT_MAX;   // maximum the exponentials are taken against (log2 domain)
        float l = 0.0f;            // this half's part of the row sum
        bool ok = true;
        // trace slots (debug builds): half 0 of tile t -> 4t .. 4t+3, half 1 of tile 0 -> 12 .. 15
        const bool tracer = g == 0 && lane == 0 && (h == 0 || t == 0);
        const int trace_slot = h == 0 ? 4 * t : 12;
        (void)tracer;
        (void)trace_slot;

        for (int j = 0; j < n_blocks; ++j) {
            // A half whose wait ran out still meets its partner at the named barrier of every block
            // left, so that the partner cannot be left waiting there.
            if (ok && !mbar_wait(&s_full[t], j & 1, status, 328)) ok = false;
            uint32_t s[2][32];
            if (tracer) ATTN3_TRACE(trace_slot + 0, j);
            if (ok) {
                tc_fence_after();
                tmem_ld_32x32(t_s, s[0]);
                tmem_ld_32x32(t_s + 32, s[1]);
                tmem_ld_wait();
                const int valid = min(64, nkv - j * BN - h * 64);   // may be <= 0 in the last block
                float m0 = -FLT_MAX, m1 = -FLT_MAX;
                if (valid == 64) {
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            m0 = max3f(m0, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                            m1 = max3f(m1, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
                        }
                } else {
#pragma unroll
                    for (int c = 0; c < 2; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i < valid) m0 = fmaxf(m0, __uint_as_float(s[c][i]));
                }
                const float part = fmaxf(m0, m1) * scale_log2;   // scale > 0 commutes with the maximum
                atomicMax(my_max, float_to_ordered(part));
            }
            pair_bar_sync(bar_id);
            if (!ok) continue;
            if (tracer) ATTN3_TRACE(trace_slot + 1, j);
            // the row's running maximum over blocks 0 .. j, the same value in both halves
            const float m_run = ordered_to_float(*reinterpret_cast<volatile int *>(my_max));
            const bool grow = (m_run - m_used) > RESCALE_THRESHOLD;
            if (j == 0) {
                m_used = m_run;
            } else if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = ex2_ftz(m_used - m_run);
                    m_used = m_run;
                    l *= alpha;
                }
                // 16 columns at a time: the 64 S values of this block stay live in registers meanwhile
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[16];
                    tmem_ld_32x16(t_o + c * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st_32x16(t_o + c * 16, o);
                }
                tmem_st_wait();
            }
            const uint64_t scale2 = pk2(scale_log2, scale_log2);
            const uint64_t negm2 = pk2(-m_used, -m_used);
            const int valid = min(64, nkv - j * BN - h * 64);
            uint64_t sum2 = pk2(0.0f, 0.0f);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t pb[16];
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const uint64_t x2 =
                        fma2(pk2(__uint_as_float(s[c][2 * k]), __uint_as_float(s[c][2 * k + 1])), scale2, negm2);
                    float x0, x1;
                    unpk2(x2, x0, x1);
                    float e0 = ex2_ftz(x0), e1 = ex2_ftz(x1);
                    if (valid < 64) {
                        if (c * 32 + 2 * k >= valid) e0 = 0.0f;
                        if (c * 32 + 2 * k + 1 >= valid) e1 = 0.0f;
                    }
                    sum2 = add2(sum2, pk2(e0, e1));
                    pb[k] = pack_bf16(e0, e1);
                }
                tmem_st_32x16(t_p + c * 16, pb);
            }
            float sum_lo, sum_hi;
            unpk2(sum2, sum_lo, sum_hi);
            l += sum_lo + sum_hi;
            if (tracer) ATTN3_TRACE(trace_slot + 2, j);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(done_bar);
            if (tracer) ATTN3_TRACE(trace_slot + 3, j);
        }

        // ---- epilogue: O / (l_0 + l_1) -> bf16 -> global, 64 columns per half ----
        if (ok && n_blocks > 0) ok = mbar_wait(&o_full[t], 0, status, 330);
        // every MMA has completed: the Q tile in shared memory is free and carries the two partial sums
        float *l_xch = reinterpret_cast<float *>(sQ + t * TILE_BYTES);    // [2][BM]
        l_xch[h * BM + row_in_tile] = l;
        pair_bar_sync(bar_id);
        if (ok && n_blocks > 0) {
            tc_fence_after();
            const float inv = 1.0f / (l + l_xch[(h ^ 1) * BM + row_in_tile]);
            const int row = q0 + t * BM + row_in_tile;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
            const bool vec32_ok = (ldo % 16 == 0) && ((reinterpret_cast<uintptr_t>(O) & 31) == 0);
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row < nq) {
                    __nv_bfloat16 *dst = O + static_cast<int64_t>(row) * ldo + h * 64 + c * 32;
                    if (vec32_ok) {
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            uint32_t w[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                w[i] = pack_bf16(__uint_as_float(o[16 * hh + 2 * i]) * inv,
                                                 __uint_as_float(o[16 * hh + 2 * i + 1]) * inv);
                            st_global_256(dst + 16 * hh, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
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
    if (warp == SOFTMAX_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, attn3::TMEM_COLS);
    }
}

// Launch of the two-threads-per-row kernel (called from attention_dispatch in attention.cu).
int attention_split_launch(gb200_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                           void *O, int64_t ldo, int64_t nq, int64_t nkv, float scale, cudaStream_t stream) {
    using namespace attn3;
    int rc = ensure_dynamic_smem(ctx, attention_bf16_split_kernel, SMEM_BYTES);
    if (rc) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    const unsigned grid = (unsigned)((nq + BM * TILES - 1) / (BM * TILES));
    GB200_CUDA_TRY(launch_pdl(attention_bf16_split_kernel, dim3(grid), dim3(NUM_THREADS), (size_t)SMEM_BYTES,
                              stream, tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv,
                              scale_log2, ctx->d_status));
    return after_launch(ctx, "attention_bf16_split_kernel");
}

int kernel_regs_attention_split() { return kernel_registers(attention_bf16_split_kernel); }

}  // namespace gb200

#ifdef GB200_ATTN_TRACE
extern "C" int gb200_attn3_trace_read(long long *out) {
    return (int)cudaMemcpyFromSymbol(out, gb200::g_attn3_trace, sizeof(long long) * 16 * 64);
}
#endif
