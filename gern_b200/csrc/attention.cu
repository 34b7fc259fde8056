// Fused GEMM -> row softmax -> GEMM chain on the sm_100a tensor cores:
//     O = softmax_rows(scale * Q K^T) V,   Q [nq,128], K [nkv,128], V [nkv,128], O [nq,128] bf16.
//
// In Gern's terms this is the program  Tile(O.row)( mm(Q,K^T -> S), softmax pieces(S -> P),
// mm(P,V -> O) )  with S and P as per-tile temporaries, the shape of the reference's chained
// matmul fusion (test/test-cpu-mm.cpp:266-408, E = (A*B)*D with C allocated per tile) with the
// five softmax ops (apps/common/annot/functions.h:9-173) between the two multiplies.  Here the
// temporaries never reach HBM: S lives in TMEM, P is re-quantised to bf16 into shared memory as
// the A operand of the second multiply, and the softmax is computed online over 128-wide blocks
// of K/V with a running row maximum and row sum.
//
// One CTA owns 128 rows of Q.  Warp 0 streams K and V blocks through 2-deep TMA rings; warp 1
// issues tcgen05.mma for S_j = Q K_j^T (two TMEM buffers, so S_{j+1} is computed while block j is
// in the softmax) and O += P_j V_j; warps 2-5 own one row of the tile per thread: they read S_j
// from TMEM, update max/sum, write P_j to shared memory in the 128-byte-swizzled K-major layout
// the MMA reads, rescale O in TMEM when the running maximum has grown by more than 2^8, and at
// the end normalise and store O.  Every wait is bounded and reports through the status word.
#include <float.h>

#include "common.cuh"

namespace gb200 {

namespace attn {
constexpr int BM = 128, BN = 128, D = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;  // 32 KiB: any 128 x 128 bf16 tile (2 swizzle chunks)
constexpr int CHUNK_BYTES = 128 * 128;     // 16 KiB: 128 rows x 64 bf16
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 192;
// Q, P, K ring, V ring, then barriers
constexpr int SMEM_BYTES = (2 + 2 * KV_STAGES) * TILE_BYTES + 1024 + 256;
constexpr uint32_t TMEM_COLS = 512;  // S0 [0,128) S1 [128,256) O [256,384)
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units
}  // namespace attn

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(attn::NUM_THREADS, 1)
attention_bf16_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, __nv_bfloat16 *__restrict__ O,
                      int64_t ldo, int nq, int nkv, float scale_log2, int *status) {
    using namespace attn;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *sQ = smem;
    unsigned char *sP = smem + TILE_BYTES;
    unsigned char *sK = smem + 2 * TILE_BYTES;
    unsigned char *sV = smem + (2 + KV_STAGES) * TILE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (2 + 2 * KV_STAGES) * TILE_BYTES);
    uint64_t *q_full = bars;           // [1]
    uint64_t *k_full = bars + 1;       // [2]
    uint64_t *k_empty = bars + 3;      // [2]
    uint64_t *v_full = bars + 5;       // [2]
    uint64_t *v_empty = bars + 7;      // [2]
    uint64_t *s_full = bars + 9;       // [2]
    uint64_t *s_free = bars + 11;      // [2]
    uint64_t *p_ready = bars + 13;     // [1]
    uint64_t *pv_done = bars + 14;     // [1]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 15);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * BM;
    const int n_blocks = (nkv + BN - 1) / BN;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmap_q);
        prefetch_tmap(&tmap_k);
        prefetch_tmap(&tmap_v);
        mbar_init(q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_full[b], 1);
            mbar_init(&s_free[b], 4);
        }
        mbar_init(p_ready, 4);
        mbar_init(pv_done, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_2d(sQ, &tmap_q, 0, q0, q_full);
            tma_load_2d(sQ + CHUNK_BYTES, &tmap_q, 64, q0, q_full);
            for (int j = 0; j < n_blocks; ++j) {
                const int st = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                if (!mbar_wait(&k_empty[st], ph ^ 1, status, 301)) break;
                mbar_expect_tx(&k_full[st], TILE_BYTES);
                tma_load_2d(sK + st * TILE_BYTES, &tmap_k, 0, j * BN, &k_full[st]);
                tma_load_2d(sK + st * TILE_BYTES + CHUNK_BYTES, &tmap_k, 64, j * BN, &k_full[st]);
                if (!mbar_wait(&v_empty[st], ph ^ 1, status, 302)) break;
                mbar_expect_tx(&v_full[st], TILE_BYTES);
                tma_load_2d(sV + st * TILE_BYTES, &tmap_v, 0, j * BN, &v_full[st]);
                tma_load_2d(sV + st * TILE_BYTES + CHUNK_BYTES, &tmap_v, 64, j * BN, &v_full[st]);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BN, 0);  // A, B both K-major
            constexpr uint32_t idesc_pv = umma_idesc_bf16(BM, D, 1);   // B (= V) is MN-major
            const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
            bool ok = mbar_wait(q_full, 0, status, 303);

            auto issue_qk = [&](int j) -> bool {
                const int st = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                const int buf = j & 1;
                if (!mbar_wait(&k_full[st], ph, status, 304)) return false;
                // S[buf] was last read by the softmax of block j-2
                if (!mbar_wait(&s_free[buf], ((j >> 1) & 1) ^ 1, status, 305)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
                    umma_f16_ss(tmem_base + buf * BN, umma_desc_sw128(q_addr + off, 16, 1024),
                                umma_desc_sw128(k_addr + off, 16, 1024), idesc_qk, ks != 0);
                }
                umma_commit(&k_empty[st]);
                umma_commit(&s_full[buf]);
                return true;
            };

            if (ok && n_blocks > 0) ok = issue_qk(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                if (j + 1 < n_blocks) {
                    ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                const int st = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1;
                if (!mbar_wait(&v_full[st], ph, status, 306)) { ok = false; break; }
                if (!mbar_wait(p_ready, j & 1, status, 307)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
                for (int ks = 0; ks < BN / 16; ++ks) {
                    // A = P: K-major, 16 kv values = 32 bytes inside the swizzle row.
                    const uint32_t a_off = (ks / 4) * CHUNK_BYTES + (ks % 4) * 32;
                    // B = V: MN-major; 16 kv rows = 2048 bytes; the two 64-wide d chunks are
                    // CHUNK_BYTES apart (leading offset), 8-row groups 1024 bytes apart.
                    const uint32_t b_off = ks * 16 * 128;
                    umma_f16_ss(tmem_o, umma_desc_sw128(p_addr + a_off, 16, 1024),
                                umma_desc_sw128(v_addr + b_off, CHUNK_BYTES, 1024), idesc_pv,
                                (j | ks) != 0);
                }
                umma_commit(&v_empty[st]);
                umma_commit(pv_done);
            }
        }
    } else {
        // ---------------- softmax / correction / epilogue: one row per thread ----------------
        const int lane_group = warp & 3;
        const int row_in_tile = lane_group * 32 + lane;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
        const uint32_t t_o = t_row + 256;
        float m_used = -FLT_MAX;  // maximum the exponentials are taken against (log2 domain)
        float l = 0.0f;           // running row sum
        bool ok = true;
        unsigned char *p_row = sP + row_in_tile * 128;
        const int sw = row_in_tile & 7;

        for (int j = 0; j < n_blocks && ok; ++j) {
            const int buf = j & 1;
            if (!mbar_wait(&s_full[buf], (j >> 1) & 1, status, 308)) { ok = false; break; }
            tc_fence_after();
            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_row + buf * BN + c * 32, sr[c]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[buf]);

            const int valid = min(BN, nkv - j * BN);
            float m_blk = -FLT_MAX;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float v = __uint_as_float(sr[c][i]) * scale_log2;
                    if (c * 32 + i >= valid) v = -FLT_MAX;
                    sr[c][i] = __float_as_uint(v);
                    m_blk = fmaxf(m_blk, v);
                }
            // Lazy rescale: keep the old reference maximum unless it has fallen behind by more
            // than the threshold, so that O is touched rarely.
            const bool grow = (m_blk - m_used) > RESCALE_THRESHOLD;
            float alpha = 1.0f;
            if (j == 0) {
                m_used = m_blk;
            } else if (grow) {
                alpha = fast_exp2(m_used - m_blk);
                m_used = m_blk;
                l *= alpha;
            }
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float p = fast_exp2(__uint_as_float(sr[c][i]) - m_used);
                    sum += p;
                    sr[c][i] = __float_as_uint(p);
                }
            l += sum;

            // P (and O) may be touched only after P_{j-1} V_{j-1} has finished.
            if (j > 0) {
                if (!mbar_wait(pv_done, (j - 1) & 1, status, 309)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32(t_o + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(t_o + c * 32, o);
                    }
                    tmem_st_wait();
                }
            }
            // P row -> shared memory, bf16, 128-byte swizzle (16-byte unit u of row r lands at
            // unit u ^ (r % 8)); kv 0-63 in the first chunk, 64-127 in the second.
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 v;
                    v.x = pack_bf16(__uint_as_float(sr[c][8 * q + 0]), __uint_as_float(sr[c][8 * q + 1]));
                    v.y = pack_bf16(__uint_as_float(sr[c][8 * q + 2]), __uint_as_float(sr[c][8 * q + 3]));
                    v.z = pack_bf16(__uint_as_float(sr[c][8 * q + 4]), __uint_as_float(sr[c][8 * q + 5]));
                    v.w = pack_bf16(__uint_as_float(sr[c][8 * q + 6]), __uint_as_float(sr[c][8 * q + 7]));
                    const int unit = (c & 1) * 4 + q;  // 16-byte unit inside the 128-byte row
                    *reinterpret_cast<uint4 *>(p_row + (c >> 1) * CHUNK_BYTES + ((unit ^ sw) << 4)) = v;
                }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
        }

        // ---- epilogue: O / l -> bf16 -> global ----
        if (ok && n_blocks > 0) ok = mbar_wait(pv_done, (n_blocks - 1) & 1, status, 310);
        if (ok && n_blocks > 0) {
            tc_fence_after();
            const float inv = 1.0f / l;
            const int row = q0 + row_in_tile;
            const bool vec_ok = (ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(O) & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(t_o + c * 32, o);
                tmem_ld_wait();
                if (row < nq) {
                    __nv_bfloat16 *dst = O + static_cast<int64_t>(row) * ldo + c * 32;
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, attn::TMEM_COLS);
    }
}

int attention_dispatch(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                       const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq, int64_t nkv,
                       int64_t d, float scale, cudaStream_t stream) {
    using namespace attn;
    GB200_REQUIRE(d == D, GB200_ERR_UNSUPPORTED, "attention: d must be %d in this build (got %lld)",
                  D, (long long)d);
    GB200_REQUIRE(ctx->encode_tiled != nullptr, GB200_ERR_NO_DEVICE, "TMA descriptors unavailable");
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
    GB200_CUDA_TRY(cudaFuncSetAttribute(attention_bf16_kernel,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    const float scale_log2 = scale * 1.4426950408889634f;
    const unsigned grid = (unsigned)((nq + BM - 1) / BM);
    attention_bf16_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(
        tq, tk, tv, static_cast<__nv_bfloat16 *>(O), ldo, (int)nq, (int)nkv, scale_log2,
        ctx->d_status);
    return after_launch(ctx, "attention_bf16_kernel");
}

static int check_attention_args(const void *Q, int64_t ldq, const void *K, int64_t ldk,
                                const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                                int64_t nkv, int64_t d) {
    GB200_REQUIRE(nq >= 0 && nkv >= 0 && d >= 0, GB200_ERR_INVALID_ARG, "negative extent");
    GB200_REQUIRE(nq < (1ll << 30) && nkv < (1ll << 30), GB200_ERR_UNSUPPORTED, "extent beyond 2^30");
    if (nq == 0 || d == 0) return 1;
    GB200_REQUIRE(nkv > 0, GB200_ERR_INVALID_ARG, "softmax over an empty row (nkv == 0)");
    GB200_REQUIRE(Q && K && V && O, GB200_ERR_INVALID_ARG, "NULL matrix pointer");
    GB200_REQUIRE(ldq >= d && ldk >= d && ldv >= d && ldo >= d, GB200_ERR_INVALID_ARG,
                  "leading dimension smaller than the row");
    return GB200_OK;
}

}  // namespace gb200

using namespace gb200;

extern "C" {

int gb200_attention_bf16(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                         const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                         int64_t nkv, int64_t d, float scale, void *stream) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d);
    if (rc) return rc < 0 ? rc : GB200_OK;
    return attention_dispatch(ctx, Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d, scale,
                              static_cast<cudaStream_t>(stream));
}

int gb200_attention_bf16_host(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K,
                              int64_t ldk, const void *V, int64_t ldv, void *O, int64_t ldo,
                              int64_t nq, int64_t nkv, int64_t d, float scale) {
    int rc = enter(ctx);
    if (rc) return rc;
    rc = check_attention_args(Q, ldq, K, ldk, V, ldv, O, ldo, nq, nkv, d);
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
    GB200_CUDA_TRY(cudaStreamSynchronize(s));
    return GB200_OK;
}

}  // extern "C"
