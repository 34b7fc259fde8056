// Static shared-memory planner of libgern_b200 (plain C++, no CUDA: usable on the host).
//
// Gern's annotation language lets a function state what it allocates -- Allocates(reg, smem),
// include/gern/annotations/stmt.h:113-121 -- but nothing in the reference's lowering reads it, and
// its emitted kernels carve dynamic shared memory at run time with a bump allocator that thread 0
// advances (gernels/mm/impl/sh_malloc.h:12-54).  The kernels here know their buffers at compile
// time, and the buffers have hardware rules a bump allocator does not know: a tile that TMA writes
// with 128-byte swizzle and tcgen05.mma reads through a shared-memory descriptor starts on a
// 1024-byte boundary, an mbarrier on 8 bytes, a TMA box row on 16.  So every kernel's layout is one
// constexpr description built with Planner below; the kernel takes its offsets from it, the launch
// takes its dynamic-shared-memory size from it, and the host layer reads the same figures through
// gb200_kernel_resources_query() to check a program's Global(..., smem_size) against them.
#pragma once

namespace gb200 {
namespace smem {

constexpr int kSwizzleTileAlign = 1024;   // SWIZZLE_128B TMA destination / UMMA operand tile
constexpr int kBarrierAlign = 8;          // mbarrier object
constexpr int kMaxDynamicBytes = 227 * 1024;   // opt-in limit of an sm_100a block

struct Region {
    int offset = 0;
    int bytes = 0;
    constexpr int end() const { return offset + bytes; }
};

// Hands out regions in declaration order, each aligned as asked, relative to a base that the
// kernel rounds up to `base_align` itself (the dynamic shared-memory window is only guaranteed 16
// bytes of alignment, so `dynamic_bytes()` includes that slack).
class Planner {
public:
    constexpr explicit Planner(int base_align = kSwizzleTileAlign) : base_align_(base_align) {}
    constexpr Region take(int bytes, int align) {
        cursor_ = (cursor_ + align - 1) / align * align;
        Region r{cursor_, bytes};
        cursor_ += bytes;
        return r;
    }
    constexpr Region tiles(int count, int tile_bytes) { return take(count * tile_bytes, kSwizzleTileAlign); }
    constexpr Region barriers(int count) { return take(count * 8, kBarrierAlign); }
    constexpr Region words(int count) { return take(count * 4, 4); }
    constexpr int payload_bytes() const { return cursor_; }
    // what the launch asks for: payload, rounded to 128 bytes, plus the slack of the base round-up
    constexpr int dynamic_bytes() const { return (cursor_ + 127) / 128 * 128 + base_align_; }

private:
    int base_align_;
    int cursor_ = 0;
};

// ---- bf16 GEMM, one CTA per tile: ring of (A 128 x 64, B tile_n x 64) stages ------------------
struct GemmTcLayout {
    static constexpr int kStages = 4, kBM = 128, kBK = 64, kThreads = 192, kTmemColumns = 512, kCluster = 1;
    int tile_n = 256;
    int stage_bytes = 0;
    Region stages, full, empty, acc_full, acc_empty, tmem_slot;
    int dynamic_bytes = 0;
};
constexpr GemmTcLayout gemm_tc_layout(int tile_n) {
    GemmTcLayout l;
    Planner p;
    l.tile_n = tile_n;
    l.stage_bytes = (GemmTcLayout::kBM + tile_n) * GemmTcLayout::kBK * 2;
    l.stages = p.tiles(GemmTcLayout::kStages, l.stage_bytes);
    l.full = p.barriers(GemmTcLayout::kStages);
    l.empty = p.barriers(GemmTcLayout::kStages);
    l.acc_full = p.barriers(2);
    l.acc_empty = p.barriers(2);
    l.tmem_slot = p.words(1);
    l.dynamic_bytes = p.dynamic_bytes();
    return l;
}

// ---- bf16 GEMM on CTA pairs: each CTA stages its 128-row halves of A and B ---------------------
struct Gemm2CtaLayout {
    static constexpr int kHalf = 128, kBK = 64, kThreads = 192, kTmemColumns = 512, kCluster = 2;
    int stages_n = 6;
    int stage_bytes = 0;
    Region stages, full, empty, acc_full, acc_empty, tmem_slot;
    int dynamic_bytes = 0;
};
constexpr Gemm2CtaLayout gemm_2cta_layout(int stages_n) {
    Gemm2CtaLayout l;
    Planner p;
    l.stages_n = stages_n;
    l.stage_bytes = 2 * Gemm2CtaLayout::kHalf * Gemm2CtaLayout::kBK * 2;
    l.stages = p.tiles(stages_n, l.stage_bytes);
    l.full = p.barriers(stages_n);
    l.empty = p.barriers(stages_n);
    l.acc_full = p.barriers(2);
    l.acc_empty = p.barriers(2);
    l.tmem_slot = p.words(1);
    l.dynamic_bytes = p.dynamic_bytes();
    return l;
}

// ---- GEMM -> softmax -> GEMM, two Q tiles per CTA -----------------------------------------------
struct AttentionLayout {
    static constexpr int kTiles = 2, kKvSlots = 5, kTileBytes = 128 * 128 * 2, kTmemColumns = 512, kCluster = 1;
    int threads = 320;
    Region q, kv, q_full, q_empty, kv_full, kv_empty, s_full, sp_ready, o_full, p_half, tmem_slot;
    int dynamic_bytes = 0;
};
constexpr AttentionLayout attention_layout(int threads) {
    AttentionLayout l;
    Planner p;
    l.threads = threads;
    l.q = p.tiles(AttentionLayout::kTiles, AttentionLayout::kTileBytes);
    l.kv = p.tiles(AttentionLayout::kKvSlots, AttentionLayout::kTileBytes);
    l.q_full = p.barriers(1);
    l.q_empty = p.barriers(1);
    l.kv_full = p.barriers(AttentionLayout::kKvSlots);
    l.kv_empty = p.barriers(AttentionLayout::kKvSlots);
    l.s_full = p.barriers(AttentionLayout::kTiles);
    l.sp_ready = p.barriers(AttentionLayout::kTiles);
    l.o_full = p.barriers(AttentionLayout::kTiles);
    l.p_half = p.barriers(AttentionLayout::kTiles);
    l.tmem_slot = p.words(1);
    l.dynamic_bytes = p.dynamic_bytes();
    return l;
}

// ---- GEMM -> softmax -> GEMM on CTA pairs, two Q tiles per CTA ------------------------------------
// Each CTA holds its two Q tiles and a ring of half blocks: 64 kv rows of K_j, or 64 head-dimension
// columns of V_j (16 KiB each).
struct AttentionPairLayout {
    static constexpr int kTiles = 2, kKvSlots = 10, kTileBytes = 128 * 128 * 2, kHalfBytes = 16 * 1024,
                         kThreads = 320, kTmemColumns = 512, kCluster = 2;
    Region q, kv, q_full, kv_full, kv_empty, s_full, sp_ready, o_full, p_half, tmem_slot;
    int dynamic_bytes = 0;
};
constexpr AttentionPairLayout attention_pair_layout() {
    AttentionPairLayout l;
    Planner p;
    l.q = p.tiles(AttentionPairLayout::kTiles, AttentionPairLayout::kTileBytes);
    l.kv = p.tiles(AttentionPairLayout::kKvSlots, AttentionPairLayout::kHalfBytes);
    l.q_full = p.barriers(1);
    l.kv_full = p.barriers(AttentionPairLayout::kKvSlots);
    l.kv_empty = p.barriers(AttentionPairLayout::kKvSlots);
    l.s_full = p.barriers(AttentionPairLayout::kTiles);
    l.sp_ready = p.barriers(AttentionPairLayout::kTiles);
    l.o_full = p.barriers(AttentionPairLayout::kTiles);
    l.p_half = p.barriers(AttentionPairLayout::kTiles);
    l.tmem_slot = p.words(1);
    l.dynamic_bytes = p.dynamic_bytes();
    return l;
}
static_assert(attention_pair_layout().dynamic_bytes <= kMaxDynamicBytes, "pair attention layout exceeds a block's shared memory");

static_assert(gemm_tc_layout(256).dynamic_bytes <= kMaxDynamicBytes, "GEMM ring exceeds a block's shared memory");
static_assert(gemm_2cta_layout(6).dynamic_bytes <= kMaxDynamicBytes, "pair GEMM ring exceeds a block's shared memory");
static_assert(attention_layout(320).dynamic_bytes <= kMaxDynamicBytes, "attention layout exceeds a block's shared memory");
static_assert(gemm_tc_layout(192).stages.offset % kSwizzleTileAlign == 0 && attention_layout(320).kv.offset % kSwizzleTileAlign == 0,
              "swizzled tiles start on 1024-byte boundaries");

}  // namespace smem
}  // namespace gb200
