// Shared host/device plumbing of libgern_b200: context, error reporting, launch accounting,
// and thin inline-PTX wrappers for the sm_100a features the kernels use (mbarrier, TMA bulk
// tensor copies, tcgen05 MMA / TMEM).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <list>
#include <map>
#include <set>
#include <mutex>
#include <string>
#include <tuple>

#include "gern_b200.h"

namespace gb200 {

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------

void set_error(const char *fmt, ...);

#define GB200_CUDA_TRY(expr)                                                              \
    do {                                                                                  \
        cudaError_t err__ = (expr);                                                       \
        if (err__ != cudaSuccess) {                                                       \
            gb200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(err__),   \
                             __FILE__, __LINE__);                                         \
            return GB200_ERR_CUDA;                                                        \
        }                                                                                 \
    } while (0)

#define GB200_REQUIRE(cond, code, ...)        \
    do {                                      \
        if (!(cond)) {                        \
            gb200::set_error(__VA_ARGS__);    \
            return (code);                    \
        }                                     \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct TmapKey {
    const void *ptr;
    uint64_t d0, d1, stride1;
    uint32_t b0, b1;
    int dtype, swizzle;
    bool operator<(const TmapKey &o) const {
        return std::tie(ptr, d0, d1, stride1, b0, b1, dtype, swizzle) <
               std::tie(o.ptr, o.d0, o.d1, o.stride1, o.b0, o.b1, o.dtype, o.swizzle);
    }
};

}  // namespace gb200

struct gb200_ctx {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
    int64_t launches = 0;
    gb200::EncodeTiledFn encode_tiled = nullptr;
    // Tensor-map cache, least recently used first in `tmap_order`; bounded (kTmapCacheEntries) so
    // that a caller who passes fresh buffers on every call cannot grow it without limit.
    struct TmapEntry {
        CUtensorMap map;
        std::list<gb200::TmapKey>::iterator pos;
    };
    std::map<gb200::TmapKey, TmapEntry> tmaps;
    std::list<gb200::TmapKey> tmap_order;
    std::set<const void *> smem_attr_done;   // kernels whose dynamic shared memory limit is raised
    std::mutex mu;
    // device status word written by kernels whose bounded waits ran out
    int *d_status = nullptr;
    int *h_status = nullptr;   // pinned landing place for d_status in the _host entry points
    // staging of the _host entry points (grown on demand, freed at destroy)
    void *stage[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t stage_bytes[4] = {0, 0, 0, 0};
    // scratch of kernels that need global memory beyond their operands (split-K slabs)
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    // arrival counters of kernels whose thread blocks merge partial results among themselves;
    // zero whenever no such kernel is running (the merging block puts its counter back)
    int *merge_counters = nullptr;
    size_t merge_counter_words = 0;
    // Halo rows that live on another device are fetched by a copy engine on `halo_stream` into a
    // ring of local slots; a flag per slot tells the kernel that its rows have landed.
    cudaStream_t halo_stream = nullptr;
    float *halo_ring = nullptr;
    size_t halo_slot_floats = 0;
    int *halo_flags = nullptr;        // device, kHaloSlots words
    int *halo_flag_values = nullptr;  // pinned host, 256 words: [i] = i + 1
    unsigned long long halo_step = 0;
    // Bands below this many input bytes read a remote halo themselves: the two copy operations of a
    // step take 7-8 us on the copy stream, which a kernel shorter than that would wait for
    // (8192-column bands at N = 8, 1024 rows: 17.2 us per step prefetched, 12.5 us read directly).
    long long halo_prefetch_min_bytes = 48ll << 20;
    const void *last_halo = nullptr;    // the halo pointer of the last band call and the device that owns it
    int last_halo_device = -1;
    signed char peer_state[64] = {0};   // per device: 0 not asked, 1 this device's kernels may read it, -1 they may not
    cudaEvent_t halo_ev[4] = {nullptr, nullptr, nullptr, nullptr};
    cudaStream_t copy_stream[2] = {nullptr, nullptr};
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
};

namespace gb200 {

// Builds (or returns the cached) 2-D tiled tensor map over a row-major matrix:
// inner extent d0 elements, outer extent d1 rows, row pitch stride1_bytes, box b0 x b1.
int get_tmap_2d(gb200_ctx *ctx, const void *ptr, CUtensorMapDataType dtype, int elem_bytes,
                uint64_t d0, uint64_t d1, uint64_t stride1_bytes, uint32_t b0, uint32_t b1,
                CUtensorMapSwizzle swizzle, CUtensorMap *out);

constexpr size_t kTmapCacheEntries = 512;
constexpr int kHaloSlots = 32;      // ring of prefetched halo rows
constexpr int kHaloEventEvery = 8;  // a slot is reused once the launch 32 steps back has finished: one event per 8 launches
constexpr int kMaxGridY = 65535;   // CUDA's limit on gridDim.y and gridDim.z

// Sets the device for the calling thread, as every entry point must before touching CUDA.
int enter(gb200_ctx *ctx);
// The same for the extent of one entry point: makes the context's device current and puts the
// caller's device back when the entry point returns, so that a call on one context does not
// change what a later context-free call (or the caller's own CUDA code) runs on.
struct DeviceScope {
    int saved = -1;
    int enter(gb200_ctx *ctx);
    ~DeviceScope();
};
// End of a _host entry point: waits for the given streams (s1 may be NULL), then reads the
// context's status word and reports a bounded wait that ran out as GB200_ERR_TIMEOUT.
int host_finish(gb200_ctx *ctx, cudaStream_t s0, cudaStream_t s1);
// Raises a kernel's dynamic shared memory limit once per context (the attribute call costs a
// microsecond of host time, which a loop of short launches would pay every iteration).
template <typename Kernel>
inline int ensure_dynamic_smem(gb200_ctx *ctx, Kernel kernel, int bytes) {
    const void *key = reinterpret_cast<const void *>(kernel);
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->smem_attr_done.count(key)) return GB200_OK;
    GB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    ctx->smem_attr_done.insert(key);
    return GB200_OK;
}
// Registers per thread of `kernel` as compiled, or -1 where the CUDA runtime cannot tell (no device).
template <typename Kernel>
inline int kernel_registers(Kernel kernel) {
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return attr.numRegs;
}
// Grows staging slot `slot` to at least `bytes`.
int stage_reserve(gb200_ctx *ctx, int slot, size_t bytes);
// Grows the context's kernel workspace to at least `bytes`.
int workspace_reserve(gb200_ctx *ctx, size_t bytes);
// Grows the context's zeroed arrival counters to at least `words`.
int merge_counters_reserve(gb200_ctx *ctx, size_t words);
// Checks the launch that was just issued and counts it.
int after_launch(gb200_ctx *ctx, const char *what);

// ---------------------------------------------------------------------------------------
// device side: inline PTX
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__

// Launch with programmatic stream serialisation: the kernel's blocks may become resident while
// the previous kernel of the stream is still draining, which hides the launch gap between short
// kernels (blur at 8192^2: 82.2 -> 79.4 us per call, back to back).  Such a kernel must call
// pdl_wait() before it reads or writes anything the previous kernel may touch; on a stream whose
// previous work is not a kernel, or without the attribute, the wait returns at once.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The same with thread-block clusters of `cluster_x` blocks chosen at run time.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Everything before this call overlaps the previous kernel's tail; nothing after it runs until
// that kernel has completed and its writes are visible.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel of the stream start launching (it still waits in its own pdl_wait()).
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Upper bound on any mbarrier wait, in wall-clock time: a single try_wait may itself block for a
// hardware-defined while, so polls are not a usable unit.  Past the limit the waiting thread
// records a status code and leaves the wait, so that a protocol error ends the kernel (in a
// second or two) instead of hanging it.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;   // 1 s

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One try_wait may park the thread in hardware for up to this long; it resumes as soon as the
// phase completes.  A parked thread takes no issue slots from the warps that do the arithmetic,
// and a long wait needs few polls.
constexpr uint32_t kTryWaitHintNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kTryWaitHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after writing `code` to *status) if `limit_ns` of wall-clock time
// ran out (on top of the clock-free polls of the fast path, at most about 20 ms).
__device__ __forceinline__ bool mbar_wait_ns(uint64_t *bar, uint32_t parity, int *status, int code,
                                             unsigned long long limit_ns) {
    // Fast path: polls without a clock.  Reading the wall-clock timer is a long-latency operation
    // (a barrier that completes while the read is outstanding is noticed late, which showed as
    // microseconds on the TMA -> MMA -> epilogue hand-offs of a short GEMM), so the timer is
    // consulted only once a wait has outlasted any wait of a healthy pipeline.  Each poll is
    // bounded by the hardware (at most the hint above).
    for (int i = 0; i < 1024; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    while (true) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > limit_ns) break;
    }
    if (status) atomicExch(status, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *status, int code) {
    return mbar_wait_ns(bar, parity, status, code, kWaitLimitNs);
}
// Bounded wait for a word in global memory that a copy engine (or another device) writes after
// the data it announces.  Returns false (after writing `code` to *status) when the time ran out.
__device__ __forceinline__ bool wait_flag_equals_ns(const int *flag, int value, int *status, int code,
                                                    unsigned long long limit_ns) {
    auto look = [&]() {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        return v == value;
    };
    for (int i = 0; i < 1024; ++i)
        if (look()) return true;
    const unsigned long long t0 = global_timer_ns();
    while (true) {
        for (int i = 0; i < 32; ++i)
            if (look()) return true;
        if (global_timer_ns() - t0 > limit_ns) break;
    }
    if (status) atomicExch(status, code);
    return false;
}
__device__ __forceinline__ bool wait_flag_equals(const int *flag, int value, int *status, int code) {
    return wait_flag_equals_ns(flag, value, status, code, kWaitLimitNs);
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// TMA: global -> shared 2-D tile, completion counted in bytes on `bar`.  x = inner
// coordinate (elements), y = row.  No multicast anywhere in this library.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, int x, int y,
                                            uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// TMA: shared -> global 2-D tile (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *tmap, const void *smem_src, int x,
                                             int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05 / TMEM ----
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc].
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Makes `bar` complete one arrival once every tcgen05 op issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32-byte global store (one full sector per thread), sm_100 and later; `p` must be 32-byte aligned.
__device__ __forceinline__ void st_global_256(void *p, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                              uint32_t e, uint32_t f, uint32_t g, uint32_t h) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a), "r"(b), "r"(c),
                 "r"(d), "r"(e), "r"(f), "r"(g), "r"(h)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// ---- CTA pairs (clusters of two CTAs sharing one MMA: cta_group::2) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// Load from the shared memory of a CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier in (possibly) the other CTA of the cluster.  Default semantics (release at
// CTA scope): a cluster-scope release costs about a thousand cycles per arrival here (measured),
// and what the waiting side consumes -- TMEM and shared-memory tiles read by the tensor core -- is
// ordered by the tcgen05 / proxy fences the arriving thread issues first.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of this CTA's operand half; the byte count is reported to the barrier at
// cluster address `bar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *tmap, int x, int y,
                                                 uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the A operand in TMEM: each CTA's 128 rows of A come from its own TMEM.
__device__ __forceinline__ void umma_f16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this shared-memory offset in both CTAs of the pair, once every
// MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
            "r"(smem_u32(bar)),
        "h"(mask)
        : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma (sm_100 format, version field = 1):
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1
//   bits [61,64) swizzle: 2 = 128 B
// K-major operand tile whose rows are 128 bytes (64 bf16) written by TMA with
// SWIZZLE_128B: 8-row groups are 1024 bytes apart (SBO); LBO is unused for this layout.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate:
//   [4,6) D format (1 = f32)   [7,10) A format (1 = bf16)   [10,13) B format (1 = bf16)
//   [15] A major (0 = K)       [16] B major (0 = K, 1 = MN) [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// Two fp32 values -> one 32-bit word of two bf16 (round to nearest even), `lo` in the low half.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// Packed fp32x2 arithmetic (sm_100 has two-wide FADD/FMUL/FFMA): the same IEEE round-to-nearest
// operations as scalar code on two lanes at once, so results are bit-identical to the scalar
// form while the instruction count halves.
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpk2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// max over floats with integer atomics: non-negative values order like signed integers,
// negative ones like unsigned integers in reverse; the target starts at -inf.
__device__ __forceinline__ void atomic_max_f32(float *addr, float v) {
    if (v >= 0.0f)
        atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
    else
        atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

#endif  // __CUDACC__

}  // namespace gb200
