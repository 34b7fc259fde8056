// Context, error reporting, tensor-map cache and staging buffers of libgern_b200.
// Stands in for what Gern's emitted hook does around each launch
// (src/codegen/codegen.cpp:31-101: device-limit asserts, launch, check_last_error), with the
// device limits read once per context instead of once per launch.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace gb200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int enter(gb200_ctx *ctx) {
    GB200_REQUIRE(ctx != nullptr, GB200_ERR_INVALID_ARG, "ctx is NULL");
    GB200_CUDA_TRY(cudaSetDevice(ctx->device));
    return GB200_OK;
}

int DeviceScope::enter(gb200_ctx *ctx) {
    GB200_REQUIRE(ctx != nullptr, GB200_ERR_INVALID_ARG, "ctx is NULL");
    int cur = -1;
    GB200_CUDA_TRY(cudaGetDevice(&cur));
    if (cur != ctx->device) {
        GB200_CUDA_TRY(cudaSetDevice(ctx->device));
        saved = cur;
    }
    return GB200_OK;
}

DeviceScope::~DeviceScope() {
    if (saved >= 0) cudaSetDevice(saved);
}

int host_finish(gb200_ctx *ctx, cudaStream_t s0, cudaStream_t s1) {
    if (s1) GB200_CUDA_TRY(cudaStreamSynchronize(s1));
    // the status word travels behind the last of the work on s0
    GB200_CUDA_TRY(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, s0));
    GB200_CUDA_TRY(cudaStreamSynchronize(s0));
    if (*ctx->h_status != 0) {
        const int st = *ctx->h_status;
        cudaMemsetAsync(ctx->d_status, 0, sizeof(int), s0);
        // a kernel that gave up may have left arrival counters half way
        if (ctx->merge_counters) cudaMemsetAsync(ctx->merge_counters, 0, ctx->merge_counter_words * sizeof(int), s0);
        cudaStreamSynchronize(s0);
        set_error("a kernel gave up a bounded wait (status code %d); the result is not valid", st);
        return GB200_ERR_TIMEOUT;
    }
    return GB200_OK;
}

int after_launch(gb200_ctx *ctx, const char *what) {
    cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        cudaGetLastError();
        set_error("launch of %s failed: %s", what, cudaGetErrorString(err));
        return GB200_ERR_CUDA;
    }
    ctx->launches += 1;
    return GB200_OK;
}

int stage_reserve(gb200_ctx *ctx, int slot, size_t bytes) {
    if (ctx->stage_bytes[slot] >= bytes) return GB200_OK;
    if (ctx->stage[slot]) {
        GB200_CUDA_TRY(cudaFree(ctx->stage[slot]));
        ctx->stage[slot] = nullptr;
        ctx->stage_bytes[slot] = 0;
    }
    GB200_CUDA_TRY(cudaMalloc(&ctx->stage[slot], bytes));
    ctx->stage_bytes[slot] = bytes;
    return GB200_OK;
}

int workspace_reserve(gb200_ctx *ctx, size_t bytes) {
    if (ctx->workspace_bytes >= bytes) return GB200_OK;
    if (ctx->workspace) {
        GB200_CUDA_TRY(cudaFree(ctx->workspace));   // cudaFree waits for work that still uses it
        ctx->workspace = nullptr;
        ctx->workspace_bytes = 0;
    }
    GB200_CUDA_TRY(cudaMalloc(&ctx->workspace, bytes));
    ctx->workspace_bytes = bytes;
    return GB200_OK;
}

int merge_counters_reserve(gb200_ctx *ctx, size_t words) {
    if (ctx->merge_counter_words >= words) return GB200_OK;
    if (ctx->merge_counters) {
        GB200_CUDA_TRY(cudaFree(ctx->merge_counters));
        ctx->merge_counters = nullptr;
        ctx->merge_counter_words = 0;
    }
    GB200_CUDA_TRY(cudaMalloc(&ctx->merge_counters, words * sizeof(int)));
    GB200_CUDA_TRY(cudaMemset(ctx->merge_counters, 0, words * sizeof(int)));
    ctx->merge_counter_words = words;
    return GB200_OK;
}

int get_tmap_2d(gb200_ctx *ctx, const void *ptr, CUtensorMapDataType dtype, int elem_bytes,
                uint64_t d0, uint64_t d1, uint64_t stride1_bytes, uint32_t b0, uint32_t b1,
                CUtensorMapSwizzle swizzle, CUtensorMap *out) {
    GB200_REQUIRE(ctx->encode_tiled != nullptr, GB200_ERR_NO_DEVICE,
                  "cuTensorMapEncodeTiled is not available from this driver");
    GB200_REQUIRE((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (stride1_bytes & 15) == 0 &&
                      ((uint64_t)b0 * elem_bytes) % 16 == 0 && b0 <= 256 && b1 <= 256,
                  GB200_ERR_UNSUPPORTED,
                  "tensor map needs a 16-byte aligned base, pitch and box row (ptr=%p pitch=%llu)",
                  ptr, (unsigned long long)stride1_bytes);
    TmapKey key{ptr, d0, d1, stride1_bytes, b0, b1, (int)dtype, (int)swizzle};
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->tmaps.find(key);
    if (it != ctx->tmaps.end()) {
        ctx->tmap_order.splice(ctx->tmap_order.end(), ctx->tmap_order, it->second.pos);
        *out = it->second.map;
        return GB200_OK;
    }
    CUtensorMap tm;
    cuuint64_t dims[2] = {d0, d1};
    cuuint64_t strides[1] = {stride1_bytes};
    cuuint32_t box[2] = {b0, b1};
    cuuint32_t estr[2] = {1, 1};
    CUresult rc = ctx->encode_tiled(&tm, dtype, 2, const_cast<void *>(ptr), dims, strides, box,
                                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, box %u x %u)",
                  (int)rc, (unsigned long long)d0, (unsigned long long)d1, b0, b1);
        return GB200_ERR_CUDA;
    }
    while (ctx->tmaps.size() >= kTmapCacheEntries) {       // evict the least recently used
        ctx->tmaps.erase(ctx->tmap_order.front());
        ctx->tmap_order.pop_front();
    }
    ctx->tmap_order.push_back(key);
    ctx->tmaps[key] = gb200_ctx::TmapEntry{tm, std::prev(ctx->tmap_order.end())};
    *out = tm;
    return GB200_OK;
}

// Self-test of the bounded wait every TMA / tcgen05 kernel relies on: one thread waits on an mbarrier
// that nobody ever arrives on, with the wall-clock limit given by the caller.  The wait gives up,
// records code 901 in the status word and the kernel returns: nothing hangs and nothing faults.
__global__ void bounded_wait_probe_kernel(int *status, unsigned long long limit_ns, int *returned) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        const bool completed = mbar_wait_ns(&bar, 0, status, 901, limit_ns);
        *returned = completed ? 2 : 1;
    }
}

// The same for the one wait on a word in global memory (the blur's halo block row waiting for its
// slot's flag): the probe waits for a value nobody writes; code 902.
__global__ void bounded_flag_wait_probe_kernel(int *status, unsigned long long limit_ns, int *returned,
                                               const int *flag) {
    if (threadIdx.x == 0) {
        const bool seen = wait_flag_equals_ns(flag, 0x7fffffff, status, 902, limit_ns);
        *returned = seen ? 2 : 1;
    }
}

}  // namespace gb200

using namespace gb200;

extern "C" {

// Test hook: the flag-wait probe; `returned` doubles as the flag (the probe never sees 0x7fffffff in it
// before it gives up and overwrites it).
int gb200_selftest_bounded_flag_wait(gb200_ctx *ctx, unsigned long long limit_ns, int *returned, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(returned != nullptr, GB200_ERR_INVALID_ARG, "returned is NULL");
    GB200_REQUIRE(limit_ns <= 100ull * 1000ull * 1000ull, GB200_ERR_INVALID_ARG,
                  "the probe's limit is capped at 100 ms");
    bounded_flag_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->d_status, limit_ns, returned,
                                                                                  returned);
    return after_launch(ctx, "bounded_flag_wait_probe_kernel");
}

// Test hook (not part of the documented surface): launches the probe above on `stream`.
// `returned` is a device int that the kernel sets to 1 when the wait gave up (2 if it completed).
int gb200_selftest_bounded_wait(gb200_ctx *ctx, unsigned long long limit_ns, int *returned, void *stream) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_REQUIRE(returned != nullptr, GB200_ERR_INVALID_ARG, "returned is NULL");
    GB200_REQUIRE(limit_ns <= 100ull * 1000ull * 1000ull, GB200_ERR_INVALID_ARG,
                  "the probe's limit is capped at 100 ms");
    bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->d_status, limit_ns, returned);
    return after_launch(ctx, "bounded_wait_probe_kernel");
}

const char *gb200_last_error_string(void) { return g_err; }

const char *gb200_version(void) { return "gern_b200 0.1 (sm_100a)"; }

int gb200_ctx_create(int device, gb200_ctx **out) {
    GB200_REQUIRE(out != nullptr, GB200_ERR_INVALID_ARG, "out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        cudaGetLastError();
        set_error("no CUDA device: %s", err == cudaSuccess ? "device count is 0"
                                                           : cudaGetErrorString(err));
        return GB200_ERR_NO_DEVICE;
    }
    GB200_REQUIRE(device >= 0 && device < count, GB200_ERR_INVALID_ARG,
                  "device %d out of range (have %d)", device, count);
    struct Restore {   // the caller's current device is put back on every return path
        int saved = -1;
        ~Restore() { if (saved >= 0) cudaSetDevice(saved); }
    } restore;
    if (cudaGetDevice(&restore.saved) != cudaSuccess) { cudaGetLastError(); restore.saved = -1; }
    GB200_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    GB200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    GB200_REQUIRE(prop.major == 10, GB200_ERR_NO_DEVICE,
                  "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major,
                  prop.minor);
    gb200_ctx *ctx = new gb200_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess)
        ctx->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    else
        cudaGetLastError();
    err = cudaMalloc(&ctx->d_status, sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(ctx->d_status, 0, sizeof(int));
    if (err == cudaSuccess) err = cudaMallocHost(&ctx->h_status, sizeof(int));
    if (err == cudaSuccess) *ctx->h_status = 0;
    for (int i = 0; i < 2 && err == cudaSuccess; ++i)
        err = cudaStreamCreateWithFlags(&ctx->copy_stream[i], cudaStreamNonBlocking);
    for (int i = 0; i < 4 && err == cudaSuccess; ++i)
        err = cudaEventCreateWithFlags(&ctx->ev[i], cudaEventDisableTiming);
    if (err != cudaSuccess) {
        set_error("context set-up failed: %s", cudaGetErrorString(err));
        gb200_ctx_destroy(ctx);
        return GB200_ERR_CUDA;
    }
    *out = ctx;
    return GB200_OK;
}

int gb200_ctx_destroy(gb200_ctx *ctx) {
    if (!ctx) return GB200_OK;
    DeviceScope scope;
    if (scope.enter(ctx) != GB200_OK) return GB200_ERR_CUDA;
    cudaDeviceSynchronize();
    for (int i = 0; i < 4; ++i)
        if (ctx->stage[i]) cudaFree(ctx->stage[i]);
    for (int i = 0; i < 2; ++i)
        if (ctx->copy_stream[i]) cudaStreamDestroy(ctx->copy_stream[i]);
    for (int i = 0; i < 4; ++i)
        if (ctx->ev[i]) cudaEventDestroy(ctx->ev[i]);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->merge_counters) cudaFree(ctx->merge_counters);
    if (ctx->halo_stream) cudaStreamDestroy(ctx->halo_stream);
    if (ctx->halo_ring) cudaFree(ctx->halo_ring);
    if (ctx->halo_flags) cudaFree(ctx->halo_flags);
    if (ctx->halo_flag_values) cudaFreeHost(ctx->halo_flag_values);
    for (int i = 0; i < 4; ++i)
        if (ctx->halo_ev[i]) cudaEventDestroy(ctx->halo_ev[i]);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    delete ctx;
    return GB200_OK;
}

int gb200_device_sync(gb200_ctx *ctx) {
    DeviceScope scope;
    int rc = scope.enter(ctx);
    if (rc) return rc;
    GB200_CUDA_TRY(cudaDeviceSynchronize());
    int st = 0;
    GB200_CUDA_TRY(cudaMemcpy(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(ctx->d_status, 0, sizeof(int));
        if (ctx->merge_counters) cudaMemset(ctx->merge_counters, 0, ctx->merge_counter_words * sizeof(int));
        set_error("a kernel gave up a bounded wait (status code %d)", st);
        return GB200_ERR_TIMEOUT;
    }
    return GB200_OK;
}

int64_t gb200_launch_count(gb200_ctx *ctx) { return ctx ? ctx->launches : 0; }

}  // extern "C"
