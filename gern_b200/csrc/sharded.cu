// Single-process multi-GPU forms of the entry points: one call enqueues one shard per device.
// The reference launches on device 0 only (src/codegen/codegen.cpp:576-611 emits no device
// selection), so these have no counterpart there; they exist for a Gern host function that owns
// all the GPUs of a box from one thread.  Each shard is a contiguous block of rows (matrix rows,
// image rows); the only data that crosses devices is the blur's two halo rows, which the band
// kernel reads from the next device's memory with ordinary loads.
#include "common.cuh"

namespace gb200 {

namespace {

// Restores the calling thread's current device on every exit path.
struct DeviceRestore {
    int saved = -1;
    DeviceRestore() { if (cudaGetDevice(&saved) != cudaSuccess) saved = -1; }
    ~DeviceRestore() { if (saved >= 0) cudaSetDevice(saved); }
};

int check_shards(const gb200_shard *shards, int n, bool need_in1) {
    GB200_REQUIRE(shards != nullptr, GB200_ERR_INVALID_ARG, "shards is NULL");
    GB200_REQUIRE(n >= 1 && n <= 64, GB200_ERR_INVALID_ARG, "number of shards %d outside 1..64", n);
    for (int g = 0; g < n; ++g) {
        GB200_REQUIRE(shards[g].ctx != nullptr, GB200_ERR_INVALID_ARG, "shard %d: ctx is NULL", g);
        GB200_REQUIRE(shards[g].rows >= 0, GB200_ERR_INVALID_ARG, "shard %d: negative rows", g);
        if (shards[g].rows == 0) continue;
        GB200_REQUIRE(shards[g].in != nullptr && shards[g].out != nullptr, GB200_ERR_INVALID_ARG,
                      "shard %d: NULL operand", g);
        if (need_in1)
            GB200_REQUIRE(shards[g].shared0 != nullptr, GB200_ERR_INVALID_ARG,
                          "shard %d: NULL replicated operand", g);
    }
    return GB200_OK;
}

// Lets kernels on `ctx`'s device load from memory of `peer`.  A second request for the same
// pair reports cudaErrorPeerAccessAlreadyEnabled, which is the state that is wanted.
int enable_peer_loads(gb200_ctx *ctx, int peer) {
    if (ctx->device == peer) return GB200_OK;
    int can = 0;
    GB200_CUDA_TRY(cudaDeviceCanAccessPeer(&can, ctx->device, peer));
    GB200_REQUIRE(can != 0, GB200_ERR_UNSUPPORTED, "device %d cannot read device %d's memory",
                  ctx->device, peer);
    GB200_CUDA_TRY(cudaSetDevice(ctx->device));
    cudaError_t err = cudaDeviceEnablePeerAccess(peer, 0);
    if (err == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return GB200_OK;
    }
    GB200_CUDA_TRY(err);
    return GB200_OK;
}

}  // namespace
}  // namespace gb200

using namespace gb200;

extern "C" int gb200_gemm_bf16_sharded(const gb200_shard *shards, int n, int64_t lda, int64_t ldb,
                                       int64_t ldc, int64_t N, int64_t K) {
    int rc = check_shards(shards, n, true);
    if (rc != GB200_OK) return rc;
    DeviceRestore restore;
    for (int g = 0; g < n; ++g) {
        const gb200_shard &s = shards[g];
        if (s.rows == 0) continue;
        rc = gb200_gemm_bf16(s.ctx, s.in, lda, s.shared0, ldb, s.out, ldc, s.rows, N, K, s.stream);
        if (rc != GB200_OK) return rc;
    }
    return GB200_OK;
}

extern "C" int gb200_softmax_rows_f32_sharded(const gb200_shard *shards, int n, int64_t ld_in,
                                              int64_t ld_out, int64_t cols) {
    int rc = check_shards(shards, n, false);
    if (rc != GB200_OK) return rc;
    DeviceRestore restore;
    for (int g = 0; g < n; ++g) {
        const gb200_shard &s = shards[g];
        if (s.rows == 0) continue;
        rc = gb200_softmax_rows_f32(s.ctx, static_cast<const float *>(s.in), ld_in,
                                    static_cast<float *>(s.out), ld_out, s.rows, cols, s.stream);
        if (rc != GB200_OK) return rc;
    }
    return GB200_OK;
}

extern "C" int gb200_attention_bf16_sharded(const gb200_shard *shards, int n, int64_t ldq,
                                            int64_t ldk, int64_t ldv, int64_t ldo, int64_t nkv,
                                            int64_t d, float scale) {
    int rc = check_shards(shards, n, true);
    if (rc != GB200_OK) return rc;
    for (int g = 0; g < n; ++g)
        GB200_REQUIRE(shards[g].rows == 0 || shards[g].shared1 != nullptr, GB200_ERR_INVALID_ARG,
                      "shard %d: NULL V", g);
    DeviceRestore restore;
    for (int g = 0; g < n; ++g) {
        const gb200_shard &s = shards[g];
        if (s.rows == 0) continue;
        rc = gb200_attention_bf16(s.ctx, s.in, ldq, s.shared0, ldk, s.shared1, ldv, s.out, ldo,
                                  s.rows, nkv, d, scale, s.stream);
        if (rc != GB200_OK) return rc;
    }
    return GB200_OK;
}

extern "C" int gb200_blur3x3_f32_sharded(const gb200_shard *shards, int n, int64_t in_ld,
                                         int64_t in_cols, int64_t out_ld) {
    int rc = check_shards(shards, n, false);
    if (rc != GB200_OK) return rc;
    for (int g = 0; g < n; ++g)
        GB200_REQUIRE(shards[g].rows >= 2, GB200_ERR_INVALID_ARG,
                      "shard %d: a band needs at least 2 rows (it lends them to the band before)", g);
    DeviceRestore restore;
    // Band g's last two output rows need the first two input rows of band g+1.
    for (int g = 0; g + 1 < n; ++g) {
        rc = enable_peer_loads(shards[g].ctx, shards[g + 1].ctx->device);
        if (rc != GB200_OK) return rc;
    }
    for (int g = 0; g < n; ++g) {
        const gb200_shard &s = shards[g];
        const float *halo = g + 1 < n ? static_cast<const float *>(shards[g + 1].in) : nullptr;
        rc = gb200_blur3x3_f32_band(s.ctx, static_cast<const float *>(s.in), in_ld, s.rows, in_cols,
                                    halo, in_ld, static_cast<float *>(s.out), out_ld, s.stream);
        if (rc != GB200_OK) return rc;
    }
    return GB200_OK;
}
