/*
 * gern_b200.h -- C ABI of libgern_b200.so: hand-written sm_100a (B200) kernels for the
 * fused data-parallel programs that Gern's lowering emits (tiled matrix multiply, row
 * softmax, the two-stage blur, and the GEMM -> softmax -> GEMM chain).
 *
 * The library stands where Gern's generic emitted `__global__ function_N` stands today:
 * the host function that `Runner::compile` builds (src/codegen/codegen.cpp:31-101 emits the
 * `extern "C" hook_<fn>(void**)`, src/codegen/runner.cpp:17-52 compiles and dlopens it)
 * calls one of the entry points below instead of launching an emitted kernel
 * (src/codegen/codegen.cpp:576-611).  Every entry point takes plain pointers and sizes,
 * never owns a caller's buffer, never calls exit(), and returns an int status.
 *
 * Conventions
 *   - All matrices are dense with an explicit leading dimension `ld*` counted in elements.
 *   - "row-major M x K, ld" means element (i,k) lives at ptr[i*ld + k].
 *   - Device entry points take device pointers valid on the context's device and enqueue
 *     work on `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream,
 *     which is what Gern's emitted hook uses).  They do not synchronise.
 *   - `_host` entry points take host pointers (pinned memory is fastest), copy the operands
 *     to the device, run the same kernels, copy the result back and return after the result
 *     is in host memory.
 *   - A context owns one scratch workspace (split-K slabs of the bf16 GEMM, split copies of the
 *     fp32 matmul's operands, partial results of the GEMM -> softmax -> GEMM chain) and one set
 *     of staging buffers: calls on the same context whose
 *     kernels could overlap on the GPU (different streams) must use different contexts, as
 *     Gern's single-stream hooks never overlap (src/codegen/codegen.cpp:576-611).
 *   - Status: 0 = success; negative = failure (see gb200_status).  A human-readable message
 *     for the calling thread's last failure is returned by gb200_last_error_string().
 *   - The calling thread's current CUDA device is the same after a call as before it.
 *   - A kernel whose bounded device-side wait ran out (a protocol error; the result is invalid) is
 *     reported as GB200_ERR_TIMEOUT by the `_host` entry point itself, and for the device entry
 *     points by the next gb200_device_sync().
 */
#ifndef GERN_B200_H
#define GERN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gb200_ctx gb200_ctx;

enum gb200_status {
    GB200_OK = 0,
    GB200_ERR_INVALID_ARG = -1,  /* null pointer, negative size, ld smaller than the row, ... */
    GB200_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed                        */
    GB200_ERR_UNSUPPORTED = -3,  /* shape or alignment this build has no kernel for            */
    GB200_ERR_NO_DEVICE = -4,    /* no sm_100 device, or the driver is missing                 */
    GB200_ERR_TIMEOUT = -5,      /* a bounded device-side wait ran out (kernel reported it)    */
    GB200_ERR_TOO_LARGE = -6     /* request exceeds a fixed capacity of the entry point        */
};

/* ---- context -------------------------------------------------------------------------- */

/* Creates a context bound to CUDA device `device`.  The context owns only library scratch:
 * cached TMA descriptors, the staging buffers of the `_host` entry points and a small status
 * word.  Replaces the per-launch `cudaGetDeviceProperties` of Gern's hook
 * (include/gern/codegen/helpers/assert_device_properties.h:15-42): device limits are read
 * once here. */
int gb200_ctx_create(int device, gb200_ctx **out);
int gb200_ctx_destroy(gb200_ctx *ctx);
/* cudaDeviceSynchronize on the context's device (Gern's callers synchronise implicitly
 * through cudaMemcpy in MatrixGPU::get(), apps/common/impl/gpu-matrix-const.h:221-225). */
int gb200_device_sync(gb200_ctx *ctx);
const char *gb200_last_error_string(void);
const char *gb200_version(void);
/* Number of kernels this library has launched on behalf of `ctx` since it was created. */
int64_t gb200_launch_count(gb200_ctx *ctx);

/* What one of the library's TMA / tcgen05 kernels allocates per thread block: the figures Gern's
 * Allocates(reg, smem) statement carries (include/gern/annotations/stmt.h:113-121; the reference's
 * lowering never reads it, and its kernels carve shared memory at run time with a bump allocator,
 * gernels/mm/impl/sh_malloc.h:12-54).  Here every kernel's shared memory is a layout planned at
 * compile time (1024-byte aligned swizzled tiles, mbarriers, TMEM slot) and this call reports it.
 * Kernel names: "gemm_bf16_tc", "gemm_bf16_2cta", "attention_bf16", "attention_bf16_pair".
 * Works without a device, except that regs_per_thread is then -1. */
typedef struct gb200_kernel_resources {
    int regs_per_thread;     /* as compiled; -1 when no device is present to ask          */
    int threads;             /* threads per block                                          */
    int dynamic_smem_bytes;  /* dynamic shared memory per block                            */
    int cluster_x;           /* thread blocks per cluster (1 = no cluster, 2 = CTA pair)   */
    int tmem_columns;        /* tensor-memory columns the block allocates                  */
} gb200_kernel_resources;
int gb200_kernel_resources_query(const char *kernel, gb200_kernel_resources *out);

/* ---- matrix multiply ------------------------------------------------------------------ */

/* fp32 C (+)= A * B, all row-major.  A: M x K (lda), B: K x N (ldb), C: M x N (ldc).
 * accumulate != 0 adds into C (Gern's leaf does `c += sum`), 0 overwrites C.  Problems above
 * 0.2 GFLOP run on the tensor cores with every fp32 operand split into three bf16 terms (fp32
 * accuracy is kept): up to 3 GFLOP in one launch that splits in shared memory, beyond that with
 * split pre-passes (the library's workspace holds the split copies); smaller ones on CUDA cores.
 * Replaces the emitted kernel of gernels/mm/kernel_10.cu:108-131 (copy:
 * gernels/mm/bench.cu:10-44) and its leaf `matrix_multiply<k_dim>`
 * (gernels/mm/impl/matrix_multiply.h:50-61); CPU twin gern::impl::matrix_multiply
 * (test/library/matrix/impl/cpu-matrix.h:196-212). */
int gb200_gemm_f32(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                   float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate,
                   void *stream);

/* bf16 inputs, fp32 accumulate (tcgen05 / TMEM), bf16 output.  A: row-major M x K (lda).
 * B: column-major K x N, i.e. stored as N rows of K contiguous elements (ldb >= K).
 * C: row-major M x N (ldc).  Same annotation as annot::MatrixMultiply
 * (gernels/mm/gern_annot/functions.h:7-60); the reference has no bf16 leaf. */
int gb200_gemm_bf16(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                    void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, void *stream);

/* The same GEMM with the thread-block cluster shape chosen by the caller: cluster_x = 1 runs
 * one CTA per 128 x 256 tile (gemm_bf16_tc kernel), cluster_x = 2 runs CTA pairs on 256 x 256 tiles
 * with tcgen05 cta_group::2 (gemm_bf16_2cta kernel); anything else is GB200_ERR_UNSUPPORTED.  It is
 * what a program's pinned cluster dimension steers: the reference reserves the level
 * (Grid::Level::BLOCK_CLUSTER, include/gern/annotations/grid.h:47-56) but its launch emitter has
 * no cluster dimension (src/codegen/codegen.cpp:576-611). */
int gb200_gemm_bf16_cluster(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                            void *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int cluster_x,
                            void *stream);

/* bf16 GEMM whose consumers run in the epilogue, while the fp32 accumulator is still in TMEM /
 * registers: the reference's elementwise and row-reduction leaves
 * (test/library/matrix/impl/cpu-matrix.h:134-194; annotations test/library/matrix/annot/cpu-matrix.h:128-257)
 * composed after annot::MatrixMultiply, generalising the GEMM -> softmax -> GEMM chain.  Per
 * element (i,j) of the product, in this order:
 *     t = alpha * (A B)(i,j);  t -= row_sub[i];  if (apply_exp) t = exp(t);  t /= row_div[i];
 * then C(i,j) = bf16(t), row_max[i] = max_j t, row_sum[i] = sum_j t (from t before rounding).
 * NULL vectors switch their step off; C may be NULL when only the reductions are wanted (the
 * product is then a temporary that never reaches memory).  row_sub / row_div / row_max / row_sum
 * are device vectors of M floats; the output vectors are initialised by the library.  Operand
 * conventions as gb200_gemm_bf16; A and B must have 16-byte aligned rows.  subtract is `t - v`, as
 * in the reference's GPU leaf (apps/common/impl/impl.h:53-78) and in the softmax it serves; the
 * reference's CPU leaf computes `v - t` (cpu-matrix.h:170-181). */
typedef struct gb200_gemm_epilogue {
    float alpha;
    const float *row_sub;
    int apply_exp;
    const float *row_div;
    float *row_max;
    float *row_sum;
} gb200_gemm_epilogue;
int gb200_gemm_bf16_epilogue(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                             void *C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                             const gb200_gemm_epilogue *epilogue, void *stream);

/* Split-K bf16 GEMM that allocates nothing and needs no context (same operand conventions as
 * gb200_gemm_bf16; `splits` = 1..16, or 0 to let the library choose).  It has no counterpart in
 * the reference.  It is for callers that cannot call cudaMalloc where they need the product: a
 * serving loop that must not take the device-wide synchronisation an allocation implies, a
 * process whose device memory already belongs entirely to another allocator, or a callback in
 * which allocation calls are not permitted.  The fp32 partial-sum workspace is a fixed array of
 * 4 Mi floats (16 MiB) inside the library, resident on every GPU that loads it until the process
 * exits; a request with splits * M * N beyond that returns GB200_ERR_TOO_LARGE.  The first call
 * on each device looks up the array's device address and sets kernel attributes: make that call
 * once, with the device current, before any stream capture begins.  All calls share the one
 * array: two calls whose kernels may overlap on the GPU (different streams) race on it; calls
 * on one stream are safe, and nothing a previous call left in the array is ever read.  Runs on
 * the calling thread's current device, and A, B and C must be device memory of that device
 * (anything else is refused with GB200_ERR_INVALID_ARG); does not synchronise.  A kernel whose
 * bounded wait ran out leaves a wrong C and records the fact in a status word that
 * gb200_static_status() reads. */
int gb200_gemm_bf16_splitk_static(const void *A, int64_t lda, const void *B, int64_t ldb, void *C,
                                  int64_t ldc, int64_t M, int64_t N, int64_t K, int splits,
                                  void *stream);
/* Status word of gb200_gemm_bf16_splitk_static on the current device: synchronises the device,
 * returns GB200_OK when no kernel gave up a wait since the last query, else GB200_ERR_TIMEOUT with
 * the kernel's code in *code (may be NULL), and clears the word.  Allocates nothing.  No
 * counterpart in the reference. */
int gb200_static_status(int *code);

/* ---- row softmax ---------------------------------------------------------------------- */

/* out(i,:) = exp(in(i,:) - max_j in(i,j)) / sum_j exp(in(i,j) - max_j in(i,j)), fp32.
 * One fused pass replacing the five annotated ops MaxRow / SubstractVec / ExpMatrix /
 * SumRow / DivideVec (apps/common/annot/functions.h:9-173; device code
 * apps/common/impl/impl.h:7-188; CPU twins test/library/matrix/impl/cpu-matrix.h:134-194). */
int gb200_softmax_rows_f32(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                           int64_t ld_out, int64_t rows, int64_t cols, void *stream);

/* ---- fused two-stage blur ------------------------------------------------------------- */

/* t(i,j) = (in(i,j)+in(i,j+1)+in(i,j+2))/3 ; out(i,j) = (t(i,j)+t(i+1,j)+t(i+2,j))/3 with
 * out of size (in_rows-2) x (in_cols-2); t never reaches HBM.  Bit-exact with the reference's
 * cpu_blur_x / cpu_blur_y (apps/blur/blur.cpp:11-25).  Replaces the emitted kernel
 * apps/blur/blur.cu:19-45 and the leaves blur_x<3>/blur_y<3>
 * (apps/common/impl/impl.h:190-250; annotations apps/common/annot/functions.h:175-249). */
int gb200_blur3x3_f32(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                      int64_t in_cols, float *out, int64_t out_ld, void *stream);

/* Row-band form used when an image is sharded by rows across GPUs: `in` holds `band_rows`
 * rows of the band this GPU owns and `halo` holds the 2 rows that follow it (they belong to
 * the next band; `halo` may point into a peer GPU's memory, it is read with ordinary loads).
 * Produces band_rows output rows.  With halo == NULL it produces band_rows-2 rows (last band).
 * When `halo` is memory of another device (and the image is 16-byte aligned and the band holds at
 * least 48 MiB), the two rows are not read by the kernel: a copy engine fetches them on a stream of the context into a local slot
 * as soon as the call is made, and the block row that needs them waits for the slot's flag.  The
 * neighbour's two rows must therefore be complete when the call is made, not merely earlier in
 * `stream`'s order, and such a call cannot be captured into a CUDA graph.
 * No counterpart in the reference, which is single-GPU. */
int gb200_blur3x3_f32_band(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t band_rows,
                           int64_t in_cols, const float *halo, int64_t halo_ld, float *out,
                           int64_t out_ld, void *stream);

/* ---- GEMM -> row softmax -> GEMM chain ------------------------------------------------- */

/* O = softmax_rows(scale * Q K^T) V with bf16 Q (nq x d), K (nkv x d), V (nkv x d), O (nq x d),
 * all row-major; S and P stay in TMEM / shared memory.  d must be 128 in this build.  The
 * nearest reference analogue is the chained-GEMM fusion with a per-tile temporary
 * (test/test-cpu-mm.cpp:266-408).  `scale` must be positive and finite (the row maximum is taken
 * before scaling); anything else is refused with GB200_ERR_INVALID_ARG.  Work is dealt out in
 * pairs of 128-row Q tiles.  When nq is too small to give every SM a pair, the K/V range is cut
 * across thread blocks and a second kernel merges the partial results.  When whole pairs would
 * leave SMs idle in their last round (157 pairs on 148 SMs), the (pair, K/V block) units are dealt
 * out in equal runs instead, and a pair shared by several thread blocks is merged inside the
 * kernel by the one that finishes last; the last bit of such a row can then depend on which
 * block merged.  Partial results live in the context's workspace either way. */
int gb200_attention_bf16(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                         const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                         int64_t nkv, int64_t d, float scale, void *stream);

/* The same chain with the thread-block cluster shape chosen by the caller: cluster_x = 1 runs one CTA
 * per two 128-row Q tiles, cluster_x = 2 runs CTA pairs that share every MMA (tcgen05 cta_group::2:
 * each CTA holds half of every K and V block); anything else is GB200_ERR_UNSUPPORTED.  Results are
 * identical bit for bit.  See gb200_gemm_bf16_cluster for what this stands for in the reference. */
int gb200_attention_bf16_cluster(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K, int64_t ldk,
                                 const void *V, int64_t ldv, void *O, int64_t ldo, int64_t nq,
                                 int64_t nkv, int64_t d, float scale, int cluster_x, void *stream);

/* ---- single-process multi-GPU forms ---------------------------------------------------- */

/* One device's part of a row-sharded call.  The reference launches on device 0 only
 * (src/codegen/codegen.cpp:576-611 emits no device selection) and has nothing like it. */
typedef struct gb200_shard {
    gb200_ctx *ctx;      /* context of the device that holds this shard's memory              */
    const void *in;      /* this shard's rows of the sharded input (A panel, softmax rows,    */
                         /* Q rows, image band)                                               */
    void *out;           /* this shard's rows of the result                                   */
    int64_t rows;        /* rows in this shard (0 = the device sits this call out)            */
    const void *shared0; /* this device's replica of the unsharded operand: B, or K           */
    const void *shared1; /* second replicated operand: V (attention only)                     */
    void *stream;        /* cudaStream_t on ctx's device; NULL = legacy default stream        */
} gb200_shard;

/* Each call enqueues shard g on shards[g].ctx's device and stream and returns without
 * synchronising; the calling thread's current device is restored.  Operand conventions are those
 * of the single-device entry point of the same name.  GEMM shards the M rows of A and C (B
 * replicated per device), softmax shards rows, attention shards the rows of Q and O (K, V
 * replicated): no data crosses devices.  The fp32 matmul has no sharded form (replicas only). */
int gb200_gemm_bf16_sharded(const gb200_shard *shards, int n, int64_t lda, int64_t ldb,
                            int64_t ldc, int64_t N, int64_t K);
int gb200_softmax_rows_f32_sharded(const gb200_shard *shards, int n, int64_t ld_in,
                                   int64_t ld_out, int64_t cols);
int gb200_attention_bf16_sharded(const gb200_shard *shards, int n, int64_t ldq, int64_t ldk,
                                 int64_t ldv, int64_t ldo, int64_t nkv, int64_t d, float scale);
/* Blur over an image cut into n consecutive row bands: shards[g].in holds shards[g].rows input
 * rows (>= 2) and shards[g].out receives as many output rows, except the last band, which
 * receives rows - 2.  Band g's kernel reads the first two rows of band g+1 directly from the
 * memory of the device that holds it (peer access is enabled on first use; ordinary loads over
 * NVLink, no copy, no extra launch).  Band g's kernel runs on shards[g].stream and reads band
 * g+1's first two input rows without any ordering against the stream that produced them: every
 * band's input must be complete (its producer synchronised, or an event of it waited on by
 * shards[g].stream) before this call. */
int gb200_blur3x3_f32_sharded(const gb200_shard *shards, int n, int64_t in_ld, int64_t in_cols,
                              int64_t out_ld);

/* ---- host-buffer forms (operands and results in host memory) -------------------------- */

int gb200_gemm_f32_host(gb200_ctx *ctx, const float *A, int64_t lda, const float *B, int64_t ldb,
                        float *C, int64_t ldc, int64_t M, int64_t N, int64_t K, int accumulate);
int gb200_gemm_bf16_host(gb200_ctx *ctx, const void *A, int64_t lda, const void *B, int64_t ldb,
                         void *C, int64_t ldc, int64_t M, int64_t N, int64_t K);
int gb200_softmax_rows_f32_host(gb200_ctx *ctx, const float *in, int64_t ld_in, float *out,
                                int64_t ld_out, int64_t rows, int64_t cols);
int gb200_blur3x3_f32_host(gb200_ctx *ctx, const float *in, int64_t in_ld, int64_t in_rows,
                           int64_t in_cols, float *out, int64_t out_ld);
int gb200_attention_bf16_host(gb200_ctx *ctx, const void *Q, int64_t ldq, const void *K,
                              int64_t ldk, const void *V, int64_t ldv, void *O, int64_t ldo,
                              int64_t nq, int64_t nkv, int64_t d, float scale);

#ifdef __cplusplus
}
#endif
#endif /* GERN_B200_H */
