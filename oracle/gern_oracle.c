/*
 * gern_oracle.c -- CPU restatement of the reference algorithms on the hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing that ships may call into this file: it exists so that the
 * tests, the smoke check and the bench's CPU-baseline leg can compare the CUDA library against
 * the reference's own arithmetic.  Each function names the reference code it restates
 * (paths are relative to the reference project's root).
 *
 * Pinning: oracle/ref_shim_matrix.cpp and oracle/ref_shim_blur.cpp compile the reference's own
 * CPU functions from its sources into oracle/_ref/, and tests/test_oracle_pin.py requires
 * bit-equality between every function here and its reference original (where the reference has
 * one), as well as the reference tests' known answers (10x10 ascending matmul,
 * test/test-cpu-mm.cpp:13-83; ascending blur, apps/blur/blur.cpp:83-108).  The softmax
 * composition, the bf16 GEMM and the attention chain have no runnable original in the reference
 * (its softmax test is commented out, test/test-cpu-matrix.cpp:69-148): parity for those is
 * "unpinned" and is anchored on an fp64 evaluation instead.
 *
 * Build: gcc -O2 -ffp-contract=off -pthread -shared -fPIC (see oracle/Makefile).  Contraction is
 * off so that a*b+c rounds twice, as the reference's default g++ build does
 * (src/codegen/runner.cpp:29-35 passes no -O and no -mfma).
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

static int g_threads = 1;

/* Minimal row-range fan-out over pthreads: body(arg, begin, end) on g_threads slices. */
typedef void (*range_fn)(void *arg, int64_t begin, int64_t end);
typedef struct {
    range_fn fn;
    void *arg;
    int64_t begin, end;
} range_job;
static void *range_thread(void *p) {
    range_job *j = (range_job *)p;
    j->fn(j->arg, j->begin, j->end);
    return NULL;
}
static void parallel_range(int64_t begin, int64_t end, range_fn fn, void *arg) {
    int nt = g_threads;
    int64_t n = end - begin;
    if (nt > n) nt = (int)(n > 0 ? n : 1);
    if (nt <= 1) {
        fn(arg, begin, end);
        return;
    }
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nt);
    range_job *jobs = (range_job *)malloc(sizeof(range_job) * (size_t)nt);
    int64_t per = (n + nt - 1) / nt;
    for (int t = 0; t < nt; t++) {
        jobs[t].fn = fn;
        jobs[t].arg = arg;
        jobs[t].begin = begin + t * per;
        jobs[t].end = jobs[t].begin + per < end ? jobs[t].begin + per : end;
        if (jobs[t].begin > end) jobs[t].begin = end;
        pthread_create(&th[t], NULL, range_thread, &jobs[t]);
    }
    for (int t = 0; t < nt; t++) pthread_join(th[t], NULL);
    free(th);
    free(jobs);
}

/* Number of host threads the row-parallel entry points use (1 = the reference's own
 * single-threaded behaviour: its emitter never produces a parallel loop,
 * src/codegen/codegen.cpp:336-344). */
void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int oracle_get_threads(void) { return g_threads; }
int oracle_max_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n < 1 ? 1 : (int)n;
}

/* ---- matrix multiply -------------------------------------------------------------------- */

/* gern::impl::matrix_multiply (test/library/matrix/impl/cpu-matrix.h:196-212):
 * for i, j: sum = 0; for k < k_dim: sum += a(i,k) * b(k,j); c(i,j) += sum.
 * a, b, c are views with leading dimensions lda, ldb, ldc; c is crow x ccol. */
void oracle_matrix_multiply(const float *a, int64_t lda, const float *b, int64_t ldb, float *c,
                            int64_t ldc, int64_t crow, int64_t ccol, int64_t k_dim) {
    for (int64_t i = 0; i < crow; i++) {
        float *c_data = c + i * ldc;
        const float *a_data = a + i * lda;
        for (int64_t j = 0; j < ccol; j++) {
            float sum = 0.0f;
            for (int64_t k = 0; k < k_dim; k++) sum += a_data[k] * b[k * ldb + j];
            c_data[j] += sum;
        }
    }
}

/* Gern's CPU code for Tile(C.row,ti)(Tile(C.col,tj)(Reduce(k_dim,tk)(matrix_multiply)))
 * (program: test/test-cpu-mm.cpp:13-83; the lowering emits nested for loops, a C.query view per
 * (i,j) tile, A.query / B.query views per k tile, the leaf call, then C.insert of the view onto
 * itself: src/codegen/concretize.cpp:67-146, test/library/matrix/impl/cpu-matrix.h:42-56).
 * Tile extents need not divide the matrix here; the last tile is clipped (the reference
 * requires divisibility). */
typedef struct {
    const float *A, *B;
    float *C;
    int64_t lda, ldb, ldc, M, N, K, ti, tj, tk;
} mm_args;
static void matmul_tiled_body(void *p, int64_t it_begin, int64_t it_end) {
    mm_args *a = (mm_args *)p;
    for (int64_t it = it_begin; it < it_end; it++) {
        int64_t i = it * a->ti;
        int64_t li = (i + a->ti <= a->M) ? a->ti : a->M - i;
        for (int64_t j = 0; j < a->N; j += a->tj) {
            int64_t lj = (j + a->tj <= a->N) ? a->tj : a->N - j;
            float *cq = a->C + i * a->ldc + j;
            for (int64_t k = 0; k < a->K; k += a->tk) {
                int64_t lk = (k + a->tk <= a->K) ? a->tk : a->K - k;
                oracle_matrix_multiply(a->A + i * a->lda + k, a->lda, a->B + k * a->ldb + j, a->ldb,
                                       cq, a->ldc, li, lj, lk);
            }
        }
    }
}
void oracle_matmul_tiled(const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                         int64_t ldc, int64_t M, int64_t N, int64_t K, int64_t ti, int64_t tj,
                         int64_t tk) {
    mm_args a = {A, B, C, lda, ldb, ldc, M, N, K, ti, tj, tk};
    parallel_range(0, (M + ti - 1) / ti, matmul_tiled_body, &a);
}

/* ---- blur ------------------------------------------------------------------------------- */

/* cpu_blur_x (apps/blur/blur.cpp:11-17): out(i,j) = (in(i,j) + in(i,j+1) + in(i,j+2)) / 3 */
typedef struct {
    const float *in;
    float *out;
    int64_t in_ld, out_ld, out_cols;
} blur_args;
static void blur_x_body(void *p, int64_t r0, int64_t r1) {
    blur_args *a = (blur_args *)p;
    const float *in = a->in;
    float *out = a->out;
    int64_t in_ld = a->in_ld, out_ld = a->out_ld;
    for (int64_t i = r0; i < r1; i++)
        for (int64_t j = 0; j < a->out_cols; j++)
            out[i * out_ld + j] =
                (in[i * in_ld + j] + in[i * in_ld + j + 1] + in[i * in_ld + j + 2]) / 3;
}
void oracle_blur_x(const float *in, int64_t in_ld, float *out, int64_t out_ld, int64_t out_rows,
                   int64_t out_cols) {
    blur_args a = {in, out, in_ld, out_ld, out_cols};
    parallel_range(0, out_rows, blur_x_body, &a);
}

/* cpu_blur_y (apps/blur/blur.cpp:19-25): out(i,j) = (in(i,j) + in(i+1,j) + in(i+2,j)) / 3 */
static void blur_y_body(void *p, int64_t r0, int64_t r1) {
    blur_args *a = (blur_args *)p;
    const float *in = a->in;
    float *out = a->out;
    int64_t in_ld = a->in_ld, out_ld = a->out_ld;
    for (int64_t i = r0; i < r1; i++)
        for (int64_t j = 0; j < a->out_cols; j++)
            out[i * out_ld + j] =
                (in[i * in_ld + j] + in[(i + 1) * in_ld + j] + in[(i + 2) * in_ld + j]) / 3;
}
void oracle_blur_y(const float *in, int64_t in_ld, float *out, int64_t out_ld, int64_t out_rows,
                   int64_t out_cols) {
    blur_args a = {in, out, in_ld, out_ld, out_cols};
    parallel_range(0, out_rows, blur_y_body, &a);
}

/* The two-stage program as the reference checks it (apps/blur/blur.cpp:97-101): blur_x into a
 * (rows, cols-2) temporary, blur_y into the (rows-2, cols-2) result.  Returns 0, or -1 if the
 * temporary cannot be allocated. */
int oracle_blur_xy(const float *in, int64_t in_ld, int64_t in_rows, int64_t in_cols, float *out,
                   int64_t out_ld) {
    if (in_rows <= 2 || in_cols <= 2) return 0;
    int64_t tc = in_cols - 2;
    float *tmp = (float *)malloc(sizeof(float) * (size_t)in_rows * (size_t)tc);
    if (!tmp) return -1;
    oracle_blur_x(in, in_ld, tmp, tc, in_rows, tc);
    oracle_blur_y(tmp, tc, out, out_ld, in_rows - 2, tc);
    free(tmp);
    return 0;
}

/* ---- softmax pieces, exactly as the reference writes them -------------------------------- */

/* max_row (cpu-matrix.h:158-168): maximum seeded with numeric_limits<float>::min(). */
void oracle_max_row_ref(const float *a, int64_t lda, int64_t rows, int64_t cols, float *b) {
    for (int64_t i = 0; i < rows; i++) {
        float maximum = FLT_MIN;
        for (int64_t j = 0; j < cols; j++) maximum = maximum < a[i * lda + j] ? a[i * lda + j] : maximum;
        b[i] = maximum;
    }
}
/* sum_row (cpu-matrix.h:146-156) */
void oracle_sum_row(const float *a, int64_t lda, int64_t rows, int64_t cols, float *b) {
    for (int64_t i = 0; i < rows; i++) {
        float sum = 0.0f;
        for (int64_t j = 0; j < cols; j++) sum += a[i * lda + j];
        b[i] = sum;
    }
}
/* exp_matrix (cpu-matrix.h:134-144) */
void oracle_exp_matrix(const float *a, int64_t lda, int64_t rows, int64_t cols, float *b,
                       int64_t ldb) {
    for (int64_t i = 0; i < rows; i++)
        for (int64_t j = 0; j < cols; j++) b[i * ldb + j] = expf(a[i * lda + j]);
}
/* subtract_vec (cpu-matrix.h:170-181): out = vec - a, as the reference writes it. */
void oracle_subtract_vec_ref(const float *vec, const float *a, int64_t lda, int64_t rows,
                             int64_t cols, float *out, int64_t ldo) {
    for (int64_t i = 0; i < rows; i++)
        for (int64_t j = 0; j < cols; j++) out[i * ldo + j] = vec[i] - a[i * lda + j];
}
/* divide_vec (cpu-matrix.h:183-194): out = a / vec */
void oracle_divide_vec(const float *vec, const float *a, int64_t lda, int64_t rows, int64_t cols,
                       float *out, int64_t ldo) {
    for (int64_t i = 0; i < rows; i++)
        for (int64_t j = 0; j < cols; j++) out[i * ldo + j] = a[i * lda + j] / vec[i];
}

/* Row softmax in the op order of the reference's pieces (max -> subtract -> expf -> sum ->
 * divide; cpu-matrix.h:134-194; the intended composition is the commented-out program at
 * test/test-cpu-matrix.cpp:69-148), with the two defects of the pieces corrected: the
 * subtraction is a - max (the reference computes max - a) and the maximum is seeded from the
 * row's first element (the reference seeds with FLT_MIN, which is wrong for all-negative rows). */
typedef struct {
    const float *in;
    void *out;
    int64_t ld_in, ld_out, cols;
} sm_args;
static void softmax_body(void *p, int64_t r0, int64_t r1) {
    sm_args *g = (sm_args *)p;
    int64_t cols = g->cols;
    for (int64_t i = r0; i < r1; i++) {
        const float *a = g->in + i * g->ld_in;
        float *o = (float *)g->out + i * g->ld_out;
        float maximum = a[0];
        for (int64_t j = 1; j < cols; j++) maximum = maximum < a[j] ? a[j] : maximum;
        for (int64_t j = 0; j < cols; j++) o[j] = a[j] - maximum;
        for (int64_t j = 0; j < cols; j++) o[j] = expf(o[j]);
        float sum = 0.0f;
        for (int64_t j = 0; j < cols; j++) sum += o[j];
        for (int64_t j = 0; j < cols; j++) o[j] = o[j] / sum;
    }
}
void oracle_softmax_rows(const float *in, int64_t ld_in, float *out, int64_t ld_out, int64_t rows,
                         int64_t cols) {
    sm_args g = {in, out, ld_in, ld_out, cols};
    parallel_range(0, rows, softmax_body, &g);
}

/* fp64 softmax, the anchor for the unpinned fp32 composition above. */
static void softmax64_body(void *p, int64_t r0, int64_t r1) {
    sm_args *g = (sm_args *)p;
    int64_t cols = g->cols;
    for (int64_t i = r0; i < r1; i++) {
        const float *a = g->in + i * g->ld_in;
        double *o = (double *)g->out + i * g->ld_out;
        double maximum = a[0];
        for (int64_t j = 1; j < cols; j++) maximum = maximum < a[j] ? a[j] : maximum;
        double sum = 0.0;
        for (int64_t j = 0; j < cols; j++) {
            o[j] = exp((double)a[j] - maximum);
            sum += o[j];
        }
        for (int64_t j = 0; j < cols; j++) o[j] /= sum;
    }
}
void oracle_softmax_rows_f64(const float *in, int64_t ld_in, double *out, int64_t ld_out,
                             int64_t rows, int64_t cols) {
    sm_args g = {in, out, ld_in, ld_out, cols};
    parallel_range(0, rows, softmax64_body, &g);
}

/* ---- bf16 GEMM and the GEMM -> softmax -> GEMM chain (no reference original) ------------- */

static inline float bf16_to_f32(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* C(i,j) = sum_k A(i,k) * B(k,j) on bf16 inputs, fp32 accumulate in ascending k (the leaf
 * semantics of cpu-matrix.h:196-212), fp32 result.  A row-major M x K; B column-major, i.e. N
 * rows of K contiguous values.  Only rows [row_begin, row_end) of C are computed; C holds
 * (row_end - row_begin) rows. */
typedef struct {
    const uint16_t *A, *B;
    float *C;
    int64_t lda, ldb, ldc, N, K, row_begin;
} gb_args;
static void gemm_bf16_body(void *p, int64_t r0, int64_t r1) {
    gb_args *g = (gb_args *)p;
    int64_t K = g->K, N = g->N;
    float *arow = (float *)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
    float *brow = (float *)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
    for (int64_t i = r0; i < r1; i++) {
        for (int64_t k = 0; k < K; k++) arow[k] = bf16_to_f32(g->A[i * g->lda + k]);
        for (int64_t j = 0; j < N; j++) {
            const uint16_t *b = g->B + j * g->ldb;
            for (int64_t k = 0; k < K; k++) brow[k] = bf16_to_f32(b[k]);
            float sum = 0.0f;
            for (int64_t k = 0; k < K; k++) sum += arow[k] * brow[k];
            g->C[(i - g->row_begin) * g->ldc + j] = sum;
        }
    }
    free(arow);
    free(brow);
}
void oracle_gemm_bf16(const uint16_t *A, int64_t lda, const uint16_t *B, int64_t ldb, float *C,
                      int64_t ldc, int64_t N, int64_t K, int64_t row_begin, int64_t row_end) {
    gb_args g = {A, B, C, lda, ldb, ldc, N, K, row_begin};
    parallel_range(row_begin, row_end, gemm_bf16_body, &g);
}

/* O = softmax_rows(scale * Q K^T) V on bf16 inputs: S in fp32 (ascending-k accumulate), the
 * softmax of oracle_softmax_rows, P V accumulated in fp32 in ascending kv, fp32 result.
 * Rows [row_begin, row_end) of Q only. */
typedef struct {
    const uint16_t *Q, *K, *V;
    float *O;
    int64_t ldq, ldk, ldv, ldo, nkv, d, row_begin;
    float scale;
} att_args;
static void attention_body(void *p, int64_t r0, int64_t r1) {
    att_args *g = (att_args *)p;
    int64_t nkv = g->nkv, d = g->d;
    float *s = (float *)malloc(sizeof(float) * (size_t)(nkv > 0 ? nkv : 1));
    float *q = (float *)malloc(sizeof(float) * (size_t)(d > 0 ? d : 1));
    for (int64_t i = r0; i < r1; i++) {
        for (int64_t k = 0; k < d; k++) q[k] = bf16_to_f32(g->Q[i * g->ldq + k]);
        for (int64_t j = 0; j < nkv; j++) {
            float sum = 0.0f;
            for (int64_t k = 0; k < d; k++) sum += q[k] * bf16_to_f32(g->K[j * g->ldk + k]);
            s[j] = sum * g->scale;
        }
        float maximum = s[0];
        for (int64_t j = 1; j < nkv; j++) maximum = maximum < s[j] ? s[j] : maximum;
        float den = 0.0f;
        for (int64_t j = 0; j < nkv; j++) {
            s[j] = expf(s[j] - maximum);
            den += s[j];
        }
        float *o = g->O + (i - g->row_begin) * g->ldo;
        for (int64_t k = 0; k < d; k++) o[k] = 0.0f;
        for (int64_t j = 0; j < nkv; j++) {
            float pj = s[j] / den;
            for (int64_t k = 0; k < d; k++) o[k] += pj * bf16_to_f32(g->V[j * g->ldv + k]);
        }
    }
    free(s);
    free(q);
}
void oracle_attention_bf16(const uint16_t *Q, int64_t ldq, const uint16_t *Kmat, int64_t ldk,
                           const uint16_t *V, int64_t ldv, float *O, int64_t ldo, int64_t nkv,
                           int64_t d, float scale, int64_t row_begin, int64_t row_end) {
    att_args g = {Q, Kmat, V, O, ldq, ldk, ldv, ldo, nkv, d, row_begin, scale};
    parallel_range(row_begin, row_end, attention_body, &g);
}
