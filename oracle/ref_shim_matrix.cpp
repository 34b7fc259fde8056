// C-callable doors onto the reference's own CPU matrix functions, compiled from the reference's
// header where it lies (test/library/matrix/impl/cpu-matrix.h).  Test infrastructure: used to pin
// oracle/gern_oracle.c and, optionally, as the timed CPU baseline.  No reference source is
// copied; this file only wraps pointers into the reference's MatrixCPU / ArrayCPU views.
#include <cstdint>

#include "library/matrix/impl/cpu-matrix.h"

using gern::impl::ArrayCPU;
using gern::impl::MatrixCPU;

extern "C" {

// gern::impl::matrix_multiply(a, b, c, k_dim): c(crow x ccol) += a * b   (cpu-matrix.h:196-212)
void ref_matrix_multiply(float *a, int64_t lda, float *b, int64_t ldb, float *c, int64_t ldc,
                         int64_t crow, int64_t ccol, int64_t k_dim) {
    gern::impl::matrix_multiply(MatrixCPU(a, crow, k_dim, lda), MatrixCPU(b, k_dim, ccol, ldb),
                                MatrixCPU(c, crow, ccol, ldc), k_dim);
}

// The loop nest Gern emits for Tile(row,ti)(Tile(col,tj)(Reduce(k_dim,tk)(matrix_multiply)))
// (test/test-cpu-mm.cpp:13-83), driven through the reference's own query / insert / leaf.
void ref_matmul_tiled(float *A, int64_t lda, float *B, int64_t ldb, float *C, int64_t ldc,
                      int64_t M, int64_t N, int64_t K, int64_t ti, int64_t tj, int64_t tk) {
    MatrixCPU a(A, M, K, lda), b(B, K, N, ldb), c(C, M, N, ldc);
    for (int64_t i = 0; i < M; i += ti)
        for (int64_t j = 0; j < N; j += tj) {
            MatrixCPU cq = c.query(i, j, ti, tj);
            for (int64_t k = 0; k < K; k += tk)
                gern::impl::matrix_multiply(a.query(i, k, ti, tk), b.query(k, j, tk, tj), cq, tk);
            c.insert(i, j, ti, tj, cq);
        }
}

void ref_max_row(float *a, int64_t lda, int64_t rows, int64_t cols, float *out) {
    gern::impl::max_row(MatrixCPU(a, rows, cols, lda), ArrayCPU(out, rows));
}
void ref_sum_row(float *a, int64_t lda, int64_t rows, int64_t cols, float *out) {
    gern::impl::sum_row(MatrixCPU(a, rows, cols, lda), ArrayCPU(out, rows));
}
void ref_exp_matrix(float *a, int64_t lda, int64_t rows, int64_t cols, float *b, int64_t ldb) {
    gern::impl::exp_matrix(MatrixCPU(a, rows, cols, lda), MatrixCPU(b, rows, cols, ldb));
}
void ref_subtract_vec(float *vec, float *a, int64_t lda, int64_t rows, int64_t cols, float *out,
                      int64_t ldo) {
    gern::impl::subtract_vec(ArrayCPU(vec, rows), MatrixCPU(a, rows, cols, lda),
                             MatrixCPU(out, rows, cols, ldo));
}
void ref_divide_vec(float *vec, float *a, int64_t lda, int64_t rows, int64_t cols, float *out,
                    int64_t ldo) {
    gern::impl::divide_vec(ArrayCPU(vec, rows), MatrixCPU(a, rows, cols, lda),
                           MatrixCPU(out, rows, cols, ldo));
}
// MatrixCPU::random_fill (cpu-matrix.h:71-81): mt19937(0) + uniform_real_distribution<float>.
void ref_random_fill(float *a, int64_t lda, int64_t rows, int64_t cols, float lo, float hi) {
    MatrixCPU(a, rows, cols, lda).random_fill(lo, hi);
}
void ref_ascending(float *a, int64_t lda, int64_t rows, int64_t cols) {
    MatrixCPU(a, rows, cols, lda).ascending();
}

}  // extern "C"
