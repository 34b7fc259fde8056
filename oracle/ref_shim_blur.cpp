// C-callable doors onto cpu_blur_x / cpu_blur_y, the reference's CPU check of the blur program
// (apps/blur/blur.cpp:11-25).  The two functions are compiled from the reference's file itself
// (see the Makefile rule for blur_app.o); this file only declares them and wraps pointers in the
// app's own MatrixCPU view type (apps/common/impl/gpu-matrix-const.h).  Test infrastructure.
#include <cstdint>

#include "impl/gpu-matrix-const.h"

void cpu_blur_x(impl::MatrixCPU &input, impl::MatrixCPU &output);
void cpu_blur_y(impl::MatrixCPU &input, impl::MatrixCPU &output);

extern "C" {

void ref_blur_x(float *in, int64_t in_ld, float *out, int64_t out_ld, int64_t out_rows,
                int64_t out_cols) {
    impl::MatrixCPU i(in, out_rows, out_cols + 2, in_ld), o(out, out_rows, out_cols, out_ld);
    cpu_blur_x(i, o);
}
void ref_blur_y(float *in, int64_t in_ld, float *out, int64_t out_ld, int64_t out_rows,
                int64_t out_cols) {
    impl::MatrixCPU i(in, out_rows + 2, out_cols, in_ld), o(out, out_rows, out_cols, out_ld);
    cpu_blur_y(i, o);
}

}  // extern "C"
