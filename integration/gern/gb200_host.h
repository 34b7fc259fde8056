// gb200_host.h -- the run-time side of the Gern binding of libgern_b200.
//
// Gern's Runner emits a hook whose body names C++ types and functions by the strings an
// AbstractDataType / AbstractFunction returns (src/codegen/codegen.cpp:31-101, :557-561).  This
// header holds what those strings name for the annotations of b200.h: matrix objects with
// run-time extents (the reference's GPU ADTs bake them into the type,
// gernels/mm/gern_annot/adt.h:18-29; one prebuilt library needs them at run time) and thin
// functions that pass pointers and sizes to the C ABI of include/gern_b200.h.  It plays the part
// of test/library/matrix/impl/cpu-matrix.h / apps/common/impl/gpu-matrix-const.h in the reference.
//
// Two kinds of object: Matrix / MatrixBf16 hold DEVICE memory and go to the device entry points
// (no synchronisation, as in the reference's hooks); HostMatrix / HostMatrixBf16 hold host memory
// and go to the `_host` entry points, which return when the result is in host memory.
//
// A failing call throws gb200_host::Error (the reference's check_last_error() prints and calls
// exit(1), include/gern/codegen/helpers/check_last_error.h:7-18; an exception leaves the
// decision to the program that called Runner::evaluate).
#pragma once

#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include "gern_b200.h"

#ifndef GB200_HOST_NO_CUDART
#include <cuda_runtime_api.h>
#endif

namespace gb200_host {

struct Error : std::runtime_error {
    int status;
    Error(int status, const std::string &what) : std::runtime_error(what), status(status) {}
};

inline void check(int rc, const char *what) {
    if (rc != GB200_OK)
        throw Error(rc, std::string(what) + " failed with status " + std::to_string(rc) + ": " +
                            gb200_last_error_string());
}

// One context per hook library, created on first use on device $GERN_B200_DEVICE (default 0:
// the reference's hooks launch on device 0 only, src/codegen/codegen.cpp:576-611).
inline gb200_ctx *ctx() {
    static gb200_ctx *c = nullptr;
    if (!c) {
        const char *dev = std::getenv("GERN_B200_DEVICE");
        check(gb200_ctx_create(dev ? std::atoi(dev) : 0, &c), "gb200_ctx_create");
    }
    return c;
}

// A row-major matrix view: element (i, j) at data[i * lda + j].  query() is a pointer view into
// the parent (so nothing is copied back: insert() is a no-op and the annotations below say
// insertQuery() == false), allocate() makes a temporary that destroy() frees.
template <typename T, bool kDevice>
struct MatrixT {
    T *data = nullptr;
    int64_t row = 0, col = 0, lda = 0;

    MatrixT() = default;
    MatrixT(T *data, int64_t row, int64_t col, int64_t lda) : data(data), row(row), col(col), lda(lda) {}

    static MatrixT allocate(int64_t, int64_t, int64_t l_x, int64_t l_y) {
        MatrixT m(nullptr, l_x, l_y, (l_y + 7) / 8 * 8);      // rows stay 16-byte aligned for TMA
        const size_t bytes = sizeof(T) * (size_t)m.row * (size_t)m.lda;
        if (kDevice) {
#ifndef GB200_HOST_NO_CUDART
            if (cudaMalloc(reinterpret_cast<void **>(&m.data), bytes ? bytes : 16) != cudaSuccess)
                throw Error(GB200_ERR_CUDA, "cudaMalloc of a temporary failed");
#else
            throw Error(GB200_ERR_UNSUPPORTED, "device temporaries need the CUDA runtime");
#endif
        } else {
            m.data = static_cast<T *>(std::malloc(bytes ? bytes : 16));
        }
        return m;
    }
    void destroy() {
        if (kDevice) {
#ifndef GB200_HOST_NO_CUDART
            cudaFree(data);
#endif
        } else {
            std::free(data);
        }
        data = nullptr;
    }
    MatrixT query(int64_t x, int64_t y, int64_t l_x, int64_t l_y) { return MatrixT(data + x * lda + y, l_x, l_y, lda); }
    void insert(int64_t, int64_t, int64_t, int64_t, MatrixT) {}
};

using bf16_t = uint16_t;   // bf16 bit patterns; the library takes them as void*
using Matrix = MatrixT<float, true>;
using MatrixBf16 = MatrixT<bf16_t, true>;
using HostMatrix = MatrixT<float, false>;
using HostMatrixBf16 = MatrixT<bf16_t, false>;

// ---- fused blur: out is (in.row - 2) x (in.col - 2) ------------------------------------------
inline void blur3x3(Matrix &in, Matrix &out) {
    check(gb200_blur3x3_f32(ctx(), in.data, in.lda, out.row + 2, out.col + 2, out.data, out.lda, nullptr),
          "gb200_blur3x3_f32");
}
inline void blur3x3(HostMatrix &in, HostMatrix &out) {
    check(gb200_blur3x3_f32_host(ctx(), in.data, in.lda, out.row + 2, out.col + 2, out.data, out.lda),
          "gb200_blur3x3_f32_host");
}

// ---- matrix multiply: C += A B over k_dim, the reference leaf's contract ---------------------
// (gern::impl::matrix_multiply, test/library/matrix/impl/cpu-matrix.h:196-212: `c += sum`)
inline void matrix_multiply(Matrix &A, Matrix &B, Matrix &C, int64_t k_dim) {
    check(gb200_gemm_f32(ctx(), A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col, k_dim, 1, nullptr),
          "gb200_gemm_f32");
}
inline void matrix_multiply(HostMatrix &A, HostMatrix &B, HostMatrix &C, int64_t k_dim) {
    check(gb200_gemm_f32_host(ctx(), A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col, k_dim, 1),
          "gb200_gemm_f32_host");
}
// bf16: A row-major M x K, B stored as N rows of K (column-major B), C = A B (overwrites C, so the
// call takes the whole of K: a program may Tile rows and columns of C but not Reduce over k_dim).
inline void matrix_multiply_bf16(MatrixBf16 &A, MatrixBf16 &B, MatrixBf16 &C, int64_t k_dim) {
    check(gb200_gemm_bf16(ctx(), A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col, k_dim, nullptr),
          "gb200_gemm_bf16");
}
inline void matrix_multiply_bf16(HostMatrixBf16 &A, HostMatrixBf16 &B, HostMatrixBf16 &C, int64_t k_dim) {
    check(gb200_gemm_bf16_host(ctx(), A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col, k_dim),
          "gb200_gemm_bf16_host");
}

// ---- row softmax -------------------------------------------------------------------------------
inline void softmax_rows(Matrix &in, Matrix &out) {
    check(gb200_softmax_rows_f32(ctx(), in.data, in.lda, out.data, out.lda, out.row, out.col, nullptr),
          "gb200_softmax_rows_f32");
}
inline void softmax_rows(HostMatrix &in, HostMatrix &out) {
    check(gb200_softmax_rows_f32_host(ctx(), in.data, in.lda, out.data, out.lda, out.row, out.col),
          "gb200_softmax_rows_f32_host");
}

// ---- O = softmax_rows(scale * Q K^T) V ----------------------------------------------------------
inline void attention(MatrixBf16 &Q, MatrixBf16 &K, MatrixBf16 &V, MatrixBf16 &O, float scale) {
    check(gb200_attention_bf16(ctx(), Q.data, Q.lda, K.data, K.lda, V.data, V.lda, O.data, O.lda, O.row, K.row,
                               O.col, scale, nullptr),
          "gb200_attention_bf16");
}
inline void attention(HostMatrixBf16 &Q, HostMatrixBf16 &K, HostMatrixBf16 &V, HostMatrixBf16 &O, float scale) {
    check(gb200_attention_bf16_host(ctx(), Q.data, Q.lda, K.data, K.lda, V.data, V.lda, O.data, O.lda, O.row,
                                    K.row, O.col, scale),
          "gb200_attention_bf16_host");
}

// cudaDeviceSynchronize on the binding's device, for programs that read device results back.
inline void sync() { check(gb200_device_sync(ctx()), "gb200_device_sync"); }

}  // namespace gb200_host
