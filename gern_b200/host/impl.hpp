// Run-time objects handed to Runner::evaluate, shaped after the reference's impl::MatrixGPU /
// impl::MatrixCPU (apps/common/impl/gpu-matrix-const.h:48-249, gernels/mm/impl/matrix-gpu.h:95-508):
// a device (or host) pointer with row / col / lda, owned by the caller, with the helpers the
// reference's apps use (vvals, ascending, get, destroy).  Sizes are run-time fields here.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "annotations.hpp"

namespace gern {
namespace b200 {
namespace impl {

inline void cudaCheck(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw error::UserError(std::string(what) + ": " + cudaGetErrorString(e));
}

class MatrixCPU {
public:
    MatrixCPU(float *data, int64_t row, int64_t col, int64_t lda) : data(data), row(row), col(col), lda(lda) {}
    MatrixCPU(int64_t row, int64_t col, int64_t lda)
        : MatrixCPU(static_cast<float *>(std::malloc(sizeof(float) * row * lda)), row, col, lda) {}
    float &operator()(int64_t x, int64_t y) { return data[x * lda + y]; }
    float operator()(int64_t x, int64_t y) const { return data[x * lda + y]; }
    void vvals(float f) {
        for (int64_t i = 0; i < row; i++)
            for (int64_t j = 0; j < col; j++) data[i * lda + j] = f;
    }
    void ascending() {
        for (int64_t i = 0; i < row; i++)
            for (int64_t j = 0; j < col; j++) data[i * lda + j] = static_cast<float>(i * col + j);
    }
    void destroy() { std::free(data); data = nullptr; }
    float *data;
    int64_t row, col, lda;
};

// fp32 or bf16 matrix in device memory.  `elem_bytes` is 4 (Float32) or 2 (BFloat16).
class MatrixGPU {
public:
    MatrixGPU(int64_t row, int64_t col, int64_t lda, Datatype dtype = Datatype::Float32)
        : row(row), col(col), lda(lda), dtype(dtype) {
        cudaCheck(cudaMalloc(&data, bytes()), "cudaMalloc");
    }
    MatrixGPU(int64_t row, int64_t col) : MatrixGPU(row, col, col) {}
    int elem_bytes() const { return dtype == Datatype::Float32 ? 4 : 2; }
    size_t bytes() const { return static_cast<size_t>(row) * lda * elem_bytes(); }
    void vvals(float f) {
        MatrixCPU h(row, col, lda);
        h.vvals(f);
        put(h);
        h.destroy();
    }
    void ascending() {
        MatrixCPU h(row, col, lda);
        h.ascending();
        put(h);
        h.destroy();
    }
    // host fp32 -> device (fp32 only), and back (the reference's get(), which also synchronises)
    void put(const MatrixCPU &h) {
        if (dtype != Datatype::Float32) throw error::UserError("put(MatrixCPU) needs a Float32 matrix");
        cudaCheck(cudaMemcpy2D(data, lda * 4, h.data, h.lda * 4, col * 4, row, cudaMemcpyHostToDevice), "cudaMemcpy2D");
    }
    MatrixCPU get() const {
        if (dtype != Datatype::Float32) throw error::UserError("get() needs a Float32 matrix");
        MatrixCPU h(row, col, col);
        cudaCheck(cudaMemcpy2D(h.data, col * 4, data, lda * 4, col * 4, row, cudaMemcpyDeviceToHost), "cudaMemcpy2D");
        return h;
    }
    void put_raw(const void *src) { cudaCheck(cudaMemcpy(data, src, bytes(), cudaMemcpyHostToDevice), "cudaMemcpy"); }
    void get_raw(void *dst) const { cudaCheck(cudaMemcpy(dst, data, bytes(), cudaMemcpyDeviceToHost), "cudaMemcpy"); }
    void destroy() {
        if (data) cudaFree(data);
        data = nullptr;
    }
    void *data = nullptr;
    int64_t row, col, lda;
    Datatype dtype;
};

// fp32 vector in device memory: the row vectors of the softmax pieces (max, sum, and the operands
// of subtract_vec / divide_vec), the reference's impl::ArrayGPU / StaticArray.
class ArrayGPU {
public:
    explicit ArrayGPU(int64_t size) : size(size) {
        cudaCheck(cudaMalloc(reinterpret_cast<void **>(&data), sizeof(float) * (size > 0 ? size : 1)), "cudaMalloc");
    }
    void put(const std::vector<float> &h) {
        if (static_cast<int64_t>(h.size()) != size) throw error::UserError("ArrayGPU::put: size mismatch");
        cudaCheck(cudaMemcpy(data, h.data(), sizeof(float) * size, cudaMemcpyHostToDevice), "cudaMemcpy");
    }
    std::vector<float> get() const {
        std::vector<float> h(size);
        cudaCheck(cudaMemcpy(h.data(), data, sizeof(float) * size, cudaMemcpyDeviceToHost), "cudaMemcpy");
        return h;
    }
    void destroy() {
        if (data) cudaFree(data);
        data = nullptr;
    }
    float *data = nullptr;
    int64_t size;
};

}  // namespace impl
}  // namespace b200
}  // namespace gern
