// b200.h -- Gern-side binding of libgern_b200: abstract data types and annotated functions that a
// Gern program composes (Tile / Reduce / Global) and hands to the unmodified Runner.  Plain Gern
// user code, the counterpart of gernels/mm/gern_annot/{adt,functions}.h,
// apps/common/annot/{adt,functions}.h and test/library/matrix/annot/cpu-matrix.h in the Gern tree:
// each AbstractFunction below has FunctionSignature.access == HOST (the default,
// include/gern/compose/compose.h:68-85), so Gern's code generator emits a plain host call
// (src/codegen/codegen.cpp:563-620 wraps only GLOBAL calls in <<<>>>) to a function of
// gb200_host.h, which forwards pointers and sizes to the C ABI of gern_b200.h.  The library
// launches its own sm_100a kernels; nothing in Gern's lowering changes.
//
// Build a program against it with Runner::Options (include/gern/compose/runner.h:19-26):
//   include = "-I <dir of this file> -I <repo>/include -I <cuda>/include"
//   ldflags = "-L <repo>/gern_b200 -lgern_b200 -Wl,-rpath,<repo>/gern_b200 -L <cuda>/lib64 -lcudart"
//   cpp_std = "c++17"
#pragma once

#include <string>
#include <vector>

#include "annotations/abstract_function.h"
#include "annotations/data_dependency_language.h"

namespace gern {
namespace annot {
namespace b200 {

// Matrix with run-time extents.  `type` is the C++ type the emitted hook casts args[i] to:
// gb200_host::Matrix (device fp32), MatrixBf16, HostMatrix, HostMatrixBf16.
class Matrix : public AbstractDataType {
public:
    Matrix(const std::string &name, const std::string &type = "gb200_host::Matrix")
        : name(name), type(type) {
    }
    std::string getName() const override { return name; }
    std::string getType() const override { return type; }
    std::vector<Variable> getFields() const override { return {x, y, l_x, l_y}; }
    FunctionSignature getAllocateFunction() const override {
        return FunctionSignature{.name = type + "::allocate", .args = {x, y, l_x, l_y}};
    }
    FunctionSignature getFreeFunction() const override {
        return FunctionSignature{.name = "destroy", .args = {}};
    }
    FunctionSignature getInsertFunction() const override {
        return FunctionSignature{.name = "insert", .args = {x, y, l_x, l_y}};
    }
    FunctionSignature getQueryFunction() const override {
        return FunctionSignature{.name = "query", .args = {x, y, l_x, l_y}};
    }
    // query() returns a pointer view into the parent: nothing to free, nothing to copy back.
    bool freeQuery() const override { return false; }
    bool insertQuery() const override { return false; }

private:
    std::string name, type;
    Variable x{"x"}, y{"y"}, l_x{"l_x"}, l_y{"l_y"};
};

inline AbstractDataTypePtr device_f32(const std::string &name) { return AbstractDataTypePtr(new const Matrix(name, "gb200_host::Matrix")); }
inline AbstractDataTypePtr device_bf16(const std::string &name) { return AbstractDataTypePtr(new const Matrix(name, "gb200_host::MatrixBf16")); }
inline AbstractDataTypePtr host_f32(const std::string &name) { return AbstractDataTypePtr(new const Matrix(name, "gb200_host::HostMatrix")); }
inline AbstractDataTypePtr host_bf16(const std::string &name) { return AbstractDataTypePtr(new const Matrix(name, "gb200_host::HostMatrixBf16")); }

inline std::vector<std::string> headers() { return {"gern_b200.h", "gb200_host.h"}; }

// The fused BlurX -> BlurY pair with stride 3 (annot::BlurX / annot::BlurY,
// apps/common/annot/functions.h:175-249, composed as in apps/blur/blur.cpp:66-73): an output
// tile {x, y, l_x, l_y} consumes the input tile {x, y, l_x + 2, l_y + 2}.
class Blur3x3 : public AbstractFunction {
public:
    Blur3x3(AbstractDataTypePtr input, AbstractDataTypePtr output)
        : input(input), output(output) {
    }
    Annotation getAnnotation() override {
        Variable x("x"), y("y"), l_x("l_x"), l_y("l_y");
        return annotate(Tileable(x = Expr(0), ADTMember(output, "row", false), l_x,
                                 Tileable(y = Expr(0), ADTMember(output, "col", false), l_y,
                                          Produces::Subset(output, {x, y, l_x, l_y}),
                                          Consumes::Subset(input, {x, y, l_x + 2, l_y + 2}))));
    }
    FunctionSignature getFunction() override {
        FunctionSignature f;
        f.name = "gb200_host::blur3x3";
        f.args = {Parameter(input), Parameter(output)};
        return f;
    }
    std::vector<std::string> getHeader() override { return headers(); }

private:
    AbstractDataTypePtr input, output;
};

// C += A B with the annotation of annot::MatrixMultiply (gernels/mm/gern_annot/functions.h:7-60;
// CPU twin test/library/matrix/annot/cpu-matrix.h:259-305): tileable over the rows and columns of
// C, reducible over k.  `bf16` selects gb200_host::matrix_multiply_bf16 (C = A B over the whole
// of K; B stored column-major), which must not sit under a Reduce.
class MatrixMultiply : public AbstractFunction {
public:
    MatrixMultiply(AbstractDataTypePtr A, AbstractDataTypePtr B, AbstractDataTypePtr C, bool bf16 = false)
        : A(A), B(B), C(C), bf16(bf16) {
    }
    Annotation getAnnotation() override {
        Variable i("i"), j("j"), k("k");
        Variable ti("ti", Datatype::Int64), tj("tj", Datatype::Int64), tk("tk", Datatype::Int64);
        return annotate(Tileable(i = Expr(0), ADTMember(C, "row", false), ti,
                                 Tileable(j = Expr(0), ADTMember(C, "col", false), tj,
                                          Produces::Subset(C, {i, j, ti, tj}),
                                          Consumes::Subsets(
                                              Reducible(k = Expr(0), k_dim, tk,
                                                        SubsetObjMany({
                                                            SubsetObj(A, {i, k, ti, tk}),
                                                            bf16 ? SubsetObj(B, {j, k, tj, tk}) : SubsetObj(B, {k, j, tk, tj}),
                                                        }))))));
    }
    FunctionSignature getFunction() override {
        FunctionSignature f;
        f.name = bf16 ? "gb200_host::matrix_multiply_bf16" : "gb200_host::matrix_multiply";
        f.args = {Parameter(A), Parameter(B), Parameter(C), k_dim};
        return f;
    }
    std::vector<std::string> getHeader() override { return headers(); }

private:
    AbstractDataTypePtr A, B, C;
    bool bf16;
    Variable k_dim{"k_dim", Datatype::Int64};
};

// The five row-softmax pieces MaxRow / SubstractVec / ExpMatrix / SumRow / DivideVec
// (apps/common/annot/functions.h:9-173) fused.  The pattern has the two tile loops of every
// matrix function here, but a softmax needs its rows whole: the annotation assumes
// l_y == output.col, which Gern turns into an assert in the emitted code, so a program may Tile
// the rows and must leave the columns alone.
class RowSoftmax : public AbstractFunction {
public:
    RowSoftmax(AbstractDataTypePtr input, AbstractDataTypePtr output)
        : input(input), output(output) {
    }
    Annotation getAnnotation() override {
        Variable x("x"), y("y"), l_x("l_x"), l_y("l_y");
        return annotate(Tileable(x = Expr(0), ADTMember(output, "row", false), l_x,
                                 Tileable(y = Expr(0), ADTMember(output, "col", false), l_y,
                                          Produces::Subset(output, {x, y, l_x, l_y}),
                                          Consumes::Subset(input, {x, y, l_x, l_y}))))
            .assumes({Constraint(l_y == ADTMember(output, "col", false))});
    }
    FunctionSignature getFunction() override {
        FunctionSignature f;
        f.name = "gb200_host::softmax_rows";
        f.args = {Parameter(input), Parameter(output)};
        return f;
    }
    std::vector<std::string> getHeader() override { return headers(); }

private:
    AbstractDataTypePtr input, output;
};

// O = softmax_rows(scale * Q K^T) V: the chained matrix multiply with a per-tile temporary
// (test/test-cpu-mm.cpp:266-408) with the softmax pieces between the two products, as one call.
// A tile of O consumes the same rows of Q and all of K and V; the head dimension stays whole
// (assumed, and asserted in the emitted code), so a program may Tile the rows of O only.
class Attention : public AbstractFunction {
public:
    Attention(AbstractDataTypePtr Q, AbstractDataTypePtr K, AbstractDataTypePtr V, AbstractDataTypePtr O)
        : Q(Q), K(K), V(V), O(O) {
    }
    Annotation getAnnotation() override {
        Variable x("x"), y("y"), l_x("l_x"), l_y("l_y");
        return annotate(Tileable(x = Expr(0), ADTMember(O, "row", false), l_x,
                                 Tileable(y = Expr(0), ADTMember(O, "col", false), l_y,
                                          Produces::Subset(O, {x, y, l_x, l_y}),
                                          Consumes::Subsets(SubsetObjMany({
                                              SubsetObj(Q, {x, y, l_x, l_y}),
                                              SubsetObj(K, {Expr(0), y, ADTMember(K, "row", false), l_y}),
                                              SubsetObj(V, {Expr(0), y, ADTMember(V, "row", false), l_y}),
                                          })))))
            .assumes({Constraint(l_y == ADTMember(O, "col", false))});
    }
    FunctionSignature getFunction() override {
        FunctionSignature f;
        f.name = "gb200_host::attention";
        f.args = {Parameter(Q), Parameter(K), Parameter(V), Parameter(O), scale};
        return f;
    }
    std::vector<std::string> getHeader() override { return headers(); }

private:
    AbstractDataTypePtr Q, K, V, O;
    Variable scale{"scale", Datatype::Float32};
};

}  // namespace b200
}  // namespace annot
}  // namespace gern
