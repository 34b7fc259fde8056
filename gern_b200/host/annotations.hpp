// Operator surface of the B200 path, shaped after Gern's: variables, grid units, abstract data
// types and annotated functions.  Names and argument meaning follow the reference
// (include/gern/annotations/{expr.h,grid.h,abstract_function.h}, gernels/mm/gern_annot/,
// apps/common/annot/); the data-dependence annotations themselves are not re-implemented: each
// annotated function here records which operator it is and which ADTs it reads and writes, which
// is what the pipeline lowering in runner.hpp needs.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace gern {
namespace b200 {

namespace error {
// Same two error kinds as the reference (include/gern/utils/error.h:21-33).
struct UserError : std::runtime_error {
    explicit UserError(const std::string &m) : std::runtime_error(m) {}
};
struct InternalError : std::runtime_error {
    explicit InternalError(const std::string &m) : std::runtime_error(m) {}
};
}  // namespace error

// include/gern/annotations/grid.h:9-29
namespace Grid {
enum Unit {
    UNDEFINED,
    SCALAR_UNIT,
    THREAD_X, THREAD_Y, THREAD_Z,
    THREAD_X_IN_WRAPS, THREAD_Y_IN_WRAPS, THREAD_Z_IN_WRAPS,
    WARP_X, WARP_Y, WARP_Z,
    BLOCK_X, BLOCK_Y, BLOCK_Z,
    BLOCK_CLUSTER_X, BLOCK_CLUSTER_Y, BLOCK_CLUSTER_Z,   // Blackwell thread-block clusters
};
inline const char *name(Unit u) {
    static const char *n[] = {"UNDEFINED", "SCALAR_UNIT", "THREAD_X", "THREAD_Y", "THREAD_Z",
                              "THREAD_X_IN_WRAPS", "THREAD_Y_IN_WRAPS", "THREAD_Z_IN_WRAPS",
                              "WARP_X", "WARP_Y", "WARP_Z", "BLOCK_X", "BLOCK_Y", "BLOCK_Z",
                              "BLOCK_CLUSTER_X", "BLOCK_CLUSTER_Y", "BLOCK_CLUSTER_Z"};
    return n[u];
}
// Launch dimensions a Global() may pin (include/gern/annotations/grid.h:31-45), with the cluster
// dimensions the reference reserves a level for but never emits (grid.h:47-56).
enum Dim {
    GRID_DIM_X, GRID_DIM_Y, GRID_DIM_Z,
    BLOCK_DIM_X, BLOCK_DIM_Y, BLOCK_DIM_Z,
    WARP_DIM_X, WARP_DIM_Y, WARP_DIM_Z,
    CLUSTER_DIM_X, CLUSTER_DIM_Y, CLUSTER_DIM_Z,
    NULL_DIM,
};
enum Level { NULL_LEVEL = 0, SCALAR = 1, THREADS = 2, THREADS_WARPS = 3, WARPS = 4, BLOCK = 5, BLOCK_CLUSTER = 6, GRID = 7 };
// src/annotations/grid.cpp:134-158, extended by the cluster units.
inline Level getLevel(Unit u) {
    switch (u) {
        case THREAD_X: case THREAD_Y: case THREAD_Z: return THREADS;
        case THREAD_X_IN_WRAPS: case THREAD_Y_IN_WRAPS: case THREAD_Z_IN_WRAPS: return THREADS_WARPS;
        case WARP_X: case WARP_Y: case WARP_Z: return WARPS;
        case BLOCK_X: case BLOCK_Y: case BLOCK_Z: return BLOCK;
        case BLOCK_CLUSTER_X: case BLOCK_CLUSTER_Y: case BLOCK_CLUSTER_Z: return BLOCK_CLUSTER;
        case SCALAR_UNIT: return SCALAR;
        default: return NULL_LEVEL;
    }
}
// The launch dimension a unit is counted in (src/annotations/grid.cpp:198-230): threads in the
// block dimensions, warps too, blocks in the grid dimensions, clusters in the cluster dimensions.
inline Dim getDim(Unit u) {
    switch (u) {
        case THREAD_X: case WARP_X: return BLOCK_DIM_X;
        case THREAD_Y: case WARP_Y: return BLOCK_DIM_Y;
        case THREAD_Z: case WARP_Z: return BLOCK_DIM_Z;
        case THREAD_X_IN_WRAPS: return WARP_DIM_X;
        case THREAD_Y_IN_WRAPS: return WARP_DIM_Y;
        case THREAD_Z_IN_WRAPS: return WARP_DIM_Z;
        case BLOCK_X: return GRID_DIM_X;
        case BLOCK_Y: return GRID_DIM_Y;
        case BLOCK_Z: return GRID_DIM_Z;
        case BLOCK_CLUSTER_X: return CLUSTER_DIM_X;
        case BLOCK_CLUSTER_Y: return CLUSTER_DIM_Y;
        case BLOCK_CLUSTER_Z: return CLUSTER_DIM_Z;
        default: return NULL_DIM;
    }
}
inline const char *levelName(Level l) {
    static const char *n[] = {"NULL_LEVEL", "SCALAR", "THREADS", "THREADS_WARPS", "WARPS", "BLOCK", "BLOCK_CLUSTER", "GRID"};
    return n[l];
}
}  // namespace Grid

// A named int64 variable; bind() fixes its value at program-construction time, as
// Variable::bind does in the reference (include/gern/annotations/expr.h:135-165).  Copies share
// the binding.
class Variable {
public:
    Variable() : Variable("") {}
    explicit Variable(const std::string &name) : state(std::make_shared<State>()) { state->name = name; }
    Variable bind(int64_t v) const {
        Variable b(state->name);
        b.state->value = v;
        return b;
    }
    const std::string &getName() const { return state->name; }
    bool isBound() const { return state->value.has_value(); }
    int64_t getInt64Val() const {
        if (!isBound()) throw error::UserError("variable " + state->name + " is not bound");
        return *state->value;
    }
    bool defined() const { return !state->name.empty(); }

private:
    struct State {
        std::string name;
        std::optional<int64_t> value;
    };
    std::shared_ptr<State> state;
};

enum class Datatype { Float32, BFloat16 };
enum class Layout { RowMajor, ColMajor };

class AbstractDataType;
struct ADTMember;

// Owning handle, used as in the reference: AbstractDataTypePtr(new const annot::MatrixGPU("A")),
// A_DS["row"], A_DS.getName()  (include/gern/annotations/expr.h:208-238).
class AbstractDataTypePtr {
public:
    AbstractDataTypePtr() = default;
    explicit AbstractDataTypePtr(const AbstractDataType *p) : ptr(p) {}
    ADTMember operator[](const std::string &field) const;
    const AbstractDataType *operator->() const { return ptr.get(); }
    const AbstractDataType *get() const { return ptr.get(); }
    bool defined() const { return ptr != nullptr; }
    std::string getName() const;
    bool operator==(const AbstractDataTypePtr &o) const { return ptr == o.ptr; }

private:
    std::shared_ptr<const AbstractDataType> ptr;
};

// ADTMember(C, "row") in the reference; produced by adt["row"].
struct ADTMember {
    AbstractDataTypePtr adt;
    std::string field;
};

// include/gern/annotations/expr.h:167-206, reduced to what the B200 path needs: a name, the
// element type and layout, and whether the object is a temporary of the fused pipeline (the
// reference marks those with a `true` constructor flag and type "auto", apps/blur/blur.cpp:48).
class AbstractDataType {
public:
    AbstractDataType(std::string name, Datatype dtype = Datatype::Float32,
                     Layout layout = Layout::RowMajor, bool temporary = false)
        : name(std::move(name)), dtype(dtype), layout(layout), temporary(temporary) {}
    virtual ~AbstractDataType() = default;
    const std::string &getName() const { return name; }
    Datatype getDatatype() const { return dtype; }
    Layout getLayout() const { return layout; }
    bool isTemporary() const { return temporary; }
    virtual std::vector<std::string> getFields() const { return {"x", "y", "row", "col"}; }

private:
    std::string name;
    Datatype dtype;
    Layout layout;
    bool temporary;
};

inline std::string AbstractDataTypePtr::getName() const { return ptr ? ptr->getName() : std::string(); }
inline ADTMember AbstractDataTypePtr::operator[](const std::string &field) const {
    if (!ptr) throw error::UserError("field access on an undefined data type");
    bool ok = false;
    for (const auto &f : ptr->getFields()) ok = ok || f == field;
    if (!ok) throw error::UserError("data type " + ptr->getName() + " has no field " + field);
    return ADTMember{*this, field};
}

namespace annot {
// Matrix on the GPU: fp32 row-major unless stated (gernels/mm/gern_annot/adt.h:9-93,
// apps/common/annot/adt.h:9-148).  Sizes are run-time fields of the impl object, not template
// constants, so one compiled library serves every shape.
class MatrixGPU : public AbstractDataType {
public:
    using AbstractDataType::AbstractDataType;
};
// Row vector temporaries of the softmax pieces (apps/common/annot/adt.h StaticArray).
class ArrayGPU : public AbstractDataType {
public:
    explicit ArrayGPU(std::string name, bool temporary = true)
        : AbstractDataType(std::move(name), Datatype::Float32, Layout::RowMajor, temporary) {}
    std::vector<std::string> getFields() const override { return {"x", "size"}; }
};
}  // namespace annot


// Which leaf an annotated function is.  The reference identifies leaves by the C++ name in
// FunctionSignature (include/gern/compose/compose.h:68-85); the names are kept in opName().
enum class Op { MatrixMultiply, BlurX, BlurY, MaxRow, SubstractVec, ExpMatrix, SumRow, DivideVec };

inline const char *opName(Op op) {
    switch (op) {
        case Op::MatrixMultiply: return "matrix_multiply";
        case Op::BlurX: return "blur_x";
        case Op::BlurY: return "blur_y";
        case Op::MaxRow: return "max_shuffle";
        case Op::SubstractVec: return "subtract_vec";
        case Op::ExpMatrix: return "exp_matrix";
        case Op::SumRow: return "sum_row";
        case Op::DivideVec: return "divide_vec";
    }
    return "?";
}

// One call of an annotated function on concrete ADTs (ComputeFunctionCall in the reference).
struct FunctionCall {
    Op op;
    std::vector<AbstractDataTypePtr> inputs;
    AbstractDataTypePtr output;
    std::map<std::string, Variable> template_args;   // e.g. stride of blur, k_dim of matmul
    float scale = 1.0f;                               // MatrixMultiply only: C = scale * A B
};

}  // namespace b200
}  // namespace gern
