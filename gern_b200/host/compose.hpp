// Composition combinators shaped after Gern's (include/gern/compose/composable.h:18-174):
// Composable trees made of function calls, Tile / Reduce loops optionally bound to grid units,
// Stage and Global wrappers.  Tiling and grid binding are checked for legality the way the
// reference checks them (a grid unit may be bound once per nest, src/compose/composable.cpp:242-262;
// tile variables must name a field of the output), but they do not steer the B200 kernels: tile
// shapes for tcgen05 / TMA are chosen inside libgern_b200 from the run-time problem size.
#pragma once

#include <initializer_list>

#include "annotations.hpp"

namespace gern {
namespace b200 {

struct Node;
class Composable {
public:
    Composable() = default;
    explicit Composable(std::shared_ptr<const Node> n) : node(std::move(n)) {}
    Composable(std::initializer_list<Composable> composed);
    Composable(const std::vector<Composable> &composed);
    bool defined() const { return node != nullptr; }
    const Node *get() const { return node.get(); }

private:
    std::shared_ptr<const Node> node;
};

struct Node {
    enum Kind { Call, Computation, Tiled, Stage, Global } kind;
    // Call
    FunctionCall call;
    // Computation / bodies
    std::vector<Composable> children;
    // Tiled
    ADTMember member;          // field being tiled (Tile)
    Variable extent;           // reduction extent (Reduce)
    Variable tile;             // tile size variable
    Grid::Unit unit = Grid::UNDEFINED;
    bool reduce = false;
    // Stage
    AbstractDataTypePtr staged;
    // Global
    std::map<Grid::Dim, Variable> launch_args;
    Variable smem_size;
};

inline Composable::Composable(std::initializer_list<Composable> composed)
    : Composable(std::vector<Composable>(composed)) {}
inline Composable::Composable(const std::vector<Composable> &composed) {
    if (composed.size() == 1) {
        node = composed[0].node;
        return;
    }
    auto n = std::make_shared<Node>();
    n->kind = Node::Computation;
    n->children = composed;
    node = n;
}

inline Composable call(const FunctionCall &c) {
    auto n = std::make_shared<Node>();
    n->kind = Node::Call;
    n->call = c;
    return Composable(n);
}

// Tile(C["row"], ti) || Grid::BLOCK_X  applied to a body  (composable.h:118-150).
class TileDummy {
public:
    TileDummy(ADTMember m, Variable v, bool reduce) : member(std::move(m)), tile(std::move(v)), reduce(reduce) {}
    TileDummy(Variable extent, Variable v) : extent(std::move(extent)), tile(std::move(v)), reduce(true) {}
    TileDummy operator||(Grid::Unit u) const {
        TileDummy t = *this;
        t.unit = u;
        return t;
    }
    template <typename... Rest>
    Composable operator()(Composable first, Rest... rest) const {
        return (*this)(Composable(std::vector<Composable>{first, rest...}));
    }
    Composable operator()(Composable body) const {
        auto n = std::make_shared<Node>();
        n->kind = Node::Tiled;
        n->member = member;
        n->extent = extent;
        n->tile = tile;
        n->unit = unit;
        n->reduce = reduce;
        n->children = {body};
        return Composable(n);
    }

private:
    ADTMember member;
    Variable extent;
    Variable tile;
    Grid::Unit unit = Grid::UNDEFINED;
    bool reduce = false;
};

inline TileDummy Tile(ADTMember m, Variable v) { return TileDummy(std::move(m), std::move(v), false); }
inline TileDummy Reduce(ADTMember m, Variable v) { return TileDummy(std::move(m), std::move(v), true); }
inline TileDummy Reduce(Variable extent, Variable v) { return TileDummy(std::move(extent), std::move(v)); }

inline Composable Stage(AbstractDataTypePtr adt, Composable body) {
    auto n = std::make_shared<Node>();
    n->kind = Node::Stage;
    n->staged = std::move(adt);
    n->children = {body};
    return Composable(n);
}

// include/gern/compose/composable.h:49-52.  launch_args pins launch dimensions to bound variables
// and smem_size asks for dynamic shared memory; both are checked (Runner::compile) and recorded,
// but the kernels of libgern_b200 size their own grids, clusters and shared memory from the
// run-time problem, so they do not steer a launch.
inline Composable Global(Composable program, std::map<Grid::Dim, Variable> launch_args = {},
                         Variable smem_size = Variable()) {
    auto n = std::make_shared<Node>();
    n->kind = Node::Global;
    n->children = {program};
    n->launch_args = std::move(launch_args);
    n->smem_size = std::move(smem_size);
    return Composable(n);
}

// include/gern/annotations/abstract_function.h:22-64: operator[] binds template variables and
// operator() applies the function to ADTs (in the reference's argument order) and yields a
// Composable.  A concrete function states how many ADTs it takes and which one it produces.
class AbstractFunction {
public:
    virtual ~AbstractFunction() = default;
    virtual Op getOp() const = 0;
    virtual std::vector<std::string> templateArgs() const { return {}; }
    virtual size_t arity() const = 0;          // number of ADT arguments, output included
    virtual size_t outputIndex() const { return arity() - 1; }
    virtual float getScale() const { return 1.0f; }

    AbstractFunction &operator[](const std::map<std::string, Variable> &bindings) {
        for (const auto &kv : bindings) {
            bool known = false;
            for (const auto &t : templateArgs()) known = known || t == kv.first;
            if (!known)
                throw error::UserError(std::string(opName(getOp())) + " has no template argument " + kv.first);
            if (!kv.second.isBound())
                throw error::UserError("template argument " + kv.first + " must be bound to a value");
            bound[kv.first] = kv.second;
        }
        return *this;
    }

    template <typename... T>
    Composable operator()(T... adts) const {
        std::vector<AbstractDataTypePtr> args{adts...};
        if (args.size() != arity())
            throw error::UserError(std::string(opName(getOp())) + " takes " + std::to_string(arity()) + " arguments");
        FunctionCall c;
        c.op = getOp();
        c.output = args[outputIndex()];
        for (size_t i = 0; i < args.size(); ++i)
            if (i != outputIndex()) c.inputs.push_back(args[i]);
        c.template_args = bound;
        c.scale = getScale();
        return call(c);
    }

protected:
    std::map<std::string, Variable> bound;
};

// ---- the annotated library of the hot path ------------------------------------------------
namespace annot {

// gernels/mm/gern_annot/functions.h:7-60 (GPU) and test/library/matrix/annot/cpu-matrix.h:259-305:
// matrix_multiply(A, B, C): C{i,j,ti,tj} is produced from A{i,k,ti,tk} and B{k,j,tk,tj},
// reducible over k.  `scale` multiplies the product (used by the fused chain; 1 otherwise).
class MatrixMultiply : public AbstractFunction {
public:
    MatrixMultiply() = default;
    explicit MatrixMultiply(float scale) : scale(scale) {}
    Op getOp() const override { return Op::MatrixMultiply; }
    std::vector<std::string> templateArgs() const override { return {"k_dim"}; }
    size_t arity() const override { return 3; }
    float getScale() const override { return scale; }

private:
    float scale = 1.0f;
};

// apps/common/annot/functions.h:175-211 / 213-249: blur_x(in, out), blur_y(in, out); output
// {x,y,lx,ly} consumes input {x,y,lx,ly+stride-1} (X) or {x,y,lx+stride-1,ly} (Y).
class BlurX : public AbstractFunction {
public:
    Op getOp() const override { return Op::BlurX; }
    std::vector<std::string> templateArgs() const override { return {"stride"}; }
    size_t arity() const override { return 2; }
};
class BlurY : public AbstractFunction {
public:
    Op getOp() const override { return Op::BlurY; }
    std::vector<std::string> templateArgs() const override { return {"stride"}; }
    size_t arity() const override { return 2; }
};

// The five softmax pieces (apps/common/annot/functions.h:9-173; CPU twins
// test/library/matrix/annot/cpu-matrix.h:128-257), argument order as in the reference:
// max_row(in, vec), subtract_vec(vec, in, out), exp_matrix(in, out), sum_row(in, vec),
// divide_vec(vec, in, out).
class MaxRow : public AbstractFunction {
public:
    Op getOp() const override { return Op::MaxRow; }
    size_t arity() const override { return 2; }
};
class SubstractVec : public AbstractFunction {   // spelled as in the reference
public:
    Op getOp() const override { return Op::SubstractVec; }
    size_t arity() const override { return 3; }
};
class ExpMatrix : public AbstractFunction {
public:
    Op getOp() const override { return Op::ExpMatrix; }
    size_t arity() const override { return 2; }
};
class SumRow : public AbstractFunction {
public:
    Op getOp() const override { return Op::SumRow; }
    size_t arity() const override { return 2; }
};
class DivideVec : public AbstractFunction {
public:
    Op getOp() const override { return Op::DivideVec; }
    size_t arity() const override { return 3; }
};

}  // namespace annot
}  // namespace b200
}  // namespace gern
