// substitute.h -- pattern substitution on a Gern program: a Composable written against the
// reference's OWN annotations is rewritten onto the annotations of b200.h when its leaf calls form
// one of the fused pipelines libgern_b200 has a kernel for.  It is a pass over the reference's
// Composable tree (include/gern/compose/composable.h) with its own visitor interface
// (include/gern/compose/composable_visitor.h:14-22); the result goes to the unmodified Runner.
//
//   Global(Tile...(blur_x<3>(in, tmp), blur_y<3>(tmp, out)))        apps/blur/blur.cpp:66-73
//       -> b200::Blur3x3(in, out)
//   Global(Tile...(Reduce...(Stage...(matrix_multiply(A, B, C)))))  gernels/mm/kernel_10.cu:108-131,
//       and its CPU twin gern::impl::matrix_multiply                test/test-cpu-mm.cpp:13-83
//       -> b200::MatrixMultiply(A, B, C, k_dim)
//   max_shuffle ; subtract_vec ; exp_matrix ; sum_row ; divide_vec  apps/common/annot/functions.h:9-173
//       -> b200::RowSoftmax(in, out)
//
// The tile loops, grid bindings and staging of the original schedule are dropped: they describe
// how the reference's generic kernel walks the data, and the library's kernels bring their own
// (TMA tiles, tcgen05 MMAs, their own grid).  Temporaries between the fused stages disappear.
// The data types keep their names and become gb200_host matrices, so Runner::evaluate takes
// gb200_host::Matrix (device) or gb200_host::HostMatrix objects under the same names.
// A program that matches no pattern is returned unchanged (`matched` == false) and lowers to
// the reference's generic kernel as before.
#pragma once

#include <string>
#include <vector>

#include "b200.h"
#include "compose/composable.h"
#include "compose/composable_visitor.h"

namespace gern {
namespace b200 {

struct Substitution {
    Composable program;       // what to hand to Runner
    bool matched = false;
    std::string kernel;       // "blur3x3", "matrix_multiply", "softmax_rows" or ""
    std::vector<std::string> arguments;   // names Runner::evaluate expects (data types, then variables)
};

namespace detail {

// Leaf calls of a program in execution order, whatever Tile / Reduce / Stage / Global wraps them.
class LeafCollector : public ComposableVisitorStrict {
public:
    using ComposableVisitorStrict::visit;
    void visit(const Computation *n) override {
        for (const auto &c : n->composed) c.accept(this);
    }
    void visit(const TiledComputation *n) override { n->tiled.accept(this); }
    void visit(const GlobalNode *n) override { n->program.accept(this); }
    void visit(const StageNode *n) override { n->body.accept(this); }
    void visit(const ComputeFunctionCall *n) override { calls.push_back(n->getCall()); }
    std::vector<FunctionCall> calls;
};

inline bool is_adt(const Argument &a) { return isa<DSArg>(a.ptr); }
inline AbstractDataTypePtr adt_of(const Argument &a) { return to<DSArg>(a.ptr)->getADTPtr(); }

// First template argument as a bound integer (blur stride, matmul k_dim), or `otherwise`.
inline int64_t bound_template_arg(const FunctionCall &f, int64_t otherwise) {
    if (f.template_args.empty() || !isa<ExprArg>(f.template_args[0].ptr)) return otherwise;
    const Variable v = to<ExprArg>(f.template_args[0].ptr)->getVar();
    return v.isBound() ? v.getInt64Val() : otherwise;
}

inline bool all_adts(const FunctionCall &f, size_t n) {
    if (f.args.size() < n) return false;
    for (size_t i = 0; i < n; ++i)
        if (!is_adt(f.args[i])) return false;
    return true;
}

}  // namespace detail

// `device`: true -> gb200_host::Matrix (device memory), false -> gb200_host::HostMatrix.
inline Substitution substitute(Composable program, bool device = true) {
    Substitution out;
    out.program = program;
    detail::LeafCollector leaves;
    program.accept(&leaves);
    const auto &c = leaves.calls;
    auto mat = [&](const AbstractDataTypePtr &a) {
        return device ? annot::b200::device_f32(a.getName()) : annot::b200::host_f32(a.getName());
    };
    auto ends_with = [](const std::string &s, const std::string &suffix) {
        return s.size() >= suffix.size() && s.compare(s.size() - suffix.size(), suffix.size(), suffix) == 0;
    };

    if (c.size() == 2 && c[0].name == "blur_x" && c[1].name == "blur_y" && detail::all_adts(c[0], 2) &&
        detail::all_adts(c[1], 2) && detail::adt_of(c[1].args[0]) == detail::adt_of(c[0].args[1]) &&
        detail::bound_template_arg(c[0], 0) == 3 && detail::bound_template_arg(c[1], 0) == 3) {
        auto in = mat(detail::adt_of(c[0].args[0])), res = mat(detail::adt_of(c[1].args[1]));
        annot::b200::Blur3x3 blur(in, res);
        out.program = Composable(blur(in, res));
        out.kernel = "blur3x3";
        out.arguments = {in.getName(), res.getName()};
    } else if (c.size() == 1 && (c[0].name == "matrix_multiply" || ends_with(c[0].name, "::matrix_multiply")) &&
               detail::all_adts(c[0], 3)) {
        auto A = mat(detail::adt_of(c[0].args[0])), B = mat(detail::adt_of(c[0].args[1])),
             C = mat(detail::adt_of(c[0].args[2]));
        annot::b200::MatrixMultiply mm(A, B, C);
        Variable k_dim("k_dim", Datatype::Int64);
        out.program = Composable(mm(A, B, C, k_dim));
        out.kernel = "matrix_multiply";
        out.arguments = {A.getName(), B.getName(), C.getName(), "k_dim"};
    } else if (c.size() == 5 && c[0].name == "max_shuffle" && c[1].name == "subtract_vec" && c[2].name == "exp_matrix" &&
               c[3].name == "sum_row" && c[4].name == "divide_vec" && detail::all_adts(c[0], 2) &&
               detail::all_adts(c[1], 3) && detail::all_adts(c[2], 2) && detail::all_adts(c[3], 2) &&
               detail::all_adts(c[4], 3)) {
        // max(m <- x); subtract(m, x -> t1); exp(t1 -> t2); sum(s <- t2); divide(s, t2 -> y)
        const auto x = detail::adt_of(c[0].args[1]), m = detail::adt_of(c[0].args[0]);
        const auto t1 = detail::adt_of(c[1].args[2]), t2 = detail::adt_of(c[2].args[1]);
        const auto s = detail::adt_of(c[3].args[0]), y = detail::adt_of(c[4].args[2]);
        const bool flow = detail::adt_of(c[1].args[0]) == m && detail::adt_of(c[1].args[1]) == x &&
                          detail::adt_of(c[2].args[0]) == t1 && detail::adt_of(c[3].args[1]) == t2 &&
                          detail::adt_of(c[4].args[0]) == s && detail::adt_of(c[4].args[1]) == t2;
        if (flow) {
            auto in = mat(x), res = mat(y);
            annot::b200::RowSoftmax sm(in, res);
            out.program = Composable(sm(in, res));
            out.kernel = "softmax_rows";
            out.arguments = {in.getName(), res.getName()};
        }
    }
    out.matched = !out.kernel.empty();
    return out;
}

}  // namespace b200
}  // namespace gern
