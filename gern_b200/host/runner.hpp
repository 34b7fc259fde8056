// Runner: compile + evaluate for the B200 path, shaped after the reference's
// (include/gern/compose/runner.h:14-46, src/codegen/runner.cpp:11-80).
//
// The reference's compile() lowers the Composable to C++/CUDA text, shells out to nvcc, dlopens
// the result and keeps the hook; evaluate() checks the argument names and calls the hook.  Here
// compile() lowers the Composable to one of the fused sm_100a kernels of libgern_b200: it strips
// the Tile / Reduce / Stage / Global structure (checking it for legality), takes the sequence of
// leaf calls and their data flow, and recognises
//     matrix_multiply                                   -> gb200_gemm_f32 / gb200_gemm_bf16
//     blur_x ; blur_y through a temporary                -> gb200_blur3x3_f32
//     max ; subtract ; exp ; sum ; divide on one matrix  -> gb200_softmax_rows_f32
//     matrix_multiply ; the softmax chain ; matrix_multiply through temporaries
//                                                        -> gb200_attention_bf16
//     matrix_multiply ; [subtract_vec] ; [exp_matrix] ; [divide_vec] ; [max_row] ; [sum_row] on
//     its product (bf16 operands)                        -> gb200_gemm_bf16_epilogue
// Anything else is a UserError: there is no generic code generator and no fallback behind this
// Runner.  evaluate() performs the reference's argument checks (every ADT of the program must be
// supplied by name, nothing else may be) and makes one C-ABI call.
#pragma once

#include <algorithm>
#include <map>
#include <set>
#include <sstream>

#include "compose.hpp"
#include "gern_b200.h"
#include "impl.hpp"

namespace gern {
namespace b200 {

class Runner {
public:
    explicit Runner(Composable c) : c(std::move(c)) {}
    // Same fields as the reference's Options (runner.h:19-26).  Only `arch` matters here: if set
    // it must be "100a", the one architecture the library holds code for.
    struct Options {
        std::string filename;
        std::string prefix = "/tmp";
        std::string cpp_std = "c++17";
        std::string include = "";
        std::string ldflags = "";
        std::string arch = "";
    };

    enum class Kernel { None, GemmF32, GemmBF16, Blur, Softmax, Attention, GemmEpilogue };

    void compile() { compile(Options{}); }
    void compile(Options config) {
        if (!config.arch.empty() && config.arch != "100a")
            throw error::UserError("libgern_b200 holds sm_100a code only (arch=" + config.arch + ")");
        calls.clear();
        launch_args.clear();
        smem_request = -1;
        std::set<int> units;
        bool in_global = false;
        flatten(c, units, in_global);
        if (calls.empty()) throw error::UserError("empty program");
        lower();
        bindLaunch();
        compiled = true;
    }

    // What the planned kernel allocates per thread block (registers, threads, dynamic shared memory,
    // cluster size, TMEM columns): the library's answer to Gern's Allocates(reg, smem)
    // (include/gern/annotations/stmt.h:113-121).  Defined for the TMA / tcgen05 kernels.
    bool hasResources() const { return !kernel_name.empty(); }
    const gb200_kernel_resources &resources() const { return kernel_resources; }
    const std::string &kernelName() const { return kernel_name; }
    // Thread blocks per cluster the program pinned with Global({{CLUSTER_DIM_X, v}}), 0 = not pinned.
    int clusterX() const { return cluster_x; }

    Kernel kernel() const { return plan; }
    std::vector<std::string> argumentOrder() const { return argument_order; }

    // Launch dimensions pinned by Global(), by dimension.  CLUSTER_DIM_X selects the kernel (see
    // bindLaunch); grid and block dimensions are checked and recorded: the library's kernels size
    // their own persistent grids.
    const std::map<Grid::Dim, int64_t> &launchArgs() const { return launch_args; }

    void evaluate(std::map<std::string, void *> args) { evaluate(std::move(args), nullptr); }
    // `stream`: the CUDA stream the kernels are enqueued on (the reference's hook has none and
    // launches on the legacy default stream, src/codegen/codegen.cpp:576-611; nullptr does the same).
    void evaluate(std::map<std::string, void *> args, cudaStream_t stream) {
        if (!compiled) throw error::UserError("Please compile the pipeline first");
        if (args.size() != argument_order.size())
            throw error::UserError("All the arguments have not been passed! Expecting " +
                                   std::to_string(argument_order.size()) + " args");
        for (const auto &a : argument_order)
            if (args.count(a) <= 0) throw error::UserError("Argument " + a + " was not passed in");
        auto M = [&](const std::string &n) -> impl::MatrixGPU & { return *static_cast<impl::MatrixGPU *>(args.at(n)); };
        gb200_ctx *ctx = context();
        int rc = 0;
        switch (plan) {
            case Kernel::GemmF32: {
                auto &A = M(names[0]), &B = M(names[1]), &C = M(names[2]);
                require(A.col == B.row && C.row == A.row && C.col == B.col, "matrix_multiply: shapes do not agree");
                // The reference's leaf accumulates into C (c += sum): keep that.
                rc = gb200_gemm_f32(ctx, (const float *)A.data, A.lda, (const float *)B.data, B.lda,
                                    (float *)C.data, C.lda, C.row, C.col, A.col, 1, stream);
                break;
            }
            case Kernel::GemmBF16: {
                auto &A = M(names[0]), &B = M(names[1]), &C = M(names[2]);
                // B is a column-major K x N matrix: its object holds N rows of K values.
                require(A.col == B.col && C.row == A.row && C.col == B.row, "matrix_multiply: shapes do not agree");
                if (cluster_x > 0)
                    rc = gb200_gemm_bf16_cluster(ctx, A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col,
                                                 A.col, cluster_x, stream);
                else
                    rc = gb200_gemm_bf16(ctx, A.data, A.lda, B.data, B.lda, C.data, C.lda, C.row, C.col, A.col, stream);
                break;
            }
            case Kernel::Blur: {
                auto &in = M(names[0]), &out = M(names[1]);
                require(in.row >= out.row + 2 && in.col >= out.col + 2, "blur: the input must exceed the output by 2 rows and columns");
                rc = gb200_blur3x3_f32(ctx, (const float *)in.data, in.lda, out.row + 2, out.col + 2,
                                       (float *)out.data, out.lda, stream);
                break;
            }
            case Kernel::Softmax: {
                auto &in = M(names[0]), &out = M(names[1]);
                require(in.row == out.row && in.col == out.col, "softmax: shapes do not agree");
                rc = gb200_softmax_rows_f32(ctx, (const float *)in.data, in.lda, (float *)out.data, out.lda,
                                            in.row, in.col, stream);
                break;
            }
            case Kernel::Attention: {
                auto &Q = M(names[0]), &K = M(names[1]), &V = M(names[2]), &O = M(names[3]);
                require(Q.col == K.col && K.row == V.row && O.row == Q.row && O.col == V.col, "attention: shapes do not agree");
                if (cluster_x > 0)
                    rc = gb200_attention_bf16_cluster(ctx, Q.data, Q.lda, K.data, K.lda, V.data, V.lda, O.data, O.lda,
                                                      Q.row, K.row, Q.col, scale, cluster_x, stream);
                else
                    rc = gb200_attention_bf16(ctx, Q.data, Q.lda, K.data, K.lda, V.data, V.lda, O.data, O.lda,
                                              Q.row, K.row, Q.col, scale, stream);
                break;
            }
            case Kernel::GemmEpilogue: {
                auto V = [&](const std::string &n) -> float * {
                    return n.empty() ? nullptr : static_cast<impl::ArrayGPU *>(args.at(n))->data;
                };
                auto &A = M(names[0]), &B = M(names[1]);
                impl::MatrixGPU *C = epi_c.empty() ? nullptr : &M(epi_c);
                require(A.col == B.col, "matrix_multiply: shapes do not agree");
                if (C) require(C->row == A.row && C->col == B.row, "matrix_multiply: shapes do not agree");
                for (const std::string *v : {&epi_sub, &epi_div, &epi_max, &epi_sum})
                    if (!v->empty())
                        require(static_cast<impl::ArrayGPU *>(args.at(*v))->size == A.row,
                                "row vector length differs from the number of rows");
                gb200_gemm_epilogue e;
                e.alpha = scale;
                e.row_sub = V(epi_sub);
                e.apply_exp = epi_exp ? 1 : 0;
                e.row_div = V(epi_div);
                e.row_max = V(epi_max);
                e.row_sum = V(epi_sum);
                rc = gb200_gemm_bf16_epilogue(ctx, A.data, A.lda, B.data, B.lda, C ? C->data : nullptr,
                                              C ? C->lda : 0, A.row, B.row, A.col, &e, stream);
                break;
            }
            default: throw error::InternalError("no kernel planned");
        }
        if (rc != 0) throw error::UserError(std::string("libgern_b200: ") + gb200_last_error_string());
    }

    // The reference's callers synchronise through cudaMemcpy in MatrixGPU::get(); so do ours.
    static gb200_ctx *context() {
        static gb200_ctx *ctx = nullptr;
        if (!ctx && gb200_ctx_create(0, &ctx) != 0)
            throw error::UserError(std::string("libgern_b200: ") + gb200_last_error_string());
        return ctx;
    }

private:
    static void require(bool ok, const char *msg) {
        if (!ok) throw error::UserError(msg);
    }

    void flatten(const Composable &n, std::set<int> units, bool in_global) {
        if (!n.defined()) throw error::UserError("undefined Composable in the program");
        const Node *p = n.get();
        switch (p->kind) {
            case Node::Call: calls.push_back(p->call); return;
            case Node::Computation:
                for (const auto &ch : p->children) flatten(ch, units, in_global);
                return;
            case Node::Global:
                if (in_global) throw error::UserError("Global inside Global");
                for (const auto &kv : p->launch_args) {
                    if (kv.first == Grid::NULL_DIM) throw error::UserError("Global: NULL_DIM cannot be pinned");
                    if (!kv.second.isBound())
                        throw error::UserError("Global: launch dimension bound to unbound variable " + kv.second.getName());
                    if (kv.second.getInt64Val() <= 0) throw error::UserError("Global: launch dimensions are positive");
                    launch_args[kv.first] = kv.second.getInt64Val();
                }
                if (p->smem_size.defined() && p->smem_size.isBound()) {
                    if (p->smem_size.getInt64Val() > 227 * 1024)
                        throw error::UserError("Global: more dynamic shared memory than an sm_100a block can have (227 KB)");
                    smem_request = p->smem_size.getInt64Val();
                }
                flatten(p->children[0], units, true);
                return;
            case Node::Stage: flatten(p->children[0], units, in_global); return;
            case Node::Tiled: {
                if (p->unit != Grid::UNDEFINED) {
                    // A grid unit can drive one loop of a nest only (composable.cpp:242-262).
                    if (units.count(p->unit))
                        throw error::UserError(std::string("grid unit ") + Grid::name(p->unit) + " is bound twice in one nest");
                    if (!in_global) throw error::UserError("a grid unit can only be bound inside Global()");
                    // Outer loops take the coarser units: what is already distributed inside must
                    // not sit above the unit it is distributed over (legalToDistribute,
                    // src/annotations/grid.cpp:121-132, checked at composable.cpp:247-258).
                    for (int outer : units)
                        if (Grid::getLevel(static_cast<Grid::Unit>(outer)) < Grid::getLevel(p->unit))
                            throw error::UserError(std::string("Trying to distribute ") +
                                                   Grid::levelName(Grid::getLevel(p->unit)) + " over unit " +
                                                   Grid::name(static_cast<Grid::Unit>(outer)));
                    units.insert(p->unit);
                }
                if (!p->reduce && !p->member.adt.defined()) throw error::UserError("Tile needs an ADT field");
                if (!p->tile.defined()) throw error::UserError("tile variable has no name");
                flatten(p->children[0], units, in_global);
                // the tiled field must belong to an output of the body (Tile) -- composable.cpp:142-192
                if (!p->reduce) {
                    bool found = false;
                    for (const auto &cl : calls) found = found || cl.output == p->member.adt;
                    if (!found)
                        throw error::UserError("Tile(" + p->member.adt.getName() + "[\"" + p->member.field +
                                               "\"]): the data type is not produced by the tiled computation");
                }
                return;
            }
        }
    }

    // Turns what Global() pinned into the launch: the cluster dimension picks between the kernels
    // the library has for the planned operator (bf16 matrix_multiply and the fused chain have one for
    // single CTAs and one for CTA pairs), and the program's shared-memory request is held
    // against the planned layout of that kernel.
    void bindLaunch() {
        cluster_x = 0;
        kernel_name.clear();
        for (Grid::Dim d : {Grid::CLUSTER_DIM_Y, Grid::CLUSTER_DIM_Z}) {
            auto it = launch_args.find(d);
            if (it != launch_args.end() && it->second != 1)
                throw error::UserError("Global: the library's kernels form clusters along x only");
        }
        auto cx = launch_args.find(Grid::CLUSTER_DIM_X);
        if (cx != launch_args.end()) cluster_x = static_cast<int>(cx->second);
        switch (plan) {
            case Kernel::GemmBF16:
                if (cluster_x != 0 && cluster_x != 1 && cluster_x != 2)
                    throw error::UserError("Global: the bf16 matrix_multiply has kernels for clusters of 1 and 2 "
                                           "thread blocks, not " + std::to_string(cluster_x));
                // not pinned: the library picks by problem size; report the pair kernel's needs (the larger)
                kernel_name = cluster_x == 1 ? "gemm_bf16_tc" : "gemm_bf16_2cta";
                break;
            case Kernel::GemmEpilogue: kernel_name = "gemm_bf16_tc"; break;
            case Kernel::Attention:
                if (cluster_x != 0 && cluster_x != 1 && cluster_x != 2)
                    throw error::UserError("Global: the fused chain has kernels for clusters of 1 and 2 thread "
                                           "blocks, not " + std::to_string(cluster_x));
                kernel_name = cluster_x == 2 ? "attention_bf16_pair" : "attention_bf16";
                break;
            default: break;
        }
        if (plan != Kernel::GemmBF16 && plan != Kernel::Attention && cluster_x > 1)
            throw error::UserError("Global: only the bf16 matrix_multiply and the fused chain have kernels for "
                                   "clusters of " + std::to_string(cluster_x) + " thread blocks");
        if (kernel_name.empty()) return;
        if (gb200_kernel_resources_query(kernel_name.c_str(), &kernel_resources) != 0)
            throw error::InternalError(std::string("libgern_b200: ") + gb200_last_error_string());
        if (smem_request >= 0 && smem_request < kernel_resources.dynamic_smem_bytes)
            throw error::UserError("Global: kernel " + kernel_name + " needs " +
                                   std::to_string(kernel_resources.dynamic_smem_bytes) +
                                   " bytes of dynamic shared memory, the program asks for " +
                                   std::to_string(smem_request));
    }

    bool isChain(size_t at, AbstractDataTypePtr &in, AbstractDataTypePtr &out) const {
        // max(in -> m); subtract(m, in -> t1); exp(t1 -> t2); sum(t2 -> s); divide(s, t2 -> out)
        if (at + 5 > calls.size()) return false;
        const auto &mx = calls[at], &sb = calls[at + 1], &ex = calls[at + 2], &sm = calls[at + 3], &dv = calls[at + 4];
        if (mx.op != Op::MaxRow || sb.op != Op::SubstractVec || ex.op != Op::ExpMatrix || sm.op != Op::SumRow ||
            dv.op != Op::DivideVec)
            return false;
        in = mx.inputs[0];
        const bool flow = sb.inputs[0] == mx.output && sb.inputs[1] == in && ex.inputs[0] == sb.output &&
                          sm.inputs[0] == ex.output && dv.inputs[0] == sm.output && dv.inputs[1] == ex.output;
        if (!flow) return false;
        out = dv.output;
        return true;
    }

    void lower() {
        names.clear();
        auto f32 = [](const AbstractDataTypePtr &a) { return a->getDatatype() == Datatype::Float32; };
        if (calls.size() == 1 && calls[0].op == Op::MatrixMultiply) {
            const auto &A = calls[0].inputs[0], &B = calls[0].inputs[1], &C = calls[0].output;
            if (f32(A) && f32(B) && f32(C)) {
                if (B->getLayout() != Layout::RowMajor) throw error::UserError("fp32 matrix_multiply takes a row-major B");
                plan = Kernel::GemmF32;
            } else if (!f32(A) && !f32(B) && !f32(C)) {
                if (B->getLayout() != Layout::ColMajor) throw error::UserError("bf16 matrix_multiply takes a column-major B");
                plan = Kernel::GemmBF16;
            } else {
                throw error::UserError("matrix_multiply: mixed element types");
            }
            names = {A.getName(), B.getName(), C.getName()};
        } else if (calls.size() == 2 && calls[0].op == Op::BlurX && calls[1].op == Op::BlurY) {
            if (!(calls[1].inputs[0] == calls[0].output))
                throw error::UserError("blur_y must consume the output of blur_x");
            for (const auto &cl : calls) {
                auto it = cl.template_args.find("stride");
                if (it == cl.template_args.end() || it->second.getInt64Val() != 3)
                    throw error::UserError("this library fuses blur_x/blur_y with stride 3 only");
            }
            plan = Kernel::Blur;
            names = {calls[0].inputs[0].getName(), calls[1].output.getName()};
        } else if (calls.size() == 5 && calls[0].op != Op::MatrixMultiply) {
            AbstractDataTypePtr in, out;
            if (!isChain(0, in, out)) throw error::UserError("unrecognised 5-call pipeline (expected the softmax chain)");
            plan = Kernel::Softmax;
            names = {in.getName(), out.getName()};
        } else if (calls.size() == 7 && calls[0].op == Op::MatrixMultiply && calls[6].op == Op::MatrixMultiply) {
            AbstractDataTypePtr in, out;
            if (!isChain(1, in, out) || !(in == calls[0].output) || !(calls[6].inputs[0] == out))
                throw error::UserError("unrecognised 7-call pipeline (expected matmul ; softmax ; matmul)");
            const auto &Q = calls[0].inputs[0], &K = calls[0].inputs[1], &V = calls[6].inputs[1], &O = calls[6].output;
            if (f32(Q) || f32(K) || f32(V) || f32(O)) throw error::UserError("the fused chain takes BFloat16 Q, K, V, O");
            if (K->getLayout() != Layout::ColMajor) throw error::UserError("the fused chain takes K as the column-major operand of Q K^T");
            plan = Kernel::Attention;
            scale = calls[0].scale;
            names = {Q.getName(), K.getName(), V.getName(), O.getName()};
        } else if (calls.size() >= 2 && calls.size() <= 6 && calls[0].op == Op::MatrixMultiply) {
            lowerEpilogue(f32);
        } else {
            std::ostringstream os;
            os << "no fused sm_100a kernel for this pipeline:";
            for (const auto &cl : calls) os << " " << opName(cl.op);
            throw error::UserError(os.str());
        }
        // Argument order = ADTs sorted by name, as the reference orders them (codegen.cpp:139-198).
        argument_order = names;
        std::sort(argument_order.begin(), argument_order.end());
        std::set<std::string> uniq(argument_order.begin(), argument_order.end());
        if (uniq.size() != argument_order.size()) throw error::UserError("two arguments share a name");
    }

    // matrix_multiply followed by consumers of its product: elementwise leaves in the order
    // subtract_vec, exp_matrix, divide_vec (each optional), then max_row and / or sum_row of the
    // last matrix.  Matrices between the stages must be temporaries (they live in TMEM and
    // registers only); the last one is stored unless it is a temporary too.
    template <typename F32>
    void lowerEpilogue(F32 f32) {
        const auto &mm = calls[0];
        const auto &A = mm.inputs[0], &B = mm.inputs[1];
        if (f32(A) || f32(B)) throw error::UserError("fused consumers need the BFloat16 matrix_multiply");
        if (B->getLayout() != Layout::ColMajor) throw error::UserError("bf16 matrix_multiply takes a column-major B");
        epi_sub = epi_div = epi_max = epi_sum = epi_c = "";
        epi_exp = false;
        AbstractDataTypePtr cur = mm.output;
        size_t at = 1;
        auto step = [&](const AbstractDataTypePtr &next) {
            if (!cur->isTemporary())
                throw error::UserError("matrix " + cur.getName() + " sits between fused stages: declare it a temporary");
            cur = next;
            ++at;
        };
        if (at < calls.size() && calls[at].op == Op::SubstractVec && calls[at].inputs[1] == cur) {
            epi_sub = calls[at].inputs[0].getName();
            step(calls[at].output);
        }
        if (at < calls.size() && calls[at].op == Op::ExpMatrix && calls[at].inputs[0] == cur) {
            epi_exp = true;
            step(calls[at].output);
        }
        if (at < calls.size() && calls[at].op == Op::DivideVec && calls[at].inputs[1] == cur) {
            epi_div = calls[at].inputs[0].getName();
            step(calls[at].output);
        }
        for (; at < calls.size(); ++at) {
            const auto &cl = calls[at];
            if (cl.op == Op::MaxRow && cl.inputs[0] == cur && epi_max.empty())
                epi_max = cl.output.getName();
            else if (cl.op == Op::SumRow && cl.inputs[0] == cur && epi_sum.empty())
                epi_sum = cl.output.getName();
            else
                throw error::UserError(std::string("no fused sm_100a kernel: ") + opName(cl.op) +
                                       " cannot follow in the epilogue of matrix_multiply here");
        }
        if (f32(cur) && !cur->isTemporary()) throw error::UserError("the stored result of the fused GEMM is BFloat16");
        if (!cur->isTemporary()) epi_c = cur.getName();
        if (epi_c.empty() && epi_max.empty() && epi_sum.empty())
            throw error::UserError("the pipeline produces nothing: its last matrix is a temporary");
        plan = Kernel::GemmEpilogue;
        scale = mm.scale;
        names = {A.getName(), B.getName()};
        for (const std::string *v : {&epi_c, &epi_sub, &epi_div, &epi_max, &epi_sum})
            if (!v->empty()) names.push_back(*v);
    }

    std::map<Grid::Dim, int64_t> launch_args;
    int64_t smem_request = -1;   // Global(..., smem_size), -1 = none
    int cluster_x = 0;
    std::string kernel_name;
    gb200_kernel_resources kernel_resources{};
    std::string epi_sub, epi_div, epi_max, epi_sum, epi_c;
    bool epi_exp = false;
    Composable c;
    std::vector<FunctionCall> calls;
    Kernel plan = Kernel::None;
    std::vector<std::string> names;           // in kernel-argument order
    std::vector<std::string> argument_order;  // sorted, as evaluate() expects them
    float scale = 1.0f;
    bool compiled = false;
};

}  // namespace b200
}  // namespace gern
