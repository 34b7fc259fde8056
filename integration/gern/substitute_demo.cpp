// Programs written exactly as the reference's apps and tests write them, with the reference's OWN
// annotation headers (apps/common/annot, gernels/mm/gern_annot, test/library/matrix/annot), are
// run through gern::b200::substitute() and then through the unmodified Runner.
//
//   gern_b200_substitute --repo <root of this repository> {blur|mm_cpu|softmax|unmatched}
//
// Built a second time with -DDEMO_PATCHED_RUNNER against a Runner that carries
// runner_substitute.patch (gern_b200_patched): the demo then hands the ORIGINAL program to
// Runner::compile with nothing but a file name, and the substitution happens inside Gern.
//
// Prints `matched: <kernel>` and, after Runner::compile, `compiled: <file>`; then calls evaluate on
// small host matrices.  Exit status as in run_program.cpp (4 = evaluate failed; without a GPU that
// is the library's "no CUDA device").  `unmatched` shows a program that is left alone.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "annot/adt.h"          // apps/common/annot/adt.h        (the reference's blur / softmax ADTs)
#include "annot/functions.h"    // apps/common/annot/functions.h  (BlurX, BlurY, MaxRow, ...)
#include "compose/runner.h"
#include "gb200_host.h"
#include "library/matrix/annot/cpu-matrix.h"   // test/library/matrix/annot/cpu-matrix.h (MatrixMultiplyCPU)
#include "substitute.h"

using namespace gern;

int main(int argc, char **argv) {
    std::vector<std::string> a(argv + 1, argv + argc);
    if (a.size() != 3 || a[0] != "--repo") {
        std::fprintf(stderr, "usage: %s --repo <root> {blur|mm_cpu|softmax|unmatched}\n", argv[0]);
        return 2;
    }
    const std::string repo = a[1], what = a[2];
    const char *cuda = std::getenv("CUDA_HOME") ? std::getenv("CUDA_HOME") : "/usr/local/cuda";
    Composable program;
    std::map<std::string, void *> args;
    constexpr int64_t R = 48, C = 64;
    // buffers large enough for every program below (the blur's 50 x 66 input, the 64 x 64 squares)
    std::vector<float> in_buf((C + 2) * (C + 2), 1.0f), out_buf(C * C, 0.0f), b_buf(C * C, 1.0f);
    gb200_host::HostMatrix in(in_buf.data(), R + 2, C + 2, C + 2), out(out_buf.data(), R, C, C);
    gb200_host::HostMatrix sq_a(in_buf.data(), C, C, C), sq_b(b_buf.data(), C, C, C), sq_c(out_buf.data(), C, C, C);
    int64_t k_dim_val = C;
    try {
        if (what == "blur" || what == "unmatched") {
            // apps/blur/blur.cpp:46-73, word for word apart from the sizes
            using InAnnot = ::annot::MatrixGPUSequential<R + 2, C + 2, 1>;
            using OutAnnot = ::annot::MatrixGPUSequential<R, C, 1>;
            auto input = AbstractDataTypePtr(new const InAnnot("input", false));
            auto output = AbstractDataTypePtr(new const OutAnnot("output", false));
            auto temp = AbstractDataTypePtr(new const OutAnnot("temp", true));
            Variable col("col"), col_inner("col_inner"), row("row"), row_inner("row_inner"), stride{"stride"};
            const int64_t stride_val = what == "blur" ? 3 : 5;     // only stride 3 has a fused kernel
            ::annot::BlurX blur_x_no_template{input, temp};
            auto blur_x_t = &blur_x_no_template[{{"stride", stride.bind(stride_val)}}];
            ::annot::BlurY blur_y{input, temp};
            auto blur_y_t = &blur_y[{{"stride", stride.bind(stride_val)}}];
            program = {Global(
                (Tile(output["col"], col.bind(32)) || Grid::BLOCK_X)(
                    (Tile(output["row"], row.bind(24)) || Grid::BLOCK_Y)(
                        (Tile(output["col"], col_inner.bind(8)) || Grid::THREAD_X)(
                            (Tile(output["row"], row_inner.bind(4)) || Grid::THREAD_Y)(
                                (*blur_x_t)(input, temp),
                                (*blur_y_t)(temp, output))))))};
            args = {{"input", &in}, {"output", &out}};
        } else if (what == "mm_cpu") {
            // test/test-cpu-mm.cpp:13-83
            auto A_DS = AbstractDataTypePtr(new const gern::annot::MatrixCPU("A"));
            auto B_DS = AbstractDataTypePtr(new const gern::annot::MatrixCPU("B"));
            auto C_DS = AbstractDataTypePtr(new const gern::annot::MatrixCPU("C"));
            gern::annot::MatrixMultiplyCPU matrix_multiply;
            Variable ti("ti"), tj("tj"), tk("tk"), k_dim("k_dim");
            program = {(Tile(C_DS["row"], ti))(Tile(C_DS["col"], tj)((Reduce(k_dim, tk))(matrix_multiply(A_DS, B_DS, C_DS, k_dim))))};
            args = {{"A", &sq_a}, {"B", &sq_b}, {"C", &sq_c}, {"k_dim", &k_dim_val}};
#ifdef DEMO_PATCHED_RUNNER
            // a caller written for the original schedule also passes its tile sizes: the patched
            // Runner::evaluate accepts and ignores them
            static int64_t tile = 16;
            args["ti"] = &tile;
            args["tj"] = &tile;
            args["tk"] = &tile;
#endif
        } else if (what == "softmax") {
            // the five row-softmax pieces of apps/common/annot/functions.h:9-173 under one row tile
            using MatAnnot = ::annot::MatrixGPUSequential<R, C, 1>;
            auto x = AbstractDataTypePtr(new const MatAnnot("input", false));
            auto y = AbstractDataTypePtr(new const MatAnnot("output", false));
            auto t1 = AbstractDataTypePtr(new const MatAnnot("shifted", true));
            auto t2 = AbstractDataTypePtr(new const MatAnnot("exped", true));
            auto m = AbstractDataTypePtr(new const ::annot::StaticArray("row_max"));
            auto sm = AbstractDataTypePtr(new const ::annot::StaticArray("row_sum"));
            Variable row("row"), stride{"stride"};
            ::annot::MaxRow max_row(x, m);
            ::annot::SubstractVec subtract_vec(m, x, t1);
            ::annot::ExpMatrix exp_matrix(t1, t2);
            ::annot::SumRow sum_row(t2, sm);
            ::annot::DivideVec divide_vec(sm, t2, y);
            auto max_t = &max_row[{{"stride", stride.bind(1)}}];
            auto sum_t = &sum_row[{{"stride", stride.bind(1)}}];
            program = {Global((Tile(y["row"], row.bind(1)) || Grid::BLOCK_X)(
                (*max_t)(m, x), subtract_vec(m, x, t1), exp_matrix(t1, t2), (*sum_t)(sm, t2), divide_vec(sm, t2, y)))};
            in = gb200_host::HostMatrix(in_buf.data(), R, C, C);
            args = {{"input", &in}, {"output", &out}};
        } else {
            std::fprintf(stderr, "unknown program %s\n", what.c_str());
            return 2;
        }
    } catch (const std::exception &e) {
        std::fprintf(stderr, "building the program failed: %s\n", e.what());
        return 3;
    }

    b200::Substitution sub = b200::substitute(program, /*device=*/false);
    std::printf("matched: %s\n", sub.matched ? sub.kernel.c_str() : "none (program left as written)");
    if (!sub.matched) return 0;
    std::printf("arguments:");
    for (const auto &n : sub.arguments) std::printf(" %s", n.c_str());
    std::printf("\n");

    Runner::Options o;
    o.prefix = "/tmp";
#ifdef DEMO_PATCHED_RUNNER
    // the patched Runner substitutes by itself and adds the include and link flags of the library
    setenv("GERN_B200_OPERANDS", "host", 1);
    Runner run(program);
    o.filename = "gern_b200_patched_" + what + ".cpp";
    o.include = " -O2 ";
    (void)cuda;
#else
    Runner run(sub.program);
    o.filename = "gern_b200_substituted_" + what + ".cpp";
    o.cpp_std = "c++17";
    o.include = " -O2 -I " + repo + "/integration/gern -I " + repo + "/include -I " + cuda + "/include";
    o.ldflags = "-L " + repo + "/gern_b200 -lgern_b200 -Wl,-rpath," + repo + "/gern_b200 -L " + cuda + "/lib64 -lcudart";
#endif
    try {
        run.compile(o);
    } catch (const std::exception &e) {
        std::fprintf(stderr, "Runner::compile failed: %s\n", e.what());
        return 3;
    }
    std::printf("compiled: %s/%s\n", o.prefix.c_str(), o.filename.c_str());
    try {
        run.evaluate(args);
    } catch (const std::exception &e) {
        std::fprintf(stderr, "evaluate failed: %s\n", e.what());
        return 4;
    }
    // a constant image is a fixed point of the blur; ones times ones sums to the inner extent
    const float want = what == "blur" ? 1.0f : what == "softmax" ? 1.0f / (float)C : (float)C;
    const size_t produced = what == "mm_cpu" ? C * C : R * C;
    for (size_t i = 0; i < produced; ++i)
        if (const float v = out_buf[i]; v != want) {
            std::fprintf(stderr, "wrong result: %g instead of %g\n", v, want);
            return 5;
        }
    std::printf("evaluated: result as expected\n");
    return 0;
}
