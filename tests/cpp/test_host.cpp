// Tests of the C++ host layer, written the way the reference's own tests and app self-checks are:
// build a Composable from annotated functions, Runner::compile, Runner::evaluate on small inputs,
// compare with a CPU loop (test/test-cpu-mm.cpp:13-83, apps/blur/blur.cpp:83-108,
// gernels/mm/kernel_10.cu:168-177, test/test-runner.cpp).
//
//   test_host cpu   composition, legality and lowering checks (no GPU needed)
//   test_host gpu   the same programs evaluated on cuda:0 against CPU loops
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <random>

#include "gern_b200.hpp"

using namespace gern::b200;

static int failures = 0;
#define CHECK(cond)                                                           \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);      \
            ++failures;                                                       \
        }                                                                     \
    } while (0)

template <typename F>
static bool throwsUserError(F f) {
    try {
        f();
    } catch (const error::UserError &) {
        return true;
    }
    return false;
}

// ---- programs ------------------------------------------------------------------------------
struct MMProgram {
    AbstractDataTypePtr A, B, C;
    Composable program;
};
// The kernel_10-style schedule of the reference (gernels/mm/kernel_10.cu:108-131): block tiles
// bound to BLOCK_X / BLOCK_Y, a K reduction, staged operands, warp and thread tiles.
static MMProgram mmProgram(Datatype t) {
    MMProgram p;
    const Layout bl = t == Datatype::Float32 ? Layout::RowMajor : Layout::ColMajor;
    p.A = AbstractDataTypePtr(new const annot::MatrixGPU("A", t));
    p.B = AbstractDataTypePtr(new const annot::MatrixGPU("B", t, bl));
    p.C = AbstractDataTypePtr(new const annot::MatrixGPU("C", t));
    Variable block_x("block_x"), block_y("block_y"), k_tiled("k_tiled"), k_dim("k_dim");
    Variable warp_x("warp_x"), warp_y("warp_y");
    annot::MatrixMultiply mm;
    p.program = {Global(
        (Tile(p.C["row"], block_x.bind(32)) || Grid::BLOCK_X)(
            (Tile(p.C["col"], block_y.bind(32)) || Grid::BLOCK_Y)(
                (Reduce(k_dim, k_tiled.bind(64)))(
                    Stage(p.A, Stage(p.B,
                        (Tile(p.C["row"], warp_x.bind(32)) || Grid::WARP_Y)(
                            (Tile(p.C["col"], warp_y.bind(32)) || Grid::WARP_X)(
                                mm(p.A, p.B, p.C)))))))))};
    return p;
}

struct BlurProgram {
    AbstractDataTypePtr input, output, temp;
    Composable program;
};
// apps/blur/blur.cpp:41-73
static BlurProgram blurProgram(int64_t stride_val = 3) {
    BlurProgram p;
    p.input = AbstractDataTypePtr(new const annot::MatrixGPU("input"));
    p.output = AbstractDataTypePtr(new const annot::MatrixGPU("output"));
    p.temp = AbstractDataTypePtr(new const annot::MatrixGPU("temp", Datatype::Float32, Layout::RowMajor, true));
    Variable col("col"), col_inner("col_inner"), row("row"), row_inner("row_inner"), stride("stride");
    annot::BlurX blur_x;
    annot::BlurY blur_y;
    auto &bx = blur_x[{{"stride", stride.bind(stride_val)}}];
    auto &by = blur_y[{{"stride", stride.bind(stride_val)}}];
    p.program = {Global(
        (Tile(p.output["col"], col.bind(128)) || Grid::BLOCK_X)(
            (Tile(p.output["row"], row.bind(24)) || Grid::BLOCK_Y)(
                (Tile(p.output["col"], col_inner.bind(8)) || Grid::THREAD_X)(
                    (Tile(p.output["row"], row_inner.bind(4)) || Grid::THREAD_Y)(
                        bx(p.input, p.temp),
                        by(p.temp, p.output))))))};
    return p;
}

struct SoftmaxProgram {
    AbstractDataTypePtr in, out;
    Composable program;
};
// The assembled five-op program the reference sketches (test/test-cpu-matrix.cpp:69-148).
static Composable softmaxChain(AbstractDataTypePtr in, AbstractDataTypePtr out, const std::string &tag) {
    auto m = AbstractDataTypePtr(new const annot::ArrayGPU("max_" + tag));
    auto s = AbstractDataTypePtr(new const annot::ArrayGPU("sum_" + tag));
    auto t1 = AbstractDataTypePtr(new const annot::MatrixGPU("sub_" + tag, Datatype::Float32, Layout::RowMajor, true));
    auto t2 = AbstractDataTypePtr(new const annot::MatrixGPU("exp_" + tag, Datatype::Float32, Layout::RowMajor, true));
    annot::MaxRow max_row;
    annot::SubstractVec subtract_vec;
    annot::ExpMatrix exp_matrix;
    annot::SumRow sum_row;
    annot::DivideVec divide_vec;
    return Composable({max_row(in, m), subtract_vec(m, in, t1), exp_matrix(t1, t2), sum_row(t2, s),
                       divide_vec(s, t2, out)});
}
static SoftmaxProgram softmaxProgram() {
    SoftmaxProgram p;
    p.in = AbstractDataTypePtr(new const annot::MatrixGPU("input"));
    p.out = AbstractDataTypePtr(new const annot::MatrixGPU("output"));
    Variable row("row");
    p.program = {Global((Tile(p.out["row"], row.bind(1)) || Grid::BLOCK_X)(softmaxChain(p.in, p.out, "a")))};
    return p;
}

struct AttentionProgram {
    AbstractDataTypePtr Q, K, V, O;
    Composable program;
};
static AttentionProgram attentionProgram(float scale) {
    AttentionProgram p;
    const Datatype bf = Datatype::BFloat16;
    p.Q = AbstractDataTypePtr(new const annot::MatrixGPU("Q", bf));
    p.K = AbstractDataTypePtr(new const annot::MatrixGPU("K", bf, Layout::ColMajor));
    p.V = AbstractDataTypePtr(new const annot::MatrixGPU("V", bf));
    p.O = AbstractDataTypePtr(new const annot::MatrixGPU("O", bf));
    auto S = AbstractDataTypePtr(new const annot::MatrixGPU("S", Datatype::Float32, Layout::RowMajor, true));
    auto P = AbstractDataTypePtr(new const annot::MatrixGPU("P", Datatype::Float32, Layout::RowMajor, true));
    annot::MatrixMultiply qk(scale), pv;
    Variable row("row");
    p.program = {Global((Tile(p.O["row"], row.bind(128)) || Grid::BLOCK_X)(
        qk(p.Q, p.K, S), softmaxChain(S, P, "s"), pv(P, p.V, p.O)))};
    return p;
}

// matrix_multiply whose product feeds the reference's elementwise / row-reduction leaves:
// E = exp(scale * A B - sub), with the row sums of E; the product and the difference are temporaries.
struct EpilogueProgram {
    AbstractDataTypePtr A, B, E, sub, sum;
    Composable program;
};
static EpilogueProgram epilogueProgram(float scale, bool temporaries = true, bool store = true) {
    EpilogueProgram p;
    const Datatype bf = Datatype::BFloat16;
    p.A = AbstractDataTypePtr(new const annot::MatrixGPU("A", bf));
    p.B = AbstractDataTypePtr(new const annot::MatrixGPU("B", bf, Layout::ColMajor));
    p.E = AbstractDataTypePtr(new const annot::MatrixGPU("E", bf, Layout::RowMajor, !store));
    p.sub = AbstractDataTypePtr(new const annot::ArrayGPU("m", false));
    p.sum = AbstractDataTypePtr(new const annot::ArrayGPU("s", false));
    auto S = AbstractDataTypePtr(new const annot::MatrixGPU("S", Datatype::Float32, Layout::RowMajor, temporaries));
    auto D = AbstractDataTypePtr(new const annot::MatrixGPU("D", Datatype::Float32, Layout::RowMajor, true));
    annot::MatrixMultiply mm(scale);
    annot::SubstractVec subtract_vec;
    annot::ExpMatrix exp_matrix;
    annot::SumRow sum_row;
    Variable row("row");
    p.program = {Global((Tile(p.sum["x"], row.bind(128)) || Grid::BLOCK_X)(
        mm(p.A, p.B, S), subtract_vec(p.sub, S, D), exp_matrix(D, p.E), sum_row(p.E, p.sum)))};
    return p;
}

// ---- CPU-only checks -------------------------------------------------------------------------
static void cpuTests() {
    {   // lowering picks the kernel and orders arguments by name
        auto p = mmProgram(Datatype::Float32);
        Runner run(p.program);
        Runner::Options o;
        o.arch = "100a";
        run.compile(o);
        CHECK(run.kernel() == Runner::Kernel::GemmF32);
        CHECK((run.argumentOrder() == std::vector<std::string>{"A", "B", "C"}));
        auto q = mmProgram(Datatype::BFloat16);
        Runner run2(q.program);
        run2.compile();
        CHECK(run2.kernel() == Runner::Kernel::GemmBF16);
    }
    {
        auto p = blurProgram();
        Runner run(p.program);
        run.compile();
        CHECK(run.kernel() == Runner::Kernel::Blur);
        CHECK((run.argumentOrder() == std::vector<std::string>{"input", "output"}));  // temp is fused away
    }
    {
        auto p = softmaxProgram();
        Runner run(p.program);
        run.compile();
        CHECK(run.kernel() == Runner::Kernel::Softmax);
    }
    {
        auto p = attentionProgram(0.5f);
        Runner run(p.program);
        run.compile();
        CHECK(run.kernel() == Runner::Kernel::Attention);
        CHECK((run.argumentOrder() == std::vector<std::string>{"K", "O", "Q", "V"}));
    }
    {   // consumers of a product go into the GEMM's epilogue
        auto p = epilogueProgram(0.25f);
        Runner run(p.program);
        run.compile();
        CHECK(run.kernel() == Runner::Kernel::GemmEpilogue);
        CHECK((run.argumentOrder() == std::vector<std::string>{"A", "B", "E", "m", "s"}));
        auto q = epilogueProgram(0.25f, true, false);   // E a temporary: only the row sums leave the kernel
        Runner run2(q.program);
        run2.compile();
        CHECK((run2.argumentOrder() == std::vector<std::string>{"A", "B", "m", "s"}));
    }
    CHECK(throwsUserError([] {   // a matrix between fused stages has nowhere to live unless it is a temporary
        auto p = epilogueProgram(1.0f, false);
        Runner run(p.program);
        run.compile();
    }));
    {   // cluster units nest above block units; Global() records pinned launch dimensions
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A", Datatype::BFloat16));
        auto B = AbstractDataTypePtr(new const annot::MatrixGPU("B", Datatype::BFloat16, Layout::ColMajor));
        auto C = AbstractDataTypePtr(new const annot::MatrixGPU("C", Datatype::BFloat16));
        Variable cl("cl"), bx("bx"), by("by"), kd("k_dim"), kt("kt"), cx("cluster_x"), smem("smem");
        annot::MatrixMultiply mm;
        Composable prog = {Global(
            (Tile(C["row"], cl.bind(256)) || Grid::BLOCK_CLUSTER_X)(
                (Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(
                    (Tile(C["col"], by.bind(256)) || Grid::BLOCK_Y)(
                        (Reduce(kd, kt.bind(64)))(mm(A, B, C))))),
            {{Grid::CLUSTER_DIM_X, cx.bind(2)}}, smem.bind(200 * 1024))};
        Runner run(prog);
        run.compile();
        CHECK(run.kernel() == Runner::Kernel::GemmBF16);
        CHECK(run.launchArgs().at(Grid::CLUSTER_DIM_X) == 2);
        // the pinned cluster dimension picks the CTA-pair kernel, whose planned layout is reported
        CHECK(run.clusterX() == 2 && run.kernelName() == "gemm_bf16_2cta" && run.hasResources());
        CHECK(run.resources().cluster_x == 2 && run.resources().threads == 192 && run.resources().tmem_columns == 512);
        CHECK(run.resources().dynamic_smem_bytes > 6 * 32 * 1024 && run.resources().dynamic_smem_bytes <= 200 * 1024);
        {   // cluster of one: the single-CTA kernel and its (different) layout
            Composable one = {Global((Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(A, B, C)),
                                     {{Grid::CLUSTER_DIM_X, Variable("c1").bind(1)}})};
            Runner r1(one);
            r1.compile();
            CHECK(r1.clusterX() == 1 && r1.kernelName() == "gemm_bf16_tc" && r1.resources().cluster_x == 1);
            CHECK(r1.resources().dynamic_smem_bytes != run.resources().dynamic_smem_bytes);
        }
        CHECK(throwsUserError([&] {   // no kernel for clusters of 4
            Composable bad = {Global((Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(A, B, C)),
                                     {{Grid::CLUSTER_DIM_X, Variable("c4").bind(4)}})};
            Runner r(bad);
            r.compile();
        }));
        CHECK(throwsUserError([&] {   // less shared memory than the planned layout of the kernel needs
            Composable bad = {Global((Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(A, B, C)),
                                     {{Grid::CLUSTER_DIM_X, Variable("c2").bind(2)}}, Variable("s").bind(64 * 1024))};
            Runner r(bad);
            r.compile();
        }));
        CHECK(throwsUserError([&] {   // the fp32 matrix_multiply has no cluster kernel
            auto fA = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
            auto fB = AbstractDataTypePtr(new const annot::MatrixGPU("B"));
            auto fC = AbstractDataTypePtr(new const annot::MatrixGPU("C"));
            Composable bad = {Global((Tile(fC["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(fA, fB, fC)),
                                     {{Grid::CLUSTER_DIM_X, Variable("c2").bind(2)}})};
            Runner r(bad);
            r.compile();
        }));
        CHECK(Grid::getLevel(Grid::BLOCK_CLUSTER_Y) == Grid::BLOCK_CLUSTER);
        CHECK(Grid::getDim(Grid::BLOCK_CLUSTER_Z) == Grid::CLUSTER_DIM_Z);
        CHECK(throwsUserError([&] {   // blocks cannot be distributed over... a cluster inside a block
            Composable bad = {Global(
                (Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(
                    (Tile(C["col"], cl.bind(256)) || Grid::BLOCK_CLUSTER_X)(mm(A, B, C))))};
            Runner r(bad);
            r.compile();
        }));
        CHECK(throwsUserError([&] {   // a pinned launch dimension needs a value
            Composable bad = {Global((Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(A, B, C)),
                                     {{Grid::GRID_DIM_X, Variable("gx")}})};
            Runner r(bad);
            r.compile();
        }));
        CHECK(throwsUserError([&] {   // more shared memory than an sm_100a block can have
            Composable bad = {Global((Tile(C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(A, B, C)), {},
                                     smem.bind(300 * 1024))};
            Runner r(bad);
            r.compile();
        }));
    }
    // errors, as the reference raises them
    CHECK(throwsUserError([] {   // evaluate before compile (src/codegen/runner.cpp:58-60)
        auto p = blurProgram();
        Runner run(p.program);
        run.evaluate({});
    }));
    CHECK(throwsUserError([] {   // wrong arch
        auto p = blurProgram();
        Runner run(p.program);
        Runner::Options o;
        o.arch = "89";
        run.compile(o);
    }));
    CHECK(throwsUserError([] {   // missing / misnamed arguments (runner.cpp:62-76)
        auto p = blurProgram();
        Runner run(p.program);
        run.compile();
        int dummy = 0;
        run.evaluate({{"input", &dummy}});
    }));
    CHECK(throwsUserError([] {
        auto p = blurProgram();
        Runner run(p.program);
        run.compile();
        int dummy = 0;
        run.evaluate({{"input", &dummy}, {"not_output", &dummy}});
    }));
    CHECK(throwsUserError([] {   // a grid unit bound twice in one nest (test-grid-constraints.cpp)
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
        auto B = AbstractDataTypePtr(new const annot::MatrixGPU("B"));
        auto C = AbstractDataTypePtr(new const annot::MatrixGPU("C"));
        annot::MatrixMultiply mm;
        Variable a("a"), b("b");
        Composable prog = {Global((Tile(C["row"], a.bind(8)) || Grid::BLOCK_X)(
            (Tile(C["col"], b.bind(8)) || Grid::BLOCK_X)(mm(A, B, C))))};
        Runner(prog).compile();
    }));
    CHECK(throwsUserError([] {   // grid binding outside Global
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
        auto B = AbstractDataTypePtr(new const annot::MatrixGPU("B"));
        auto C = AbstractDataTypePtr(new const annot::MatrixGPU("C"));
        annot::MatrixMultiply mm;
        Variable a("a");
        Composable prog = {(Tile(C["row"], a.bind(8)) || Grid::BLOCK_X)(mm(A, B, C))};
        Runner(prog).compile();
    }));
    CHECK(throwsUserError([] {   // tiling a field of something the body does not produce
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
        auto B = AbstractDataTypePtr(new const annot::MatrixGPU("B"));
        auto C = AbstractDataTypePtr(new const annot::MatrixGPU("C"));
        annot::MatrixMultiply mm;
        Variable a("a");
        Composable prog = {Tile(A["row"], a.bind(8))(mm(A, B, C))};
        Runner(prog).compile();
    }));
    CHECK(throwsUserError([] {   // unknown field
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
        (void)A["depth"];
    }));
    CHECK(throwsUserError([] {   // unbound template argument
        annot::BlurX bx;
        Variable stride("stride");
        bx[{{"stride", stride}}];
    }));
    CHECK(throwsUserError([] { blurProgram(5); Runner(blurProgram(5).program).compile(); }));
    CHECK(throwsUserError([] {   // a pipeline with no fused kernel: no generic fallback exists
        auto A = AbstractDataTypePtr(new const annot::MatrixGPU("A"));
        auto B = AbstractDataTypePtr(new const annot::MatrixGPU("B"));
        annot::ExpMatrix e;
        Runner(Composable({e(A, B)})).compile();
    }));
}

// ---- GPU checks -----------------------------------------------------------------------------
static void gpuTests() {
    {   // blur, ascending input, exact equality with the CPU loops (apps/blur/blur.cpp:83-108)
        const int64_t rows = 24 * 6, cols = 128 * 3;
        auto p = blurProgram();
        Runner run(p.program);
        Runner::Options o;
        o.arch = "100a";
        run.compile(o);
        impl::MatrixGPU in(rows + 4, cols + 4, cols + 4), out(rows, cols, cols);
        in.ascending();
        out.vvals(0.0f);
        run.evaluate({{p.input.getName(), &in}, {p.output.getName(), &out}});
        auto got = out.get();
        auto hin = in.get();
        impl::MatrixCPU bx(rows + 2, cols, cols), by(rows, cols, cols);
        for (int64_t i = 0; i < rows + 2; i++)
            for (int64_t j = 0; j < cols; j++) bx(i, j) = (hin(i, j) + hin(i, j + 1) + hin(i, j + 2)) / 3;
        for (int64_t i = 0; i < rows; i++)
            for (int64_t j = 0; j < cols; j++) by(i, j) = (bx(i, j) + bx(i + 1, j) + bx(i + 2, j)) / 3;
        bool equal = true;
        for (int64_t i = 0; i < rows; i++)
            for (int64_t j = 0; j < cols; j++) equal = equal && got(i, j) == by(i, j);
        CHECK(equal);
        // the same program on a stream of the caller's: identical result once that stream is done
        cudaStream_t stream;
        impl::cudaCheck(cudaStreamCreate(&stream), "cudaStreamCreate");
        out.vvals(0.0f);
        run.evaluate({{p.input.getName(), &in}, {p.output.getName(), &out}}, stream);
        impl::cudaCheck(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        auto again = out.get();
        bool same = true;
        for (int64_t i = 0; i < rows; i++)
            for (int64_t j = 0; j < cols; j++) same = same && again(i, j) == by(i, j);
        CHECK(same);
        impl::cudaCheck(cudaStreamDestroy(stream), "cudaStreamDestroy");
        again.destroy();
        got.destroy(); hin.destroy(); bx.destroy(); by.destroy(); in.destroy(); out.destroy();
    }
    {   // fp32 matmul, ascending % 10 inputs, |delta| < 1e-3 (gernels/mm/kernel_10.cu:140-177)
        const int64_t n = 256;
        auto p = mmProgram(Datatype::Float32);
        Runner run(p.program);
        run.compile();
        impl::MatrixGPU A(n, n), B(n, n), C(n, n);
        impl::MatrixCPU ha(n, n, n), hb(n, n, n);
        for (int64_t i = 0; i < n * n; i++) {
            ha.data[i] = static_cast<float>(i % 10);
            hb.data[i] = static_cast<float>((i * 7) % 10);
        }
        A.put(ha); B.put(hb); C.vvals(0.0f);
        run.evaluate({{"A", &A}, {"B", &B}, {"C", &C}});
        auto got = C.get();
        float worst = 0.f;
        for (int64_t i = 0; i < n; i++)
            for (int64_t j = 0; j < n; j++) {
                float sum = 0.f;
                for (int64_t k = 0; k < n; k++) sum += ha(i, k) * hb(k, j);
                worst = std::fmax(worst, std::fabs(sum - got(i, j)));
            }
        CHECK(worst < 1e-3f);
        // the leaf accumulates into C: a second evaluate doubles the result
        run.evaluate({{"A", &A}, {"B", &B}, {"C", &C}});
        auto twice = C.get();
        CHECK(std::fabs(twice(3, 5) - 2 * got(3, 5)) < 1e-2f);
        got.destroy(); twice.destroy(); ha.destroy(); hb.destroy(); A.destroy(); B.destroy(); C.destroy();
    }
    {   // softmax chain against the CPU pieces in the corrected order
        const int64_t rows = 33, cols = 1000;
        auto p = softmaxProgram();
        Runner run(p.program);
        run.compile();
        impl::MatrixGPU in(rows, cols), out(rows, cols);
        impl::MatrixCPU h(rows, cols, cols);
        std::mt19937 gen(0);
        std::normal_distribution<float> dist(0.f, 3.f);
        for (int64_t i = 0; i < rows * cols; i++) h.data[i] = dist(gen);
        in.put(h);
        run.evaluate({{"input", &in}, {"output", &out}});
        auto got = out.get();
        double worst = 0;
        for (int64_t i = 0; i < rows; i++) {
            float m = h(i, 0);
            for (int64_t j = 1; j < cols; j++) m = std::fmax(m, h(i, j));
            double sum = 0;
            for (int64_t j = 0; j < cols; j++) sum += std::exp(double(h(i, j)) - m);
            for (int64_t j = 0; j < cols; j++) {
                const double want = std::exp(double(h(i, j)) - m) / sum;
                worst = std::fmax(worst, std::fabs(got(i, j) - want) / std::fmax(want, 1e-30));
            }
        }
        CHECK(worst <= 1e-5);
        got.destroy(); h.destroy(); in.destroy(); out.destroy();
    }
    {   // bf16 matmul and the fused chain: small-integer operands are exact in bf16
        const int64_t m = 128, n = 256, k = 64;
        auto p = mmProgram(Datatype::BFloat16);
        Runner run(p.program);
        run.compile();
        impl::MatrixGPU A(m, k, k, Datatype::BFloat16), B(n, k, k, Datatype::BFloat16), C(m, n, n, Datatype::BFloat16);
        std::vector<uint16_t> ha(m * k), hb(n * k), hc(m * n);
        auto bf = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); return static_cast<uint16_t>(u >> 16); };
        auto fl = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; };
        for (int64_t i = 0; i < m * k; i++) ha[i] = bf(static_cast<float>(int(i % 7) - 3));
        for (int64_t i = 0; i < n * k; i++) hb[i] = bf(static_cast<float>(int(i % 5) - 2));
        A.put_raw(ha.data()); B.put_raw(hb.data());
        run.evaluate({{"A", &A}, {"B", &B}, {"C", &C}});
        C.get_raw(hc.data());
        bool exact = true;
        for (int64_t i = 0; i < m; i++)
            for (int64_t j = 0; j < n; j++) {
                float sum = 0.f;
                for (int64_t kk = 0; kk < k; kk++) sum += fl(ha[i * k + kk]) * fl(hb[j * k + kk]);
                exact = exact && fl(hc[i * n + j]) == sum;
            }
        CHECK(exact);
        // Global({{CLUSTER_DIM_X, c}}) steers the launch: c = 1 the single-CTA kernel, c = 2 CTA pairs;
        // both produce the same exact product
        for (int64_t c : {1, 2}) {
            Variable bx("bx"), cx("cx");
            annot::MatrixMultiply mm;
            Composable pinned = {Global((Tile(p.C["row"], bx.bind(128)) || Grid::BLOCK_X)(mm(p.A, p.B, p.C)),
                                        {{Grid::CLUSTER_DIM_X, cx.bind(c)}})};
            Runner rc(pinned);
            rc.compile();
            CHECK(rc.clusterX() == c && rc.resources().cluster_x == c);
            std::vector<uint16_t> hz(m * n, 0x7fc0), hc2(m * n);
            C.put_raw(hz.data());
            rc.evaluate({{"A", &A}, {"B", &B}, {"C", &C}});
            C.get_raw(hc2.data());
            CHECK(hc2 == hc);
        }
        A.destroy(); B.destroy(); C.destroy();
    }
    {   // exp(0.25 * A B - m) with row sums, against a CPU loop on the same small integers
        const int64_t m = 160, n = 300, k = 64;
        auto p = epilogueProgram(0.25f);
        Runner run(p.program);
        run.compile();
        const Datatype bfd = Datatype::BFloat16;
        impl::MatrixGPU A(m, k, k, bfd), B(n, k, k, bfd), E(m, n, 304, bfd);
        impl::ArrayGPU sub(m), sum(m);
        std::vector<uint16_t> ha(m * k), hb(n * k), he(m * 304);
        std::vector<float> hsub(m);
        auto bf = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); return static_cast<uint16_t>(u >> 16); };
        auto fl = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; };
        for (int64_t i = 0; i < m * k; i++) ha[i] = bf(static_cast<float>(int(i % 3) - 1));
        for (int64_t i = 0; i < n * k; i++) hb[i] = bf(static_cast<float>(int(i % 5) - 2));
        for (int64_t i = 0; i < m; i++) hsub[i] = 0.5f * static_cast<float>(i % 7);
        A.put_raw(ha.data()); B.put_raw(hb.data()); sub.put(hsub);
        run.evaluate({{"A", &A}, {"B", &B}, {"E", &E}, {"m", &sub}, {"s", &sum}});
        E.get_raw(he.data());
        const std::vector<float> hsum = sum.get();
        bool ok = true;
        for (int64_t i = 0; i < m; i++) {
            float rs = 0.f;
            for (int64_t j = 0; j < n; j++) {
                float acc = 0.f;
                for (int64_t kk = 0; kk < k; kk++) acc += fl(ha[i * k + kk]) * fl(hb[j * k + kk]);
                const float want = std::exp(0.25f * acc - hsub[i]);
                rs += want;
                ok = ok && std::fabs(fl(he[i * 304 + j]) - want) <= 0.01f * want + 1e-6f;
            }
            ok = ok && std::fabs(hsum[i] - rs) <= 1e-3f * rs;
        }
        CHECK(ok);
        A.destroy(); B.destroy(); E.destroy(); sub.destroy(); sum.destroy();
    }
    {   // fused chain with all-zero Q: uniform weights, O = column means of V
        const int64_t nq = 128, nkv = 256, d = 128;
        auto p = attentionProgram(1.0f);
        Runner run(p.program);
        run.compile();
        const Datatype bfd = Datatype::BFloat16;
        impl::MatrixGPU Q(nq, d, d, bfd), K(nkv, d, d, bfd), V(nkv, d, d, bfd), O(nq, d, d, bfd);
        std::vector<uint16_t> hq(nq * d, 0), hk(nkv * d), hv(nkv * d), ho(nq * d);
        auto bf = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); return static_cast<uint16_t>(u >> 16); };
        auto fl = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; };
        for (int64_t i = 0; i < nkv * d; i++) {
            hk[i] = bf(static_cast<float>(int(i % 3) - 1));
            hv[i] = bf(static_cast<float>(int((i / d) % 4)));
        }
        Q.put_raw(hq.data()); K.put_raw(hk.data()); V.put_raw(hv.data());
        run.evaluate({{"Q", &Q}, {"K", &K}, {"V", &V}, {"O", &O}});
        O.get_raw(ho.data());
        bool ok = true;
        for (int64_t i = 0; i < nq * d; i++) ok = ok && std::fabs(fl(ho[i]) - 1.5f) < 0.02f;
        CHECK(ok);
        {   // the same chain pinned to CTA pairs: the kernel for clusters of two, same bits
            Composable pinned = {Global(p.program.get()->children[0], {{Grid::CLUSTER_DIM_X, Variable("cx").bind(2)}})};
            Runner rp(pinned);
            rp.compile();
            CHECK(rp.kernelName() == "attention_bf16_pair" && rp.resources().cluster_x == 2);
            std::vector<uint16_t> ho2(nq * d, 0);
            O.put_raw(ho2.data());
            rp.evaluate({{"Q", &Q}, {"K", &K}, {"V", &V}, {"O", &O}});
            O.get_raw(ho2.data());
            CHECK(ho2 == ho);
        }
        Q.destroy(); K.destroy(); V.destroy(); O.destroy();
    }
}

int main(int argc, char **argv) {
    const std::string mode = argc > 1 ? argv[1] : "cpu";
    try {
        cpuTests();
        if (mode == "gpu") gpuTests();
    } catch (const std::exception &e) {
        std::printf("FAIL uncaught exception: %s\n", e.what());
        return 1;
    }
    if (failures == 0) std::printf("all host-layer checks passed (%s)\n", mode.c_str());
    return failures == 0 ? 0 : 1;
}
