// Runs Gern's real CPU path for a tiled matrix multiply and dumps the result: builds the
// Composable  Tile(C.row,ti)(Tile(C.col,tj)(Reduce(k_dim,tk)(matrix_multiply)))  with the
// reference's own annotated function and ADTs, has Runner::compile lower it, shell out to g++
// and dlopen the hook, and calls Runner::evaluate on seeded inputs.  It is the producer of the
// matmul fixtures under tests/golden/ (see tests/golden/make_golden.py) and exists only where
// the reference tree is present.  Test infrastructure; links the reference's library objects.
//
//   gern_cpu_mm M N K ti tj tk {ascending|random} out.bin [O-flag]
//
// "random" is MatrixCPU::random_fill(-1, 1) for A and for B: the reference re-seeds
// std::mt19937(0) inside every call (test/library/matrix/impl/cpu-matrix.h:71-81), so A and B
// hold the same stream, which is the reference's own behaviour and is kept.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "compose/composable.h"
#include "compose/runner.h"
#include "config.h"
#include "library/matrix/annot/cpu-matrix.h"
#include "library/matrix/impl/cpu-matrix.h"

using namespace gern;

int main(int argc, char **argv) {
    if (argc < 9) {
        std::fprintf(stderr, "usage: %s M N K ti tj tk {ascending|random} out.bin [-O3]\n", argv[0]);
        return 2;
    }
    int64_t M = std::atoll(argv[1]), N = std::atoll(argv[2]), K = std::atoll(argv[3]);
    int64_t ti_val = std::atoll(argv[4]), tj_val = std::atoll(argv[5]), tk_val = std::atoll(argv[6]);
    const bool ascending = std::strcmp(argv[7], "ascending") == 0;
    const char *out_path = argv[8];
    const std::string oflag = argc > 9 ? argv[9] : "";

    auto A_DS = AbstractDataTypePtr(new const annot::MatrixCPU("A"));
    auto B_DS = AbstractDataTypePtr(new const annot::MatrixCPU("B"));
    auto C_DS = AbstractDataTypePtr(new const annot::MatrixCPU("C"));
    annot::MatrixMultiplyCPU matrix_multiply;
    Variable ti("ti"), tj("tj"), tk("tk"), k_dim("k_dim");

    Composable program = {
        (Tile(C_DS["row"], ti))(
            Tile(C_DS["col"], tj)(
                (Reduce(k_dim, tk))(
                    matrix_multiply(A_DS, B_DS, C_DS, k_dim))))};

    Runner run(program);
    Runner::Options o;
    o.filename = "gern_cpu_mm_golden.cpp";
    o.prefix = "/tmp";
    o.include = " " + oflag + " -I " + std::string(GERN_ROOT_DIR) + "/test/" +
                " -I " + std::string(GERN_ROOT_DIR) + "/test/library/matrix/impl";
    run.compile(o);

    impl::MatrixCPU a(M, K, K), b(K, N, N), c(M, N, N);
    if (ascending) {
        a.ascending();
        b.ascending();
    } else {
        a.random_fill(-1.0f, 1.0f);
        b.random_fill(-1.0f, 1.0f);
    }
    c.vvals(0.0f);
    int64_t k_dim_val = K;
    auto t0 = std::chrono::steady_clock::now();
    run.evaluate({
        {A_DS.getName(), &a},
        {B_DS.getName(), &b},
        {C_DS.getName(), &c},
        {ti.getName(), &ti_val},
        {tj.getName(), &tj_val},
        {tk.getName(), &tk_val},
        {k_dim.getName(), &k_dim_val},
    });
    auto t1 = std::chrono::steady_clock::now();
    std::fprintf(stderr, "evaluate: %.3f ms\n",
                 std::chrono::duration<double, std::milli>(t1 - t0).count());
    FILE *f = std::fopen(out_path, "wb");
    if (!f) return 3;
    std::fwrite(c.data, sizeof(float), (size_t)(M * N), f);
    std::fclose(f);
    return 0;
}
