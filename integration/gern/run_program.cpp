// Drives libgern_b200 through the UNMODIFIED Gern front end: builds a Composable from the
// annotations of b200.h, has gern::Runner::compile lower it, shell out to g++ and dlopen the hook
// (src/codegen/runner.cpp:11-55), and calls Runner::evaluate (runner.cpp:57-80) on matrices read
// from files.  The shape of test/test-cpu-mm.cpp:13-83 with the library behind the leaf.
//
//   gern_b200_runner --repo <root of this repository> <space> <program> <sizes...> <in...> <out>
//     space    host   : operands stay in host memory (gb200_host::HostMatrix, `_host` entry points)
//              device : operands are copied to device memory first (gb200_host::Matrix)
//     program  blur rows cols band in.bin out.bin          Tile(out.row, band)(Blur3x3); band 0 = untiled
//              mm M N K ti tj tk a.bin b.bin c.bin          Tile(C.row,ti)(Tile(C.col,tj)(Reduce(k_dim,tk)(mm)))
//              mm_bf16 M N K ti tj a.bin b.bin c.bin        Tile(C.row,ti)(Tile(C.col,tj)(mm_bf16)), B as N x K
//              softmax rows cols band in.bin out.bin        Tile(out.row, band)(RowSoftmax)
//              attention nq nkv band scale q.bin k.bin v.bin o.bin   Tile(O.row, band)(Attention), d = 128
//   exit status: 0 ok, 2 usage, 3 Runner::compile failed, 4 evaluate failed (the library's message
//   is printed: without a GPU that is "no CUDA device", status -4)
//
// Links the reference's library objects (built from the Gern tree where it lies); exists only
// where that tree is present at build time.  The hook it compiles at run time includes only
// gern_b200.h and gb200_host.h, so the built driver also runs where the Gern tree is absent.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "b200.h"
#include "compose/composable.h"
#include "compose/runner.h"
#include "gb200_host.h"

using namespace gern;

namespace {

std::vector<char> read_file(const std::string &path, size_t bytes) {
    std::vector<char> buf(bytes);
    FILE *f = std::fopen(path.c_str(), "rb");
    if (!f || std::fread(buf.data(), 1, bytes, f) != bytes) {
        std::fprintf(stderr, "cannot read %zu bytes from %s\n", bytes, path.c_str());
        std::exit(2);
    }
    std::fclose(f);
    return buf;
}

void write_file(const std::string &path, const void *data, size_t bytes) {
    FILE *f = std::fopen(path.c_str(), "wb");
    if (!f || std::fwrite(data, 1, bytes, f) != bytes) {
        std::fprintf(stderr, "cannot write %s\n", path.c_str());
        std::exit(2);
    }
    std::fclose(f);
}

// One operand: host bytes plus, in device space, a device copy; `view` is what evaluate() gets
// (all four gb200_host matrix types share the layout {pointer, row, col, lda}).
struct Operand {
    std::vector<char> host;
    void *dev = nullptr;
    gb200_host::MatrixT<char, false> view;
    size_t elem = 4;

    void init(bool device, std::vector<char> bytes, int64_t rows, int64_t cols, size_t elem_size) {
        host = std::move(bytes);
        elem = elem_size;
        void *p = host.data();
        if (device) {
            if (cudaMalloc(&dev, host.size() ? host.size() : 16) != cudaSuccess ||
                cudaMemcpy(dev, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
                std::fprintf(stderr, "evaluate failed: cannot place an operand in device memory: %s\n",
                             cudaGetErrorString(cudaGetLastError()));
                std::exit(4);
            }
            p = dev;
        }
        view = gb200_host::MatrixT<char, false>(static_cast<char *>(p), rows, cols, cols);
    }
    void fetch() {
        if (dev && cudaMemcpy(host.data(), dev, host.size(), cudaMemcpyDeviceToHost) != cudaSuccess) {
            std::fprintf(stderr, "evaluate failed: %s\n", cudaGetErrorString(cudaGetLastError()));
            std::exit(4);
        }
    }
};

}  // namespace

int main(int argc, char **argv) {
    std::vector<std::string> a(argv + 1, argv + argc);
    if (a.size() < 4 || a[0] != "--repo") {
        std::fprintf(stderr, "usage: %s --repo <root> {host|device} <program> <sizes...> <files...>\n", argv[0]);
        return 2;
    }
    const std::string repo = a[1];
    const bool device = a[2] == "device";
    const std::string prog = a[3];
    auto num = [&](size_t i) { return (int64_t)std::atoll(a.at(i).c_str()); };
    const char *cuda = std::getenv("CUDA_HOME") ? std::getenv("CUDA_HOME") : "/usr/local/cuda";

    Runner::Options o;
    o.filename = "gern_b200_" + prog + "_" + a[2] + ".cpp";
    o.prefix = "/tmp";
    o.cpp_std = "c++17";
    o.include = " -O2 -I " + repo + "/integration/gern -I " + repo + "/include -I " + cuda + "/include";
    o.ldflags = "-L " + repo + "/gern_b200 -lgern_b200 -Wl,-rpath," + repo + "/gern_b200 -L " + cuda +
                "/lib64 -lcudart";
    auto f32 = [&](const std::string &n) { return device ? annot::b200::device_f32(n) : annot::b200::host_f32(n); };
    auto b16 = [&](const std::string &n) { return device ? annot::b200::device_bf16(n) : annot::b200::host_bf16(n); };

    std::map<std::string, void *> args;
    std::vector<Operand> ops(4);
    std::vector<int64_t> ints(8);
    float scale = 1.0f;
    Composable program;
    std::string out_path;
    int out_index = 0;
    try {
        if (prog == "blur" && a.size() == 9) {
            const int64_t rows = num(4), cols = num(5);
            ints[0] = num(6);
            auto in = f32("input"), out = f32("output");
            annot::b200::Blur3x3 blur(in, out);
            Variable band("band");
            program = ints[0] > 0 ? Composable(Tile(out["row"], band)(blur(in, out))) : Composable(blur(in, out));
            ops[0].init(device, read_file(a[7], (size_t)rows * cols * 4), rows, cols, 4);
            ops[1].init(device, std::vector<char>((size_t)(rows - 2) * (cols - 2) * 4), rows - 2, cols - 2, 4);
            args = {{"input", &ops[0].view}, {"output", &ops[1].view}};
            if (ints[0] > 0) args["band"] = &ints[0];
            out_path = a[8];
            out_index = 1;
        } else if (prog == "mm" && a.size() == 13) {
            const int64_t M = num(4), N = num(5), K = num(6);
            ints[0] = num(7), ints[1] = num(8), ints[2] = num(9), ints[3] = K;
            auto A = f32("A"), B = f32("B"), C = f32("C");
            annot::b200::MatrixMultiply mm(A, B, C);
            Variable ti("ti"), tj("tj"), tk("tk"), k_dim("k_dim");
            program = Composable(Tile(C["row"], ti)(Tile(C["col"], tj)(Reduce(k_dim, tk)(mm(A, B, C, k_dim)))));
            ops[0].init(device, read_file(a[10], (size_t)M * K * 4), M, K, 4);
            ops[1].init(device, read_file(a[11], (size_t)K * N * 4), K, N, 4);
            ops[2].init(device, std::vector<char>((size_t)M * N * 4), M, N, 4);      // C starts at zero
            args = {{"A", &ops[0].view}, {"B", &ops[1].view}, {"C", &ops[2].view},
                    {"ti", &ints[0]}, {"tj", &ints[1]}, {"tk", &ints[2]}, {"k_dim", &ints[3]}};
            out_path = a[12];
            out_index = 2;
        } else if (prog == "mm_bf16" && a.size() == 12) {
            const int64_t M = num(4), N = num(5), K = num(6);
            ints[0] = num(7), ints[1] = num(8), ints[3] = K;
            auto A = b16("A"), B = b16("B"), C = b16("C");
            annot::b200::MatrixMultiply mm(A, B, C, true);
            Variable ti("ti"), tj("tj"), k_dim("k_dim");
            program = Composable(Tile(C["row"], ti)(Tile(C["col"], tj)(mm(A, B, C, k_dim))));
            ops[0].init(device, read_file(a[9], (size_t)M * K * 2), M, K, 2);
            ops[1].init(device, read_file(a[10], (size_t)N * K * 2), N, K, 2);
            ops[2].init(device, std::vector<char>((size_t)M * N * 2), M, N, 2);
            args = {{"A", &ops[0].view}, {"B", &ops[1].view}, {"C", &ops[2].view},
                    {"ti", &ints[0]}, {"tj", &ints[1]}, {"k_dim", &ints[3]}};
            out_path = a[11];
            out_index = 2;
        } else if (prog == "softmax" && a.size() == 9) {
            const int64_t rows = num(4), cols = num(5);
            ints[0] = num(6), ints[1] = 0, ints[2] = cols;
            auto in = f32("input"), out = f32("output");
            annot::b200::RowSoftmax sm(in, out);
            Variable band("band");
            program = Composable(Tile(out["row"], band)(sm(in, out)));
            ops[0].init(device, read_file(a[7], (size_t)rows * cols * 4), rows, cols, 4);
            ops[1].init(device, std::vector<char>((size_t)rows * cols * 4), rows, cols, 4);
            args = {{"input", &ops[0].view}, {"output", &ops[1].view}, {"band", &ints[0]}};
            out_path = a[8];
            out_index = 1;
        } else if (prog == "attention" && a.size() == 12) {
            const int64_t nq = num(4), nkv = num(5), d = 128;
            ints[0] = num(6), ints[1] = 0, ints[2] = d, ints[3] = nkv;
            scale = (float)std::atof(a[7].c_str());
            auto Q = b16("Q"), K = b16("K"), V = b16("V"), O = b16("O");
            annot::b200::Attention att(Q, K, V, O);
            Variable band("band"), sc("scale", Datatype::Float32);
            program = Composable(Tile(O["row"], band)(att(Q, K, V, O, sc)));
            ops[0].init(device, read_file(a[8], (size_t)nq * d * 2), nq, d, 2);
            ops[1].init(device, read_file(a[9], (size_t)nkv * d * 2), nkv, d, 2);
            ops[2].init(device, read_file(a[10], (size_t)nkv * d * 2), nkv, d, 2);
            ops[3].init(device, std::vector<char>((size_t)nq * d * 2), nq, d, 2);
            args = {{"Q", &ops[0].view}, {"K", &ops[1].view}, {"V", &ops[2].view}, {"O", &ops[3].view},
                    {"band", &ints[0]}, {"scale", &scale}};
            out_path = a[11];
            out_index = 3;
        } else {
            std::fprintf(stderr, "unknown program or wrong number of arguments: %s\n", prog.c_str());
            return 2;
        }
    } catch (const std::exception &e) {
        std::fprintf(stderr, "building the program failed: %s\n", e.what());
        return 3;
    }

    Runner run(program);
    try {
        run.compile(o);
    } catch (const std::exception &e) {
        std::fprintf(stderr, "Runner::compile failed: %s\n", e.what());
        return 3;
    }
    std::printf("compiled: %s/%s\n", o.prefix.c_str(), o.filename.c_str());
    // Matrix views are measured in elements: give each its element type's row pitch.
    for (auto &op : ops) {
        if (!op.view.data) continue;
        op.view.lda = op.view.col;
    }
    try {
        run.evaluate(args);
        if (device) gb200_host::sync();
    } catch (const std::exception &e) {
        std::fprintf(stderr, "evaluate failed: %s\n", e.what());
        return 4;
    }
    ops[out_index].fetch();
    write_file(out_path, ops[out_index].host.data(), ops[out_index].host.size());
    std::printf("evaluated: wrote %s\n", out_path.c_str());
    return 0;
}
