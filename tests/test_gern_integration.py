"""libgern_b200 behind the UNMODIFIED Gern front end: integration/gern/b200.h (annotations) and
gb200_host.h (run-time objects) are composed into Gern programs by integration/gern/run_program.cpp,
lowered by the reference's own Runner::compile (code generation, g++, dlopen) and run by
Runner::evaluate -- the flow of the reference's test/test-cpu-mm.cpp:13-83 with the library behind
the leaf function.

The driver links the reference's library objects, so it is built only where the Gern tree is present
(`make -C integration/gern`, also done by __graft_entry__.build()); the built binary travels with the
tree.  Without it these tests are skipped with that reason.  CPU part: every program is generated,
compiled, linked and loaded, and evaluate reaches the library, which reports that there is no
device.  GPU part: results against the oracle and the reference-made fixtures."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "integration", "_ref", "gern_b200_runner")

needs_runner = pytest.mark.skipif(not os.path.exists(RUNNER),
                                  reason="integration/_ref/gern_b200_runner not built (needs the Gern tree at build time)")


def run(space, program, *args, cwd):
    cmd = [RUNNER, "--repo", ROOT, space, program] + [str(a) for a in args]
    return subprocess.run(cmd, capture_output=True, text=True, cwd=cwd, timeout=600)


def have_gpu():
    import torch
    return torch.cuda.is_available()


PROGRAMS = {
    "blur": (lambda d: [40, 52, 8, d / "in.bin", d / "out.bin"], "gb200_host::blur3x3(", {"in.bin": (40 * 52, np.float32)}),
    "mm": (lambda d: [64, 64, 64, 32, 32, 32, d / "a.bin", d / "b.bin", d / "c.bin"], "gb200_host::matrix_multiply(",
           {"a.bin": (64 * 64, np.float32), "b.bin": (64 * 64, np.float32)}),
    "mm_bf16": (lambda d: [64, 64, 64, 32, 32, d / "a.bin", d / "b.bin", d / "c.bin"], "gb200_host::matrix_multiply_bf16(",
                {"a.bin": (64 * 64, np.uint16), "b.bin": (64 * 64, np.uint16)}),
    "softmax": (lambda d: [64, 64, 16, d / "in.bin", d / "out.bin"], "gb200_host::softmax_rows(", {"in.bin": (64 * 64, np.float32)}),
    "attention": (lambda d: [128, 256, 64, 0.125, d / "q.bin", d / "k.bin", d / "v.bin", d / "o.bin"], "gb200_host::attention(",
                  {"q.bin": (128 * 128, np.uint16), "k.bin": (256 * 128, np.uint16), "v.bin": (256 * 128, np.uint16)}),
}


@needs_runner
@pytest.mark.parametrize("program", sorted(PROGRAMS))
def test_runner_generates_compiles_and_loads_every_program(tmp_path, program):
    """No GPU needed: Runner::compile must succeed (the hook is generated, compiled against
    gb200_host.h, linked with -lgern_b200 and dlopen'ed) and evaluate must reach the library."""
    make_args, call, files = PROGRAMS[program]
    for name, (count, dtype) in files.items():
        np.zeros(count, dtype).tofile(tmp_path / name)
    res = run("host", program, *make_args(tmp_path), cwd=tmp_path)
    assert "compiled: /tmp/gern_b200_" + program + "_host.cpp" in res.stdout, res.stderr
    src = open(f"/tmp/gern_b200_{program}_host.cpp").read()
    assert call in src and 'extern "C"' in src and "hook_function_" in src
    assert '#include "gb200_host.h"' in src and '#include "gern_b200.h"' in src
    if have_gpu():
        assert res.returncode == 0, res.stderr
    else:
        # the library is reached and refuses loudly: GB200_ERR_NO_DEVICE, never a CPU fallback
        assert res.returncode == 4
        assert "status -4" in res.stderr and "no CUDA device" in res.stderr


@needs_runner
def test_softmax_annotation_puts_its_whole_row_assumption_into_the_emitted_code(tmp_path):
    """The RowSoftmax annotation assumes l_y == output.col; Gern prints the assumption as an assert
    at the top of the generated function."""
    np.zeros(64 * 64, np.float32).tofile(tmp_path / "in.bin")
    run("host", "softmax", 64, 64, 16, tmp_path / "in.bin", tmp_path / "out.bin", cwd=tmp_path)
    src = open("/tmp/gern_b200_softmax_host.cpp").read()
    assert "assert((output.col == output.col))" in src.replace("  ", " ")


# ---------------------------------------------------------------------------------------------
gpu = pytest.mark.gpu


@needs_runner
@gpu
@pytest.mark.parametrize("space", ["host", "device"])
@pytest.mark.parametrize("rows,cols,band", [(514, 1030, 0), (514, 1030, 128), (66, 70, 16)])
def test_blur_through_gern_matches_the_oracle(tmp_path, oracle, space, rows, cols, band):
    x = np.random.default_rng(rows + cols).random((rows, cols), dtype=np.float32)
    x.tofile(tmp_path / "in.bin")
    res = run(space, "blur", rows, cols, band, tmp_path / "in.bin", tmp_path / "out.bin", cwd=tmp_path)
    assert res.returncode == 0, res.stderr
    got = np.fromfile(tmp_path / "out.bin", np.float32).reshape(rows - 2, cols - 2)
    assert np.array_equal(got, oracle.blur_xy(x))


@needs_runner
@gpu
@pytest.mark.parametrize("space", ["host", "device"])
def test_fp32_matmul_512_through_gern_matches_gerns_cpu_path(tmp_path, golden, space):
    """Configuration 0 (512^3, A = B = random_fill(-1, 1)), tiled 256 / 256 / 256 under Gern's
    Tile / Reduce, against the fixture Gern's own CPU path produced (tiles 64 / 64 / 64): the
    apps' bar |delta| < 1e-3 (gernels/mm/float-error.h) and relative Frobenius error < 1e-5."""
    from oracle import pyoracle
    a = pyoracle.mt19937_uniform(512 * 512, -1.0, 1.0).reshape(512, 512)
    a.tofile(tmp_path / "a.bin")
    res = run(space, "mm", 512, 512, 512, 256, 256, 256, tmp_path / "a.bin", tmp_path / "a.bin", tmp_path / "c.bin", cwd=tmp_path)
    assert res.returncode == 0, res.stderr
    c = np.fromfile(tmp_path / "c.bin", np.float32).reshape(512, 512)
    want = golden["mm512_sub"]
    got = c[::8, ::8]
    assert np.abs(got - want).max() < 1e-3
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5
    assert abs(c.astype(np.float64).sum() - float(golden["mm512_sum"])) < 1e-3 * 512


@needs_runner
@gpu
def test_bf16_matmul_softmax_and_chain_through_gern(tmp_path, oracle, golden, golden_maker):
    from oracle import pyoracle
    a, b = golden_maker.bf16_inputs("gemm512")
    a.tofile(tmp_path / "a.bin")
    b.tofile(tmp_path / "b.bin")
    res = run("device", "mm_bf16", 512, 512, 512, 256, 256, tmp_path / "a.bin", tmp_path / "b.bin", tmp_path / "c.bin", cwd=tmp_path)
    assert res.returncode == 0, res.stderr
    c = pyoracle.bf16_bits_to_f32(np.fromfile(tmp_path / "c.bin", np.uint16).reshape(512, 512))
    want = golden["gemmbf512_sub"]
    assert np.linalg.norm(c[::8, ::8] - want) / np.linalg.norm(want) <= 3e-3

    x = (np.random.default_rng(5).standard_normal((256, 4096)) * 3).astype(np.float32)
    x.tofile(tmp_path / "in.bin")
    res = run("device", "softmax", 256, 4096, 64, tmp_path / "in.bin", tmp_path / "out.bin", cwd=tmp_path)
    assert res.returncode == 0, res.stderr
    got = np.fromfile(tmp_path / "out.bin", np.float32).reshape(256, 4096)
    ref = oracle.softmax_rows(x)
    assert (np.abs(got.astype(np.float64) - ref) / np.maximum(ref, 1e-30)).max() <= 1e-5

    q, k, v = golden_maker.bf16_inputs("attn")
    for name, t in (("q.bin", q), ("k.bin", k), ("v.bin", v)):
        t.tofile(tmp_path / name)
    res = run("host", "attention", 64, 256, 32, golden_maker.ATTN_SCALE, tmp_path / "q.bin", tmp_path / "k.bin",
              tmp_path / "v.bin", tmp_path / "o.bin", cwd=tmp_path)
    assert res.returncode == 0, res.stderr
    o = pyoracle.bf16_bits_to_f32(np.fromfile(tmp_path / "o.bin", np.uint16).reshape(64, 128))
    assert np.linalg.norm(o - golden["attn_o"]) / np.linalg.norm(golden["attn_o"]) <= 1e-2


# ---------------------------------------------------------------------------------------------
# Pattern substitution: programs written against the reference's OWN annotation headers.
# `substitute`: the program is rewritten by gern::b200::substitute() and handed to the unmodified
# Runner.  `patched`: the ORIGINAL program is handed to a Runner built from the reference's
# runner.cpp plus integration/gern/runner_substitute.patch, which rewrites it inside
# Runner::compile and adds the library's include and link flags itself.
DEMOS = {"substitute": (os.path.join(ROOT, "integration", "_ref", "gern_b200_substitute"), "gern_b200_substituted_"),
         "patched": (os.path.join(ROOT, "integration", "_ref", "gern_b200_patched"), "gern_b200_patched_")}
SUBSTITUTED = {"blur": ("blur3x3", "gb200_host::blur3x3(input, output)"),
               "mm_cpu": ("matrix_multiply", "gb200_host::matrix_multiply(A, B, C, k_dim)"),
               "softmax": ("softmax_rows", "gb200_host::softmax_rows(input, output)")}


def run_demo(how, what, cwd):
    binary = DEMOS[how][0]
    if not os.path.exists(binary):
        pytest.skip(f"{os.path.relpath(binary, ROOT)} not built (needs the Gern tree at build time)")
    return subprocess.run([binary, "--repo", ROOT, what], capture_output=True, text=True, cwd=cwd, timeout=600)


@pytest.mark.parametrize("how", sorted(DEMOS))
@pytest.mark.parametrize("what", sorted(SUBSTITUTED))
def test_reference_programs_are_rewritten_onto_the_library(tmp_path, what, how):
    """The blur program of apps/blur/blur.cpp:46-73, the tiled matmul of test/test-cpu-mm.cpp:13-83 and
    the five softmax pieces of apps/common/annot/functions.h, built with the reference's own
    annotation classes, are recognised by gern::b200::substitute() -- called by the demo, or by the
    patched Runner::compile (src/codegen/runner.cpp:11) -- and the generated hook is one call into
    the library.  The patched Runner::evaluate also takes the tile sizes the original schedule's
    caller passes (the matmul demo passes ti, tj, tk) and ignores them."""
    kernel, call = SUBSTITUTED[what]
    res = run_demo(how, what, tmp_path)
    generated = f"/tmp/{DEMOS[how][1]}{what}.cpp"
    assert f"matched: {kernel}" in res.stdout, res.stdout + res.stderr
    assert f"compiled: {generated}" in res.stdout, res.stderr
    src = open(generated).read()
    assert call in src and "for(" not in src        # one library call, the schedule's loops are gone
    if have_gpu():
        assert res.returncode == 0 and "evaluated: result as expected" in res.stdout, res.stderr
    else:
        assert res.returncode == 4 and "status -4" in res.stderr and "no CUDA device" in res.stderr


@pytest.mark.parametrize("how", sorted(DEMOS))
def test_programs_without_a_fused_kernel_are_left_alone(tmp_path, how):
    res = run_demo(how, "unmatched", tmp_path)      # blur with stride 5
    assert res.returncode == 0 and "matched: none" in res.stdout


def test_the_runner_patch_applies_to_the_reference_source(tmp_path):
    """runner_substitute.patch is a unified diff of src/codegen/runner.cpp; it has to apply cleanly
    to the tree the oracle was built from, and everything it adds sits under GERN_B200_ROOT."""
    from oracle import pyoracle
    ref = pyoracle.find_reference()
    if ref is None:
        pytest.skip("no Gern tree here")
    import shutil
    os.makedirs(tmp_path / "src" / "codegen")
    shutil.copy(os.path.join(ref, "src", "codegen", "runner.cpp"), tmp_path / "src" / "codegen" / "runner.cpp")
    patch = os.path.join(ROOT, "integration", "gern", "runner_substitute.patch")
    res = subprocess.run(["patch", "-p1", "--dry-run", "-i", patch], cwd=tmp_path, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    added = [l[1:] for l in open(patch) if l.startswith("+") and not l.startswith("+++")]
    depth = 0
    for line in added:
        if line.startswith("#ifdef GERN_B200_ROOT"):
            depth += 1
        elif line.startswith("#endif"):
            depth -= 1
        else:
            assert depth == 1 or not line.strip(), line


@gpu
@pytest.mark.parametrize("how", sorted(DEMOS))
@pytest.mark.parametrize("what", sorted(SUBSTITUTED))
def test_substituted_programs_evaluate_on_the_gpu(tmp_path, what, how):
    res = run_demo(how, what, tmp_path)
    assert res.returncode == 0 and "evaluated: result as expected" in res.stdout, res.stdout + res.stderr
