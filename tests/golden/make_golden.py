"""Generates tests/golden/golden.npz from the reference itself.  Run only where the reference tree
is present and oracle/_ref has been built (`make -C oracle ref`):

    python tests/golden/make_golden.py [/path/to/reference]

What it records (all produced by the reference's own code, none by this repository's oracle):
  * mm10_c            Gern's real CPU path (Composable -> Runner::compile(g++) -> evaluate) on the
                      10x10 ascending matmul of test/test-cpu-mm.cpp:13-83, tiles 5/5/5
  * mm64_c            same path, 64^3, A = B = MatrixCPU::random_fill(-1,1), tiles 16/16/16
  * mm512_sub, mm512_sum   same path at 512^3 with tiles 64/64/64 (every 8th row and column of C,
                      and the fp64 sum of all of C); the hook is compiled with the reference's
                      default flags (no -O)
  * fill32            first 32 values of random_fill(-1,1)
  * blur_in/blur_out  cpu_blur_x then cpu_blur_y (apps/blur/blur.cpp:11-25) on an ascending 20x24
                      image (the app's own check uses ascending input) and on a random 37x70 one
  * sm_*              the five softmax pieces of test/library/matrix/impl/cpu-matrix.h:134-194 on a
                      random 5x33 matrix, exactly as the reference computes them
  * gemmbf96_c, gemmbf512_sub, gemmbf512_sum
                      gern::impl::matrix_multiply (cpu-matrix.h:196-212) on bf16-rounded operands
                      widened to fp32: a 96 x 80 x 64 case in full, and a 512^3 case as every 8th
                      row and column plus the fp64 sum.  The operands are bf16_inputs() below
  * attn_o            the chain matrix_multiply -> max_row -> subtract_vec (negated) -> exp_matrix
                      -> sum_row -> divide_vec -> matrix_multiply of the same header on bf16-rounded
                      Q (64 x 128), K, V (256 x 128), the shape of the reference's chained-GEMM test
                      with a per-tile temporary (test/test-cpu-mm.cpp:266-336).  The scale 1/8 is a
                      power of two and is applied to Q before the first product, which is exact
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pyoracle  # noqa: E402


def run_gern_cpu_mm(m, n, k, ti, tj, tk, fill, oflag=None):
    with tempfile.NamedTemporaryFile(suffix=".bin") as f:
        cmd = [pyoracle.REF_MM_DRIVER] + [str(v) for v in (m, n, k, ti, tj, tk)] + [fill, f.name]
        if oflag:
            cmd.append(oflag)
        subprocess.run(cmd, check=True)
        return np.fromfile(f.name, dtype=np.float32).reshape(m, n)


def bf16_inputs(tag):
    """Operands of the bf16 fixtures as bf16 bit patterns.  They come from the reference's own
    random_fill stream (std::mt19937(0)), which pyoracle.mt19937_uniform rebuilds without the
    reference, so the tests regenerate them instead of storing them."""
    u = pyoracle.mt19937_uniform
    if tag == "gemm96":       # A 96 x 64 row-major, B as 80 rows of K = 64 (column-major B)
        s = u(96 * 64 + 80 * 64, -1.0, 1.0)
        return pyoracle.to_bf16_bits(s[: 96 * 64].reshape(96, 64)), pyoracle.to_bf16_bits(s[96 * 64:].reshape(80, 64))
    if tag == "gemm512":
        s = u(2 * 512 * 512, -1.0, 1.0) * np.float32(0.25)
        return (pyoracle.to_bf16_bits(s[: 512 * 512].reshape(512, 512)),
                pyoracle.to_bf16_bits(s[512 * 512:].reshape(512, 512)))
    if tag == "attn":         # Q 64 x 128, K and V 256 x 128
        s = u(64 * 128 + 2 * 256 * 128, -2.0, 2.0)
        q = s[: 64 * 128].reshape(64, 128)
        k = s[64 * 128: 64 * 128 + 256 * 128].reshape(256, 128)
        v = s[64 * 128 + 256 * 128:].reshape(256, 128)
        return tuple(pyoracle.to_bf16_bits(t) for t in (q, k, v))
    raise KeyError(tag)


ATTN_SCALE = 0.125


def reference_bf16_fixtures(ref):
    """bf16 GEMM and the GEMM -> softmax -> GEMM chain, computed by the reference's CPU leaves."""
    f32 = lambda bits: np.ascontiguousarray(pyoracle.bf16_bits_to_f32(bits))
    out = {}
    a, b = bf16_inputs("gemm96")
    out["gemmbf96_c"] = ref.matrix_multiply(f32(a), np.ascontiguousarray(f32(b).T))
    a, b = bf16_inputs("gemm512")
    c = ref.matrix_multiply(f32(a), np.ascontiguousarray(f32(b).T))
    out["gemmbf512_sub"] = np.ascontiguousarray(c[::8, ::8])
    out["gemmbf512_sum"] = np.array(c.astype(np.float64).sum())
    q, k, v = (f32(t) for t in bf16_inputs("attn"))
    s = ref.matrix_multiply(np.ascontiguousarray(q * np.float32(ATTN_SCALE)), np.ascontiguousarray(k.T))
    mx = ref.max_row(s)
    assert (mx > 0).all(), "the reference's max_row is seeded with FLT_MIN: rows need a positive maximum"
    e = ref.exp_matrix(np.ascontiguousarray(-ref.subtract_vec(mx, s)))       # exp(s - max)
    p = ref.divide_vec(ref.sum_row(e), e)
    out["attn_o"] = ref.matrix_multiply(p, v)
    return out


def main():
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else (pyoracle.find_reference() or "")
    if not os.path.isdir(os.path.join(ref_dir, "src")):
        raise SystemExit("usage: make_golden.py /path/to/reference  (or set GERN_REFERENCE_DIR)")
    pyoracle.build(ref_dir)
    ref = pyoracle.Reference()
    out = {}
    out["mm10_c"] = run_gern_cpu_mm(10, 10, 10, 5, 5, 5, "ascending")
    out["mm64_c"] = run_gern_cpu_mm(64, 64, 64, 16, 16, 16, "random")
    c512 = run_gern_cpu_mm(512, 512, 512, 64, 64, 64, "random")
    out["mm512_sub"] = np.ascontiguousarray(c512[::8, ::8])
    out["mm512_sum"] = np.array(c512.astype(np.float64).sum())
    out["fill32"] = ref.random_fill(1, 32, -1.0, 1.0).ravel()

    asc = np.arange(20 * 24, dtype=np.float32).reshape(20, 24)
    rnd = np.random.default_rng(7).random((37, 70), dtype=np.float32)
    out["blur_in_asc"], out["blur_out_asc"] = asc, ref.blur_xy(asc)
    out["blur_in_rnd"], out["blur_out_rnd"] = rnd, ref.blur_xy(rnd)

    x = (np.random.default_rng(11).standard_normal((5, 33)) * 3).astype(np.float32)
    out["sm_in"] = x
    out["sm_max"] = ref.max_row(x)
    out["sm_sub"] = ref.subtract_vec(out["sm_max"], x)          # max - x, as the reference does
    out["sm_exp"] = ref.exp_matrix(-out["sm_sub"])              # exp(x - max)
    out["sm_sum"] = ref.sum_row(out["sm_exp"])
    out["sm_div"] = ref.divide_vec(out["sm_sum"], out["sm_exp"])
    out.update(reference_bf16_fixtures(ref))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
