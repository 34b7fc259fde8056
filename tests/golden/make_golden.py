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


def main():
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
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
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
