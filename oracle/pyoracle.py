"""ctypes doors onto the test oracle (oracle/libgern_oracle.so) and, where it was built, the
reference's own compiled CPU code (oracle/_ref/libgern_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU
baseline / reference arm.  The library package never imports this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libgern_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libgern_ref.so")
REF_MM_DRIVER = os.path.join(HERE, "_ref", "gern_cpu_mm")

_i64 = ctypes.c_int64
_fp = ctypes.POINTER(ctypes.c_float)
_dp = ctypes.POINTER(ctypes.c_double)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def find_reference() -> str | None:
    """The reference's source tree: $GERN_REFERENCE_DIR, else a directory named `reference` beside
    this repository; None where neither holds the reference's src/."""
    for cand in (os.environ.get("GERN_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")):
            return cand
    return None


def build(reference_dir: str | None = None) -> None:
    """Compiles the restatement and, when a reference tree is given, oracle/_ref."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    if reference_dir and os.path.isdir(os.path.join(reference_dir, "src")):
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={reference_dir}"], check=True)


def _f(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_fp)


def _u16(a: np.ndarray):
    assert a.dtype == np.uint16 and a.flags.c_contiguous
    return a.ctypes.data_as(_u16p)


class Oracle:
    """The CPU restatement (oracle/gern_oracle.c)."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(None)
        self.lib = ctypes.CDLL(ORACLE_SO)
        L = self.lib
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        L.oracle_max_threads.restype = ctypes.c_int
        L.oracle_matrix_multiply.argtypes = [_fp, _i64, _fp, _i64, _fp, _i64, _i64, _i64, _i64]
        L.oracle_matmul_tiled.argtypes = [_fp, _i64, _fp, _i64, _fp, _i64] + [_i64] * 6
        L.oracle_blur_x.argtypes = [_fp, _i64, _fp, _i64, _i64, _i64]
        L.oracle_blur_y.argtypes = [_fp, _i64, _fp, _i64, _i64, _i64]
        L.oracle_blur_xy.argtypes = [_fp, _i64, _i64, _i64, _fp, _i64]
        L.oracle_blur_xy.restype = ctypes.c_int
        L.oracle_max_row_ref.argtypes = [_fp, _i64, _i64, _i64, _fp]
        L.oracle_sum_row.argtypes = [_fp, _i64, _i64, _i64, _fp]
        L.oracle_exp_matrix.argtypes = [_fp, _i64, _i64, _i64, _fp, _i64]
        L.oracle_subtract_vec_ref.argtypes = [_fp, _fp, _i64, _i64, _i64, _fp, _i64]
        L.oracle_divide_vec.argtypes = [_fp, _fp, _i64, _i64, _i64, _fp, _i64]
        L.oracle_softmax_rows.argtypes = [_fp, _i64, _fp, _i64, _i64, _i64]
        L.oracle_softmax_rows_f64.argtypes = [_fp, _i64, _dp, _i64, _i64, _i64]
        L.oracle_gemm_bf16.argtypes = [_u16p, _i64, _u16p, _i64, _fp, _i64, _i64, _i64, _i64, _i64]
        L.oracle_attention_bf16.argtypes = [_u16p, _i64, _u16p, _i64, _u16p, _i64, _fp, _i64, _i64,
                                            _i64, ctypes.c_float, _i64, _i64]

    def set_threads(self, n: int) -> None:
        self.lib.oracle_set_threads(int(n))

    def max_threads(self) -> int:
        return int(self.lib.oracle_max_threads())

    def matrix_multiply(self, a, b, c=None):
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32) if c is None else c
        self.lib.oracle_matrix_multiply(_f(a), k, _f(b), n, _f(c), n, m, n, k)
        return c

    def matmul_tiled(self, a, b, ti, tj, tk, c=None):
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32) if c is None else c
        self.lib.oracle_matmul_tiled(_f(a), k, _f(b), n, _f(c), n, m, n, k, ti, tj, tk)
        return c

    def blur_x(self, x):
        r, c = x.shape
        out = np.empty((r, c - 2), np.float32)
        self.lib.oracle_blur_x(_f(x), c, _f(out), c - 2, r, c - 2)
        return out

    def blur_y(self, x):
        r, c = x.shape
        out = np.empty((r - 2, c), np.float32)
        self.lib.oracle_blur_y(_f(x), c, _f(out), c, r - 2, c)
        return out

    def blur_xy(self, x):
        r, c = x.shape
        out = np.empty((max(r - 2, 0), max(c - 2, 0)), np.float32)
        if out.size:
            rc = self.lib.oracle_blur_xy(_f(x), c, r, c, _f(out), c - 2)
            assert rc == 0
        return out

    def max_row_ref(self, a):
        out = np.empty(a.shape[0], np.float32)
        self.lib.oracle_max_row_ref(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out))
        return out

    def sum_row(self, a):
        out = np.empty(a.shape[0], np.float32)
        self.lib.oracle_sum_row(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out))
        return out

    def exp_matrix(self, a):
        out = np.empty_like(a)
        self.lib.oracle_exp_matrix(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out), a.shape[1])
        return out

    def subtract_vec_ref(self, vec, a):
        out = np.empty_like(a)
        self.lib.oracle_subtract_vec_ref(_f(vec), _f(a), a.shape[1], a.shape[0], a.shape[1], _f(out),
                                         a.shape[1])
        return out

    def divide_vec(self, vec, a):
        out = np.empty_like(a)
        self.lib.oracle_divide_vec(_f(vec), _f(a), a.shape[1], a.shape[0], a.shape[1], _f(out),
                                   a.shape[1])
        return out

    def softmax_rows(self, x):
        out = np.empty_like(x)
        if x.size:
            self.lib.oracle_softmax_rows(_f(x), x.shape[1], _f(out), x.shape[1], x.shape[0], x.shape[1])
        return out

    def softmax_rows_f64(self, x):
        out = np.empty(x.shape, np.float64)
        if x.size:
            self.lib.oracle_softmax_rows_f64(_f(x), x.shape[1], out.ctypes.data_as(_dp), x.shape[1],
                                             x.shape[0], x.shape[1])
        return out

    def gemm_bf16(self, a_bits, b_bits, row_begin=0, row_end=None):
        """a_bits: (M,K) uint16 bf16 bit patterns; b_bits: (N,K) (column-major B)."""
        m, k = a_bits.shape
        n = b_bits.shape[0]
        row_end = m if row_end is None else row_end
        out = np.empty((row_end - row_begin, n), np.float32)
        self.lib.oracle_gemm_bf16(_u16(a_bits), k, _u16(b_bits), k, _f(out), n, n, k, row_begin, row_end)
        return out

    def gemm_bf16_epilogue(self, a_bits, b_bits, alpha=1.0, row_sub=None, apply_exp=False, row_div=None):
        """The reference's leaves composed after the product, in the order the fused epilogue applies
        them: t = alpha * (A B); t - row_sub (the GPU leaf's direction, apps/common/impl/impl.h:53-78);
        exp_matrix (cpu-matrix.h:134-144); divide_vec (cpu-matrix.h:183-194).  Returns the fp32 matrix
        t, its row maxima (max_row without the reference's FLT_MIN seed, cpu-matrix.h:158-168) and its
        row sums (sum_row, cpu-matrix.h:146-156)."""
        t = self.gemm_bf16(a_bits, b_bits) * np.float32(alpha)
        if row_sub is not None:
            t = (t - np.asarray(row_sub, np.float32)[:, None]).astype(np.float32)
        if apply_exp:
            t = self.exp_matrix(np.ascontiguousarray(t))
        if row_div is not None:
            t = self.divide_vec(np.asarray(row_div, np.float32), np.ascontiguousarray(t))
        t = np.ascontiguousarray(t, dtype=np.float32)
        return t, t.max(axis=1), self.sum_row(t)

    def attention_bf16(self, q_bits, k_bits, v_bits, scale, row_begin=0, row_end=None):
        nq, d = q_bits.shape
        nkv = k_bits.shape[0]
        row_end = nq if row_end is None else row_end
        out = np.empty((row_end - row_begin, d), np.float32)
        self.lib.oracle_attention_bf16(_u16(q_bits), d, _u16(k_bits), d, _u16(v_bits), d, _f(out), d,
                                       nkv, d, ctypes.c_float(scale), row_begin, row_end)
        return out


class Reference:
    """The reference's own CPU functions, compiled from its sources (oracle/_ref)."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = ctypes.CDLL(REF_SO)
        L = self.lib
        L.ref_matrix_multiply.argtypes = [_fp, _i64, _fp, _i64, _fp, _i64, _i64, _i64, _i64]
        L.ref_matmul_tiled.argtypes = [_fp, _i64, _fp, _i64, _fp, _i64] + [_i64] * 6
        L.ref_blur_x.argtypes = [_fp, _i64, _fp, _i64, _i64, _i64]
        L.ref_blur_y.argtypes = [_fp, _i64, _fp, _i64, _i64, _i64]
        L.ref_max_row.argtypes = [_fp, _i64, _i64, _i64, _fp]
        L.ref_sum_row.argtypes = [_fp, _i64, _i64, _i64, _fp]
        L.ref_exp_matrix.argtypes = [_fp, _i64, _i64, _i64, _fp, _i64]
        L.ref_subtract_vec.argtypes = [_fp, _fp, _i64, _i64, _i64, _fp, _i64]
        L.ref_divide_vec.argtypes = [_fp, _fp, _i64, _i64, _i64, _fp, _i64]
        L.ref_random_fill.argtypes = [_fp, _i64, _i64, _i64, ctypes.c_float, ctypes.c_float]
        L.ref_ascending.argtypes = [_fp, _i64, _i64, _i64]

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def matrix_multiply(self, a, b, c=None):
        m, k = a.shape
        n = b.shape[1]
        c = np.zeros((m, n), np.float32) if c is None else c
        self.lib.ref_matrix_multiply(_f(a), k, _f(b), n, _f(c), n, m, n, k)
        return c

    def matmul_tiled(self, a, b, ti, tj, tk, c=None):
        m, k = a.shape
        n = b.shape[1]
        assert m % ti == 0 and n % tj == 0 and k % tk == 0, "the reference needs divisible tiles"
        c = np.zeros((m, n), np.float32) if c is None else c
        self.lib.ref_matmul_tiled(_f(a), k, _f(b), n, _f(c), n, m, n, k, ti, tj, tk)
        return c

    def blur_x(self, x):
        r, c = x.shape
        out = np.empty((r, c - 2), np.float32)
        self.lib.ref_blur_x(_f(x), c, _f(out), c - 2, r, c - 2)
        return out

    def blur_y(self, x):
        r, c = x.shape
        out = np.empty((r - 2, c), np.float32)
        self.lib.ref_blur_y(_f(x), c, _f(out), c, r - 2, c)
        return out

    def blur_xy(self, x):
        return self.blur_y(self.blur_x(x))

    def max_row(self, a):
        out = np.empty(a.shape[0], np.float32)
        self.lib.ref_max_row(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out))
        return out

    def sum_row(self, a):
        out = np.empty(a.shape[0], np.float32)
        self.lib.ref_sum_row(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out))
        return out

    def exp_matrix(self, a):
        out = np.empty_like(a)
        self.lib.ref_exp_matrix(_f(a), a.shape[1], a.shape[0], a.shape[1], _f(out), a.shape[1])
        return out

    def subtract_vec(self, vec, a):
        out = np.empty_like(a)
        self.lib.ref_subtract_vec(_f(vec), _f(a), a.shape[1], a.shape[0], a.shape[1], _f(out), a.shape[1])
        return out

    def divide_vec(self, vec, a):
        out = np.empty_like(a)
        self.lib.ref_divide_vec(_f(vec), _f(a), a.shape[1], a.shape[0], a.shape[1], _f(out), a.shape[1])
        return out

    def random_fill(self, rows, cols, lo=0.0, hi=1.0):
        out = np.empty((rows, cols), np.float32)
        self.lib.ref_random_fill(_f(out), cols, rows, cols, lo, hi)
        return out


def mt19937_uniform(n: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    """The stream MatrixCPU::random_fill(lo, hi) produces (std::mt19937(0) +
    std::uniform_real_distribution<float>, test/library/matrix/impl/cpu-matrix.h:71-81), rebuilt
    with numpy so that it needs neither the reference nor a C++ runtime: one 32-bit draw per
    value, scaled by 2^-32 in float, clamped below 1, then v * (hi - lo) + lo in float."""
    bg = np.random.MT19937()
    bg._legacy_seeding(0)
    raw = bg.random_raw(n).astype(np.uint32)
    u = raw.astype(np.float32) * np.float32(2.0 ** -32)
    u = np.minimum(u, np.nextafter(np.float32(1.0), np.float32(0.0)))
    return (u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)
