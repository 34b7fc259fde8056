"""ctypes binding of include/gern_b200.h.  Device entry points take torch CUDA tensors (used only
as owners of device memory); `_host` entry points take numpy arrays or CPU torch tensors."""
from __future__ import annotations

import ctypes
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libgern_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m gern_b200.build` (there is no CPU or "
        "PyTorch fallback for the gern_b200 kernels)")

lib = ctypes.CDLL(LIB_PATH)

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_int = ctypes.c_int

# name -> argtypes (after the leading ctx pointer); every function returns int unless noted.
SIGNATURES = {
    "gb200_ctx_create": None,
    "gb200_ctx_destroy": None,
    "gb200_device_sync": None,
    "gb200_last_error_string": None,
    "gb200_version": None,
    "gb200_launch_count": None,
    "gb200_gemm_f32": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp],
    "gb200_gemm_f32_variant": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp, _int],
    "gb200_gemm_bf16": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp],
    "gb200_gemm_bf16_cluster": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp],
    "gb200_gemm_bf16_splitk": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _int],
    "gb200_gemm_bf16_variant": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp, _int],
    "gb200_gemm_bf16_splitk_static": None,
    "gb200_softmax_rows_f32": [_vp, _i64, _vp, _i64, _i64, _i64, _vp],
    "gb200_softmax_rows_f32_variant": [_vp, _i64, _vp, _i64, _i64, _i64, _vp, _int],
    "gb200_blur3x3_f32": [_vp, _i64, _i64, _i64, _vp, _i64, _vp],
    "gb200_blur3x3_f32_variant": [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _int],
    "gb200_blur3x3_f32_band": [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp],
    "gb200_attention_bf16": [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                             ctypes.c_float, _vp],
    "gb200_attention_bf16_cluster": [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                     ctypes.c_float, _int, _vp],
    "gb200_attention_bf16_splitkv": [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                     ctypes.c_float, _vp, _int],
    "gb200_attention_bf16_variant": [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                     ctypes.c_float, _vp, _int],
    "gb200_gemm_f32_host": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int],
    "gb200_gemm_bf16_host": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64],
    "gb200_softmax_rows_f32_host": [_vp, _i64, _vp, _i64, _i64, _i64],
    "gb200_blur3x3_f32_host": [_vp, _i64, _i64, _i64, _vp, _i64],
    "gb200_attention_bf16_host": [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                  ctypes.c_float],
}

lib.gb200_ctx_create.argtypes = [_int, ctypes.POINTER(_vp)]
lib.gb200_ctx_destroy.argtypes = [_vp]
lib.gb200_device_sync.argtypes = [_vp]
lib.gb200_last_error_string.restype = ctypes.c_char_p
lib.gb200_version.restype = ctypes.c_char_p
lib.gb200_selftest_bounded_wait.argtypes = [_vp, ctypes.c_ulonglong, _vp, _vp]
lib.gb200_selftest_bounded_wait.restype = _int
lib.gb200_selftest_bounded_flag_wait.argtypes = [_vp, ctypes.c_ulonglong, _vp, _vp]
lib.gb200_selftest_bounded_flag_wait.restype = _int
lib.gb200_launch_count.argtypes = [_vp]
lib.gb200_launch_count.restype = _i64
lib.gb200_gemm_bf16_splitk_static.argtypes = [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _int, _vp]
lib.gb200_gemm_bf16_splitk_static.restype = _int
lib.gb200_static_status.argtypes = [ctypes.POINTER(_int)]
lib.gb200_static_status.restype = _int
SIGNATURES["gb200_static_status"] = None


class KernelResources(ctypes.Structure):
    """gb200_kernel_resources."""
    _fields_ = [("regs_per_thread", _int), ("threads", _int), ("dynamic_smem_bytes", _int), ("cluster_x", _int),
                ("tmem_columns", _int)]


lib.gb200_kernel_resources_query.argtypes = [ctypes.c_char_p, ctypes.POINTER(KernelResources)]
lib.gb200_kernel_resources_query.restype = _int
SIGNATURES["gb200_kernel_resources_query"] = None


def kernel_resources(name: str) -> KernelResources:
    out = KernelResources()
    _check(lib.gb200_kernel_resources_query(name.encode(), ctypes.byref(out)), "gb200_kernel_resources_query")
    return out


class GemmEpilogue(ctypes.Structure):
    """gb200_gemm_epilogue."""
    _fields_ = [("alpha", ctypes.c_float), ("row_sub", _vp), ("apply_exp", _int), ("row_div", _vp),
                ("row_max", _vp), ("row_sum", _vp)]


lib.gb200_gemm_bf16_epilogue.argtypes = [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64,
                                         ctypes.POINTER(GemmEpilogue), _vp]
lib.gb200_gemm_bf16_epilogue.restype = _int
lib.gb200_gemm_bf16_epilogue_variant.argtypes = lib.gb200_gemm_bf16_epilogue.argtypes + [_int]
lib.gb200_gemm_bf16_epilogue_variant.restype = _int
SIGNATURES["gb200_gemm_bf16_epilogue"] = None


class Shard(ctypes.Structure):
    """gb200_shard: one device's rows of a sharded call."""
    _fields_ = [("ctx", _vp), ("in_", _vp), ("out", _vp), ("rows", _i64), ("shared0", _vp),
                ("shared1", _vp), ("stream", _vp)]


_shards_p = ctypes.POINTER(Shard)
lib.gb200_gemm_bf16_sharded.argtypes = [_shards_p, _int, _i64, _i64, _i64, _i64, _i64]
lib.gb200_softmax_rows_f32_sharded.argtypes = [_shards_p, _int, _i64, _i64, _i64]
lib.gb200_attention_bf16_sharded.argtypes = [_shards_p, _int, _i64, _i64, _i64, _i64, _i64, _i64,
                                             ctypes.c_float]
lib.gb200_blur3x3_f32_sharded.argtypes = [_shards_p, _int, _i64, _i64, _i64]
for _name in ("gb200_gemm_bf16_sharded", "gb200_softmax_rows_f32_sharded",
              "gb200_attention_bf16_sharded", "gb200_blur3x3_f32_sharded"):
    SIGNATURES[_name] = None
    getattr(lib, _name).restype = _int
for _name, _args in SIGNATURES.items():
    if _args is not None and hasattr(lib, _name):
        getattr(lib, _name).argtypes = [_vp] + _args
        getattr(lib, _name).restype = _int


class GernB200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        msg = lib.gb200_last_error_string().decode(errors="replace")
        super().__init__(f"{what} failed with status {code}: {msg}")


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise GernB200Error(rc, what)


def _ptr(t) -> int:
    """Address of a torch tensor's / numpy array's first element (None -> NULL)."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


def _stream(stream) -> int | None:
    if stream is None:
        return None
    return getattr(stream, "cuda_stream", stream)


def _ld(t) -> int:
    if isinstance(t, np.ndarray):
        assert t.strides[1] == t.itemsize, "rows must be contiguous"
        return t.strides[0] // t.itemsize
    assert t.stride(1) == 1, "rows must be contiguous"
    return t.stride(0)


def gemm_bf16_splitk_static(A, Bt, C, splits=0, stream=None):
    """Context-free, allocation-free split-K GEMM on the current device (see gern_b200.h)."""
    M, K = A.shape
    N = Bt.shape[0]
    _check(lib.gb200_gemm_bf16_splitk_static(_ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C), _ld(C), M, N, K,
                                             int(splits), _stream(stream)), "gb200_gemm_bf16_splitk_static")


def static_status():
    """gb200_static_status: raises GernB200Error(-5) if a kernel of the static entry gave up a wait."""
    code = _int(0)
    _check(lib.gb200_static_status(ctypes.byref(code)), "gb200_static_status")


def _shard_array(parts):
    """parts: list of (Context, in, out, shared0, shared1, stream); rows come from `in`."""
    arr = (Shard * len(parts))()
    for g, (ctx, x, out, s0, s1, stream) in enumerate(parts):
        arr[g] = Shard(ctx.handle, _ptr(x), _ptr(out), x.shape[0], _ptr(s0), _ptr(s1), _stream(stream))
    return arr


def gemm_bf16_sharded(parts):
    """parts: one (Context, A_panel, C_panel, Bt_replica) per device."""
    a0, c0, b0 = parts[0][1], parts[0][2], parts[0][3]
    arr = _shard_array([(c, a, o, b, None, None) for c, a, o, b in parts])
    _check(lib.gb200_gemm_bf16_sharded(arr, len(parts), _ld(a0), _ld(b0), _ld(c0), b0.shape[0],
                                       a0.shape[1]), "gb200_gemm_bf16_sharded")


def softmax_rows_sharded(parts):
    """parts: one (Context, x_rows, out_rows) per device."""
    x0, o0 = parts[0][1], parts[0][2]
    arr = _shard_array([(c, x, o, None, None, None) for c, x, o in parts])
    _check(lib.gb200_softmax_rows_f32_sharded(arr, len(parts), _ld(x0), _ld(o0), x0.shape[1]),
           "gb200_softmax_rows_f32_sharded")


def attention_bf16_sharded(parts, scale):
    """parts: one (Context, Q_rows, O_rows, K_replica, V_replica) per device."""
    q0, o0, k0, v0 = parts[0][1], parts[0][2], parts[0][3], parts[0][4]
    arr = _shard_array([(c, q, o, k, v, None) for c, q, o, k, v in parts])
    _check(lib.gb200_attention_bf16_sharded(arr, len(parts), _ld(q0), _ld(k0), _ld(v0), _ld(o0),
                                            k0.shape[0], q0.shape[1], ctypes.c_float(scale)),
           "gb200_attention_bf16_sharded")


def blur3x3_sharded(parts):
    """parts: one (Context, band, out_band) per device, bands in image order."""
    x0, o0 = parts[0][1], parts[0][2]
    arr = _shard_array([(c, x, o, None, None, None) for c, x, o in parts])
    _check(lib.gb200_blur3x3_f32_sharded(arr, len(parts), _ld(x0), x0.shape[1], _ld(o0)),
           "gb200_blur3x3_f32_sharded")


class Context:
    """Owner of a gb200_ctx (one per process and device)."""

    def __init__(self, device: int = 0):
        h = _vp()
        _check(lib.gb200_ctx_create(int(device), ctypes.byref(h)), "gb200_ctx_create")
        self.handle = h
        self.device = device

    def close(self) -> None:
        if getattr(self, "handle", None):
            lib.gb200_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self) -> None:
        _check(lib.gb200_device_sync(self.handle), "gb200_device_sync")

    def launch_count(self) -> int:
        return int(lib.gb200_launch_count(self.handle))

    # ---- device entry points (torch CUDA tensors) ----
    def gemm_f32(self, A, B, C, accumulate=False, stream=None, variant=None):
        M, K = A.shape
        N = B.shape[1]
        if variant is not None:
            _check(lib.gb200_gemm_f32_variant(self.handle, _ptr(A), _ld(A), _ptr(B), _ld(B), _ptr(C), _ld(C),
                                              M, N, K, int(bool(accumulate)), _stream(stream), int(variant)),
                   "gb200_gemm_f32_variant")
            return
        _check(lib.gb200_gemm_f32(self.handle, _ptr(A), _ld(A), _ptr(B), _ld(B), _ptr(C), _ld(C), M, N, K,
                                  int(bool(accumulate)), _stream(stream)), "gb200_gemm_f32")

    def gemm_bf16(self, A, Bt, C, stream=None, splits=None, variant=None):
        """A: (M,K) bf16; Bt: (N,K) bf16 (column-major B); C: (M,N) bf16."""
        M, K = A.shape
        N = Bt.shape[0]
        if variant is not None:
            _check(lib.gb200_gemm_bf16_variant(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C),
                                               _ld(C), M, N, K, _stream(stream), int(variant)),
                   "gb200_gemm_bf16_variant")
            return
        if splits is not None:
            _check(lib.gb200_gemm_bf16_splitk(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C),
                                              _ld(C), M, N, K, _stream(stream), int(splits)),
                   "gb200_gemm_bf16_splitk")
            return
        _check(lib.gb200_gemm_bf16(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C), _ld(C), M, N,
                                   K, _stream(stream)), "gb200_gemm_bf16")

    def gemm_bf16_epilogue(self, A, Bt, C=None, alpha=1.0, row_sub=None, apply_exp=False, row_div=None,
                           row_max=None, row_sum=None, stream=None, variant=None):
        """C = bf16(epilogue(alpha * A Bt^T)); any of C / row_max / row_sum may be left out."""
        M, K = A.shape
        N = Bt.shape[0]
        e = GemmEpilogue(ctypes.c_float(alpha), _ptr(row_sub), int(bool(apply_exp)), _ptr(row_div),
                         _ptr(row_max), _ptr(row_sum))
        if variant is not None:
            _check(lib.gb200_gemm_bf16_epilogue_variant(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C),
                                                        _ld(C) if C is not None else 0, M, N, K, ctypes.byref(e),
                                                        _stream(stream), int(variant)), "gb200_gemm_bf16_epilogue_variant")
            return
        _check(lib.gb200_gemm_bf16_epilogue(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C),
                                            _ld(C) if C is not None else 0, M, N, K, ctypes.byref(e),
                                            _stream(stream)), "gb200_gemm_bf16_epilogue")

    def softmax_rows(self, x, out, stream=None, variant=None):
        rows, cols = x.shape
        if variant is not None:
            _check(lib.gb200_softmax_rows_f32_variant(self.handle, _ptr(x), _ld(x), _ptr(out), _ld(out),
                                                      rows, cols, _stream(stream), int(variant)),
                   "gb200_softmax_rows_f32_variant")
            return
        _check(lib.gb200_softmax_rows_f32(self.handle, _ptr(x), _ld(x), _ptr(out), _ld(out), rows, cols,
                                          _stream(stream)), "gb200_softmax_rows_f32")

    def blur3x3(self, x, out, stream=None, variant=None):
        rows, cols = x.shape
        if variant is None:
            _check(lib.gb200_blur3x3_f32(self.handle, _ptr(x), _ld(x), rows, cols, _ptr(out), _ld(out),
                                         _stream(stream)), "gb200_blur3x3_f32")
        else:
            _check(lib.gb200_blur3x3_f32_variant(self.handle, _ptr(x), _ld(x), rows, cols, _ptr(out),
                                                 _ld(out), _stream(stream), int(variant)),
                   "gb200_blur3x3_f32_variant")

    def blur3x3_band(self, x, halo, out, stream=None, halo_ptr=None, halo_ld=None):
        """x: this rank's band; halo: tensor with the 2 rows that follow it (or None)."""
        rows, cols = x.shape
        hp = halo_ptr if halo_ptr is not None else _ptr(halo)
        hl = halo_ld if halo_ld is not None else (_ld(halo) if halo is not None else 0)
        _check(lib.gb200_blur3x3_f32_band(self.handle, _ptr(x), _ld(x), rows, cols, hp, hl, _ptr(out),
                                          _ld(out), _stream(stream)), "gb200_blur3x3_f32_band")

    def attention_bf16(self, Q, K, V, O, scale, stream=None, variant=None, splits=None):
        """splits (test hook): 0 = the library's choice, 1 = whole Q tile pairs per thread block,
        n > 1 = that many K/V ranges and a combine pass, -1 = equal runs of (pair, K/V block) units
        per thread block, merged inside the kernel, -9 = whole pairs through the same instantiation
        as the equal runs."""
        nq, d = Q.shape
        nkv = K.shape[0]
        if splits is not None:
            _check(lib.gb200_attention_bf16_splitkv(self.handle, _ptr(Q), _ld(Q), _ptr(K), _ld(K), _ptr(V),
                                                    _ld(V), _ptr(O), _ld(O), nq, nkv, d,
                                                    ctypes.c_float(scale), _stream(stream), int(splits)),
                   "gb200_attention_bf16_splitkv")
            return
        if variant is not None:
            _check(lib.gb200_attention_bf16_variant(self.handle, _ptr(Q), _ld(Q), _ptr(K), _ld(K), _ptr(V),
                                                    _ld(V), _ptr(O), _ld(O), nq, nkv, d,
                                                    ctypes.c_float(scale), _stream(stream), int(variant)),
                   "gb200_attention_bf16_variant")
            return
        _check(lib.gb200_attention_bf16(self.handle, _ptr(Q), _ld(Q), _ptr(K), _ld(K), _ptr(V), _ld(V),
                                        _ptr(O), _ld(O), nq, nkv, d, ctypes.c_float(scale),
                                        _stream(stream)), "gb200_attention_bf16")

    # ---- host entry points (numpy arrays / CPU tensors) ----
    def gemm_f32_host(self, A, B, C, accumulate=False):
        M, K = A.shape
        N = B.shape[1]
        _check(lib.gb200_gemm_f32_host(self.handle, _ptr(A), _ld(A), _ptr(B), _ld(B), _ptr(C), _ld(C), M,
                                       N, K, int(bool(accumulate))), "gb200_gemm_f32_host")

    def gemm_bf16_host(self, A, Bt, C):
        M, K = A.shape
        N = Bt.shape[0]
        _check(lib.gb200_gemm_bf16_host(self.handle, _ptr(A), _ld(A), _ptr(Bt), _ld(Bt), _ptr(C), _ld(C),
                                        M, N, K), "gb200_gemm_bf16_host")

    def softmax_rows_host(self, x, out):
        rows, cols = x.shape
        _check(lib.gb200_softmax_rows_f32_host(self.handle, _ptr(x), _ld(x), _ptr(out), _ld(out), rows,
                                               cols), "gb200_softmax_rows_f32_host")

    def blur3x3_host(self, x, out):
        rows, cols = x.shape
        _check(lib.gb200_blur3x3_f32_host(self.handle, _ptr(x), _ld(x), rows, cols, _ptr(out), _ld(out)),
               "gb200_blur3x3_f32_host")

    def attention_bf16_host(self, Q, K, V, O, scale):
        nq, d = Q.shape
        nkv = K.shape[0]
        _check(lib.gb200_attention_bf16_host(self.handle, _ptr(Q), _ld(Q), _ptr(K), _ld(K), _ptr(V),
                                             _ld(V), _ptr(O), _ld(O), nq, nkv, d, ctypes.c_float(scale)),
               "gb200_attention_bf16_host")
