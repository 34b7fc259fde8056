"""gern_b200: B200 (sm_100a) kernels for the fused programs Gern's lowering emits, behind a C ABI.

The product is gern_b200/libgern_b200.so (sources in gern_b200/csrc, declarations in
include/gern_b200.h).  This package is the thin Python door onto that C ABI used by the tests and
the benchmark; it holds no compute of its own and has no fallback: if the shared library is
missing, importing `gern_b200.api` raises.
"""
__all__ = ["api", "build"]
