"""The C-ABI library loads without a GPU, exports every symbol include/gern_b200.h declares, and
fails loudly (never silently falls back) when there is no device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gern_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gb200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gern_b200 import api
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(api.lib, name), f"{name} is declared in gern_b200.h but not exported"
    # and the binding covers every declared entry point
    for name in names:
        assert name in api.SIGNATURES, f"{name} has no ctypes signature in gern_b200/api.py"


def test_version_string():
    from gern_b200 import api
    assert b"sm_100a" in api.lib.gb200_version()


def test_no_device_is_a_loud_error():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from gern_b200 import api
    with pytest.raises(api.GernB200Error) as e:
        api.Context(0)
    assert e.value.code == -4  # GB200_ERR_NO_DEVICE
    assert "no CUDA device" in str(e.value)


def test_null_context_is_rejected():
    from gern_b200 import api
    rc = api.lib.gb200_blur3x3_f32(None, None, 0, 0, 0, None, 0, None)
    assert rc == -1
    assert b"ctx is NULL" in api.lib.gb200_last_error_string()
    assert api.lib.gb200_ctx_destroy(None) == 0


def test_product_does_not_touch_the_oracle():
    """Nothing under gern_b200/ or include/ may import, link or name the oracle."""
    for base in ("gern_b200", "include"):
        for dirpath, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                    src = open(os.path.join(dirpath, f), errors="replace").read()
                    assert "oracle" not in src.lower(), f"{f} names the oracle"


def test_kernel_resources_come_from_the_planned_layouts():
    """gb200_kernel_resources_query answers without a device (registers are then -1): dynamic shared
    memory within an sm_100a block's 227 KB, the pair kernels in clusters of two, 512 TMEM columns."""
    from gern_b200 import api
    seen = {}
    for name in ("gemm_bf16_tc", "gemm_bf16_2cta", "attention_bf16", "attention_bf16_pair"):
        r = api.kernel_resources(name)
        assert 64 * 1024 < r.dynamic_smem_bytes <= 227 * 1024, name
        assert r.dynamic_smem_bytes % 128 == 0 and r.tmem_columns == 512 and r.threads % 32 == 0
        assert r.cluster_x == (2 if name in ("gemm_bf16_2cta", "attention_bf16_pair") else 1)
        seen[name] = r.dynamic_smem_bytes
    # four stages of (128 + 256) x 64 bf16 and six stages of 2 x 128 x 64 bf16, plus barriers and slack
    assert seen["gemm_bf16_tc"] >= 4 * 49152 + 1024 and seen["gemm_bf16_2cta"] >= 6 * 32768 + 1024
    with pytest.raises(api.GernB200Error) as e:
        api.kernel_resources("no_such_kernel")
    assert e.value.code == -1


def test_timeline_tool_imports_and_shipped_library_has_no_trace_code():
    """gern_b200.timeline builds its own debug libraries; the shipped one exports no trace reader."""
    import ctypes
    from gern_b200 import timeline, build
    assert timeline.OUT_DIR.startswith(os.path.join(build.ROOT, "build"))
    lib = ctypes.CDLL(build.LIB_PATH)
    for name in ("gb200_attn_trace_read", "gb200_blur_trace_read"):
        assert not hasattr(lib, name)
