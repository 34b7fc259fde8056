"""The allocation-free split-K GEMM entry point (gb200_gemm_bf16_splitk_static), called through
the C ABI.  It serves callers that may not call cudaMalloc (see include/gern_b200.h), so its
workspace is a fixed array inside the library that every call shares.  The checks: two calls in a
row with different shapes and split counts give exactly the bits of the context-based entry point
(stale workspace contents must not leak into a later result), and an oversized request is refused
with a clear error instead of overrunning the array.  Collected last on purpose."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make(m, n, k, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = (torch.randn((m, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    return a, b


def test_matches_the_context_entry_point_on_two_calls_in_a_row(ctx):
    from gern_b200 import api
    torch.cuda.set_device(0)
    # first call: big slabs (fills most of the fixed workspace with this problem's partial sums)
    a1, b1 = make(512, 512, 4096, seed=1)
    want1 = torch.zeros((512, 512), dtype=torch.bfloat16, device="cuda")
    got1 = torch.zeros_like(want1)
    ctx.gemm_bf16(a1, b1, want1, splits=8)
    api.gemm_bf16_splitk_static(a1, b1, got1, splits=8)
    # second call straight after, smaller and differently shaped: reads nothing the first left
    a2, b2 = make(200, 328, 2048, seed=2)
    want2 = torch.zeros((200, 328), dtype=torch.bfloat16, device="cuda")
    got2 = torch.zeros_like(want2)
    ctx.gemm_bf16(a2, b2, want2, splits=3)
    api.gemm_bf16_splitk_static(a2, b2, got2, splits=3)
    torch.cuda.synchronize()
    # same kernels, same split points: bit-identical (tolerance of the GEMM tests not needed)
    assert torch.equal(got1, want1)
    assert torch.equal(got2, want2)
    # and against an fp32 evaluation within the bf16 GEMM tolerance used elsewhere (3e-3)
    ref = a2.float() @ b2.float().T
    err = float(torch.linalg.norm(got2.float() - ref) / torch.linalg.norm(ref))
    assert err <= 3e-3
    # unsplit and library-chosen forms go through the same door
    got3 = torch.zeros_like(want2)
    api.gemm_bf16_splitk_static(a2, b2, got3, splits=1)
    want3 = torch.zeros_like(want2)
    ctx.gemm_bf16(a2, b2, want3, splits=1)
    torch.cuda.synchronize()
    assert torch.equal(got3, want3)


def test_requests_beyond_the_fixed_workspace_are_refused():
    from gern_b200 import api
    a, b = make(2048, 2048, 2048, seed=3)
    c = torch.full((2048, 2048), 7.0, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(api.GernB200Error) as e:
        api.gemm_bf16_splitk_static(a, b, c, splits=2)      # 2 * 2048 * 2048 floats = 32 MiB > 16 MiB
    assert e.value.code == -6
    assert "exceeds the fixed workspace" in str(e.value)
    torch.cuda.synchronize()
    assert bool((c == 7.0).all()), "a refused call must not touch the output"
    api.gemm_bf16_splitk_static(a, b, c, splits=1)          # no workspace needed: accepted
    torch.cuda.synchronize()
    ref = a.float() @ b.float().T
    assert float(torch.linalg.norm(c.float() - ref) / torch.linalg.norm(ref)) <= 3e-3
