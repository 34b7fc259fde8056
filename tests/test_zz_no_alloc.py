"""The allocation-free split-K GEMM entry point (gb200_gemm_bf16_splitk_static), called through
the C ABI.  It serves callers that may not call cudaMalloc (see include/gern_b200.h), so its
workspace is a fixed array inside the library that every call shares.  The checks: two calls in a
row with different shapes and split counts give exactly the bits of the context-based entry point
(stale workspace contents must not leak into a later result), and an oversized request is refused
with a clear error instead of overrunning the array; a warmed call leaves the device's free memory
unchanged; operands that are not memory of the current device are refused.  Collected last on
purpose."""
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


@pytest.mark.parametrize("mnk,splits", [((200, 330, 2048), 3),     # N % 4 != 0: scalar slab stores and reduce
                                        ((128, 256, 128), 4),      # more splits than 64-wide K blocks: empty slabs
                                        ((512, 512, 8192), 0)])    # library-chosen split count
def test_slab_paths_match_the_context_entry_point(ctx, mnk, splits):
    from gern_b200 import api
    m, n, k = mnk
    # a call that leaves the shared array full of another problem's partial sums comes first
    af, bf = make(512, 512, 4096, seed=9)
    api.gemm_bf16_splitk_static(af, bf, torch.empty((512, 512), dtype=torch.bfloat16, device="cuda"), splits=8)
    a, b = make(m, n, k, seed=m + n + k)
    want = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    got = torch.zeros_like(want)
    ctx.gemm_bf16(a, b, want, splits=splits)
    api.gemm_bf16_splitk_static(a, b, got, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    api.static_status()      # no kernel gave up a wait


def test_a_warmed_call_allocates_no_device_memory(ctx):
    from gern_b200 import api
    a, b = make(512, 512, 4096, seed=4)
    c = torch.zeros((512, 512), dtype=torch.bfloat16, device="cuda")
    api.gemm_bf16_splitk_static(a, b, c, splits=8)           # first call on the device: set-up
    api.static_status()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for splits in (8, 2, 0, 1):
        api.gemm_bf16_splitk_static(a, b, c, splits=splits)
    api.static_status()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0, "the entry point changed the device's free memory"


def test_operands_outside_the_current_device_are_refused():
    from gern_b200 import api
    a, b = make(128, 256, 256, seed=5)
    c = torch.full((128, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    host_a = torch.zeros((128, 256), dtype=torch.bfloat16).pin_memory()
    with pytest.raises(api.GernB200Error) as e:
        api.gemm_bf16_splitk_static(host_a, b, c, splits=1)
    assert e.value.code == -1 and "not device memory of the current device" in str(e.value)
    torch.cuda.synchronize()
    assert bool((c == 7.0).all())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_second_device_has_its_own_array(ctx):
    from gern_b200 import api
    with torch.cuda.device(1):
        g = torch.Generator(device="cuda:1").manual_seed(6)
        a = (torch.randn((256, 2048), generator=g, device="cuda:1") * 0.02).to(torch.bfloat16)
        b = (torch.randn((512, 2048), generator=g, device="cuda:1") * 0.02).to(torch.bfloat16)
        c = torch.zeros((256, 512), dtype=torch.bfloat16, device="cuda:1")
        api.gemm_bf16_splitk_static(a, b, c, splits=4)
        api.static_status()
        torch.cuda.synchronize()
        ref = a.float() @ b.float().T
        assert float(torch.linalg.norm(c.float() - ref) / torch.linalg.norm(ref)) <= 3e-3
        # a context call on device 0 in between must not move this thread off device 1
        x = torch.zeros((64, 64), device="cuda:0")
        ctx.softmax_rows(x, torch.empty_like(x))
        assert torch.cuda.current_device() == 1
        c0 = torch.zeros((128, 256), dtype=torch.bfloat16, device="cuda:0")
        with pytest.raises(api.GernB200Error):
            api.gemm_bf16_splitk_static(a[:128, :256].contiguous(), b[:256, :256].contiguous(), c0, splits=1)
