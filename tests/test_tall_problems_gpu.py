"""Problems with more row blocks than one grid dimension holds (65535): the kernels that put row
blocks in grid.y go out as several row panels (or taller strips), and the result is the same."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bf16_plain_kernel_beyond_65535_row_blocks(ctx):
    m, n, k = 65535 * 16 + 40, 8, 4              # pitch of 4 elements: the plain CUDA-core kernel
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randint(-3, 4, (m, k), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randint(-3, 4, (n, k), device="cuda", generator=g).to(torch.bfloat16)
    c = torch.full((m, n), 99.0, dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a, b, c)
    ctx.sync()
    assert torch.equal(c, (a.float() @ b.float().T).to(torch.bfloat16))


def test_f32_cuda_core_kernel_beyond_65535_row_blocks(ctx):
    m, n, k = 65535 * 32 + 70, 4, 4
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randint(-3, 4, (m, k), device="cuda", generator=g).float()
    b = torch.randint(-3, 4, (k, n), device="cuda", generator=g).float()
    c = torch.full((m, n), 99.0, device="cuda")
    ctx.gemm_f32(a, b, c, variant=1)
    ctx.sync()
    assert torch.equal(c, a @ b)


def test_blur_generic_kernel_beyond_65535_row_strips(ctx, oracle):
    rows, cols = 65535 * 32 + 100, 7             # 7-float rows: the generic (unaligned) kernel
    x = torch.rand((rows, cols), device="cuda")
    out = torch.empty((rows - 2, cols - 2), device="cuda")
    ctx.blur3x3(x, out)
    ctx.sync()
    for r0 in (0, 65535 * 32 - 8, rows - 2 - 16):
        xs = np.ascontiguousarray(x[r0:r0 + 18].cpu().numpy())
        assert np.array_equal(out[r0:r0 + 16].cpu().numpy(), oracle.blur_xy(xs))
    # the constant image is a fixed point everywhere
    x.fill_(0.5)
    ctx.blur3x3(x, out)
    ctx.sync()
    assert bool((out == 0.5).all())
