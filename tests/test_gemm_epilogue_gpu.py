"""bf16 GEMM with the reference's elementwise / row-reduction leaves fused into its epilogue
(gb200_gemm_bf16_epilogue) against the oracle's pieces composed on the CPU.

Bars: C (rounded to bf16) within 1e-2 relative Frobenius error; row maxima and row sums, taken from
the unrounded fp32 values, within 1e-3 relative (tensor-core accumulation order and the fast
exponential differ from the oracle's ascending-k loop and expf in the last bits)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def frob(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) /
                 max(np.linalg.norm(want.astype(np.float64)), 1e-30))


def operands(M, N, K, seed, std=0.25):
    g = torch.Generator().manual_seed(seed)
    A = (torch.randn((M, K), generator=g) * std).to(torch.bfloat16).cuda()
    Bt = (torch.randn((N, K), generator=g) * std).to(torch.bfloat16).cuda()
    return A, Bt


def run(ctx, oracle, M, N, K, seed, alpha=1.0, sub=False, exp=False, div=False, want_c=True,
        want_max=True, want_sum=True, variant=None):
    A, Bt = operands(M, N, K, seed)
    rng = np.random.default_rng(seed)
    row_sub = rng.standard_normal(M).astype(np.float32) if sub else None
    row_div = (rng.random(M).astype(np.float32) + 0.5) if div else None
    C = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda") if want_c else None
    rmax = torch.full((M,), 123.0, device="cuda") if want_max else None
    rsum = torch.full((M,), 123.0, device="cuda") if want_sum else None
    ctx.gemm_bf16_epilogue(A, Bt, C, alpha=alpha,
                           row_sub=torch.from_numpy(row_sub).cuda() if sub else None, apply_exp=exp,
                           row_div=torch.from_numpy(row_div).cuda() if div else None,
                           row_max=rmax, row_sum=rsum, variant=variant)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    t, tmax, tsum = oracle.gemm_bf16_epilogue(bits(A), bits(Bt), alpha, row_sub, exp, row_div)
    oracle.set_threads(1)
    if want_c:
        assert frob(C.float().cpu().numpy(), t) <= 1e-2
    if want_max:
        np.testing.assert_allclose(rmax.cpu().numpy(), tmax, rtol=1e-3, atol=1e-4)
    if want_sum:
        np.testing.assert_allclose(rsum.cpu().numpy(), tsum, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 128), (300, 700, 192), (1, 8, 8),
                                   (129, 257, 72), (1024, 1024, 512)])
def test_plain_product_with_reductions(ctx, oracle, shape):
    run(ctx, oracle, *shape, seed=sum(shape))


@pytest.mark.parametrize("shape", [(256, 512, 128), (300, 700, 192), (77, 1000, 256)])
def test_exp_matrix_consumer(ctx, oracle, shape):
    run(ctx, oracle, *shape, seed=1 + sum(shape), exp=True)


@pytest.mark.parametrize("shape", [(256, 512, 128), (513, 300, 64)])
def test_subtract_exp_divide_chain(ctx, oracle, shape):
    run(ctx, oracle, *shape, seed=2 + sum(shape), alpha=0.5, sub=True, exp=True, div=True)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("shape", [(256, 512, 128), (300, 700, 192), (1, 8, 8), (129, 257, 72), (1024, 1280, 512)])
def test_both_kernels_with_every_consumer(ctx, oracle, shape, variant):
    """Single-CTA tiles (1) and CTA pairs (2), forced; large outputs take the pair kernel by default."""
    run(ctx, oracle, *shape, seed=7 + sum(shape), alpha=0.5, sub=True, exp=True, div=True, variant=variant)
    run(ctx, oracle, *shape, seed=8 + sum(shape), want_c=False, variant=variant)


def test_large_output_takes_the_pair_kernel(ctx, oracle):
    run(ctx, oracle, 2560, 2560, 256, seed=11, exp=True)      # 100 tiles of 256 x 256 >= 74 pairs


def test_negative_values_take_the_right_maximum(ctx, oracle):
    # every entry negative after the subtraction: exercises the unsigned branch of the float max
    M, N, K = 200, 600, 64
    A, Bt = operands(M, N, K, 3)
    sub = np.full(M, 50.0, np.float32)
    rmax = torch.zeros((M,), device="cuda")
    ctx.gemm_bf16_epilogue(A, Bt, None, row_sub=torch.from_numpy(sub).cuda(), row_max=rmax)
    ctx.sync()
    t, tmax, _ = oracle.gemm_bf16_epilogue(bits(A), bits(Bt), 1.0, sub)
    assert (tmax < 0).all()
    np.testing.assert_allclose(rmax.cpu().numpy(), tmax, rtol=1e-4)


def test_reductions_without_storing_the_product(ctx, oracle):
    run(ctx, oracle, 384, 768, 128, seed=4, want_c=False)


def test_two_pass_softmax_of_a_product(ctx, oracle):
    """softmax_rows(alpha * A B) from two fused GEMMs: pass 1 keeps only the row maxima, pass 2
    subtracts them, exponentiates and sums; P / sum must match the oracle's softmax of the product."""
    M, N, K = 512, 1536, 128
    A, Bt = operands(M, N, K, 5, std=1.0)
    alpha = 1.0 / np.sqrt(K)
    rmax = torch.empty((M,), device="cuda")
    ctx.gemm_bf16_epilogue(A, Bt, None, alpha=alpha, row_max=rmax)
    P = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    rsum = torch.empty((M,), device="cuda")
    ctx.gemm_bf16_epilogue(A, Bt, P, alpha=alpha, row_sub=rmax, apply_exp=True, row_sum=rsum)
    ctx.sync()
    got = P.float().cpu().numpy() / rsum.cpu().numpy()[:, None]
    oracle.set_threads(oracle.max_threads())
    s = oracle.gemm_bf16(bits(A), bits(Bt)) * np.float32(alpha)
    want = oracle.softmax_rows(np.ascontiguousarray(s))
    oracle.set_threads(1)
    assert frob(got, want) <= 1e-2
    assert abs(got.sum(axis=1) - 1.0).max() < 1e-2


def test_bad_arguments(ctx):
    from gern_b200 import api
    A, Bt = operands(128, 128, 64, 6)
    with pytest.raises(api.GernB200Error) as e:      # nothing to produce
        ctx.gemm_bf16_epilogue(A, Bt, None)
    assert e.value.code == -1
    assert api.lib.gb200_gemm_bf16_epilogue(ctx.handle, A.data_ptr(), 64, Bt.data_ptr(), 64, None, 0,
                                            128, 128, 64, None, None) == -1
    C = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(api.GernB200Error) as e:      # rows of A not 16-byte aligned
        ctx.gemm_bf16_epilogue(A[:, 1:], Bt[:, 1:], C)
    assert e.value.code == -3
