"""Matrix multiply: CUDA paths against the CPU oracle.
fp32: |delta| <= 1e-3 absolute as in the reference's app self-checks (gernels/mm/float-error.h:2-4)
and relative Frobenius error <= 1e-5 against the tiled Gern CPU path (fma vs mul+add rounding and
K-tile reassociation are the only differences).
bf16: relative Frobenius error <= 1e-2 against the fp32 oracle on the same bf16-rounded inputs."""
import numpy as np
import pytest
import torch

from oracle import pyoracle

pytestmark = pytest.mark.gpu


def frob(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_f32_golden_10x10(ctx, golden):
    a = torch.arange(100, dtype=torch.float32, device="cuda").reshape(10, 10)
    c = torch.zeros((10, 10), device="cuda")
    ctx.gemm_f32(a, a, c)
    ctx.sync()
    assert np.array_equal(c.cpu().numpy(), golden["mm10_c"])  # integers: exact


def test_f32_512_against_gern_cpu_path(ctx, oracle, golden):
    a_np = pyoracle.mt19937_uniform(512 * 512, -1.0, 1.0).reshape(512, 512)
    a = torch.from_numpy(a_np).cuda()
    c = torch.zeros((512, 512), device="cuda")
    ctx.gemm_f32(a, a, c)
    ctx.sync()
    got = c.cpu().numpy()
    assert np.abs(got[::8, ::8] - golden["mm512_sub"]).max() < 1e-3
    assert frob(got[::8, ::8], golden["mm512_sub"]) < 1e-5
    assert abs(got.astype(np.float64).sum() - float(golden["mm512_sum"])) < 1e-2 * 512


@pytest.mark.parametrize("mnk", [(1, 1, 1), (5, 7, 3), (33, 65, 17), (64, 64, 64), (100, 130, 250), (257, 129, 513),
                                 (2048, 2304, 96)])
def test_f32_shapes(ctx, oracle, mnk):
    m, n, k = mnk
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    oracle.set_threads(oracle.max_threads())
    want = oracle.matmul_tiled(a, b, 64, 64, 64, c0.copy())
    oracle.set_threads(1)
    ag, bg, cg = (torch.from_numpy(t).cuda() for t in (a, b, c0))
    ctx.gemm_f32(ag, bg, cg, accumulate=True)
    ctx.sync()
    got = cg.cpu().numpy()
    assert np.abs(got - want).max() < 1e-3
    assert frob(got, want) < 1e-5
    ctx.gemm_f32(ag, bg, cg, accumulate=False)
    ctx.sync()
    assert frob(cg.cpu().numpy(), want - c0) < 1e-5


@pytest.mark.parametrize("variant", [1, 2, 3, 5])
@pytest.mark.parametrize("mnk", [(1, 1, 1), (5, 7, 3), (64, 64, 64), (100, 130, 250), (257, 129, 513), (512, 512, 512),
                                 (1024, 768, 300), (256, 256, 256), (130, 70, 1100)])
def test_f32_kernel_variants(ctx, oracle, mnk, variant):
    """CUDA-core kernels (1), the tensor-core path with three-way bf16 splits in pre-passes (2) and
    the single-launch kernel that splits in shared memory (3: with a cluster per tile sharing the K
    range when there are few tiles; 5: without clusters), forced: all must meet the fp32 bars (|delta| < 1e-3, relative Frobenius error < 1e-5), with and
    without accumulation into C."""
    m, n, k = mnk
    rng = np.random.default_rng(m * 77 + n * 3 + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    oracle.set_threads(oracle.max_threads())
    want = oracle.matmul_tiled(a, b, 64, 64, 64, c0.copy())
    oracle.set_threads(1)
    pad = 5   # rows of C not 16-byte aligned, guard columns behind them
    ag, bg = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    cg = torch.full((m, n + pad), 9.0, device="cuda")
    cg[:, :n] = torch.from_numpy(c0).cuda()
    ctx.gemm_f32(ag, bg, cg[:, :n], accumulate=True, variant=variant)
    ctx.sync()
    got = cg[:, :n].cpu().numpy()
    assert bool((cg[:, n:] == 9.0).all()), "wrote past the row"
    assert np.abs(got - want).max() < 1e-3
    assert frob(got, want) < 1e-5
    ctx.gemm_f32(ag, bg, cg[:, :n], accumulate=False, variant=variant)
    ctx.sync()
    assert frob(cg[:, :n].cpu().numpy(), want - c0) < 1e-5


def test_f32_tensor_core_path_is_exact_on_small_integers(ctx):
    # the reference's own check: 10 x 10 ascending integers, == (test/test-cpu-mm.cpp:13-83); on the
    # split path integers below 2^8 are their own first bf16 term, so every product is exact
    m = n = k = 160
    a = (torch.arange(m * k, device="cuda") % 13).float().reshape(m, k)
    b = (torch.arange(k * n, device="cuda") % 7).float().reshape(k, n)
    c = torch.zeros((m, n), device="cuda")
    for variant in (2, 3, 5):
        c.zero_()
        ctx.gemm_f32(a, b, c, variant=variant)
        ctx.sync()
        assert torch.equal(c, a.double().matmul(b.double()).float()), variant


def test_f32_large_goes_to_the_tensor_cores_and_keeps_fp32_accuracy(ctx, oracle):
    m, n, k = 2048, 1536, 1024          # 6.4 GFLOP: above the switch-over
    rng = np.random.default_rng(9)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    ag, bg = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.zeros((m, n), device="cuda")
    ctx.gemm_f32(ag, bg, c)
    ctx.sync()
    rows = np.arange(0, m, 37)
    want = a[rows].astype(np.float64) @ b.astype(np.float64)
    got = c.cpu().numpy()[rows]
    assert frob(got, want) < 1e-6
    c1 = torch.zeros((m, n), device="cuda")
    ctx.gemm_f32(ag, bg, c1, variant=1)
    ctx.sync()
    assert frob(c1.cpu().numpy()[rows], want) < 1e-6


def test_f32_cta_pair_path(ctx):
    # 10 x 9 tiles of 256 x 256: enough for the CTA-pair kernel; ragged K, accumulation into C
    m, n, k = 2560, 2300, 328
    rng = np.random.default_rng(21)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c0 = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    ag, bg, cg = (torch.from_numpy(t).cuda() for t in (a, b, c0))
    ctx.gemm_f32(ag, bg, cg, accumulate=True)
    ctx.sync()
    rows = np.arange(0, m, 53)
    want = a[rows].astype(np.float64) @ b.astype(np.float64) + c0[rows]
    assert frob(cg.cpu().numpy()[rows], want) < 1e-6
    ctx.gemm_f32(ag, bg, cg, accumulate=False)
    ctx.sync()
    assert frob(cg.cpu().numpy()[rows], want - c0[rows]) < 1e-6


def test_f32_k_zero_and_empty(ctx):
    c = torch.full((4, 4), 3.0, device="cuda")
    a = torch.zeros((4, 0), device="cuda")
    b = torch.zeros((0, 4), device="cuda")
    from gern_b200 import api
    assert api.lib.gb200_gemm_f32(ctx.handle, None, 0, None, 4, c.data_ptr(), 4, 4, 4, 0, 1, None) == 0
    ctx.sync()
    assert bool((c == 3.0).all())
    assert api.lib.gb200_gemm_f32(ctx.handle, None, 0, None, 4, c.data_ptr(), 4, 0, 4, 4, 0, None) == 0


def run_bf16(ctx, m, n, k, seed, std=0.02, pad=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = (torch.randn((m, k + pad), generator=g, device="cuda") * std).to(torch.bfloat16)
    b = (torch.randn((n, k + pad), generator=g, device="cuda") * std).to(torch.bfloat16)
    c = torch.zeros((m, n + pad), dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a[:, :k], b[:, :k], c[:, :n])
    ctx.sync()
    return a[:, :k], b[:, :k], c[:, :n]


@pytest.mark.parametrize("mnk", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (100, 200, 72), (130, 258, 136),
                                 (1, 8, 8), (384, 768, 1024), (1024, 1024, 1024)])
def test_bf16_against_oracle(ctx, oracle, mnk):
    m, n, k = mnk
    a, b, c = run_bf16(ctx, m, n, k, seed=m + n + k)
    oracle.set_threads(oracle.max_threads())
    want = oracle.gemm_bf16(np.ascontiguousarray(bits(a.contiguous())), np.ascontiguousarray(bits(b.contiguous())))
    oracle.set_threads(1)
    got = c.float().cpu().numpy()
    assert frob(got, want) <= 1e-2
    # tighter: the only error beyond fp32 accumulation order is the final bf16 rounding (2^-9)
    assert frob(got, want) <= 3e-3


@pytest.mark.parametrize("mnk,splits", [((256, 512, 2048), 0), ((256, 512, 2048), 1), ((256, 512, 2048), 2),
                                        ((256, 512, 2048), 5), ((130, 258, 1100), 3), ((128, 256, 8192), 16),
                                        ((100, 203, 1024), 4), ((128, 256, 64), 4)])
def test_bf16_split_k(ctx, oracle, mnk, splits):
    """K split into slabs of fp32 partial sums (workspace) + reduce kernel; 0 = library's choice."""
    m, n, k = mnk
    g = torch.Generator(device="cuda").manual_seed(m + n + k + splits)
    a = (torch.randn((m, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a, b, c, splits=splits)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    want = oracle.gemm_bf16(np.ascontiguousarray(bits(a)), np.ascontiguousarray(bits(b)))
    oracle.set_threads(1)
    assert frob(c.float().cpu().numpy(), want) <= 3e-3
    # a second call reuses the workspace and must not depend on what the first left there
    c2 = torch.zeros_like(c)
    ctx.gemm_bf16(a, b, c2, splits=splits)
    ctx.sync()
    assert torch.equal(c, c2)


@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("mnk", [(256, 256, 64), (512, 768, 1024), (300, 500, 200), (130, 258, 136), (1, 8, 8),
                                 (1024, 1280, 512), (1000, 3000, 328)])
def test_bf16_kernel_variants(ctx, oracle, mnk, variant):
    """Single-CTA 128x256 tiles (1), CTA-pair tiles with the width picked (2), single-CTA tiles of 192
    (3) and 128 (4) columns, CTA-pair tiles of 224 (5) and 256 (6) columns, forced, ragged shapes
    included."""
    m, n, k = mnk
    g = torch.Generator(device="cuda").manual_seed(m * 3 + n * 5 + k)
    a = (torch.randn((m, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    c = torch.full((m, n + 8), 9.0, dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a, b, c[:, :n], variant=variant)
    ctx.sync()
    assert bool((c[:, n:] == 9.0).all()), "wrote past the row"
    oracle.set_threads(oracle.max_threads())
    want = oracle.gemm_bf16(np.ascontiguousarray(bits(a)), np.ascontiguousarray(bits(b)))
    oracle.set_threads(1)
    assert frob(c[:, :n].float().cpu().numpy(), want) <= 3e-3


def test_bf16_pair_kernel_exact_on_integers(ctx):
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(-3, 4, (2048, 1024), device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randint(-3, 4, (1536, 1024), device="cuda", generator=g).to(torch.bfloat16)
    c = torch.empty((2048, 1536), dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a, b, c, variant=2)
    ctx.sync()
    assert torch.equal(c, (a.float() @ b.float().T).to(torch.bfloat16))


def test_bf16_unaligned_falls_to_simple_kernel(ctx, oracle):
    a, b, c = run_bf16(ctx, 70, 90, 50, seed=1, pad=3)   # pitch not a multiple of 8 elements
    want = oracle.gemm_bf16(np.ascontiguousarray(bits(a.contiguous())), np.ascontiguousarray(bits(b.contiguous())))
    assert frob(c.float().cpu().numpy(), want) <= 3e-3


def test_bf16_structured_exact(ctx):
    """Identity and small-integer operands are exact in bf16, so the result must be exact: checks
    operand layout (row-major A, column-major B) and tile addressing without any tolerance."""
    m = n = k = 512
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randint(-4, 5, (m, k), device="cuda", generator=g).to(torch.bfloat16)
    eye = torch.eye(k, device="cuda", dtype=torch.bfloat16)
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.gemm_bf16(a, eye, c)
    ctx.sync()
    assert torch.equal(c, a)
    b = torch.randint(-4, 5, (n, k), device="cuda", generator=g).to(torch.bfloat16)
    ctx.gemm_bf16(a[:, :64].contiguous(), b[:, :64].contiguous(), c)
    ctx.sync()
    # integer sums are exact in fp32; the only rounding left is the final one to bf16
    want = (a[:, :64].float() @ b[:, :64].float().T).to(torch.bfloat16)
    assert torch.equal(c, want)


def test_bf16_against_reference_leaf_fixture(ctx, golden, golden_maker):
    """The CUDA kernels against gern::impl::matrix_multiply (test/library/matrix/impl/cpu-matrix.h:196-212)
    run by the reference itself on the same bf16-rounded operands (tests/golden/make_golden.py)."""
    for tag, variants in (("gemm96", (None, 1, 4)), ("gemm512", (None, 1, 2))):
        a_bits, b_bits = golden_maker.bf16_inputs(tag)
        a = torch.from_numpy(a_bits.view(np.int16)).cuda().view(torch.bfloat16)
        b = torch.from_numpy(b_bits.view(np.int16)).cuda().view(torch.bfloat16)
        for variant in variants:
            c = torch.zeros((a.shape[0], b.shape[0]), dtype=torch.bfloat16, device="cuda")
            ctx.gemm_bf16(a, b, c, variant=variant)
            ctx.sync()
            got = c.float().cpu().numpy()
            if tag == "gemm96":
                want = golden["gemmbf96_c"]
            else:
                got, want = got[::8, ::8], golden["gemmbf512_sub"]
            # fp32 reassociation inside the tensor core plus the final bf16 rounding (2^-9 relative)
            assert frob(got, want) <= 3e-3, (tag, variant)


def test_bf16_full_size_sampled(ctx, oracle):
    """8192^3 (the benchmark size): sampled rows against the oracle, plus linearity A(2B) = 2(AB)."""
    n = 8192
    a, b, c = run_bf16(ctx, n, n, n, seed=0)
    # one row in every 128-row block (both halves of every 256-row CTA-pair tile), at a lane that
    # moves through the block, plus the corners
    rows = sorted({0, 1, 127, 128, 4095, 8191} | {blk * 128 + (blk * 37) % 128 for blk in range(n // 128)})
    a_s = np.ascontiguousarray(bits(a[rows].contiguous()))
    oracle.set_threads(oracle.max_threads())
    want = oracle.gemm_bf16(a_s, np.ascontiguousarray(bits(b.contiguous())))
    oracle.set_threads(1)
    assert frob(c[rows].float().cpu().numpy(), want) <= 1e-2
    c2 = torch.empty_like(c)
    ctx.gemm_bf16(a, (b * 2).contiguous(), c2)
    ctx.sync()
    assert torch.equal(c2.float(), c.float() * 2)


def test_host_entry_points(ctx, oracle):
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (200, 300)).astype(np.float32)
    b = rng.uniform(-1, 1, (300, 150)).astype(np.float32)
    c = np.zeros((200, 150), np.float32)
    ctx.gemm_f32_host(a, b, c)
    assert frob(c, oracle.matrix_multiply(a, b)) < 1e-5
    ab = pyoracle.to_bf16_bits((rng.standard_normal((256, 320)) * 0.02).astype(np.float32))
    bb = pyoracle.to_bf16_bits((rng.standard_normal((512, 320)) * 0.02).astype(np.float32))
    cb = np.zeros((256, 512), np.uint16)
    ctx.gemm_bf16_host(ab, bb, cb)
    assert frob(pyoracle.bf16_bits_to_f32(cb), oracle.gemm_bf16(ab, bb)) <= 3e-3


@pytest.mark.parametrize("cluster_x", [1, 2])
def test_bf16_cluster_entry_point(ctx, oracle, cluster_x):
    """gb200_gemm_bf16_cluster: 1 = single-CTA tiles, 2 = CTA pairs; other sizes are refused."""
    from gern_b200 import api
    m, n, k = 300, 520, 200
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (torch.randn((m, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    rc = api.lib.gb200_gemm_bf16_cluster(ctx.handle, a.data_ptr(), k, b.data_ptr(), k, c.data_ptr(), n, m, n, k,
                                         cluster_x, None)
    assert rc == 0
    ctx.sync()
    want = oracle.gemm_bf16(np.ascontiguousarray(bits(a)), np.ascontiguousarray(bits(b)))
    assert frob(c.float().cpu().numpy(), want) <= 3e-3
    assert api.lib.gb200_gemm_bf16_cluster(ctx.handle, a.data_ptr(), k, b.data_ptr(), k, c.data_ptr(), n, m, n, k,
                                           4, None) == -3
