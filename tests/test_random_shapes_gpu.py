"""Seeded random shapes, paddings and kernel variants for every entry point, against the oracle.
The fixed-shape files test the cases the reference tests and the tile boundaries; this one walks
shapes nobody picked."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return np.ascontiguousarray(t.view(torch.int16).cpu().numpy().view(np.uint16))


def frob(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
                 max(np.linalg.norm(b.astype(np.float64)), 1e-30))


@pytest.fixture(scope="module")
def many_threads(oracle):
    oracle.set_threads(oracle.max_threads())
    yield oracle
    oracle.set_threads(1)


def test_blur(ctx, many_threads):
    rng = np.random.default_rng(101)
    for i in range(32):
        r, c = int(rng.integers(3, 700)), int(rng.integers(3, 1500))
        pad_in, pad_out = int(rng.integers(0, 6)), int(rng.integers(0, 6))
        x = rng.random((r, c), dtype=np.float32)
        xin = torch.zeros((r, c + pad_in), device="cuda")
        xin[:, :c] = torch.from_numpy(x).cuda()
        out = torch.full((r - 2, c - 2 + pad_out), -5.0, device="cuda")
        variant = [None, 1, 2, 3, 40, 42, 44, 52][i % 8]
        ctx.blur3x3(xin[:, :c], out[:, :c - 2], variant=variant)
        ctx.sync()
        assert np.array_equal(out[:, :c - 2].cpu().numpy(), many_threads.blur_xy(x)), (r, c, pad_in, pad_out, variant)
        assert bool((out[:, c - 2:] == -5.0).all()), (r, c, variant)


def test_softmax(ctx, many_threads):
    rng = np.random.default_rng(102)
    for _ in range(24):
        r, c = int(rng.integers(1, 300)), int(rng.integers(1, 9000))
        x = (rng.standard_normal((r, c)) * 3).astype(np.float32)
        xg = torch.from_numpy(x).cuda()
        og = torch.empty_like(xg)
        ctx.softmax_rows(xg, og)
        ctx.sync()
        want = many_threads.softmax_rows_f64(x)
        rel = np.abs(og.cpu().numpy() - want) / np.maximum(want, 1e-300)
        assert rel[want > 1e-30].max() <= 1e-5, (r, c)


def test_gemm_bf16(ctx, many_threads):
    rng = np.random.default_rng(103)
    torch.manual_seed(103)
    for i in range(30):
        m, n, k = int(rng.integers(1, 700)), int(rng.integers(1, 900)), int(rng.integers(1, 600))
        k_alloc = (k + 7) // 8 * 8 if i % 3 else k      # every third case: rows not 16-byte aligned
        a = (torch.randn((m, k_alloc), device="cuda") * 0.1).to(torch.bfloat16)[:, :k]
        b = (torch.randn((n, k_alloc), device="cuda") * 0.1).to(torch.bfloat16)[:, :k]
        c = torch.full((m, n + 3), 7.0, dtype=torch.bfloat16, device="cuda")
        variant = [None, 1, 2, 3, 4][i % 5]
        ctx.gemm_bf16(a, b, c[:, :n], variant=variant)
        ctx.sync()
        want = many_threads.gemm_bf16(bits(a.contiguous()), bits(b.contiguous()))
        assert frob(c[:, :n].float().cpu().numpy(), want) <= 1e-2, (m, n, k, variant)
        assert bool((c[:, n:] == 7.0).all()), (m, n, k, variant)


def test_gemm_f32(ctx):
    rng = np.random.default_rng(104)
    for i in range(20):
        m, n, k = int(rng.integers(1, 500)), int(rng.integers(1, 500)), int(rng.integers(1, 400))
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        want = a.astype(np.float64) @ b.astype(np.float64)
        cg = torch.zeros((m, n), device="cuda")
        ctx.gemm_f32(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), cg, variant=1 + i % 2)
        ctx.sync()
        assert frob(cg.cpu().numpy(), want) < 1e-5, (m, n, k, 1 + i % 2)


def test_attention(ctx, many_threads):
    rng = np.random.default_rng(105)
    torch.manual_seed(105)
    for i in range(18):
        nq, nkv = int(rng.integers(1, 700)), int(rng.integers(1, 1500))
        q = torch.randn((nq, 128), device="cuda").to(torch.bfloat16)
        k = torch.randn((nkv, 128), device="cuda").to(torch.bfloat16)
        v = torch.randn((nkv, 128), device="cuda").to(torch.bfloat16)
        o = torch.zeros_like(q)
        variant = [None, 1, 2][i % 3]
        ctx.attention_bf16(q, k, v, o, 0.0884, variant=variant)
        ctx.sync()
        want = many_threads.attention_bf16(bits(q), bits(k), bits(v), 0.0884)
        assert frob(o.float().cpu().numpy(), want) <= 1e-2, (nq, nkv, variant)
