"""Fused blur: CUDA path (through the C ABI) against the CPU oracle.  Bar: equal under `==`
(the reference checks its GPU result against cpu_blur_x/y with ==, apps/blur/blur.cpp:104-108)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def run_blur(ctx, x_np, variant=None, in_pad=0, out_pad=0):
    rows, cols = x_np.shape
    xin = torch.zeros((rows, cols + in_pad), dtype=torch.float32, device="cuda")
    xin[:, :cols] = torch.from_numpy(x_np).cuda()
    out = torch.full((max(rows - 2, 0), max(cols - 2, 0) + out_pad), -7.0, dtype=torch.float32, device="cuda")
    ctx.blur3x3(xin[:, :cols], out[:, :max(cols - 2, 0)], variant=variant)
    ctx.sync()
    o = out.cpu().numpy()
    if out_pad:
        assert (o[:, max(cols - 2, 0):] == -7.0).all(), "wrote past the output row"
    return np.ascontiguousarray(o[:, :max(cols - 2, 0)])


def test_golden_fixtures(ctx, golden):
    for tag in ("asc", "rnd"):
        x = np.ascontiguousarray(golden[f"blur_in_{tag}"])
        for variant in (None, 1, 2):
            assert np.array_equal(run_blur(ctx, x, variant), golden[f"blur_out_{tag}"])


@pytest.mark.parametrize("shape", [(3, 3), (4, 7), (16, 64), (17, 65), (64, 260), (67, 131), (130, 259),
                                   (300, 1028), (257, 2050), (1024, 1024), (1026, 516)])
@pytest.mark.parametrize("variant", [None, 1, 2, 3, 40, 44, 52])
def test_matches_oracle(ctx, oracle, shape, variant):
    x = np.random.default_rng(shape[0] * 7919 + shape[1]).random(shape, dtype=np.float32)
    assert np.array_equal(run_blur(ctx, x, variant), oracle.blur_xy(x))


@pytest.mark.parametrize("shape", [(16, 66), (40, 262), (130, 1030), (600, 2054)])
def test_aligned_output_rows_take_vector_stores(ctx, oracle, shape):
    # cols - 2 is a multiple of 4: output rows are 16-byte aligned, so the 128-bit store path runs
    x = np.random.default_rng(shape[1]).random(shape, dtype=np.float32)
    want = oracle.blur_xy(x)
    for variant in (None, 1, 2, 3, 41, 43, 52):
        assert np.array_equal(run_blur(ctx, x, variant, in_pad=2), want)
    assert np.array_equal(run_blur(ctx, x, None, in_pad=2, out_pad=4), want)


def test_padded_leading_dimensions_and_unaligned(ctx, oracle):
    x = np.random.default_rng(1).random((200, 777), dtype=np.float32)
    want = oracle.blur_xy(x)
    assert np.array_equal(run_blur(ctx, x, None, in_pad=3, out_pad=5), want)   # ld not multiple of 4
    assert np.array_equal(run_blur(ctx, x, None, in_pad=7, out_pad=1), want)   # TMA-eligible input


def test_tall_image_beyond_the_grid_y_limit(ctx, oracle):
    # 300000 output rows: more block rows than a grid's y extent (65535) could index
    rows, cols = 300002, 70
    x = np.random.default_rng(5).random((rows, cols), dtype=np.float32)
    xin = torch.zeros((rows, cols + 2), dtype=torch.float32, device="cuda")
    xin[:, :cols] = torch.from_numpy(x).cuda()
    out = torch.empty((rows - 2, cols - 2), dtype=torch.float32, device="cuda")
    ctx.blur3x3(xin[:, :cols], out)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    want = oracle.blur_xy(x)
    oracle.set_threads(1)
    assert np.array_equal(out.cpu().numpy(), want)


def test_empty_outputs_are_no_ops(ctx):
    for shape in ((0, 0), (2, 100), (100, 2), (1, 1)):
        x = np.zeros(shape, np.float32)
        assert run_blur(ctx, x).size == 0


def test_signed_and_large_values(ctx, oracle):
    rng = np.random.default_rng(9)
    x = (rng.standard_normal((260, 520)) * 1e6).astype(np.float32)
    x[5, 5:9] = 0.0
    x[100, :] = 3.0e38 / 4
    assert np.array_equal(run_blur(ctx, x), oracle.blur_xy(x))


def test_bad_arguments(ctx):
    from gern_b200 import api
    x = torch.zeros((8, 8), device="cuda")
    rc = api.lib.gb200_blur3x3_f32(ctx.handle, x.data_ptr(), 4, 8, 8, x.data_ptr(), 8, None)
    assert rc == -1 and b"leading dimension" in api.lib.gb200_last_error_string()
    rc = api.lib.gb200_blur3x3_f32(ctx.handle, None, 8, 8, 8, x.data_ptr(), 8, None)
    assert rc == -1


def test_band_form_with_halo(ctx, oracle):
    """Row-band form used for multi-GPU sharding: each band + 2 halo rows == rows of the whole."""
    x = np.random.default_rng(2).random((515, 1030), dtype=np.float32)
    want = oracle.blur_xy(x)
    xg = torch.from_numpy(x).cuda()
    out_rows = x.shape[0] - 2
    n = 4
    per = (out_rows + n - 1) // n
    got = torch.empty((out_rows, x.shape[1] - 2), device="cuda")
    for r in range(n):
        r0, r1 = r * per, min((r + 1) * per, out_rows)
        if r < n - 1:
            band = xg[r0:r1].contiguous()            # band_rows rows owned by this rank
            halo = xg[r1:r1 + 2].contiguous()        # first two rows of the next band
            ctx.blur3x3_band(band, halo, got[r0:r1])
        else:
            ctx.blur3x3_band(xg[r0:].contiguous(), None, got[r0:r1])
    ctx.sync()
    assert np.array_equal(got.cpu().numpy(), want)


def test_full_size_properties(ctx, oracle):
    """8192^2 (the benchmark size): every output element against the oracle, a constant image is a fixed point,
    and the TMA and direct kernels agree everywhere."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.rand((n, n), generator=g, device="cuda")
    # the benchmark's shape: 8188 x 8188 out of the 8192 x 8192 stored image (ld 8192 / 8188)
    xin = x[: n - 2, : n - 2]
    a = torch.empty((n - 4, n - 4), device="cuda")
    b = torch.empty((n - 4, n - 4), device="cuda")
    ctx.blur3x3(xin, a)
    for variant in (1, 2, 3):
        b.zero_()
        ctx.blur3x3(xin, b, variant=variant)
        ctx.sync()
        assert torch.equal(a, b), variant
    # the whole 8188 x 8188 output against the oracle, bit for bit
    oracle.set_threads(oracle.max_threads())
    want = oracle.blur_xy(np.ascontiguousarray(xin.cpu().numpy()))
    oracle.set_threads(1)
    assert np.array_equal(a.cpu().numpy(), want)
    del want
    # whole image, unaligned output rows (8190 wide)
    c = torch.empty((n - 2, n - 2), device="cuda")
    ctx.blur3x3(x, c)
    ctx.sync()
    assert torch.equal(c[: n - 4, : n - 4], a)
    x.fill_(0.75)
    ctx.blur3x3(xin, a)
    ctx.sync()
    assert bool((a == 0.75).all())


def test_host_entry_point(ctx, oracle):
    x = np.random.default_rng(3).random((1500, 2051), dtype=np.float32)
    out = np.empty((1498, 2049), np.float32)
    ctx.blur3x3_host(x, out)
    assert np.array_equal(out, oracle.blur_xy(x))
    xs = x[:40, :50].copy()
    outs = np.empty((38, 48), np.float32)
    ctx.blur3x3_host(xs, outs)
    assert np.array_equal(outs, oracle.blur_xy(xs))
