"""Single-process multi-GPU entry points (`gb200_*_sharded`): every shard against the oracle.

With one GPU the shards are placed on the same device through separate contexts, which runs the
whole host path (argument checks, per-shard launches, halo pointers into the next band); with two
or more GPUs the same tests place one shard per device, and the blur halo is a peer load."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def frob(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) /
                 max(np.linalg.norm(want.astype(np.float64)), 1e-30))


def placements():
    """(label, device per shard) for 3 shards: all on cuda:0, and spread when more GPUs exist."""
    out = [("one-device", [0, 0, 0])]
    n = torch.cuda.device_count()
    if n >= 2:
        out.append(("spread", [g % n for g in range(3)]))
    return out


@pytest.fixture(scope="module")
def ctxs():
    from gern_b200 import api
    made = {}

    def get(device):
        if device not in made:
            made[device] = []
        c = api.Context(device)
        made[device].append(c)
        return c

    yield get
    for cs in made.values():
        for c in cs:
            c.sync()
            c.close()


def split_rows(total, parts):
    base = total // parts
    cuts = [0]
    for g in range(parts):
        cuts.append(cuts[-1] + base + (1 if g < total % parts else 0))
    return cuts


@pytest.mark.parametrize("label,devices", placements())
def test_blur_bands(ctxs, oracle, label, devices):
    from gern_b200 import api
    rows, cols = 389, 1030
    x = np.random.default_rng(11).random((rows, cols), dtype=np.float32)
    want = oracle.blur_xy(x)
    cuts = split_rows(rows, len(devices))
    parts, outs = [], []
    for g, dev in enumerate(devices):
        band = torch.from_numpy(x[cuts[g]:cuts[g + 1]]).to(f"cuda:{dev}")
        n_out = band.shape[0] - (2 if g == len(devices) - 1 else 0)
        out = torch.full((n_out, cols - 2), -7.0, dtype=torch.float32, device=f"cuda:{dev}")
        parts.append((ctxs(dev), band, out))
        outs.append(out)
    api.blur3x3_sharded(parts)
    for c, _, _ in parts:
        c.sync()
    got = np.concatenate([o.cpu().numpy() for o in outs], axis=0)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("label,devices", placements())
def test_softmax_row_blocks(ctxs, oracle, label, devices):
    from gern_b200 import api
    rows, cols = 301, 4096
    x = (np.random.default_rng(3).standard_normal((rows, cols)) * 3).astype(np.float32)
    want = oracle.softmax_rows(x)
    cuts = split_rows(rows, len(devices))
    parts, outs = [], []
    for g, dev in enumerate(devices):
        xs = torch.from_numpy(x[cuts[g]:cuts[g + 1]]).to(f"cuda:{dev}")
        out = torch.empty_like(xs)
        parts.append((ctxs(dev), xs, out))
        outs.append(out)
    api.softmax_rows_sharded(parts)
    for c, _, _ in parts:
        c.sync()
    got = np.concatenate([o.cpu().numpy() for o in outs], axis=0)
    rel = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert rel[want > 1e-30].max() <= 1e-5


@pytest.mark.parametrize("label,devices", placements())
def test_gemm_m_panels(ctxs, oracle, label, devices):
    from gern_b200 import api
    M, N, K = 700, 384, 512
    g0 = torch.Generator().manual_seed(5)
    A = (torch.randn((M, K), generator=g0) * 0.5).to(torch.bfloat16)
    Bt = (torch.randn((N, K), generator=g0) * 0.5).to(torch.bfloat16)
    want = oracle.gemm_bf16(bits(A), bits(Bt))
    cuts = split_rows(M, len(devices))
    parts, outs = [], []
    for g, dev in enumerate(devices):
        a = A[cuts[g]:cuts[g + 1]].to(f"cuda:{dev}")
        b = Bt.to(f"cuda:{dev}")
        c = torch.zeros((a.shape[0], N), dtype=torch.bfloat16, device=f"cuda:{dev}")
        parts.append((ctxs(dev), a, c, b))
        outs.append(c)
    api.gemm_bf16_sharded(parts)
    for c, *_ in parts:
        c.sync()
    got = np.concatenate([o.float().cpu().numpy() for o in outs], axis=0)
    assert frob(got, want) <= 1e-2


@pytest.mark.parametrize("label,devices", placements())
def test_attention_q_blocks(ctxs, oracle, label, devices):
    from gern_b200 import api
    nq, nkv, d = 500, 384, 128
    g0 = torch.Generator().manual_seed(9)
    Q = torch.randn((nq, d), generator=g0).to(torch.bfloat16)
    K = torch.randn((nkv, d), generator=g0).to(torch.bfloat16)
    V = torch.randn((nkv, d), generator=g0).to(torch.bfloat16)
    scale = 1.0 / np.sqrt(d)
    want = oracle.attention_bf16(bits(Q), bits(K), bits(V), scale)
    cuts = split_rows(nq, len(devices))
    parts, outs = [], []
    for g, dev in enumerate(devices):
        q = Q[cuts[g]:cuts[g + 1]].to(f"cuda:{dev}")
        o = torch.zeros_like(q)
        parts.append((ctxs(dev), q, o, K.to(f"cuda:{dev}"), V.to(f"cuda:{dev}")))
        outs.append(o)
    api.attention_bf16_sharded(parts, scale)
    for c, *_ in parts:
        c.sync()
    got = np.concatenate([o.float().cpu().numpy() for o in outs], axis=0)
    assert frob(got, want) <= 1e-2


def test_bad_shard_arguments(ctxs):
    from gern_b200 import api
    c = ctxs(0)
    x = torch.zeros((1, 64), device="cuda")
    o = torch.zeros((1, 62), device="cuda")
    with pytest.raises(api.GernB200Error) as e:     # a band lends 2 rows: 1 row is not a band
        api.blur3x3_sharded([(c, x, o), (c, x, o)])
    assert e.value.code == -1
    arr = (api.Shard * 1)()                          # ctx NULL
    assert api.lib.gb200_softmax_rows_f32_sharded(arr, 1, 64, 64, 64) == -1
    assert api.lib.gb200_softmax_rows_f32_sharded(arr, 0, 64, 64, 64) == -1
    assert api.lib.gb200_softmax_rows_f32_sharded(None, 1, 64, 64, 64) == -1
    a = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    arr[0] = api.Shard(c.handle, a.data_ptr(), a.data_ptr(), 128, None, None, None)
    assert api.lib.gb200_gemm_bf16_sharded(arr, 1, 64, 64, 64, 64, 64) == -1   # B replica missing


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs the halo rows on a second GPU")
def test_band_with_halo_rows_on_another_device_over_many_steps(ctxs, oracle):
    """A halo pointer into another device's memory is not read by the kernel: a copy engine brings
    the two rows into the next of 32 local slots and sets the slot's flag.  A hundred steps with
    fresh halo rows each time walk the ring three times (slot reuse behind the event of the launch
    32 steps back); every step's last output rows are compared bit for bit with the oracle, and a
    second band size in between makes the ring grow."""
    from gern_b200 import api
    c0 = ctxs(0)
    # small bands read a remote halo directly by default: make this context prefetch at any size
    assert api.lib.gb200_ctx_set_halo_prefetch_min_bytes(c0.handle, ctypes.c_longlong(0)) == 0
    rng = np.random.default_rng(5)
    for rows, cols, steps in ((64, 1024, 70), (48, 2048, 40), (64, 1024, 10)):
        band = rng.random((rows, cols), dtype=np.float32)
        x = torch.from_numpy(band).to("cuda:0")
        out = torch.empty((rows, cols - 2), device="cuda:0")
        halos = [rng.random((2, cols), dtype=np.float32) for _ in range(steps)]
        remote = [torch.from_numpy(h).to("cuda:1") for h in halos]    # complete before any call
        torch.cuda.synchronize("cuda:1")
        outs = []
        for s in range(steps):
            c0.blur3x3_band(x, remote[s], out)
            outs.append(out[-4:].clone())          # stream order: after this step's kernel
        c0.sync()
        for s in range(steps):
            want = oracle.blur_xy(np.concatenate([band[-4:], halos[s]]))
            assert np.array_equal(outs[s].cpu().numpy(), want), (rows, cols, s)
        assert np.array_equal(out[:8].cpu().numpy(), oracle.blur_xy(band[:10]))
    # and the same band with the default threshold: the kernel reads the other device's rows itself
    assert api.lib.gb200_ctx_set_halo_prefetch_min_bytes(c0.handle, ctypes.c_longlong(48 << 20)) == 0
    c0.blur3x3_band(x, remote[-1], out)
    c0.sync()
    assert np.array_equal(out[-4:].cpu().numpy(), oracle.blur_xy(np.concatenate([band[-4:], halos[-1]])))
