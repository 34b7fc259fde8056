"""GEMM -> row softmax -> GEMM chain: CUDA path against the fp32 CPU oracle on the same
bf16-rounded inputs.  Tolerance: relative Frobenius error <= 1e-2."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def frob(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def bits(t):
    return np.ascontiguousarray(t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))


def make(nq, nkv, seed, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn((nq, 128), generator=g, device="cuda") * std).to(torch.bfloat16)
    k = (torch.randn((nkv, 128), generator=g, device="cuda") * std).to(torch.bfloat16)
    v = (torch.randn((nkv, 128), generator=g, device="cuda") * std).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("nq,nkv", [(128, 128), (128, 256), (256, 1024), (100, 200), (1, 1), (130, 129), (384, 4096)])
def test_against_oracle(ctx, oracle, nq, nkv):
    q, k, v = make(nq, nkv, nq + nkv)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / np.sqrt(128.0)
    ctx.attention_bf16(q, k, v, o, scale)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), scale)
    oracle.set_threads(1)
    assert frob(o.float().cpu().numpy(), want) <= 1e-2


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("nq,nkv", [(256, 128), (256, 1024), (100, 200), (130, 129), (1, 1), (640, 2048), (300, 190),
                                    (512, 384), (1100, 700)])
def test_kernel_variants(ctx, oracle, nq, nkv, variant):
    """One CTA per two Q tiles (1) and CTA pairs with two Q tiles per CTA (2), forced."""
    q, k, v = make(nq, nkv, nq * 7 + nkv)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / np.sqrt(128.0)
    ctx.attention_bf16(q, k, v, o, scale, variant=variant)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), scale)
    oracle.set_threads(1)
    assert frob(o.float().cpu().numpy(), want) <= 1e-2


def test_pair_kernel_rescale_path(ctx, oracle):
    nq, nkv = 256, 1024
    q, k, v = make(nq, nkv, 5, std=1.0)
    ramp = torch.linspace(0.2, 3.0, nkv, device="cuda").unsqueeze(1)
    k = (k.float() * ramp).to(torch.bfloat16)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q, k, v, o, 1.0, variant=2)
    ctx.sync()
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), 1.0)
    assert frob(o.float().cpu().numpy(), want) <= 1e-2


@pytest.mark.parametrize("variant", [None, 1, 2])
def test_peaked_rows_exercise_the_rescale(ctx, oracle, variant):
    """Large logits whose maximum keeps growing along kv force the running-max correction."""
    nq, nkv = 256, 1024
    q, k, v = make(nq, nkv, 5, std=1.0)
    ramp = torch.linspace(0.2, 3.0, nkv, device="cuda").unsqueeze(1)
    k = (k.float() * ramp).to(torch.bfloat16)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q, k, v, o, 1.0, variant=variant)
    ctx.sync()
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), 1.0)
    assert frob(o.float().cpu().numpy(), want) <= 1e-2


def test_uniform_scores_average_v(ctx):
    nq, nkv = 128, 512
    q = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    _, k, v = make(nq, nkv, 3)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q, k, v, o, 1.0)
    ctx.sync()
    want = v.float().mean(dim=0, keepdim=True).expand(nq, 128)
    assert float((o.float() - want).abs().max()) < 2e-2


def test_unsupported_head_dim_is_reported(ctx):
    from gern_b200 import api
    x = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(api.GernB200Error) as e:
        ctx.attention_bf16(x, x, x, x, 1.0)
    assert e.value.code == -3


def test_against_reference_chain_fixture(ctx, golden, golden_maker):
    """The CUDA kernels against the reference's own CPU leaves chained as matrix_multiply -> max_row ->
    subtract_vec -> exp_matrix -> sum_row -> divide_vec -> matrix_multiply
    (test/library/matrix/impl/cpu-matrix.h:134-212) on the same bf16-rounded Q, K, V."""
    q, k, v = (torch.from_numpy(t.view(np.int16)).cuda().view(torch.bfloat16) for t in golden_maker.bf16_inputs("attn"))
    for variant in (None, 1, 2):
        o = torch.zeros((q.shape[0], 128), dtype=torch.bfloat16, device="cuda")
        ctx.attention_bf16(q, k, v, o, golden_maker.ATTN_SCALE, variant=variant)
        ctx.sync()
        assert frob(o.float().cpu().numpy(), golden["attn_o"]) <= 1e-2, variant


def test_full_size_sampled(ctx, oracle):
    nq, nkv = 32768, 4096
    q, k, v = make(nq, nkv, 0)
    scale = 1.0 / np.sqrt(128.0)
    # two rows of every 128-row Q tile (so both tiles of every CTA, first and last CTA included),
    # at lanes that move through the tile, plus one whole tile
    idx = sorted({t * 128 + (t * 53) % 128 for t in range(nq // 128)} | {t * 128 + (t * 29 + 64) % 128 for t in range(nq // 128)}
                 | set(range(16000, 16128)))
    sel = torch.tensor(idx, device="cuda")
    oracle.set_threads(oracle.max_threads())
    want = oracle.attention_bf16(bits(q[sel]), bits(k), bits(v), scale)
    oracle.set_threads(1)
    outs = {}
    # 1: every CTA walks the whole K/V range of its pair (what the library picks at this size);
    # -1: equal runs per CTA, the shared pairs merged inside the kernel
    for splits in (1, -1):
        o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
        ctx.attention_bf16(q, k, v, o, scale, splits=splits)
        ctx.sync()
        got = o[sel].float().cpu().numpy()
        assert frob(got, want) <= 1e-2, splits
        # and row by row, so that one bad row cannot hide in the norm of 640
        err = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
        assert err.max() <= 2e-2, (splits, idx[int(err.argmax())], float(err.max()))
        outs[splits] = o
    # the two schedules differ by fp32 reassociation and one bf16 rounding, on every row
    diff = (outs[-1].float() - outs[1].float()).norm(dim=1) / outs[1].float().norm(dim=1)
    assert float(diff.max()) <= 1e-2
    # rows are independent: any row block alone gives the same bits (with the K/V range left whole)
    o2 = torch.zeros((256, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q[1024:1280].contiguous(), k, v, o2, scale, splits=1)
    ctx.sync()
    assert torch.equal(o2, outs[1][1024:1280])


def test_host_entry_point(ctx, oracle):
    from oracle import pyoracle
    rng = np.random.default_rng(1)
    q = pyoracle.to_bf16_bits(rng.standard_normal((200, 128)).astype(np.float32))
    k = pyoracle.to_bf16_bits(rng.standard_normal((300, 128)).astype(np.float32))
    v = pyoracle.to_bf16_bits(rng.standard_normal((300, 128)).astype(np.float32))
    o = np.zeros((200, 128), np.uint16)
    scale = 1.0 / np.sqrt(128.0)
    ctx.attention_bf16_host(q, k, v, o, scale)
    assert frob(pyoracle.bf16_bits_to_f32(o), oracle.attention_bf16(q, k, v, scale)) <= 1e-2


@pytest.mark.parametrize("scale", [0.0, -0.1, float("nan"), float("inf")])
def test_non_positive_or_non_finite_scale_is_refused(ctx, scale):
    """The kernels scale the row maximum of the raw scores, which is only right for scale > 0."""
    from gern_b200 import api
    q, k, v = make(128, 128, 1)
    o = torch.full((128, 128), 5.0, dtype=torch.bfloat16, device="cuda")
    for variant in (None, 2):
        with pytest.raises(api.GernB200Error) as e:
            ctx.attention_bf16(q, k, v, o, scale, variant=variant)
        assert e.value.code == -1 and "scale must be positive" in str(e.value)
    ctx.sync()
    assert bool((o == 5.0).all())


@pytest.mark.parametrize("nq,nkv,splits", [(256, 1024, 1), (256, 1024, 2), (256, 1024, 8), (100, 1000, 3), (640, 4096, 16),
                                           (130, 300, 5), (1, 129, 2), (512, 2048, 0), (300, 700, 64)])
def test_kv_ranges_split_across_ctas(ctx, oracle, nq, nkv, splits):
    """Few Q tiles: the K/V range is cut across CTAs (each keeps its unnormalised O, reference
    maximum and row sum) and a combine pass merges the ranges.  splits = 1 forces the unsplit
    kernel, 0 lets the library choose, more splits than blocks are clamped."""
    q, k, v = make(nq, nkv, nq * 3 + nkv + splits)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / np.sqrt(128.0)
    ctx.attention_bf16(q, k, v, o, scale, splits=splits)
    ctx.sync()
    oracle.set_threads(oracle.max_threads())
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), scale)
    oracle.set_threads(1)
    got = o.float().cpu().numpy()
    assert frob(got, want) <= 1e-2
    # the unsplit kernel on the same input: the combine adds only fp32 reassociation and one bf16 rounding
    o1 = torch.zeros_like(o)
    ctx.attention_bf16(q, k, v, o1, scale, splits=1)
    ctx.sync()
    assert frob(got, o1.float().cpu().numpy().astype(np.float64)) <= 4e-3


def test_split_ranges_with_growing_maxima(ctx, oracle):
    """Ranges whose reference maxima differ widely: the combine's 2^(m_s - M) weights must hold."""
    nq, nkv = 256, 2048
    q, k, v = make(nq, nkv, 9)
    ramp = torch.linspace(0.2, 3.0, nkv, device="cuda").unsqueeze(1)
    k = (k.float() * ramp).to(torch.bfloat16)
    o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q, k, v, o, 1.0, splits=8)
    ctx.sync()
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), 1.0)
    assert frob(o.float().cpu().numpy(), want) <= 1e-2


def test_split_output_with_a_padded_pitch(ctx, oracle):
    nq, nkv = 200, 1536
    q, k, v = make(nq, nkv, 21)
    o = torch.full((nq, 130), 3.0, dtype=torch.bfloat16, device="cuda")     # rows not 8-byte aligned
    ctx.attention_bf16(q, k, v, o[:, :128], 0.1, splits=4)
    ctx.sync()
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), 0.1)
    assert frob(o[:, :128].float().cpu().numpy(), want) <= 1e-2
    assert bool((o[:, 128:] == 3.0).all())


@pytest.mark.parametrize("nq,nkv", [(2048, 1024),      # 8 pairs x 8 blocks on 148 SMs: one block per CTA, 8 sharers per pair
                                    (5000, 3000),      # ragged rows and a ragged last block: runs of 4 of 24 blocks
                                    (40000, 1100),     # runs longer than a pair: whole pairs and shared ones in one CTA
                                    (300, 128),        # one block: nothing to share
                                    (38000, 2048)])    # 149 pairs: a second wave of whole pairs avoided
def test_equal_runs_merged_inside_the_kernel(ctx, oracle, nq, nkv):
    """splits = -1: the (Q tile pair, K/V block) units are dealt out in equal runs, one per CTA; a
    pair shared by several CTAs is merged by the one that finishes last.  Checked against the
    whole-pair schedule on every row, against the oracle on sampled rows, and launched twice so
    that the arrival counters are seen to come back to zero."""
    q, k, v = make(nq, nkv, nq + nkv)
    scale = 1.0 / np.sqrt(128.0)
    o1 = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
    ctx.attention_bf16(q, k, v, o1, scale, splits=1)
    outs = []
    for _ in range(2):
        o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
        ctx.attention_bf16(q, k, v, o, scale, splits=-1)
        outs.append(o)
    ctx.sync()
    for o in outs:
        diff = (o.float() - o1.float()).norm(dim=1) / o1.float().norm(dim=1)
        assert float(diff.max()) <= 1e-2
    # the same sharer normally merges on every launch; if another one did, the fp32 sums were taken
    # in another order: a few bf16 roundings fall the other way
    a, b = outs[0].float(), outs[1].float()
    assert float(((a - b).norm(dim=1) / a.norm(dim=1)).max()) <= 2e-3
    idx = sorted({(i * 9973) % nq for i in range(96)} | {0, nq - 1})
    sel = torch.tensor(idx, device="cuda")
    oracle.set_threads(oracle.max_threads())
    want = oracle.attention_bf16(bits(q[sel]), bits(k), bits(v), scale)
    oracle.set_threads(1)
    assert frob(outs[1][sel].float().cpu().numpy(), want) <= 1e-2


@pytest.mark.parametrize("nq,nkv", [(5000, 3000), (300, 128), (38000, 2048)])
def test_runs_of_whole_pairs_give_the_bits_of_the_whole_pair_kernel(ctx, nq, nkv):
    """splits = -9: the segment-walking instantiation with runs of exactly one pair (what the library
    picks for whole pairs from 16 K/V blocks up): nothing is shared, so the bits are those of the
    plain whole-pair kernel (splits = 1)."""
    q, k, v = make(nq, nkv, nq + 7 * nkv)
    outs = []
    for splits in (1, -9):
        o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
        ctx.attention_bf16(q, k, v, o, 0.11, splits=splits)
        outs.append(o)
    ctx.sync()
    assert torch.equal(outs[0], outs[1])


def test_equal_runs_after_a_different_shape_and_with_a_padded_pitch(ctx, oracle):
    """The counters and the partial-result workspace are shared by all launches of a context."""
    scale = 0.1
    for nq, nkv in ((2048, 1024), (700, 2500), (2048, 1024)):
        q, k, v = make(nq, nkv, nq)
        o = torch.full((nq, 130), 3.0, dtype=torch.bfloat16, device="cuda")     # rows not 8-byte aligned
        ctx.attention_bf16(q, k, v, o[:, :128], scale, splits=-1)
        ctx.sync()
        oracle.set_threads(oracle.max_threads())
        want = oracle.attention_bf16(bits(q[:256]), bits(k), bits(v), scale)
        oracle.set_threads(1)
        assert frob(o[:256, :128].float().cpu().numpy(), want) <= 1e-2
        assert bool((o[:, 128:] == 3.0).all())


def test_cluster_entry_point(ctx, oracle):
    """gb200_attention_bf16_cluster: clusters of one and of two thread blocks give the same bits
    (with the K/V range left whole); other sizes are refused."""
    from gern_b200 import api
    import ctypes
    nq, nkv = 1100, 256            # few K/V blocks: no range splitting in either kernel
    q, k, v = make(nq, nkv, 77)
    outs = []
    for cluster_x in (1, 2):
        o = torch.zeros((nq, 128), dtype=torch.bfloat16, device="cuda")
        rc = api.lib.gb200_attention_bf16_cluster(ctx.handle, q.data_ptr(), 128, k.data_ptr(), 128, v.data_ptr(), 128,
                                                  o.data_ptr(), 128, nq, nkv, 128, ctypes.c_float(0.09), cluster_x, None)
        assert rc == 0
        ctx.sync()
        outs.append(o)
    assert torch.equal(outs[0], outs[1])
    want = oracle.attention_bf16(bits(q), bits(k), bits(v), 0.09)
    assert frob(outs[0].float().cpu().numpy(), want) <= 1e-2
    assert api.lib.gb200_attention_bf16_cluster(ctx.handle, q.data_ptr(), 128, k.data_ptr(), 128, v.data_ptr(), 128,
                                                outs[0].data_ptr(), 128, nq, nkv, 128, ctypes.c_float(0.09), 3, None) == -3
