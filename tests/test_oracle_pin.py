"""Pins the CPU oracle (oracle/gern_oracle.c): against the fixtures the reference itself produced
(tests/golden/golden.npz, made by tests/golden/make_golden.py), against the known answers of the
reference's own tests, and -- where oracle/_ref was built from the reference tree -- bit for bit
against the reference's compiled CPU code."""
import numpy as np
import pytest

from oracle import pyoracle


def test_random_fill_stream_matches_reference(golden):
    got = pyoracle.mt19937_uniform(32, -1.0, 1.0)
    assert np.array_equal(got, golden["fill32"])


def test_matmul_10x10_ascending_known_answer(oracle, golden):
    # test/test-cpu-mm.cpp:13-83: tiled result == untiled leaf, ascending inputs.
    a = np.arange(100, dtype=np.float32).reshape(10, 10)
    tiled = oracle.matmul_tiled(a, a, 5, 5, 5)
    assert np.array_equal(tiled, golden["mm10_c"])
    assert np.array_equal(tiled, oracle.matrix_multiply(a, a))
    assert np.array_equal(tiled, (a.astype(np.float64) @ a.astype(np.float64)).astype(np.float32))
    # the test's own nested tiling 5 -> 1 gives the same
    assert np.array_equal(oracle.matmul_tiled(a, a, 1, 1, 1), tiled)


def test_matmul_64_matches_gern_cpu_path(oracle, golden):
    a = pyoracle.mt19937_uniform(64 * 64, -1.0, 1.0).reshape(64, 64)
    assert np.array_equal(oracle.matmul_tiled(a, a, 16, 16, 16), golden["mm64_c"])


def test_matmul_512_matches_gern_cpu_path(oracle, golden):
    a = pyoracle.mt19937_uniform(512 * 512, -1.0, 1.0).reshape(512, 512)
    oracle.set_threads(oracle.max_threads())
    c = oracle.matmul_tiled(a, a, 64, 64, 64)
    oracle.set_threads(1)
    assert np.array_equal(c[::8, ::8], golden["mm512_sub"])
    assert c.astype(np.float64).sum() == float(golden["mm512_sum"])


def test_blur_matches_reference_fixtures(oracle, golden):
    for tag in ("asc", "rnd"):
        x = np.ascontiguousarray(golden[f"blur_in_{tag}"])
        assert np.array_equal(oracle.blur_xy(x), golden[f"blur_out_{tag}"])
        assert np.array_equal(oracle.blur_y(oracle.blur_x(x)), golden[f"blur_out_{tag}"])


def test_softmax_pieces_match_reference_fixtures(oracle, golden):
    x = np.ascontiguousarray(golden["sm_in"])
    mx = oracle.max_row_ref(x)
    assert np.array_equal(mx, golden["sm_max"])
    sub = oracle.subtract_vec_ref(mx, x)
    assert np.array_equal(sub, golden["sm_sub"])
    ex = oracle.exp_matrix(-sub)
    assert np.array_equal(ex, golden["sm_exp"])
    sm = oracle.sum_row(ex)
    assert np.array_equal(sm, golden["sm_sum"])
    assert np.array_equal(oracle.divide_vec(sm, ex), golden["sm_div"])
    # The corrected composition equals the chain of reference pieces whenever the row maximum is
    # positive (then the FLT_MIN seed is harmless) -- true for this fixture.
    assert (mx > 0).all()
    assert np.array_equal(oracle.softmax_rows(x), golden["sm_div"])


def test_softmax_against_fp64(oracle):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((64, 4096)) * 3).astype(np.float32)
    got = oracle.softmax_rows(x)
    want = oracle.softmax_rows_f64(x)
    rel = np.abs(got - want) / np.maximum(want, 1e-30)
    assert rel.max() < 1e-5
    assert np.allclose(got.sum(axis=1), 1.0, atol=1e-5)
    # all-negative rows: the corrected max seed matters
    y = -np.abs(x) - 5.0
    rel = np.abs(oracle.softmax_rows(y) - oracle.softmax_rows_f64(y)) / np.maximum(oracle.softmax_rows_f64(y), 1e-30)
    assert rel.max() < 1e-5


def test_bf16_helpers_and_gemm_attention_against_fp64(oracle):
    rng = np.random.default_rng(5)
    a = pyoracle.to_bf16_bits((rng.standard_normal((48, 96)) * 0.02).astype(np.float32))
    b = pyoracle.to_bf16_bits((rng.standard_normal((40, 96)) * 0.02).astype(np.float32))
    af, bf = pyoracle.bf16_bits_to_f32(a).astype(np.float64), pyoracle.bf16_bits_to_f32(b).astype(np.float64)
    c = oracle.gemm_bf16(a, b)
    want = af @ bf.T
    assert np.linalg.norm(c - want) / np.linalg.norm(want) < 1e-6
    assert np.array_equal(oracle.gemm_bf16(a, b, 8, 24), c[8:24])
    q = pyoracle.to_bf16_bits(rng.standard_normal((16, 128)).astype(np.float32))
    k = pyoracle.to_bf16_bits(rng.standard_normal((200, 128)).astype(np.float32))
    v = pyoracle.to_bf16_bits(rng.standard_normal((200, 128)).astype(np.float32))
    scale = 1.0 / np.sqrt(128.0)
    o = oracle.attention_bf16(q, k, v, scale)
    qf, kf, vf = (pyoracle.bf16_bits_to_f32(t).astype(np.float64) for t in (q, k, v))
    s = qf @ kf.T * scale
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    want = p @ vf
    assert np.linalg.norm(o - want) / np.linalg.norm(want) < 1e-5


def test_gemm_bf16_matches_reference_leaf_fixture(oracle, golden, golden_maker):
    # The fixtures hold gern::impl::matrix_multiply (cpu-matrix.h:196-212) on the bf16-rounded
    # operands widened to fp32: same ascending-k fp32 accumulation, so equality is exact.
    a, b = golden_maker.bf16_inputs("gemm96")
    assert np.array_equal(oracle.gemm_bf16(a, b), golden["gemmbf96_c"])
    a, b = golden_maker.bf16_inputs("gemm512")
    oracle.set_threads(oracle.max_threads())
    c = oracle.gemm_bf16(a, b)
    oracle.set_threads(1)
    assert np.array_equal(c[::8, ::8], golden["gemmbf512_sub"])
    assert c.astype(np.float64).sum() == float(golden["gemmbf512_sum"])


def test_attention_matches_reference_chain_fixture(oracle, golden, golden_maker):
    # matrix_multiply -> max_row -> subtract_vec -> exp_matrix -> sum_row -> divide_vec ->
    # matrix_multiply of the reference's CPU library on the same bf16-rounded Q, K, V.  The
    # restatement performs the same fp32 operations in the same order (the power-of-two scale
    # commutes with the rounding of the first product), so the bound is zero.
    q, k, v = golden_maker.bf16_inputs("attn")
    o = oracle.attention_bf16(q, k, v, golden_maker.ATTN_SCALE)
    assert np.array_equal(o, golden["attn_o"])


@pytest.mark.skipif(not pyoracle.Reference.available(), reason="oracle/_ref not built (no reference tree)")
class TestAgainstCompiledReference:
    """Bit-equality between the restatement and the reference's own compiled functions."""

    def test_matmul(self, oracle):
        ref = pyoracle.Reference()
        rng = np.random.default_rng(1)
        a = rng.uniform(-1, 1, (96, 64)).astype(np.float32)
        b = rng.uniform(-1, 1, (64, 80)).astype(np.float32)
        assert np.array_equal(oracle.matrix_multiply(a, b), ref.matrix_multiply(a, b))
        assert np.array_equal(oracle.matmul_tiled(a, b, 32, 16, 8), ref.matmul_tiled(a, b, 32, 16, 8))
        c0 = rng.uniform(-1, 1, (96, 80)).astype(np.float32)
        assert np.array_equal(oracle.matmul_tiled(a, b, 32, 16, 8, c0.copy()),
                              ref.matmul_tiled(a, b, 32, 16, 8, c0.copy()))

    def test_blur(self, oracle):
        ref = pyoracle.Reference()
        rng = np.random.default_rng(2)
        for shape in ((3, 3), (9, 17), (130, 259)):
            x = rng.random(shape, dtype=np.float32)
            assert np.array_equal(oracle.blur_x(x), ref.blur_x(x))
            assert np.array_equal(oracle.blur_y(x), ref.blur_y(x))
            assert np.array_equal(oracle.blur_xy(x), ref.blur_xy(x))

    def test_softmax_pieces(self, oracle):
        ref = pyoracle.Reference()
        x = (np.random.default_rng(4).standard_normal((17, 257)) * 3).astype(np.float32)
        assert np.array_equal(oracle.max_row_ref(x), ref.max_row(x))
        assert np.array_equal(oracle.sum_row(x), ref.sum_row(x))
        assert np.array_equal(oracle.exp_matrix(x), ref.exp_matrix(x))
        v = ref.max_row(x)
        assert np.array_equal(oracle.subtract_vec_ref(v, x), ref.subtract_vec(v, x))
        assert np.array_equal(oracle.divide_vec(v, x), ref.divide_vec(v, x))

    def test_bf16_gemm_and_chain(self, oracle, golden_maker):
        # what make_golden.py records, recomputed live and compared with the restatement
        ref = pyoracle.Reference()
        fx = golden_maker.reference_bf16_fixtures(ref)
        a, b = golden_maker.bf16_inputs("gemm96")
        assert np.array_equal(oracle.gemm_bf16(a, b), fx["gemmbf96_c"])
        q, k, v = golden_maker.bf16_inputs("attn")
        assert np.array_equal(oracle.attention_bf16(q, k, v, golden_maker.ATTN_SCALE), fx["attn_o"])

    def test_random_fill(self):
        ref = pyoracle.Reference()
        assert np.array_equal(ref.random_fill(7, 33, -1.0, 1.0).ravel(), pyoracle.mt19937_uniform(7 * 33, -1.0, 1.0))
