"""Pins the CPU checker (C restatement and numpy mirror) to NSL's golden vectors.

Tolerances are the ones NSL's own tests state: int8 activations bit-exact,
f32 scales/outputs 1e-6 relative or 1e-7 absolute
(crates/nsl-codegen/tests/bitnet_reference.rs:245-327).
"""
import itertools

import numpy as np
import pytest


def close_f32(actual, expected):
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    ad = np.abs(actual - expected)
    rd = ad / np.maximum(np.abs(expected), 1e-30)
    return bool(np.all((rd <= 1e-6) | (ad < 1e-7)))


def test_forward_fixtures_c(kat, oracle):
    assert len(kat["forward"]) == 10
    for fx in kat["forward"]:
        r, h, o = fx["rows"], fx["hidden"], fx["out_dim"]
        x = np.array(fx["x"], np.float32).reshape(r, h)
        w = np.array(fx["w_kn"], np.int8).reshape(h, o)
        s, q, acc, y = oracle.forward_reference(x, w)
        assert close_f32(s, fx["scale"]), fx["name"]
        assert np.array_equal(q.ravel(), np.array(fx["q"], np.int8)), fx["name"]
        assert close_f32(y.ravel(), fx["y"]), fx["name"]
        # the packed-layout forward is the same arithmetic
        s2, q2, acc2, y2 = oracle.bitlinear_forward_packed(x, oracle.pack_weight_kn(w), o, 1.0)
        assert np.array_equal(q, q2) and np.array_equal(acc, acc2)
        assert np.array_equal(y.view(np.uint32), y2.view(np.uint32)), fx["name"]


def test_forward_fixtures_numpy_mirror(kat, oracle):
    for fx in kat["forward"]:
        r, h, o = fx["rows"], fx["hidden"], fx["out_dim"]
        x = np.array(fx["x"], np.float32).reshape(r, h)
        w = np.array(fx["w_kn"], np.int8).reshape(h, o)
        s, q, acc, y = oracle.np_bitlinear(x, w.T)
        assert close_f32(s, fx["scale"])
        assert np.array_equal(q.ravel(), np.array(fx["q"], np.int8)), fx["name"]
        assert close_f32(y.ravel(), fx["y"]), fx["name"]
        _, _, acc_c, y_c = oracle.forward_reference(x, w)
        assert np.array_equal(acc, acc_c)
        assert np.array_equal(y.view(np.uint32), y_c.view(np.uint32))


def test_absmax_quant_fixtures(kat, oracle):
    for fx in kat["absmax_quant"]:
        s = oracle.absmax_scale_row(fx["x"])
        assert abs(s - fx["scale"]) < 1e-6
        assert oracle.quantize_row_int8(fx["x"], s).tolist() == fx["q"]
        s2, q2 = oracle.np_act_quant(np.array([fx["x"]], np.float32))
        assert q2[0].tolist() == fx["q"]


def test_rounding_is_half_away(kat, oracle):
    row = kat["rounding_row"]
    s = oracle.absmax_scale_row(row["x"])
    assert s == 127.0
    assert oracle.quantize_row_int8(row["x"], s).tolist() == row["q"]
    assert oracle.np_act_quant(np.array([row["x"]], np.float32))[1][0].tolist() == row["q"]
    # the value where "add 0.5 then truncate" differs from a true half-away round
    x = np.array([0.49999997, -0.49999997, 127.0], np.float32)
    assert oracle.quantize_row_int8(x, 127.0).tolist() == [0, 0, 127]


def test_nan_inf_and_zero_rows(oracle):
    x = np.array([1.0, np.nan, -2.0, 0.5], np.float32)
    s = oracle.absmax_scale_row(x)
    assert s == 2.0
    assert oracle.quantize_row_int8(x, s).tolist() == [64, 0, -127, 32]
    assert oracle.np_act_quant(x[None])[1][0].tolist() == [64, 0, -127, 32]
    z = np.zeros(8, np.float32)
    assert oracle.absmax_scale_row(z) == 0.0
    assert oracle.quantize_row_int8(z, 0.0).tolist() == [0] * 8
    xi = np.array([1.0, np.inf, -3.0, 0.0], np.float32)
    assert oracle.absmax_scale_row(xi) == np.inf
    assert oracle.quantize_row_int8(xi, np.inf).tolist() == [0, 0, 0, 0]


def test_pack_layout(kat, oracle):
    p = kat["pack"]
    assert oracle.pack_trit_slice(p["trits"]).tolist() == [p["byte"]]
    assert oracle.unpack_byte_slice([p["byte"]]).tolist() == p["trits"]
    for b in p["invalid_bytes"]:
        assert oracle.try_unpack_byte(b) is None
    assert oracle.try_unpack_byte(p["byte"]) is not None
    for t in itertools.product([-1, 0, 1], repeat=4):
        b = oracle.pack_trit_slice(list(t))
        assert oracle.unpack_byte_slice(b).tolist() == list(t)
    trits = np.array([1, 0, -1, 1, 0, 0, -1, -1, 1, 1, 0, -1], np.int8)
    b = oracle.pack_trit_slice(trits)
    assert b.size == 3 and oracle.unpack_byte_slice(b).tolist() == trits.tolist()
    assert np.array_equal(oracle.np_pack_trits_nk(trits[None]).ravel(), b)
    with pytest.raises(ValueError):
        oracle.pack_trit_slice([2, 0, 0, 0])
    with pytest.raises(ValueError):
        oracle.pack_trit_slice([1, 0, 0])


def test_loader_vector(kat, oracle):
    ld = kat["loader"]
    packed, trits, scale = oracle.quantize_float_to_ternary(ld["values"])
    assert trits.tolist() == ld["trits"]
    assert abs(scale - ld["scale"]) < ld["scale_tol"]
    assert packed.tolist() == oracle.pack_trit_slice(ld["trits"]).tolist()
    p0, t0, s0 = oracle.quantize_float_to_ternary(np.zeros(8, np.float32))
    assert s0 == 0.0 and t0.tolist() == [0] * 8
    with pytest.raises(ValueError):
        oracle.quantize_float_to_ternary(np.ones(6, np.float32))


def test_f10_generator_reproduces_fixture(kat, oracle):
    fx = [f for f in kat["forward"] if f["name"].startswith("f10")][0]
    acts, w = oracle.make_f10_inputs()
    assert w.ravel().tolist() == fx["w_kn"]          # integer stream: exact
    assert np.allclose(acts, np.array(fx["x"], np.float32), rtol=2e-6, atol=1e-6)


def test_gpu_random_cases_have_negative_q(kat, oracle):
    for rows, hidden, out in kat["gpu_random_cases"]:
        acts, w = oracle.make_gpu_random_case(rows, hidden, out)
        assert acts.min() >= -1.0 and acts.max() < 1.0
        assert set(np.unique(w).tolist()) <= {-1, 0, 1}
        s, q, acc, y = oracle.forward_reference(acts, w)
        assert (q < 0).sum() > 0
        s2, q2, acc2, y2 = oracle.np_bitlinear(acts, w.T)
        assert np.array_equal(q, q2) and np.array_equal(acc, acc2)
        assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))


def test_threaded_oracle_is_identical(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 256)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(96, 256)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    a = oracle.bitlinear_forward_packed(x, packed, 96, 0.37, threads=1)
    b = oracle.bitlinear_forward_packed(x, packed, 96, 0.37, threads=4)
    for u, v in zip(a, b):
        assert np.array_equal(u, v)


# ------------------------------------------------------------------ W4 / AWQ / QuantizedTensor
def test_awq_unit_constants(kat, oracle):
    a = kat["awq"]
    s, z = oracle.awq_group_params(a["group"]["values"])
    assert abs(s - a["group"]["scale"]) < 1e-10 and z == a["group"]["zero"]
    c = a["clamp"]
    assert oracle.awq_quantize_int4(c["value"], c["scale"], c["zero"]) == c["q"]
    r = a["roundtrip"]
    q = oracle.awq_quantize_int4(r["value"], r["scale"], r["zero"])
    assert abs(oracle.awq_dequantize_int4(q, r["scale"], r["zero"]) - r["value"]) < r["scale"]
    sm = a["small_matrix"]
    w = (np.arange(16, dtype=np.float64) * 0.1).reshape(sm["k"], sm["n"])
    data, sc, ze = oracle.awq_quantize(w, sm["gs"])
    assert sc.size == sm["n"] and data.size == 8
    rec = oracle.awq_dequantize(data, sc, ze, sm["k"], sm["n"], sm["gs"])
    assert np.abs(rec - w).max() < sm["max_abs_err"]
    mm = a["matmul"]
    x = np.array(mm["input"], np.float64).reshape(mm["m"], mm["k"])
    wm = np.array(mm["weights"], np.float64).reshape(mm["k"], mm["n"])
    data, sc, ze = oracle.awq_quantize(wm, mm["gs"])
    got = oracle.awq_matmul(x, data, sc, ze, mm["k"], mm["n"], mm["gs"])
    ref = x @ wm
    assert np.all(np.abs(ref - got) < np.abs(ref) * mm["rel"] + mm["abs"])
    got4 = oracle.awq_matmul(x, data, sc, ze, mm["k"], mm["n"], mm["gs"], threads=3)
    assert np.array_equal(got, got4)


def test_awq_nibble_order(oracle):
    # flat index row*N+col, low nibble = even index (crates/nsl-runtime/src/awq.rs:82-98)
    w = np.array([[0.0, 15.0], [5.0, 10.0]], np.float64)  # K=2, N=2, one group per column
    data, sc, ze = oracle.awq_quantize(w, 2)
    # col0: min 0,max 5 -> codes 0,15 ; col1: min 10,max 15 -> codes 15,0
    assert data.tolist() == [0x0 | (0xF << 4), 0xF | (0x0 << 4)]


def test_qtensor_roundtrips_like_m16(oracle):
    """The tolerance asserts of NSL's tests/m16_test.nsl, on seeded inputs."""
    rng = np.random.default_rng(16)

    def close(a, b, rtol, atol):
        return np.all(np.abs(a - b) <= atol + rtol * np.abs(b))

    t = rng.standard_normal((4, 8))
    d, s, z = oracle.qtensor_quantize(t, 0, 0)
    assert close(oracle.qtensor_dequantize(d, s, z, t.shape, 0, 0), t, 0.1, 0.1)
    d, s, z = oracle.qtensor_quantize(t, 0, 1, 0)
    assert s.size == 4
    assert close(oracle.qtensor_dequantize(d, s, z, t.shape, 0, 1, 0), t, 0.1, 0.2)
    t = rng.standard_normal((8, 16))
    d, s, z = oracle.qtensor_quantize(t, 1, 2, 0, 4)
    # axis 0, gs 4 on [8,16]: the reference allocates 16*2 scale slots
    # (quantize.rs:72-96) but its loop fills only outer_size(1) * 2 groups of them.
    assert s.size == 32 and d.size == 64
    assert close(oracle.qtensor_dequantize(d, s, z, t.shape, 1, 2, 0, 4), t, 0.5, 0.5)
    t = np.full((4,), 0.5)
    d, s, z = oracle.qtensor_quantize(t, 1, 0)
    assert close(oracle.qtensor_dequantize(d, s, z, t.shape, 1, 0), t, 0.2, 0.2)
    t = np.full((8, 8), 3.0)
    d, s, z = oracle.qtensor_quantize(t, 0, 0)
    deq = oracle.qtensor_dequantize(d, s, z, t.shape, 0, 0)
    assert np.all(np.isfinite(deq)) and close(deq, t, 0.01, 0.01)
    x, w = rng.standard_normal((4, 8)), rng.standard_normal((8, 16))
    d, s, z = oracle.qtensor_quantize(w, 0, 1, 0)
    got = oracle.qtensor_matmul_mixed(x, d, s, z, w.shape, 0, 1, 0)
    assert close(got, x @ w, 1.0, 0.15)
    with pytest.raises(ValueError):
        oracle.qtensor_quantize(t, 3, 0)
    with pytest.raises(ValueError):
        oracle.qtensor_matmul_mixed(rng.standard_normal((4, 7)), d, s, z, w.shape, 0, 1, 0)


def test_qtensor_int4_group_axis1_is_the_w4a16_layout(oracle):
    """[N,K] INT4 per-group along axis 1: scale index n*G+g, nibble index n*K+k
    (crates/nsl-runtime/src/quantize.rs:366-417)."""
    rng = np.random.default_rng(3)
    n, k, gs = 6, 256, 128
    w = rng.standard_normal((n, k))
    d, s, z = oracle.qtensor_quantize(w, 1, 2, 1, gs)
    assert s.size == n * (k // gs) and d.size == n * k // 2
    deq = oracle.qtensor_dequantize(d, s, z, w.shape, 1, 2, 1, gs)
    codes = np.stack([d & 0xF, d >> 4], -1).reshape(n, k).astype(np.float64)
    sc = np.repeat(s.reshape(n, -1), gs, 1).astype(np.float64)
    zz = np.repeat(z.reshape(n, -1), gs, 1).astype(np.float64)
    assert np.array_equal(deq, (codes - zz) * sc)
    x = rng.standard_normal((3, k)).astype(np.float32)
    got = oracle.w4a16_matmul_nk(x, d, s, z, n, k, gs)
    want = x.astype(np.float64) @ deq.T
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
    assert np.array_equal(got, oracle.w4a16_matmul_nk(x, d, s, z, n, k, gs, threads=3))


def test_rmsnorm_restatement_known_answers(oracle):
    """nsl_tensor_rmsnorm (crates/nsl-runtime/src/tensor/mod.rs:3016-3035) on rows whose result is
    known in closed form: x = c * ones -> x / sqrt(c^2 + eps) * w; and against the same formula in
    numpy f64 with a sequential sum."""
    n = 8
    w = np.arange(1, n + 1, dtype=np.float32)
    x = np.full((1, n), 3.0, np.float32)
    want = (3.0 / np.sqrt(9.0 + 1e-5) * w.astype(np.float64)).astype(np.float32)
    assert np.array_equal(oracle.rmsnorm_f32(x, w, 1e-5)[0], want)
    rng = np.random.default_rng(1)
    x = rng.standard_normal((4, 100)).astype(np.float32)
    w = rng.standard_normal(100).astype(np.float32)
    got = oracle.rmsnorm_f32(x, w, 1e-5)
    for r in range(4):
        s = 0.0
        for v in x[r].astype(np.float64):
            s += v * v
        rms = np.sqrt(s / 100 + 1e-5)
        assert np.array_equal(got[r], (x[r].astype(np.float64) / rms * w.astype(np.float64)).astype(np.float32))
