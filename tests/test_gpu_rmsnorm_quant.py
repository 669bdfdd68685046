"""RMSNorm fused in front of the activation quantisation, against the CPU restatement of
nsl_tensor_rmsnorm followed by the reference quantiser.

The normalised rows are floating point: the GPU sums the squares as a tree, the reference
sequentially, both in f64, so h may differ in the last bit of an f32 now and then.  Bars: h equal to
the oracle within 1 ulp (rel 2e-7) everywhere and bit-equal in at least 99.9 % of the elements; the
int8 codes are the exact quantisation of the GPU's own h (bit-exact against the oracle quantiser run
on that h), and differ from the oracle's end-to-end codes by at most 1 in at most 0.1 % of places."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, dev, host, perm_index  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


@pytest.mark.parametrize("M,K", [(1, 3200), (5, 8640), (33, 4096), (3, 64), (300, 3200)])
@pytest.mark.parametrize("xdt", ["f32", "bf16"])
def test_rmsnorm_then_quant(ops, oracle, M, K, xdt):
    rng = np.random.default_rng(M * 31 + K)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30.0, size=(M, 1))).astype(np.float32)
    if xdt == "bf16":
        x = bf16_round(x)
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    xd = dev(x).to(torch.bfloat16) if xdt == "bf16" else dev(x)
    out = ops.rmsnorm_act_quant_i8(xd, dev(w), 1e-5, plain=True, perm=True, return_h=True)
    torch.cuda.synchronize()
    h, q, qp = host(out["h"]), host(out["q_plain"]), host(out["q_perm"])
    h_ref = oracle.rmsnorm_f32(x, w, 1e-5)
    assert np.all(np.abs(h - h_ref) <= 2e-7 * np.abs(h_ref) + 1e-30)
    assert (h.view(np.uint32) == h_ref.view(np.uint32)).mean() >= 0.999
    # exact quantisation of the GPU's own h
    for r in range(M):
        s = oracle.absmax_scale_row(h[r])
        assert np.float32(host(out["scale"])[r]) == np.float32(s)
        assert np.array_equal(q[r], oracle.quantize_row_int8(h[r], s))
    assert np.array_equal(qp, q[:, perm_index(K)])
    assert np.array_equal(host(out["rowsum"]), q.astype(np.int32).sum(axis=1))
    # end to end against the oracle
    q_ref = np.stack([oracle.quantize_row_int8(h_ref[r], oracle.absmax_scale_row(h_ref[r])) for r in range(M)])
    d = np.abs(q.astype(np.int32) - q_ref.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 1e-3


def test_feeds_bitlinear(ops, oracle):
    """The fused prologue hands BitLinear the same accumulators as norm -> quantise -> matmul done apart."""
    rng = np.random.default_rng(7)
    M, N, K = 6, 200, 1024
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = np.ones(K, np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    layer = ops.BitLinear(dev(packed), 0.5)
    qa = ops.rmsnorm_act_quant_i8(dev(x), dev(w), 1e-5, return_h=True)
    y, acc = layer.forward_quantized(qa, return_acc=True)
    y2, acc2 = layer.forward(qa["h"], return_acc=True)
    torch.cuda.synchronize()
    assert np.array_equal(host(acc), host(acc2)) and np.array_equal(host(y), host(y2))


@pytest.mark.parametrize("M,K", [(1, 8640), (9, 8640), (64, 8640), (65, 3200), (130, 1024), (2, 64), (3, 12288), (2, 9600)])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_swiglu_then_quant(ops, oracle, M, K, dt):
    """h = silu(gate) * up in fp32 against float64 (rel 1e-6 + a floor for the tiny outputs), the
    codes exact for the GPU's own h, and within 1 of the float64 pipeline in at most 0.1 % of places."""
    rng = np.random.default_rng(M + K)
    g = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    u = rng.standard_normal((M, K)).astype(np.float32)
    if dt == "bf16":
        g, u = bf16_round(g), bf16_round(u)
    to = (lambda a: dev(a).to(torch.bfloat16)) if dt == "bf16" else dev
    out = ops.swiglu_act_quant_i8(to(g), to(u), plain=True, perm=True, return_h=True)
    torch.cuda.synchronize()
    h, q = host(out["h"]), host(out["q_plain"])
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    want = g64 / (1.0 + np.exp(-g64)) * u64
    assert np.all(np.abs(h - want) <= 1e-6 * np.abs(want) + 1e-9)
    for r in range(M):
        s = oracle.absmax_scale_row(h[r])
        assert np.float32(host(out["scale"])[r]) == np.float32(s)
        assert np.array_equal(q[r], oracle.quantize_row_int8(h[r], s))
    assert np.array_equal(host(out["q_perm"]), q[:, perm_index(K)])
    assert np.array_equal(host(out["rowsum"]), q.astype(np.int32).sum(axis=1))
    w32 = want.astype(np.float32)
    q_ref = np.stack([oracle.quantize_row_int8(w32[r], oracle.absmax_scale_row(w32[r])) for r in range(M)])
    d = np.abs(q.astype(np.int32) - q_ref.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 1e-3


def test_swiglu_on_column_slices(ops):
    """gate and up as the two halves of one fused projection output (row stride 2K)."""
    M, K = 5, 8640
    g = torch.Generator(device="cuda"); g.manual_seed(11)
    gu = torch.randn(M, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
    a = ops.swiglu_act_quant_i8(gu[:, :K], gu[:, K:], plain=True, return_h=True)
    b = ops.swiglu_act_quant_i8(gu[:, :K].contiguous(), gu[:, K:].contiguous(), plain=True, return_h=True)
    torch.cuda.synchronize()
    for key in ("h", "q_plain", "q_perm", "scale", "rowsum"):
        assert torch.equal(a[key], b[key]), key


def test_swiglu_cluster_rows_equal_single_cta_rows(ops):
    """Up to 64 rows a cluster of CTAs shares a row, beyond that one CTA takes it: same bits either way."""
    g_ = torch.Generator(device="cuda")
    g_.manual_seed(5)
    M, K = 70, 8640
    g = (torch.randn(M, K, device="cuda", generator=g_) * 3).to(torch.bfloat16)
    u = torch.randn(M, K, device="cuda", generator=g_).to(torch.bfloat16)
    big = ops.swiglu_act_quant_i8(g, u, plain=True, perm=True, return_h=True)
    small = ops.swiglu_act_quant_i8(g[:7].contiguous(), u[:7].contiguous(), plain=True, perm=True, return_h=True)
    torch.cuda.synchronize()
    for key in ("h", "q_plain", "q_perm", "scale", "rowsum"):
        assert torch.equal(big[key][:7], small[key]), key


def test_rmsnorm_bits_when_the_sum_of_squares_is_exact(ops, oracle):
    """Power-of-two magnitudes make the f64 sum of squares independent of the summation order, so every
    normalised value must equal the oracle's bit for bit -- including the elements that leave the fast
    path of the kernel's arithmetic (zeros, results below the normal float range)."""
    rng = np.random.default_rng(77)
    M, K = 6, 256
    x = (np.exp2(rng.integers(-12, 13, size=(M, K))) * rng.choice([-1.0, 1.0], size=(M, K))).astype(np.float32)
    x[:, 5] = 0.0
    x[:, 9] = -0.0
    x[:, 17] = np.float32(1.2e-38)
    x[:, 33] = np.float32(-3e-41)            # denormal input
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    w[40] = np.float32(1e-30)                # pushes one product below the normal range
    out = ops.rmsnorm_act_quant_i8(dev(x), dev(w), 1e-5, plain=True, perm=True, return_h=True)
    torch.cuda.synchronize()
    h, h_ref = host(out["h"]), oracle.rmsnorm_f32(x, w, 1e-5)
    assert np.array_equal(h.view(np.uint32), h_ref.view(np.uint32))
