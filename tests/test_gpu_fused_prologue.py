"""nslq_bitlinear_forward_rmsnorm / _swiglu: the RMSNorm or SiLU(gate)*up in front of a projection, formed
inside the projection's launch for one token (the same call issues the two launches above that).

Bars.  (1) Where the f64 sum of squares does not depend on the summation order (power-of-two magnitudes)
the int32 accumulators and the fp32 outputs must equal the CPU checker's norm -> quantise -> matmul bit
for bit.  (2) On Gaussian rows the normalised value may differ from the checker's in the last bit of an
f32 now and then (tree against sequential f64 sum), which can move a code by one: the accumulators must
then equal, exactly, those of the library's own two-launch path in at least 99 % of the outputs and
the outputs must agree with the checker within 2e-3 of the row's rms.  (3) SiLU(gate)*up is fp32
arithmetic identical to nslq_swiglu_act_quant_i8: accumulators bit-equal to the two-launch path."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, bits_equal, dev, host  # noqa: E402
from nsl_b200 import ops  # noqa: E402
from nsl_b200 import NslqError  # noqa: E402
from oracle import oracle as o  # noqa: E402


def _layer(rng, N, K, ws=0.043):
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = o.np_pack_trits_nk(trits)
    return packed, ops.BitLinear(dev(packed), ws), ws


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(200, 256), (96, 3200), (130, 8640), (64, 11008)])
def test_rmsnorm_prologue_exact_when_the_sum_is_exact(M, N, K):
    rng = np.random.default_rng(M * 1000 + K)
    packed, layer, ws = _layer(rng, N, K)
    x = (np.exp2(rng.integers(-6, 7, size=(M, K))) * rng.choice([-1.0, 1.0], size=(M, K))).astype(np.float32)
    x[:, 5] = 0.0
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    h = o.rmsnorm_f32(x, w, 1e-5)
    _, _, acc_ref, y_ref = o.bitlinear_forward_packed(h, packed, N, ws)
    y_ref = ((y_ref + bias[None, :]).astype(np.float32) + res).astype(np.float32)      # separate roundings
    y, acc = layer.forward_rmsnorm(dev(x), dev(w), 1e-5, return_acc=True, bias=dev(bias), residual=dev(res))
    torch.cuda.synchronize()
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)
    assert ops.device_status() == 0


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7])
@pytest.mark.parametrize("xdt", ["f32", "bf16"])
def test_rmsnorm_prologue_on_gaussian_rows(M, xdt):
    rng = np.random.default_rng(M + 17)
    N, K = 320, 3200
    packed, layer, ws = _layer(rng, N, K)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30.0, size=(M, 1))).astype(np.float32)
    if xdt == "bf16":
        x = bf16_round(x)
    xd = dev(x).to(torch.bfloat16) if xdt == "bf16" else dev(x)
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    y, acc = layer.forward_rmsnorm(xd, dev(w), 1e-5, return_acc=True)
    qa = ops.rmsnorm_act_quant_i8(xd, dev(w), 1e-5, plain=False, perm=True)
    y2, acc2 = layer.forward_quantized(qa, return_acc=True)
    torch.cuda.synchronize()
    assert (host(acc) == host(acc2)).mean() >= 0.99
    h = o.rmsnorm_f32(x, w, 1e-5)
    _, _, _, y_ref = o.bitlinear_forward_packed(h, packed, N, ws)
    rms = np.sqrt((y_ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(host(y) - y_ref) <= 2e-3 * rms)
    if M > 1:                                             # above one token the call is the two launches
        assert np.array_equal(host(acc), host(acc2))


@pytest.mark.parametrize("M", [1, 2, 3, 4, 6])
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("N,K", [(192, 8640), (100, 1024)])
def test_swiglu_prologue_equals_the_two_launches(M, dt, N, K):
    rng = np.random.default_rng(M * 7 + K)
    packed, layer, ws = _layer(rng, N, K)
    g = (rng.standard_normal((M, K)) * 3).astype(np.float32)
    u = rng.standard_normal((M, K)).astype(np.float32)
    if dt == "bf16":
        g, u = bf16_round(g), bf16_round(u)
    to = (lambda a: dev(a).to(torch.bfloat16)) if dt == "bf16" else dev
    res = rng.standard_normal((M, N)).astype(np.float32)
    y, acc = layer.forward_swiglu(to(g), to(u), return_acc=True, residual=dev(res))
    qa = ops.swiglu_act_quant_i8(to(g), to(u), plain=False, perm=True, return_h=True)
    y2, acc2 = layer.forward_quantized(qa, return_acc=True, residual=dev(res))
    torch.cuda.synchronize()
    assert np.array_equal(host(acc), host(acc2))
    assert bits_equal(host(y), host(y2))
    # and the checker's BitLinear on the library's own h
    _, _, acc_ref, y_ref = o.bitlinear_forward_packed(host(qa["h"]), packed, N, ws)
    y_ref = (y_ref + res).astype(np.float32)
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)


def test_errors():
    rng = np.random.default_rng(3)
    _, layer, _ = _layer(rng, 64, 256)
    x = torch.zeros(2, 256, device="cuda")
    with pytest.raises(ValueError):
        layer.forward_rmsnorm(x, torch.ones(128, device="cuda"))
    with pytest.raises(ValueError):
        layer.forward_swiglu(x, torch.zeros(2, 256, device="cuda", dtype=torch.bfloat16))
    _, odd, _ = _layer(rng, 64, 48)                        # K % 64 != 0: no fused form
    with pytest.raises(NslqError):
        odd.forward_rmsnorm(torch.zeros(1, 48, device="cuda"), torch.ones(48, device="cuda"))


@pytest.mark.parametrize("M", [1, 2, 5, 8, 16, 40])
@pytest.mark.parametrize("normed", [True, False])
@pytest.mark.parametrize("K,Ns", [(3200, (3200, 200, 72)), (2560, (6912, 6912)), (8640, (130,)), (8640, (3200, 40)),
                                  (256, (64, 64, 64, 50))])
def test_sibling_projections_in_one_call_equal_the_separate_calls(M, normed, K, Ns):
    """nslq_bitlinear_forward_multi: q/k/v (gate/up) of the same rows; every output has the bits of the
    layer's own forward_rmsnorm / forward call, and in an exact-sum case those of the CPU checker."""
    rng = np.random.default_rng(M * 31 + K + len(Ns))
    layers = [_layer(rng, N, K, ws=0.02 + 0.01 * i) for i, N in enumerate(Ns)]
    x = (np.exp2(rng.integers(-6, 7, size=(M, K))) * rng.choice([-1.0, 1.0], size=(M, K))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, size=K).astype(np.float32)
    xd, wd = dev(x), dev(w)
    for out_dtype in (torch.float32, torch.bfloat16):
        ys = ops.BitLinear.forward_multi([l[1] for l in layers], xd, wd if normed else None, 1e-5, out_dtype=out_dtype)
        torch.cuda.synchronize()
        for (packed, layer, ws), y, N in zip(layers, ys, Ns):
            one = layer.forward_rmsnorm(xd, wd, 1e-5, out_dtype=out_dtype) if normed else layer.forward(xd, out_dtype=out_dtype)
            torch.cuda.synchronize()
            assert y.shape == (M, N)
            assert torch.equal(y.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32),
                               one.view(torch.int16 if out_dtype == torch.bfloat16 else torch.int32))
            if out_dtype == torch.float32:
                h = o.rmsnorm_f32(x, w, 1e-5) if normed else x
                _, _, _, y_ref = o.bitlinear_forward_packed(h, packed, N, ws)
                assert bits_equal(host(y), y_ref)
    assert ops.device_status() == 0


def test_sibling_projections_refuse_mismatched_layers():
    rng = np.random.default_rng(3)
    a = _layer(rng, 64, 256)[1]
    b = _layer(rng, 64, 320)[1]
    x = dev(rng.standard_normal((1, 256)).astype(np.float32))
    with pytest.raises(ValueError):
        ops.BitLinear.forward_multi([a, b], x)
    with pytest.raises(ValueError):
        ops.BitLinear.forward_multi([a] * 5, x)
