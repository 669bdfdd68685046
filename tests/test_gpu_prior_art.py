"""The benchmark's GPU baseline (oracle/gpu_prior_art.cu: the design of the one kernel NSL emits for a BitLinear
forward pass, restated) computes the reference's arithmetic: accumulators and fp32 outputs equal to the CPU
checker's, and therefore to the library's, bit for bit.  A baseline that computed something else would make the
comparison in the benchmark meaningless."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bits_equal, dev, host  # noqa: E402
from nsl_b200 import ops  # noqa: E402
from oracle import oracle as o  # noqa: E402


@pytest.mark.parametrize("M,N,K", [(1, 130, 256), (5, 8640, 3200), (33, 200, 8640), (2, 128, 4)])
def test_prior_art_kernel_equals_the_checker_and_the_library(M, N, K):
    rng = np.random.default_rng(M + N + K)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = o.np_pack_trits_nk(trits)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.01, 50.0, size=(M, 1))).astype(np.float32)
    x[0, : K // 2] = 0.0
    if M > 1:
        x[1] = 0.0                                            # a zero row: scale 0, all codes 0
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    _, _, acc_ref, y_ref = o.bitlinear_forward_packed(x, packed, N, 0.043)
    y_ref = ((y_ref + bias[None, :]).astype(np.float32) + res).astype(np.float32)
    y, acc = o.gpu_prior_art_bitlinear(dev(x), dev(packed), 0.043, return_acc=True, bias=dev(bias), residual=dev(res))
    torch.cuda.synchronize()
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)
    if K % 64 == 0:
        y2 = ops.BitLinear(dev(packed), 0.043).forward(dev(x), bias=dev(bias), residual=dev(res))
        torch.cuda.synchronize()
        assert bits_equal(host(y2), host(y))


@pytest.mark.parametrize("M", [1, 16, 40])
def test_prior_art_w4_route_dequantises_like_the_checker(M):
    """The W4 baseline (dequantise the whole weight, then a dense TF32 matmul): its dequantised weights equal
    dequantize_val's (q - zp) * scale in f64, rounded once, bit for bit, and its product agrees with the f64 product of
    those weights within TF32's rounding of the operands (1e-2 of the row rms)."""
    rng = np.random.default_rng(M)
    N, K, GS = 320, 512, 128
    codes = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    scale = (np.abs(rng.standard_normal((N, K // GS))) * 0.003).astype(np.float32)
    zp = rng.integers(0, 16, size=(N, K // GS), dtype=np.uint8)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda().to(torch.bfloat16)
    w_gpu = o.gpu_prior_art_w4_dequant(dev(codes), dev(scale), dev(zp), GS)
    y = o.gpu_prior_art_w4_matmul(x, dev(codes), dev(scale), dev(zp), GS)
    torch.cuda.synchronize()
    q = np.stack([codes & 15, codes >> 4], axis=-1).reshape(N, K).astype(np.float64)
    w_ref = ((q - np.repeat(zp, GS, axis=1).astype(np.float64)) * np.repeat(scale, GS, axis=1).astype(np.float64)).astype(np.float32)
    assert bits_equal(host(w_gpu), w_ref)
    want = x.double().cpu().numpy() @ w_ref.astype(np.float64).T
    rms = np.sqrt((want ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(host(y).astype(np.float64) - want) <= 1e-2 * rms)
