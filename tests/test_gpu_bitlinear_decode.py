"""BitLinear decode (M <= 16) on shapes that reach the tensor-memory streaming kernel
(ternary_decode_kernel): packed weights of 12 MB and more at M <= 4, 28 MB at M <= 8, any size
above that.  Same bar as everywhere: int32 accumulators bit-exact, fp32 outputs bit-equal to the
CPU oracle's separately rounded finalisation."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, bits_equal, dev, host  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


@pytest.fixture(scope="module")
def big(oracle):
    """[16400, 3072] ternary, 12.6 MB packed: N is not a multiple of the 128-row tile."""
    rng = np.random.default_rng(2024)
    N, K = 16400, 3072
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    return N, K, oracle.np_pack_trits_nk(trits)


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("xdt", ["f32", "bf16"])
def test_large_weight_small_batch(ops, oracle, big, M, xdt):
    N, K, packed = big
    rng = np.random.default_rng(M)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if M > 1:
        x[1, :] *= 37.5                      # rows with different scales
    if xdt == "bf16":
        x = bf16_round(x)
    layer = ops.BitLinear(dev(packed), 0.043)
    xd = dev(x).to(torch.bfloat16) if xdt == "bf16" else dev(x)
    y, acc = layer.forward(xd, return_acc=True)
    torch.cuda.synchronize()
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.043, threads=8)
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)


def test_zero_row_and_nan(ops, oracle, big):
    N, K, packed = big
    x = np.zeros((2, K), np.float32)
    x[1, 5] = np.nan
    x[1, 6:40] = 3.0
    layer = ops.BitLinear(dev(packed), 1.0)
    y, acc = layer.forward(dev(x), return_acc=True)
    torch.cuda.synchronize()
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 1.0, threads=8)
    assert np.array_equal(host(acc), acc_ref)
    assert np.array_equal(np.isnan(host(y)), np.isnan(y_ref))
    assert bits_equal(np.nan_to_num(host(y)), np.nan_to_num(y_ref))


@pytest.mark.parametrize("M,N,K", [(7, 36000, 3200), (16, 1000, 8640), (12, 130, 64), (9, 257, 1088), (16, 8640, 3200)])
def test_batched_decode_shapes(ops, oracle, M, N, K):
    rng = np.random.default_rng(M * 131 + N)
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    layer = ops.BitLinear(dev(packed), 0.5)
    y, acc = layer.forward(dev(x), return_acc=True)
    torch.cuda.synchronize()
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.5, threads=8)
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)


def test_bias_residual_bf16_out(ops, oracle):
    rng = np.random.default_rng(5)
    M, N, K = 12, 777, 2048
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    _, _, _, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.25, threads=4)
    want = ((y_ref + bias[None, :]).astype(np.float32) + res).astype(np.float32)      # separate roundings
    layer = ops.BitLinear(dev(packed), 0.25)
    y = layer.forward(dev(x), bias=dev(bias), residual=dev(res))
    yb = layer.forward(dev(x), bias=dev(bias), residual=dev(res), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert bits_equal(host(y), want)
    assert bits_equal(host(yb), bf16_round(want))


def test_no_wait_expired(ops):
    assert ops.device_status() == 0
