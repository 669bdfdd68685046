"""BitLinear prefill GEMM (tcgen05, M > 16) through the C ABI vs the CPU oracle:
int32 accumulators and fp32 outputs bit-exact; no bounded wait may expire."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, bits_equal, dev, host  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def case(rng, M, N, K):
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    return x, trits


@pytest.mark.parametrize("M,N,K", [
    (17, 192, 128), (64, 256, 64), (128, 192, 256), (129, 200, 320), (300, 448, 1088),
    (128, 8, 128), (40, 260, 192), (257, 1000, 3200), (130, 3200, 8640),
    (64, 3200, 8640), (33, 19200, 640), (50, 8640, 3200),     # the 64-token tile: long K, two tiles per CTA
])
def test_gemm_shapes(ops, oracle, M, N, K):
    rng = np.random.default_rng(M * 1009 + N * 17 + K)
    x, trits = case(rng, M, N, K)
    packed = oracle.np_pack_trits_nk(trits)
    layer = ops.BitLinear(dev(packed), 0.0173)
    y, acc = layer.forward(dev(x), return_acc=True)
    assert ops.device_status() == 0
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.0173, threads=8)
    assert np.array_equal(host(acc), acc_ref)
    assert bits_equal(host(y), y_ref)
    y2 = layer.forward(dev(x))                    # without the accumulator output
    assert ops.device_status() == 0
    assert bits_equal(host(y2), y_ref)


def test_gemm_epilogue_options(ops, oracle):
    rng = np.random.default_rng(99)
    M, N, K = 150, 320, 256
    x, trits = case(rng, M, N, K)
    packed = oracle.np_pack_trits_nk(trits)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    _, _, _, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.5, threads=4)
    want = ((y_ref + bias[None, :]).astype(np.float32) + res).astype(np.float32)
    layer = ops.BitLinear(dev(packed), 0.5)
    y = layer.forward(dev(x), bias=dev(bias), residual=dev(res))
    assert bits_equal(host(y), want)
    yb = layer.forward(dev(x), out_dtype=torch.bfloat16)
    assert bits_equal(host(yb), bf16_round(y_ref))
    yh = layer.forward(dev(x), out_dtype=torch.float16)
    assert np.array_equal(host(yh), y_ref.astype(np.float16))
    assert ops.device_status() == 0


def test_gemm_matches_gemv_and_shards(ops, oracle):
    """Rows of a long batch equal the same rows run as decode calls; row shards of W equal the full result."""
    rng = np.random.default_rng(5)
    M, N, K = 96, 384, 512
    x, trits = case(rng, M, N, K)
    packed = oracle.np_pack_trits_nk(trits)
    layer = ops.BitLinear(dev(packed), 0.25)
    xd = dev(x)
    y_full = layer.forward(xd)
    y_rows = torch.cat([layer.forward(xd[i:i + 8].contiguous()) for i in range(0, M, 8)])
    assert torch.equal(y_full, y_rows)
    qa = ops.act_quant_i8(xd, plain=False, perm=True)
    parts = []
    for r in range(4):
        r0, n = ops.shard_rows(N, 4, r)
        parts.append(ops.BitLinear(dev(packed[r0:r0 + n]), 0.25).forward_quantized(qa))
    assert torch.equal(torch.cat(parts, 1), y_full)
    assert ops.device_status() == 0


@pytest.mark.parametrize("N,K", [(8640, 3200), (3200, 8640)])
def test_prefill_workload_size(ops, oracle, N, K):
    """M=2048 at the benchmark's sizes: sampled token rows against the oracle, all rows
    against a weight_scale linearity property (x4 is exact in fp32)."""
    rng = np.random.default_rng(0)
    M = 2048
    x, trits = case(rng, M, N, K)
    packed = oracle.np_pack_trits_nk(trits)
    xd, pd = dev(x), dev(packed)
    y, acc = ops.BitLinear(pd, 0.02).forward(xd, return_acc=True)
    y4 = ops.BitLinear(pd, 0.08).forward(xd)
    assert ops.device_status() == 0
    rows = np.array([0, 1, 127, 128, 777, 1023, 1024, 2046, 2047])
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x[rows], packed, N, 0.02, threads=8)
    assert np.array_equal(host(acc)[rows], acc_ref)
    assert bits_equal(host(y)[rows], y_ref)
    # int32 accumulators of every row: checksum against an int64 matmul of a column sample
    cols = np.arange(0, N, 97)
    q = host(ops.act_quant_i8(xd, plain=True, perm=False)["q_plain"]).astype(np.int64)
    want = q @ trits[cols].astype(np.int64).T
    assert np.array_equal(host(acc)[:, cols].astype(np.int64), want)
    ya, yb = host(y), host(y4)
    nz = ya != 0
    assert np.allclose(yb[nz], ya[nz] * 4.0, rtol=2e-7, atol=0)
