"""W4A16 parity through the C ABI vs the f64 CPU oracle.

Tolerance (stated by the workload): bf16 outputs within rel 1e-2, fp32 outputs
within rel 1e-3, measured against the largest magnitude of the row's outputs
plus the same relative bound per element.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, dev, host, make_w4_case  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def close(got, want, rel):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    tol = rel * np.abs(want) + rel * np.abs(want).max(axis=-1, keepdims=True) * 0.05
    return bool(np.all(np.abs(got - want) <= tol)), float(np.max(np.abs(got - want) / (np.abs(want) + 1e-9)))


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 20])
@pytest.mark.parametrize("N,K,gs", [(48, 256, 128), (100, 512, 128), (130, 1024, 256), (32, 4096, 128)])
def test_streaming_kernel_bf16(ops, oracle, M, N, K, gs):
    rng = np.random.default_rng(M * 131 + N + K)
    q, codes, scale, zp = make_w4_case(rng, N, K, gs)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = ops.W4A16.from_nk(dev(codes), dev(scale).to(torch.bfloat16), dev(zp), gs)
    y32 = host(w.forward(dev(x).to(torch.bfloat16), out_dtype=torch.float32))
    ybf = host(w.forward(dev(x).to(torch.bfloat16)))
    want = oracle.w4a16_matmul_nk(x, codes, scale, zp, N, K, gs, threads=4)
    ok, worst = close(y32, want, 1e-3)
    assert ok, worst
    ok, worst = close(ybf, want, 1e-2)
    assert ok, worst


def test_fp16_activations_and_packed_zero_points(ops, oracle):
    rng = np.random.default_rng(77)
    N, K, gs, M = 64, 512, 128, 4
    q, codes, scale, zp = make_w4_case(rng, N, K, gs, scale_bf16=False)
    zp_flat = zp.ravel()
    zp_packed = (zp_flat[0::2] | (zp_flat[1::2] << 4)).astype(np.uint8)
    x = rng.standard_normal((M, K)).astype(np.float16)
    w = ops.W4A16.from_nk(dev(codes), dev(scale), dev(zp_packed), gs, zp_packed=True)
    y = host(w.forward(dev(x), out_dtype=torch.float32))
    want = oracle.w4a16_matmul_nk(x.astype(np.float32), codes, scale, zp, N, K, gs)
    ok, worst = close(y, want, 1e-3)
    assert ok, worst


@pytest.mark.parametrize("M", [1, 16])
def test_workload_size(ops, oracle, M):
    """N=11008, K=4096, group 128, the benchmark's distributions."""
    rng = np.random.default_rng(0)
    N, K, gs = 11008, 4096, 128
    q, codes, scale, zp = make_w4_case(rng, N, K, gs)
    x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = ops.W4A16.from_nk(dev(codes), dev(scale).to(torch.bfloat16), dev(zp), gs)
    y = host(w.forward(dev(x).to(torch.bfloat16)))
    want = oracle.w4a16_matmul_nk(x, codes, scale, zp, N, K, gs, threads=8)
    ok, worst = close(y, want, 1e-2)
    assert ok, worst


def test_scalar_kernel_small_groups_and_f32_x(ops, oracle):
    rng = np.random.default_rng(5)
    for N, K, gs, M in [(10, 64, 32, 3), (7, 96, 32, 2), (33, 256, 64, 5)]:
        q, codes, scale, zp = make_w4_case(rng, N, K, gs, scale_bf16=False)
        x = rng.standard_normal((M, K)).astype(np.float32)
        w = ops.W4A16.from_nk(dev(codes), dev(scale), dev(zp), gs)
        y = host(w.forward(dev(x), out_dtype=torch.float32))
        want = oracle.w4a16_matmul_nk(x, codes, scale, zp, N, K, gs)
        assert np.allclose(y, want, rtol=1e-5, atol=1e-6)


def test_awq_layout(ops, oracle):
    """AwqPackedWeight form: [K,N] nibbles, f64 scales / float zeros (awq.rs:104-144, :202-226)."""
    rng = np.random.default_rng(9)
    for K, N, gs, M in [(256, 48, 128, 2), (128, 30, 128, 1), (64, 12, 32, 3)]:
        wmat = rng.standard_normal((K, N)) * 0.05
        data, scales, zeros = oracle.awq_quantize(wmat, gs)
        x = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
        want = oracle.awq_matmul(x.astype(np.float64), data, scales, zeros, K, N, gs)
        w = ops.W4A16.from_awq_kn(dev(data), dev(scales), dev(zeros), K, N, gs)
        y = host(w.forward(dev(x).to(torch.bfloat16), out_dtype=torch.float32))
        ok, worst = close(y, want, 1e-3)
        assert ok, (K, N, gs, worst)
