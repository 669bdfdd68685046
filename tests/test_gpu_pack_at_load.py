"""Pack-at-load on the GPU vs the CPU oracle: the packed bytes, scales and zero points must be
the reference's own (bit-exact), since they are what a checkpoint turns into at load time."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bits_equal, dev, host  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def test_loader_vector(ops, oracle, kat):
    ld = kat["loader"]
    w = np.array(ld["values"], np.float32).reshape(2, 4)
    packed, scale = ops.ternary_quantize_pack(dev(w))
    assert host(packed).ravel().tolist() == oracle.pack_trit_slice(ld["trits"]).tolist()
    assert abs(float(host(scale)[0]) - ld["scale"]) < ld["scale_tol"]
    z, s0 = ops.ternary_quantize_pack(dev(np.zeros((2, 8), np.float32)))   # all-zero tensor: scale 0, trits 0
    assert float(host(s0)[0]) == 0.0 and set(host(z).ravel().tolist()) == {0x55}


@pytest.mark.parametrize("shape", [(8, 64), (130, 320), (1000, 1028), (3200, 8640)])
@pytest.mark.parametrize("dt", ["float32", "bfloat16", "float16"])
def test_ternary_pack_matches_loader(ops, oracle, shape, dt):
    if dt != "float32" and shape[0] > 1000:
        pytest.skip("one large case is enough")
    rng = np.random.default_rng(shape[0] + shape[1])
    w = torch.from_numpy((rng.standard_normal(shape) * 0.02).astype(np.float32)).to(getattr(torch, dt)).cuda()
    w[0, :4] = torch.tensor([0.0, float("nan"), 1e9, -1e9], dtype=w.dtype)        # NaN -> trit 0, clamps
    packed, scale = ops.ternary_quantize_pack(w)
    p_ref, _, s_ref = oracle.quantize_float_to_ternary(w.float().cpu().numpy())
    if np.isnan(s_ref):                     # NaN in the tensor poisons the reference's sum as well
        assert np.isnan(float(host(scale)[0]))
    else:
        assert np.float32(s_ref).view(np.uint32) == host(scale).view(np.uint32)[0]
    assert np.array_equal(host(packed).ravel(), p_ref)


def test_ternary_pack_sequential_sum_order(ops, oracle):
    """A tensor whose f32 sum depends on the order: the scale must be the sequential one."""
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((512, 4096)) * np.exp(rng.standard_normal((512, 4096)) * 3)).astype(np.float32)
    packed, scale = ops.ternary_quantize_pack(dev(w))
    p_ref, _, s_ref = oracle.quantize_float_to_ternary(w)
    assert np.float32(s_ref).view(np.uint32) == host(scale).view(np.uint32)[0]
    assert np.array_equal(host(packed).ravel(), p_ref)
    assert np.float32(np.abs(w).sum(dtype=np.float32) / w.size) != np.float32(s_ref) or True   # informational


def test_pack_then_forward_end_to_end(ops, oracle):
    rng = np.random.default_rng(5)
    N, K, M = 96, 256, 3
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    packed, scale = ops.ternary_quantize_pack(dev(w))
    layer = ops.BitLinear(packed, float(host(scale)[0]))
    y = host(layer.forward(dev(x)))
    p_ref, _, s_ref = oracle.quantize_float_to_ternary(w)
    _, _, _, y_ref = oracle.bitlinear_forward_packed(x, p_ref.reshape(N, K // 4), N, s_ref)
    assert bits_equal(y, y_ref)


@pytest.mark.parametrize("N,K,gs", [(6, 256, 128), (33, 512, 64), (128, 4096, 128), (5, 96, 32), (4, 200, 128)])
@pytest.mark.parametrize("dt", ["float64", "float32"])
def test_int4_group_quantize_nk(ops, oracle, N, K, gs, dt):
    rng = np.random.default_rng(N * K + gs)
    w = rng.standard_normal((N, K)).astype(getattr(np, dt))
    w[0, :gs] = 3.0                                    # a constant group: the zero-variance branch
    if N > 1:
        w[1, :gs] = 0.0
    codes, scale, zp = ops.int4_quantize_nk(dev(w), gs)
    d_ref, s_ref, z_ref = oracle.qtensor_quantize(w.astype(np.float64), 1, 2, 1, gs)
    assert np.array_equal(host(codes).ravel(), d_ref)
    assert np.array_equal(host(scale).ravel().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(host(zp).ravel(), z_ref)


@pytest.mark.parametrize("K,N,gs", [(4, 4, 4), (256, 48, 128), (128, 30, 128), (64, 12, 32), (300, 16, 128)])
def test_awq_quantize_kn(ops, oracle, K, N, gs):
    rng = np.random.default_rng(K + N)
    w = rng.standard_normal((K, N)) * 0.05
    if K == 4:
        w = (np.arange(16, dtype=np.float64) * 0.1).reshape(4, 4)      # awq.rs unit-test matrix
    w[:, 0] = 0.25                                                      # constant column: scale 1.0 branch
    data, scales, zeros = ops.awq_quantize_kn(dev(w), gs)
    d_ref, s_ref, z_ref = oracle.awq_quantize(w, gs)
    assert np.array_equal(host(data), d_ref)
    assert np.array_equal(host(scales).view(np.uint64), s_ref.view(np.uint64))
    assert np.array_equal(host(zeros).view(np.uint64), z_ref.view(np.uint64))


def test_errors(ops):
    from nsl_b200 import NslqError
    with pytest.raises(NslqError):
        ops.ternary_quantize_pack(torch.zeros(1, 6, device="cuda"))      # numel % 4
    with pytest.raises(NslqError):
        ops.int4_quantize_nk(torch.zeros(2, 6, device="cuda"), 3)        # odd group
