"""BitLinear parity through the C ABI vs the CPU oracle: int8 activations and int32
accumulators bit-exact, fp32 outputs bit-equal (tolerance stated by NSL: 1e-6 rel)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, bits_equal, dev, host  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def run(ops, x_np, packed_np, ws, **kw):
    layer = ops.BitLinear(dev(packed_np), ws)
    y, acc = layer.forward(dev(x_np), return_acc=True, **kw)
    torch.cuda.synchronize()
    return host(y), host(acc)


def test_golden_forward_fixtures(ops, oracle, kat):
    for fx in kat["forward"]:
        r, h, o = fx["rows"], fx["hidden"], fx["out_dim"]
        x = np.array(fx["x"], np.float32).reshape(r, h)
        w = np.array(fx["w_kn"], np.int8).reshape(h, o)
        y, acc = run(ops, x, oracle.pack_weight_kn(w), 1.0)
        want = np.array(fx["y"], np.float64).reshape(r, o)
        ad = np.abs(y - want)
        assert np.all((ad / np.maximum(np.abs(want), 1e-30) <= 1e-6) | (ad < 1e-7)), fx["name"]
        _, _, acc_ref, y_ref = oracle.forward_reference(x, w)
        assert np.array_equal(acc, acc_ref) and bits_equal(y, y_ref), fx["name"]


def test_reference_gpu_random_cases(ops, oracle, kat):
    """The four shapes of NSL's own GPU test (bitnet_gpu_correctness.rs:571-576), same generator."""
    for rows, hidden, out in kat["gpu_random_cases"]:
        acts, w = oracle.make_gpu_random_case(rows, hidden, out)
        y, acc = run(ops, acts, oracle.pack_weight_kn(w), 1.0)
        _, q, acc_ref, y_ref = oracle.forward_reference(acts, w)
        assert (q < 0).sum() > 0
        assert np.array_equal(acc, acc_ref), (rows, hidden, out)
        assert bits_equal(y, y_ref), (rows, hidden, out)


@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("N,K", [(100, 64), (48, 256), (300, 320), (16, 1088), (130, 3200)])
def test_streaming_kernel_shapes(ops, oracle, M, N, K):
    rng = np.random.default_rng(M * 7919 + N * 31 + K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    y, acc = run(ops, x, packed, 0.731)
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.731, threads=4)
    assert np.array_equal(acc, acc_ref)
    assert bits_equal(y, y_ref)


@pytest.mark.parametrize("N,K", [(8640, 3200), (3200, 8640), (4096, 4096), (11008, 4096)])
def test_decode_sizes_m1(ops, oracle, N, K):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((1, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    y, acc = run(ops, x, packed, 0.02)
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.02, threads=8)
    assert np.array_equal(acc, acc_ref)
    assert bits_equal(y, y_ref)


def test_scalar_kernel_odd_shapes(ops, oracle):
    rng = np.random.default_rng(11)
    for M, N, K in [(3, 7, 4), (2, 33, 100), (1, 5, 60)]:
        x = rng.standard_normal((M, K)).astype(np.float32)
        trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
        packed = oracle.np_pack_trits_nk(trits)
        y, acc = run(ops, x, packed, 1.25)
        _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 1.25)
        assert np.array_equal(acc, acc_ref) and bits_equal(y, y_ref)


def test_weight_scale_is_multiplicative(ops, oracle):
    """bitnet_gpu_correctness.rs:756-766: a power-of-two weight_scale scales the output exactly."""
    rows, hidden, out = 2, 64, 32
    x = np.array([[k * 0.03125 - 1.0 + r * 0.5 for k in range(hidden)] for r in range(rows)], np.float32)
    w = np.array([[(k + c) % 3 - 1 for c in range(out)] for k in range(hidden)], np.int8)
    packed = oracle.pack_weight_kn(w)
    base, _ = run(ops, x, packed, 1.0)
    scaled, _ = run(ops, x, packed, 4.0)
    nz = base != 0
    assert nz.sum() > 0 and np.array_equal(scaled[nz], base[nz] * 4.0)


def test_bias_residual_and_half_outputs(ops, oracle):
    rng = np.random.default_rng(21)
    M, N, K = 5, 96, 256
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    _, _, _, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.5)
    want = ((y_ref + bias[None, :]).astype(np.float32) + res).astype(np.float32)   # separate roundings
    y, _ = run(ops, x, packed, 0.5, bias=dev(bias), residual=dev(res))
    assert bits_equal(y, want)
    yb, _ = run(ops, x, packed, 0.5, out_dtype=torch.bfloat16)
    assert bits_equal(yb, bf16_round(y_ref))
    yh, _ = run(ops, x, packed, 0.5, out_dtype=torch.float16)
    assert np.array_equal(yh, y_ref.astype(np.float16))


def test_shared_quantisation_and_column_shards(ops, oracle):
    """gate/up share one activation quantisation; row shards of W reproduce the full result bit for bit."""
    rng = np.random.default_rng(31)
    M, N, K, G = 3, 64, 512, 4
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    full = ops.BitLinear(dev(packed), 0.3)
    qa = ops.act_quant_i8(dev(x), plain=False, perm=True)
    y_full, acc_full = full.forward_quantized(qa, return_acc=True)
    parts = []
    for r in range(G):
        r0, n = ops.shard_rows(N, G, r)
        shard = ops.BitLinear(dev(packed[r0:r0 + n]), 0.3)
        parts.append(shard.forward_quantized(qa))
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(parts, 1), y_full)
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 0.3)
    assert np.array_equal(host(acc_full), acc_ref) and bits_equal(host(y_full), y_ref)


def test_errors(ops):
    from nsl_b200 import NslqError
    with pytest.raises(NslqError):
        ops.BitLinear(torch.zeros(4, 0, dtype=torch.uint8, device="cuda"))
    layer = ops.BitLinear(torch.zeros(16, 16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError):
        layer.forward(torch.zeros(1, 60, device="cuda"))
    small = torch.empty(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(NslqError):
        layer.forward(torch.zeros(64, 64, device="cuda"), workspace=small)


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5])
def test_fused_decode_kernel_input_dtypes(ops, oracle, dt, M):
    """M <= 2 runs the kernel with the activation quantisation fused in; it must equal the
    two-kernel path (M = 3, 4, 5 here) and the oracle for every activation dtype."""
    rng = np.random.default_rng(400 + M)
    N, K = 208, 1216
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(getattr(torch, dt)).cuda()
    x_np = x.float().cpu().numpy()
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    layer = ops.BitLinear(dev(packed), 0.11)
    y, acc = layer.forward(x, return_acc=True)
    torch.cuda.synchronize()
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x_np, packed, N, 0.11)
    assert np.array_equal(host(acc), acc_ref) and bits_equal(host(y), y_ref)
    qa = ops.act_quant_i8(x, plain=False, perm=True)          # the unfused route on the same input
    assert torch.equal(layer.forward_quantized(qa), y)


def test_fused_kernel_adversarial_rows(ops, oracle):
    K, N = 64, 40
    rows = [np.zeros(K, np.float32)]
    r = np.full(K, 127.0, np.float32); r[1:9] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49999997, -0.49999997]; rows.append(r)
    r = np.linspace(-1, 1, K).astype(np.float32); r[3] = np.nan; rows.append(r)
    r = np.ones(K, np.float32); r[7] = np.inf; rows.append(r)
    x = np.stack(rows)
    rng = np.random.default_rng(8)
    packed = oracle.np_pack_trits_nk(rng.integers(-1, 2, size=(N, K)).astype(np.int8))
    y, acc = run(ops, x, packed, 1.0)
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, 1.0)
    assert np.array_equal(acc, acc_ref)
    assert np.array_equal(np.isnan(y), np.isnan(y_ref)) and bits_equal(np.nan_to_num(y), np.nan_to_num(y_ref))


def test_dependent_launch_switch_changes_nothing(ops, oracle):
    from nsl_b200 import lib
    rng = np.random.default_rng(12)
    M, N, K = 6, 320, 1024
    x = dev(rng.standard_normal((M, K)).astype(np.float32))
    layer = ops.BitLinear(dev(oracle.np_pack_trits_nk(rng.integers(-1, 2, size=(N, K)).astype(np.int8))), 0.2)
    try:
        lib().nslq_set_dependent_launch(0)
        a = [layer.forward(x) for _ in range(3)][-1].clone()
    finally:
        lib().nslq_set_dependent_launch(1)
    b = [layer.forward(x) for _ in range(3)][-1]
    torch.cuda.synchronize()
    assert torch.equal(a, b)
