"""Stage 1 parity: nslq_act_quant_i8 through the C ABI vs the CPU oracle (bit-exact)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import dev, host, perm_index  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from nsl_b200 import ops as o
    return o


def check(ops, oracle, x_np, torch_dtype=None):
    x = dev(x_np)
    if torch_dtype is not None:
        x = x.to(torch_dtype)
        x_np = x.float().cpu().numpy()
    M, K = x_np.shape
    want_perm = K % 16 == 0
    out = ops.act_quant_i8(x, plain=True, perm=want_perm)
    torch.cuda.synchronize()
    s_ref = np.array([oracle.absmax_scale_row(r) for r in x_np], np.float32)
    q_ref = np.stack([oracle.quantize_row_int8(r, s) for r, s in zip(x_np, s_ref)])
    assert np.array_equal(host(out["scale"]).view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(host(out["q_plain"]), q_ref)
    assert np.array_equal(host(out["rowsum"]), q_ref.astype(np.int32).sum(1))
    if want_perm:
        assert np.array_equal(host(out["q_perm"]), q_ref[:, perm_index(K)])
    return q_ref


def test_golden_rows(ops, oracle, kat):
    for fx in kat["absmax_quant"]:
        x = np.array([fx["x"]], np.float32)
        assert check(ops, oracle, x)[0].tolist() == fx["q"]
    row = kat["rounding_row"]
    assert check(ops, oracle, np.array([row["x"]], np.float32))[0].tolist() == row["q"]
    for fx in kat["forward"]:
        x = np.array(fx["x"], np.float32).reshape(fx["rows"], fx["hidden"])
        assert check(ops, oracle, x).ravel().tolist() == fx["q"]


@pytest.mark.parametrize("M,K", [(1, 3200), (7, 8640), (33, 4096), (3, 64), (2, 16), (5, 100), (4, 4), (2048, 3200)])
def test_random_normal(ops, oracle, M, K):
    rng = np.random.default_rng(1000 + M + K)
    q = check(ops, oracle, rng.standard_normal((M, K)).astype(np.float32))
    assert (q < 0).any() and (q > 0).any()


def test_adversarial_rows(ops, oracle):
    K = 64
    rows = []
    r = np.zeros(K, np.float32); rows.append(r)                                   # all-zero row
    r = np.full(K, 127.0, np.float32); r[1:9] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49999997, -0.49999997]
    rows.append(r)                                                               # exact ties, scale 127
    r = np.linspace(-1, 1, K).astype(np.float32); r[3] = np.nan; rows.append(r)   # NaN element
    r = np.full(K, 1e-42, np.float32); r[5] = -3e-41; rows.append(r)              # denormals
    r = np.ones(K, np.float32); r[7] = np.inf; rows.append(r)                     # infinite absmax
    r = np.full(K, -2.5, np.float32); rows.append(r)                              # uniform negative
    r = (np.arange(K) - 31.5).astype(np.float32) * 1e30; rows.append(r)           # huge magnitudes
    check(ops, oracle, np.stack(rows))


def test_every_tie_and_its_neighbours(ops, oracle):
    """Scale 127 makes x*inv = x: every k + 0.5 and the floats on either side of it, both signs."""
    k = np.arange(0, 127, dtype=np.float32) + np.float32(0.5)
    below, above = np.nextafter(k, np.float32(-1e9)), np.nextafter(k, np.float32(1e9))
    vals = np.concatenate([k, below, above])
    row = np.concatenate([vals, -vals, [np.float32(127.0)]]).astype(np.float32)
    row = np.concatenate([row, np.zeros((-len(row)) % 16, np.float32)])
    q = check(ops, oracle, np.stack([row, row[::-1].copy()]))
    assert q[0, 0] == 1 and q[0, 127] == 0 and q[0, 254] == 1          # 0.5, just below, just above


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_half_inputs(ops, oracle, dt):
    rng = np.random.default_rng(5)
    check(ops, oracle, rng.standard_normal((9, 256)).astype(np.float32), getattr(torch, dt))
    check(ops, oracle, rng.standard_normal((3, 100)).astype(np.float32), getattr(torch, dt))


def test_errors(ops):
    from nsl_b200 import NslqError
    x = torch.zeros(2, 100, device="cuda")
    with pytest.raises(NslqError):
        ops.act_quant_i8(x, plain=True, perm=True)      # q_perm needs K % 16 == 0
    with pytest.raises(NslqError):                      # int32 has a tensor tag, but the quantiser takes floats only
        ops.act_quant_i8(torch.zeros(2, 16, device="cuda", dtype=torch.int32))
    with pytest.raises(TypeError):                      # a dtype with no NSL tensor tag at all
        ops.act_quant_i8(torch.zeros(2, 16, device="cuda", dtype=torch.int64))
    with pytest.raises(ValueError):
        ops.act_quant_i8(torch.zeros(2, 16))            # CPU tensor: no CPU path
