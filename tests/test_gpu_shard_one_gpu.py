"""The column-block output path on ONE GPU: two row shards of a weight, computed one after the
other, each writing its column block into two copies of the result at once (what two ranks do to
each other's memory), must reproduce the CPU checker's unsharded output bit for bit; and the
world-size-1 communicator runs every entry point of the sharding API."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from gpu_util import bf16_round, bits_equal, dev, host  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nsl_b200 import ops as o
    return o


@pytest.mark.parametrize("M", [1, 7, 16, 40, 256, 300])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_shards_into_two_copies(ops, oracle, M, dtype):
    rng = np.random.default_rng(5 + M)
    N, K, ws = 384, 1024, 0.041
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = oracle.np_pack_trits_nk(trits)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, _, _, y_ref = oracle.bitlinear_forward_packed(x, packed, N, ws, threads=4)
    want = y_ref if dtype == torch.float32 else bf16_round(y_ref)
    qa = ops.act_quant_i8(dev(x), plain=False, perm=True)
    a = torch.full((M, N), 7.0, device="cuda", dtype=dtype)
    b = torch.full((M, N), 7.0, device="cuda", dtype=dtype)
    half = N // 2
    bias = rng.standard_normal(N).astype(np.float32)
    for r, copies in ((0, [a, b]), (1, [b, a])):
        layer = ops.BitLinear(dev(packed[r * half:(r + 1) * half]), ws)
        layer.forward_quantized_cols(qa, copies, r * half)
    torch.cuda.synchronize()
    assert bits_equal(host(a), want) and bits_equal(host(b), want)
    # with a bias: each shard adds its own slice
    for r, copies in ((0, [a, b]), (1, [b, a])):
        layer = ops.BitLinear(dev(packed[r * half:(r + 1) * half]), ws)
        layer.forward_quantized_cols(qa, copies, r * half, bias=dev(bias[r * half:(r + 1) * half]))
    torch.cuda.synchronize()
    wb = (y_ref + bias[None, :]).astype(np.float32)
    wb = wb if dtype == torch.float32 else bf16_round(wb)
    assert bits_equal(host(a), wb) and bits_equal(host(b), wb)
    assert ops.device_status() == 0


@pytest.mark.parametrize("M", [1, 5, 64])
def test_world_one_communicator(ops, oracle, M):
    from nsl_b200 import sharding
    comm = sharding.Comm(0, 1)
    rng = np.random.default_rng(11)
    N, K, ws = 256, 512, 0.05
    packed = oracle.np_pack_trits_nk(rng.integers(-1, 2, size=(N, K)).astype(np.int8))
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, _, acc_ref, y_ref = oracle.bitlinear_forward_packed(x, packed, N, ws)
    layer = ops.BitLinear(dev(packed), ws)
    yg = comm.symm_empty((M, N), torch.float32)
    assert float(yg.abs().sum()) == 0.0                      # fresh shared buffers are zero-filled
    comm.barrier()
    layer.forward_gathered(comm, dev(x), yg)
    comm.barrier()
    y_l, acc_l = layer.forward(dev(x), return_acc=True)
    y_full = torch.empty(M, N, device="cuda")
    g = comm.allgather_cols(y_l, y_full=y_full)
    comm.wait(10000)
    assert bits_equal(host(yg), y_ref) and bits_equal(host(y_full), y_ref) and bits_equal(host(g[0]), y_ref)
    assert np.array_equal(host(acc_l), acc_ref)
    y2 = comm.symm_empty((M, N), torch.float32)
    comm.peer_allgather_cols(y_l, y2)
    torch.cuda.synchronize()
    assert bits_equal(host(y2), y_ref)
    assert comm.status() == 0
    comm.close()
