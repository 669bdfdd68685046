"""Column-parallel host logic on CPU: 2 gloo ranks, each computes its row shard with the CPU
checker, the shards are all-gathered and reassembled, and the result must equal the unsharded
one bit for bit (replicated quantisation => identical int32 accumulators)."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, N, K, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from nsl_b200 import sharding
    from oracle import oracle as o
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(1234)                      # same inputs on every rank
    x = rng.standard_normal((M, K)).astype(np.float32)
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = o.np_pack_trits_nk(trits)
    shard = sharding.shard_weight_rows(torch.from_numpy(packed), world, rank).numpy()
    assert shard.shape[0] == N // world
    _, _, acc_l, y_l = o.bitlinear_forward_packed(x, shard, shard.shape[0], 0.05)
    g = sharding.all_gather_columns(torch.from_numpy(y_l))
    y = sharding.assemble(g).contiguous().numpy()
    ga = sharding.all_gather_columns(torch.from_numpy(acc_l))
    acc = sharding.assemble(ga).contiguous().numpy()
    _, _, acc_ref, y_ref = o.bitlinear_forward_packed(x, packed, N, 0.05)
    ok = np.array_equal(acc, acc_ref) and np.array_equal(y.view(np.uint32), y_ref.view(np.uint32))
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("ok" if ok else "mismatch")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_two_rank_column_shards_reassemble_bit_exact(tmp_path, M):
    world, N, K = 2, 96, 256
    mp.spawn(_worker, args=(world, _free_port(), M, N, K, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "ok"


def test_shard_math_matches_reference_rules():
    sys.path.insert(0, ROOT)
    from nsl_b200 import NslqError, ops
    assert [ops.shard_rows(8640, 8, r) for r in (0, 7)] == [(0, 1080), (7560, 1080)]
    assert ops.shard_rows(3200, 4, 2) == (1600, 800)
    with pytest.raises(NslqError):
        ops.shard_rows(8641, 8, 0)          # not divisible: the reference asserts, we return an error
