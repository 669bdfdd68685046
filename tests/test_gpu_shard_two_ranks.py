"""Column-sharded BitLinear and W4A16 on two GPUs, one process per GPU, through the C ABI:
the gathered result must equal the CPU checker's unsharded result -- int32 accumulators and
fp32 bits for BitLinear -- on both data planes (NCCL all-gather called from the library, and the
shards stored straight into every rank's copy by the kernels).  Skipped below two visible GPUs."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from gpu_util import bf16_round, bits_equal, dev, host, make_w4_case
    from nsl_b200 import ops, sharding
    from oracle import oracle as o
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # carries the unique id only
    comm = sharding.Comm.from_torch()
    fails = []
    rng = np.random.default_rng(77)                                   # same inputs on every rank
    N, K, ws = 512, 1024, 0.037
    trits = rng.integers(-1, 2, size=(N, K)).astype(np.int8)
    packed = o.np_pack_trits_nk(trits)
    r0, rows = ops.shard_rows(N, world, rank)
    layer = ops.BitLinear(dev(packed[r0:r0 + rows]), ws)
    for M in (1, 16, 256, 300):
        x = rng.standard_normal((M, K)).astype(np.float32)
        _, _, acc_ref, y_ref = o.bitlinear_forward_packed(x, packed, N, ws, threads=4)
        xd = dev(x)
        # plane 1: NCCL all-gather, called from the library
        y_l, acc_l = layer.forward(xd, return_acc=True)
        y_full = torch.empty(M, N, device="cuda")
        acc_full = torch.empty(M, N, device="cuda", dtype=torch.int32)
        comm.allgather_cols(y_l, y_full=y_full)
        comm.allgather_cols(acc_l, y_full=acc_full)
        comm.wait(60000)
        if not np.array_equal(host(acc_full), acc_ref):
            fails.append("nccl acc M=%d" % M)
        if not bits_equal(host(y_full), y_ref):
            fails.append("nccl y M=%d" % M)
        # plane 2: the kernels store their shard into every rank's copy
        for dt in (torch.float32, torch.bfloat16):
            yg = comm.symm_empty((M, N), dt)
            comm.barrier()
            layer.forward_gathered(comm, xd, yg)
            comm.barrier()
            torch.cuda.synchronize()
            want = y_ref if dt == torch.float32 else bf16_round(y_ref)
            if not bits_equal(host(yg), want):
                fails.append("peer y M=%d %s" % (M, dt))
    # W4A16 shards (codes, scales and zero points split by rows), NCCL plane
    N4, K4, gs = 256, 1024, 128
    q, codes, scale, zp = make_w4_case(rng, N4, K4, gs)
    r0, rows = ops.shard_rows(N4, world, rank)
    w4 = ops.W4A16.from_nk(dev(codes[r0:r0 + rows]), dev(scale[r0:r0 + rows]).to(torch.bfloat16), dev(zp[r0:r0 + rows]), gs)
    for M in (1, 16, 64):
        xb = bf16_round(rng.standard_normal((M, K4)).astype(np.float32))
        want = o.w4a16_matmul_nk(xb, codes, scale, zp, N4, K4, gs, threads=4)
        y_l = w4.forward(dev(xb).to(torch.bfloat16), out_dtype=torch.float32)
        y_full = torch.empty(M, N4, device="cuda")
        comm.allgather_cols(y_l, y_full=y_full)
        comm.wait(60000)
        got = host(y_full)
        rms = np.sqrt((want.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
        if not np.all(np.abs(got - want) <= 1e-3 * np.maximum(np.abs(want), rms)):
            fails.append("w4 M=%d" % M)
    # two decode layers of a small decoder, column-sharded over the two ranks, against the same layers
    # unsharded on this GPU (every linear is bit-exact and heads are independent, so the residual
    # stream must come out bit-equal)
    from nsl_b200 import sharded_decoder

    class Small:
        hidden, heads, head_dim, ffn, layers, vocab = 512, 4, 128, 1024, 2, 1000
        eps, rope_theta = 1e-5, 10000.0

    for batch in (8, 48):
        sh = sharded_decoder.ShardedDecodeLayers(comm, batch, 60, 2, cfg=Small, seed=3, kv_from_full=True)
        one = sharded_decoder.ShardedDecodeLayers(sharding.Comm(0, 1), batch, 60, 2, cfg=Small, seed=3, kv_from_full=True)
        one.x.copy_(sh.x)
        sh.step()
        one.step()
        torch.cuda.synchronize()
        if not torch.equal(sh.x, one.x):
            fails.append("sharded decoder layers differ from the unsharded ones (batch %d)" % batch)
    if comm.status() != 0 or ops.device_status() != 0:
        fails.append("status word set")
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("ok" if not fails else "; ".join(fails))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def test_two_rank_gather_equals_oracle(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / ("rank%d.txt" % r)).read() == "ok"
