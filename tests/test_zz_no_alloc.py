"""nslq_bitlinear_forward_noalloc through the C ABI.

Some callers of this library cannot hand it device memory: NSL's runtime owns every
device allocation through its caching allocator, a decode loop cannot stall on
cudaMalloc, a late-loaded plug-in may find the device already reserved.  For them the
library keeps a fixed 512 KiB scratch area in its own device image.  This test checks
that the entry point gives exactly what nslq_bitlinear_forward gives (bit-equal
outputs; the other BitLinear tests already pin that one to the CPU checker), on two
calls in a row that share the area, and that oversized requests are refused in words.

The file name sorts last on purpose: a run that stops at the first failure has
already run every other test by the time it gets here.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _layer(ops, rng, N, K, ws):
    c = rng.integers(0, 3, size=(N, K // 4, 4), dtype=np.uint8)
    packed = ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).astype(np.uint8)
    return ops.BitLinear(torch.from_numpy(packed).cuda(), ws)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    from nsl_b200 import ops
    rng = np.random.default_rng(2024)
    layer = _layer(ops, rng, 272, 3200, 0.031)
    # two different inputs back to back: the second call finds the first call's bytes in the area
    for M in (3, 1):
        x = torch.from_numpy(rng.standard_normal((M, 3200)).astype(np.float32)).cuda()
        want = layer.forward(x)                                   # caller-workspace entry point
        got = torch.full((M, 272), float("nan"), device="cuda")
        layer.forward_noalloc(x, got)
        torch.cuda.synchronize()
        assert torch.equal(got, want), "M=%d" % M
    # a prefill-sized call (tensor-core path) that still fits the area, then decode again
    x = torch.from_numpy(rng.standard_normal((96, 3200)).astype(np.float32)).cuda()
    want = layer.forward(x, out_dtype=torch.bfloat16)
    got = torch.zeros(96, 272, dtype=torch.bfloat16, device="cuda")
    layer.forward_noalloc(x, got)
    x1 = torch.from_numpy(rng.standard_normal((2, 3200)).astype(np.float32)).cuda()
    want1 = layer.forward(x1)
    got1 = torch.zeros(2, 272, device="cuda")
    layer.forward_noalloc(x1, got1)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(got1, want1)
    assert ops.device_status() == 0


def test_noalloc_refuses_what_does_not_fit():
    from nsl_b200 import NslqError, lib, ops
    cap = int(lib().nslq_noalloc_scratch_bytes())
    assert cap == 512 * 1024
    rng = np.random.default_rng(7)
    layer = _layer(ops, rng, 32, 8192, 1.0)
    M = cap // 8192 + 1                                           # one token row too many
    x = torch.zeros(M, 8192, device="cuda")
    out = torch.zeros(M, 32, device="cuda")
    with pytest.raises(NslqError) as e:
        layer.forward_noalloc(x, out)
    assert e.value.code == -5 and "built-in" in str(e.value)
    ok_rows = (cap - 1024) // 8192                                # the largest M that fits
    x = torch.from_numpy(rng.standard_normal((ok_rows, 8192)).astype(np.float32)).cuda()
    out = torch.zeros(ok_rows, 32, device="cuda")
    layer.forward_noalloc(x, out)
    torch.cuda.synchronize()
    assert torch.equal(out, layer.forward(x))
