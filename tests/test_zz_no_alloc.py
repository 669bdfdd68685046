"""nslq_bitlinear_forward_noalloc through the C ABI.

Some callers of this library cannot hand it device memory: NSL's runtime owns every
device allocation through its caching allocator, a decode loop cannot stall on
cudaMalloc, a late-loaded plug-in may find the device already reserved.  For them the
library keeps a fixed 512 KiB scratch area in its own device image.  These tests check
that the entry point gives exactly what nslq_bitlinear_forward gives and what the CPU
checker gives (bit-equal), on calls in a row that share the area -- including calls
issued back to back on one stream with no synchronisation between them, with and
without dependent launch -- that a call leaves the free device memory as it found it,
and that oversized requests are refused in words.

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


@pytest.mark.parametrize("pdl", [1, 0])
def test_back_to_back_calls_share_the_area_and_match_the_cpu_checker(oracle, pdl):
    """Three calls that all use the built-in area (tensor-core path at M = 96 and 40, quantise + decode
    kernel at M = 8), different inputs, separate outputs, one stream, no synchronisation in between:
    each must still equal the workspace entry point and the CPU checker; free device memory must not
    move across the calls."""
    from nsl_b200 import lib, ops
    rng = np.random.default_rng(99)
    N, K, ws = 272, 3200, 0.031
    c = rng.integers(0, 3, size=(N, K // 4, 4), dtype=np.uint8)
    packed = ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).astype(np.uint8)
    layer = ops.BitLinear(torch.from_numpy(packed).cuda(), ws)
    xs = [rng.standard_normal((M, K)).astype(np.float32) for M in (96, 40, 8)]
    xd = [torch.from_numpy(x).cuda() for x in xs]
    outs = [torch.full((x.shape[0], N), float("nan"), device="cuda") for x in xs]
    wants = [layer.forward(x) for x in xd]
    lib().nslq_set_dependent_launch(pdl)
    try:
        layer.forward_noalloc(xd[2], outs[2])                    # first use on this device (address look-up) outside the measured window
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        for x, o in zip(xd, outs):
            layer.forward_noalloc(x, o)                          # no synchronisation between the three
        torch.cuda.synchronize()
        free1 = torch.cuda.mem_get_info()[0]
    finally:
        lib().nslq_set_dependent_launch(1)
    assert free1 == free0, "a no-allocation call changed the free device memory"
    for x, o, w in zip(xs, outs, wants):
        assert torch.equal(o, w), "M=%d differs from the workspace entry point" % x.shape[0]
        _, _, _, y_ref = oracle.bitlinear_forward_packed(x, packed, N, ws, threads=4)
        assert np.array_equal(o.cpu().numpy().view(np.uint32), y_ref.view(np.uint32)), "M=%d differs from the CPU checker" % x.shape[0]
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
