"""nsl_qtensor_quantize / nsl_qtensor_dequantize on the GPU against the CPU checker: every dtype,
granularity and axis the reference has (crates/nsl-runtime/src/quantize.rs:283-537), byte for byte."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from gpu_util import dev, host  # noqa: E402
from nsl_b200 import ops  # noqa: E402
from nsl_b200 import NslqError  # noqa: E402
from oracle import oracle as o  # noqa: E402

pytestmark = pytest.mark.gpu

CASES = [
    # shape, granularity, axis, group size
    ((1000,), 0, 0, 0),
    ((37, 53), 0, 0, 0),
    ((37, 53), 1, 0, 0),
    ((37, 53), 1, 1, 0),
    ((64, 256), 2, 1, 128),
    ((64, 250), 2, 1, 64),          # ragged last group
    ((96, 40), 2, 0, 32),
    ((5, 12, 7), 1, 1, 0),
    ((5, 12, 7), 2, 1, 5),          # ragged, inner > 1
    ((3, 4, 5, 6), 2, 2, 2),
    ((3, 4, 5, 6), 1, 3, 0),
    ((1, 1), 0, 0, 0),
    ((7,), 2, 0, 16),               # one group larger than the axis
]


def _used_scales(shape, gran, axis, gs):
    if gran == 0:
        return 1
    if gran == 1:
        return shape[axis]
    return int(np.prod(shape[:axis], dtype=np.int64)) * ((shape[axis] + gs - 1) // gs)


def _src(rng, shape, kind):
    x = rng.standard_normal(shape) * 3.0
    if kind == "const":             # constant groups take the reference's other branch (quantize.rs:236-248)
        x[...] = 0.731
    elif kind == "zero":
        x[...] = 0.0
    elif kind == "mixed":           # some constant channels, some huge, some tiny
        x.reshape(-1)[:: 7] *= 1e4
        x[..., 0] = -2.5
    return x


@pytest.mark.parametrize("dtype", [0, 1])
@pytest.mark.parametrize("kind", ["normal", "const", "zero", "mixed"])
@pytest.mark.parametrize("src_dtype", [np.float64, np.float32])
def test_quantize_matches_reference_bytes(dtype, kind, src_dtype):
    rng = np.random.default_rng(11 + dtype)
    for shape, gran, axis, gs in CASES:
        x = _src(rng, shape, kind).astype(src_dtype)
        want = o.qtensor_quantize(x.astype(np.float64), dtype, gran, axis, gs)
        got = ops.qtensor_quantize(dev(x), dtype, gran, axis, gs)
        used = _used_scales(shape, gran, axis, gs)
        for name, w, g in zip(("data", "scale", "zero_point"), want, got):
            g = host(g)
            assert g.dtype == w.dtype and g.shape == w.shape, (name, shape, gran, axis)
            if name == "scale":         # the reference leaves the entries its loops never write uninitialised
                assert not g[used:].any()
                w, g = w[:used], g[:used]
            assert np.array_equal(g.view(np.uint8), w.view(np.uint8)), (name, shape, gran, axis, gs)
        ref = o.qtensor_dequantize(*want, shape, dtype, gran, axis, gs)
        back = ops.qtensor_dequantize(*got, shape, dtype, gran, axis, gs)
        assert np.array_equal(host(back).view(np.uint64), ref.view(np.uint64)), (shape, gran, axis, gs)
        back32 = ops.qtensor_dequantize(*got, shape, dtype, gran, axis, gs, out_dtype=torch.float32)
        assert np.array_equal(host(back32), ref.astype(np.float32)), (shape, gran, axis, gs)


def test_nan_never_wins_and_large_tensor_round_trip():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 96))
    x[3, 5] = np.nan
    want = o.qtensor_quantize(x, 0, 1, 0, 0)
    got = ops.qtensor_quantize(dev(x), 0, 1, 0, 0)
    assert np.array_equal(host(got[1]).view(np.uint32), want[1].view(np.uint32))
    assert np.array_equal(host(got[2]), want[2])
    assert np.array_equal(host(got[0]), want[0])
    # size-independent property at a weight-sized tensor: |dequantise(quantise(x)) - x| <= scale / 2 (+ rounding of the scale)
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    w = torch.randn(4096, 11008, device="cuda", generator=g)
    for dtype, gran, axis, gs in ((0, 1, 0, 0), (1, 2, 1, 128)):
        data, scale, zp = ops.qtensor_quantize(w, dtype, gran, axis, gs)
        back = ops.qtensor_dequantize(data, scale, zp, w.shape, dtype, gran, axis, gs, out_dtype=torch.float32)
        s = scale.view(4096, -1).repeat_interleave(w.shape[1] // scale.view(4096, -1).shape[1], dim=1)
        assert bool(((back - w).abs() <= 0.5001 * s + 1e-6).all())


def test_errors():
    x = torch.zeros(4, 4, device="cuda")
    with pytest.raises(ValueError):
        ops.qtensor_quantize(x, 0, 1, 2, 0)           # axis out of range
    with pytest.raises(ValueError):
        ops.qtensor_quantize(x, 0, 2, 1, 0)           # group size 0
    with pytest.raises(NslqError):
        ops.qtensor_quantize(x, 3, 0, 0, 0)           # unknown dtype
    with pytest.raises(NslqError):
        ops.qtensor_quantize(x.half(), 0, 0, 0, 0)    # only f32 / f64 sources
