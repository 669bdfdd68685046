"""Host-side logic of the library that runs without a GPU: the safetensors container reader of
nslq_bitnet_load_safetensors (every refusal happens before the first CUDA call) and the geometry of
nsl_qtensor_quantize (nslq_qtensor_num_scales against the CPU checker's compute_num_scales)."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

from nsl_b200._lib import lib
from oracle import oracle as o


def _container(tensors, metadata=None):
    header, data = {}, b""
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dt, shape, raw in tensors:
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


def _load(path):
    L = lib()
    handle = C.c_void_p()
    rc = L.nslq_bitnet_load_safetensors(str(path).encode(), None, C.byref(handle))
    n = int(L.nslq_ternary_set_size(handle)) if rc == 0 else None
    if rc == 0:
        L.nslq_ternary_set_destroy(handle)
    return rc, L.nslq_last_error().decode(), n


UP = "model.layers.0.mlp.up_proj.weight"


def test_loader_refusals_need_no_gpu(tmp_path):
    rc, msg, _ = _load(tmp_path / "missing.safetensors")
    assert rc == -8 and "io" in msg
    cases = {
        "short": (b"\x01\x02", -8, "shorter than a header length"),
        "long_header": (struct.pack("<Q", 1 << 40) + b"{}", -8, "does not fit the file"),
        "not_json": (struct.pack("<Q", 8) + b"nonsense", -8, "invalid header"),
        "trailing": (struct.pack("<Q", 4) + b"{} x", -8, "invalid header"),
        "no_offsets": (lambda: (lambda h: struct.pack("<Q", len(h)) + h)(json.dumps({UP: {"dtype": "F32", "shape": [2, 4]}}).encode()))(),
        "range": (_container([(UP, "F32", (2, 4), bytes(32))])[:-1], -8, "byte range"),
        "shape_bytes": (_container([(UP, "F32", (2, 4), bytes(28))]), -8, "byte range"),
        "dtype": (_container([(UP, "I64", (2, 4), bytes(64))]), -4, "unsupported dtype I64"),
        "align": (_container([(UP, "F16", (3, 3), bytes(18))]), -2, "not a multiple of 4"),
        "empty_tensor": (_container([(UP, "F32", (0, 4), b"")]), -2, "is empty"),
    }
    cases["no_offsets"] = (cases["no_offsets"], -8, "without dtype, shape or data_offsets")
    for name, (raw, want, text) in cases.items():
        p = tmp_path / (name + ".safetensors")
        p.write_bytes(raw)
        rc, msg, _ = _load(p)
        assert rc == want and text in msg, (name, rc, msg)


def test_loader_skips_what_is_not_a_projection(tmp_path):
    """Nothing selected: an empty set, and no byte of the other tensors is looked at (their dtype may be anything)."""
    raw = _container([("model.embed_tokens.weight", "I64", (2, 3), bytes(48)), ("model.norm.weight", "F32", (8,), bytes(32)),
                      ("model.layers.0.mlp.up_proj.bias", "F32", (8,), bytes(32))],
                     metadata={"format": "pt", "nested": "a \"quoted\" \\ value é \n"})
    p = tmp_path / "skip.safetensors"
    p.write_bytes(raw)
    rc, msg, n = _load(p)
    assert rc == 0 and n == 0, msg
    p.write_bytes(struct.pack("<Q", 2) + b"{}")
    assert _load(p)[0] == 0


def test_qtensor_num_scales_matches_the_checker():
    L = lib()
    rng = np.random.default_rng(0)
    for _ in range(300):
        nd = int(rng.integers(1, 6))
        shape = [int(v) for v in rng.integers(1, 9, size=nd)]
        gran, axis, gs = int(rng.integers(0, 3)), int(rng.integers(0, nd)), int(rng.integers(1, 7))
        arr = (C.c_int64 * nd)(*shape)
        assert int(L.nslq_qtensor_num_scales(arr, nd, gran, axis, gs)) == int(o.qtensor_num_scales(tuple(shape), gran, axis, gs)), (shape, gran, axis, gs)
    arr = (C.c_int64 * 2)(4, 4)
    assert int(L.nslq_qtensor_num_scales(arr, 2, 1, 2, 0)) == -1          # axis out of range
    assert int(L.nslq_qtensor_num_scales(arr, 2, 2, 1, 0)) == -1          # group size 0
    assert int(L.nslq_qtensor_num_scales(arr, 2, 3, 0, 0)) == -1          # unknown granularity


def test_new_entry_points_refuse_bad_arguments_before_any_cuda_call():
    L = lib()
    null = C.c_void_p(0)
    one = C.c_void_p(16)                       # a non-null pointer that is never dereferenced: the checks come first
    assert L.nslq_embed_gather(null, 3, 10, 8, one, 1, one, null) == -1
    assert L.nslq_embed_gather(one, 3, 0, 8, one, 1, one, null) == -2
    assert L.nslq_embed_gather(one, 7, 10, 8, one, 1, one, null) == -1          # dtype tag outside F32/FP16/BF16
    assert L.nslq_embed_gather(one, 3, 10, 8, one, 0, one, null) == 0           # nothing to do
    assert L.nslq_rmsnorm_rows(null, one, 1e-5, 1, 8, one, 1, null) == -1
    assert L.nslq_rmsnorm_rows(one, one, 1e-5, 1, 0, one, 1, null) == -2
    assert L.nslq_rmsnorm_rows(one, one, 1e-5, 1, 8, one, 0, null) == -1        # F64 output is not offered
    assert L.nslq_argmax_rows(null, 3, 1, 8, 8, one, null, null) == -1
    assert L.nslq_rope_kv_prefill(null, one, one, 8, 8, 8, one, one, one, one, 1, 1, 0, 1, 1, 8, 4, null) == -1
    assert L.nslq_rope_kv_prefill(one, one, one, 8, 8, 8, one, one, one, one, 1, 4, 1, 1, 1, 8, 4, null) == -2   # pos0 + T past the cache
    assert L.nslq_rope_kv_prefill(one, one, one, 8, 8, 8, one, one, one, one, 1, 1, 0, 1, 1, 7, 4, null) == -2   # odd head dimension
    assert L.nslq_argmax_rows(one, 3, 1, 8, 4, one, null, null) == -2           # row stride shorter than the row
    shape = (C.c_int64 * 2)(4, 4)
    assert L.nslq_qtensor_quantize(null, 1, shape, 2, 0, 0, 0, 0, one, one, one, null) == -1
    assert L.nslq_qtensor_quantize(one, 1, shape, 2, 5, 0, 0, 0, one, one, one, null) == -1   # unknown dtype
    assert L.nslq_qtensor_quantize(one, 1, shape, 9, 0, 0, 0, 0, one, one, one, null) == -2   # ndim
    assert L.nslq_qtensor_dequantize(one, one, one, shape, 2, 0, 1, 3, 0, one, 1, null) == -1  # axis out of range
    assert L.nslq_bitlinear_forward_rmsnorm(null, one, 1, 1, one, 1e-5, one, 1, null, null, null, null, 0, null) == -1
    assert L.nslq_bitlinear_forward_swiglu(null, one, one, 3, 1, one, 1, null, null, null, null, 0, null) == -1
    assert L.nslq_bitlinear_forward_multi(one, 5, one, 3, 1, null, 1e-5, one, 1, null, 0, null) == -1
    assert L.nslq_bitlinear_forward_multi(null, 1, one, 3, 1, null, 1e-5, one, 1, null, 0, null) == -1
    assert b"null" in L.nslq_last_error()
