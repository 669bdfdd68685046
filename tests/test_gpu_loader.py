"""nslq_bitnet_load_safetensors against the reference's own loader tests
(crates/nsl-codegen/tests/bitnet_loader.rs: missing file, corrupt header, F32 and F16 storage of the
pinned VALUES -> EXPECTED_TRITS with scale 0.925, an unsupported dtype) and against the CPU checker's
quantize_float_to_ternary on a file of layer-shaped tensors.  The container is written by hand, as the
reference's tests do (u64 header length, JSON header, data)."""
import json
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from gpu_util import bf16_round, host  # noqa: E402
from nsl_b200 import loader, ops  # noqa: E402
from nsl_b200 import NslqError  # noqa: E402
from oracle import oracle as o  # noqa: E402

VALUES = np.array([-2.0, 0.0, 0.2, 1.0, -1.0, 2.0, -0.2, 1.0], np.float32)
EXPECTED_TRITS = [-1, 0, 0, 1, -1, 1, 0, 1]


def _expected_packed():
    c = [t + 1 for t in EXPECTED_TRITS]
    return [(c[i] << 6) | (c[i + 1] << 4) | (c[i + 2] << 2) | c[i + 3] for i in (0, 4)]


def _container(tensors, metadata=None, pad=0):
    """tensors: list of (name, dtype string, shape, bytes)."""
    header, data = {}, b""
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dt, shape, raw in tensors:
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [len(data), len(data) + len(raw)]}
        data += raw
    h = json.dumps(header).encode() + b" " * pad
    return struct.pack("<Q", len(h)) + h + data


def _write(tmp_path, raw, name="weights.safetensors"):
    p = tmp_path / name
    p.write_bytes(raw)
    return p


def test_missing_file_and_corrupt_header(tmp_path):
    with pytest.raises(NslqError, match="io"):
        loader.load_bitnet_b158_safetensors(tmp_path / "nope.safetensors")
    with pytest.raises(NslqError, match="safetensors"):
        loader.load_bitnet_b158_safetensors(_write(tmp_path, b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!"))
    with pytest.raises(NslqError, match="safetensors"):
        loader.load_bitnet_b158_safetensors(_write(tmp_path, b"\x03\x00"))
    with pytest.raises(NslqError, match="safetensors"):          # header longer than the file
        loader.load_bitnet_b158_safetensors(_write(tmp_path, struct.pack("<Q", 1 << 40) + b"{}"))
    raw = _container([("model.layers.0.mlp.up_proj.weight", "F32", (2, 4), VALUES.tobytes())])
    with pytest.raises(NslqError, match="byte range"):           # data cut short
        loader.load_bitnet_b158_safetensors(_write(tmp_path, raw[:-4]))


def test_pinned_values_in_f32_f16_bf16_storage(tmp_path):
    for dt, raw in (("F32", VALUES.tobytes()), ("F16", VALUES.astype(np.float16).tobytes()),
                    ("BF16", (VALUES.view(np.uint32) >> 16).astype(np.uint16).tobytes())):
        got = loader.load_bitnet_b158_safetensors(_write(tmp_path, _container([("model.layers.0.mlp.up_proj.weight", dt, (2, 4), raw)])))
        assert len(got) == 1 and got[0].shape == (2, 4) and got[0].name == "model.layers.0.mlp.up_proj.weight"
        assert host(got[0].packed).ravel().tolist() == _expected_packed()
        if dt == "F32":
            assert abs(got[0].scale - 0.925) < 1e-5
            assert np.float32(got[0].scale) == np.float32(o.quantize_float_to_ternary(VALUES)[2])


def test_unsupported_dtype_and_alignment(tmp_path):
    raw = _container([("model.layers.0.mlp.down_proj.weight", "I64", (2, 4), bytes(64))])
    with pytest.raises(NslqError, match="unsupported dtype I64"):
        loader.load_bitnet_b158_safetensors(_write(tmp_path, raw))
    raw = _container([("model.layers.0.mlp.down_proj.weight", "F32", (2, 3), bytes(24))])
    with pytest.raises(NslqError, match="not a multiple of 4"):
        loader.load_bitnet_b158_safetensors(_write(tmp_path, raw))
    # the same defects in a tensor that is not a BitLinear projection do not matter: it is skipped
    raw = _container([("model.embed_tokens.weight", "I64", (2, 3), bytes(48)),
                      ("model.layers.0.mlp.up_proj.weight", "F32", (2, 4), VALUES.tobytes())])
    assert len(loader.load_bitnet_b158_safetensors(_write(tmp_path, raw))) == 1


def test_layer_shaped_file_against_the_cpu_checker(tmp_path):
    """All seven projection suffixes, mixed storage, other tensors in between, metadata and header padding."""
    rng = np.random.default_rng(12)
    shapes = {"self_attn.q_proj": (320, 256), "self_attn.k_proj": (64, 256), "self_attn.v_proj": (64, 256),
              "self_attn.o_proj": (256, 320), "mlp.gate_proj": (704, 256), "mlp.up_proj": (704, 256), "mlp.down_proj": (256, 704)}
    tensors, want = [("model.embed_tokens.weight", "F32", (10, 256), bytes(10 * 256 * 4))], {}
    for li in range(2):
        tensors.append(("model.layers.%d.input_layernorm.weight" % li, "F32", (256,), np.ones(256, np.float32).tobytes()))
        for i, (nm, shp) in enumerate(shapes.items()):
            w = (rng.standard_normal(shp) * 0.02).astype(np.float32)
            name = "model.layers.%d.%s.weight" % (li, nm)
            kind = ("F32", "F16", "BF16")[(i + li) % 3]
            if kind == "F16":
                w = w.astype(np.float16).astype(np.float32)
                raw = w.astype(np.float16).tobytes()
            elif kind == "BF16":
                w = bf16_round(w)
                raw = (w.view(np.uint32) >> 16).astype(np.uint16).tobytes()
            else:
                raw = w.tobytes()
            tensors.append((name, kind, shp, raw))
            want[name] = (o.quantize_float_to_ternary(w), shp)
    tensors.append(("lm_head.weight", "F16", (10, 256), bytes(10 * 256 * 2)))
    path = _write(tmp_path, _container(tensors, metadata={"format": "pt", 'note': 'a "quoted" value \u00e9'}, pad=5))
    got = loader.load_bitnet_b158_safetensors(path)
    assert [g.name for g in got] == [t[0] for t in tensors if t[0] in want]        # file order
    for g in got:
        (packed, _, scale), shp = want[g.name]
        assert g.shape == shp and tuple(g.packed.shape) == (shp[0], shp[1] // 4)
        assert np.array_equal(host(g.packed).ravel(), packed)
        assert np.float32(g.scale) == np.float32(scale)
    # a loaded weight is a layer: same result as the layer built from the checker's bytes
    g = got[0]
    x = rng.standard_normal((3, g.shape[1])).astype(np.float32)
    y = g.bitlinear().forward(torch.from_numpy(x).cuda())
    (packed, _, scale), shp = want[g.name]
    _, _, _, y_ref = o.bitlinear_forward_packed(x, packed.reshape(shp[0], shp[1] // 4), shp[0], scale)
    assert np.array_equal(host(y).view(np.uint32), y_ref.view(np.uint32))


def test_empty_selection(tmp_path):
    raw = _container([("model.norm.weight", "F32", (8,), bytes(32))])
    assert loader.load_bitnet_b158_safetensors(_write(tmp_path, raw)) == []
    assert loader.load_bitnet_b158_safetensors(_write(tmp_path, struct.pack("<Q", 2) + b"{}")) == []
