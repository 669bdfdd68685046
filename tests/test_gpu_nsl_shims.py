"""The entry points with NSL's calling convention: fabricate NslTensor / QuantizedTensor /
AwqPackedWeight structs the way the Rust runtime lays them out, call through the i64-handle
functions, compare with the CPU oracle.  The cases are NSL's own (tests/m16_test.nsl asserts,
awq.rs unit matrix, bitnet fixtures)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


class NslTensor(C.Structure):
    _fields_ = [("magic", C.c_uint32), ("data", C.c_void_p), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("ndim", C.c_int64), ("len", C.c_int64), ("refcount", C.c_int64),
                ("device", C.c_uint8), ("dtype", C.c_uint16), ("owns_data", C.c_uint8), ("data_owner", C.c_int64),
                ("slab_managed", C.c_uint8), ("tape_id", C.c_int64)]


class QuantizedTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scale", C.c_void_p), ("zero_point", C.c_void_p), ("shape", C.POINTER(C.c_int64)),
                ("ndim", C.c_int64), ("dtype", C.c_int64), ("granularity", C.c_int64), ("gran_axis", C.c_int64),
                ("group_size", C.c_int64), ("num_scales", C.c_int64), ("refcount", C.c_int64)]


class AwqPackedWeight(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p), ("k", C.c_int64), ("n", C.c_int64),
                ("group_size", C.c_int64), ("num_groups", C.c_int64), ("refcount", C.c_int64)]


TAG = {torch.float64: 0, torch.float32: 1, torch.float16: 2, torch.bfloat16: 3}


def nsl_tensor(t):
    """An NslTensor describing a torch CUDA tensor (device field is 1-based)."""
    assert C.sizeof(NslTensor) == 88
    shape = (C.c_int64 * t.dim())(*t.shape)
    strides = (C.c_int64 * t.dim())(*t.stride())
    s = NslTensor(0x4E534C54, t.data_ptr(), shape, strides, t.dim(), t.numel(), 1, t.device.index + 1, TAG[t.dtype], 0, 0, 0, 0)
    s._keep = (shape, strides, t)
    return s


@pytest.fixture(scope="module")
def lib():
    from nsl_b200 import lib as l
    return l()


def test_struct_sizes():
    assert C.sizeof(NslTensor) == 88 and C.sizeof(QuantizedTensor) == 88 and C.sizeof(AwqPackedWeight) == 64
    assert NslTensor.device.offset == 56 and NslTensor.dtype.offset == 58 and NslTensor.tape_id.offset == 80


def test_bitlinear_trio_on_golden_fixtures(lib, oracle, kat):
    for fx in kat["forward"]:
        r, h, o = fx["rows"], fx["hidden"], fx["out_dim"]
        x = np.array(fx["x"], np.float32).reshape(r, h)
        w = np.array(fx["w_kn"], np.int8).reshape(h, o)
        packed = np.ascontiguousarray(oracle.pack_weight_kn(w))          # host bytes, as the loader leaves them
        handle = lib.nsl_bitlinear_pack(packed.ctypes.data, o, h, 1.0)
        assert handle != 0
        xt = torch.from_numpy(x).cuda()
        yt = torch.empty(r, o, device="cuda")
        xs, ys = nsl_tensor(xt), nsl_tensor(yt)
        assert lib.nsl_bitlinear_forward(handle, C.addressof(xs), C.addressof(ys)) == C.addressof(ys)
        torch.cuda.synchronize()
        _, _, _, y_ref = oracle.forward_reference(x, w)
        assert np.array_equal(yt.cpu().numpy().view(np.uint32), y_ref.view(np.uint32)), fx["name"]
        lib.nsl_bitlinear_free(handle)


def test_bitlinear_trio_decode_and_prefill_shapes(lib, oracle):
    rng = np.random.default_rng(4)
    N, K = 320, 1024
    packed = oracle.np_pack_trits_nk(rng.integers(-1, 2, size=(N, K)).astype(np.int8))
    handle = lib.nsl_bitlinear_pack(packed.ctypes.data, N, K, 0.125)
    for M, dt in [(1, torch.float32), (7, torch.bfloat16), (200, torch.float32)]:
        xt = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(dt).cuda()
        yt = torch.empty(M, N, device="cuda")
        xs, ys = nsl_tensor(xt), nsl_tensor(yt)
        assert lib.nsl_bitlinear_forward(handle, C.addressof(xs), C.addressof(ys)) != 0
        torch.cuda.synchronize()
        _, _, _, y_ref = oracle.bitlinear_forward_packed(xt.float().cpu().numpy(), packed, N, 0.125, threads=4)
        assert np.array_equal(yt.cpu().numpy().view(np.uint32), y_ref.view(np.uint32))
    lib.nsl_bitlinear_free(handle)


def make_awq(oracle, w, gs):
    k, n = w.shape
    data, scales, zeros = oracle.awq_quantize(w, gs)
    keep = (np.ascontiguousarray(data), np.ascontiguousarray(scales), np.ascontiguousarray(zeros))
    s = AwqPackedWeight(keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data, k, n, gs, (k + gs - 1) // gs, 1)
    s._keep = keep
    return s, keep


def test_awq_matmul_cuda(lib, oracle, kat):
    mm = kat["awq"]["matmul"]                                             # awq.rs:491-512
    x = np.array(mm["input"], np.float64).reshape(mm["m"], mm["k"])
    w = np.array(mm["weights"], np.float64).reshape(mm["k"], mm["n"])
    cases = [(x, w, mm["gs"])]
    rng = np.random.default_rng(2)
    cases.append((rng.standard_normal((3, 256)), rng.standard_normal((256, 48)) * 0.05, 128))
    for x, w, gs in cases:
        pw, (data, scales, zeros) = make_awq(oracle, w, gs)
        xt = torch.from_numpy(x.astype(np.float32)).cuda()
        yt = torch.empty(x.shape[0], w.shape[1], device="cuda")
        xs, ys = nsl_tensor(xt), nsl_tensor(yt)
        for _ in range(2):                                                # second call hits the cached device copy
            assert lib.nsl_awq_matmul_cuda(C.addressof(xs), C.addressof(pw), gs, C.addressof(ys)) == C.addressof(ys)
        torch.cuda.synchronize()
        want = oracle.awq_matmul(x.astype(np.float32).astype(np.float64), data, scales, zeros, w.shape[0], w.shape[1], gs)
        # fp32 accumulation and f32 scale/zero tables against the reference's f64: an output moves by a few 1e-7 of
        # the row's magnitude, so the bound is relative to max(|y|, row rms) -- 1e-5, a hundredth of the 1e-3 asked for
        rms = np.sqrt((want ** 2).mean(axis=1, keepdims=True))
        assert np.all(np.abs(yt.cpu().numpy() - want) <= 1e-5 * np.maximum(np.abs(want), rms))
        if w.shape == (mm["k"], mm["n"]):                                  # the reference test's own matrix and bound
            ref = x @ w
            assert np.all(np.abs(ref - yt.cpu().numpy()) < np.abs(ref) * mm["rel"] + mm["abs"])
        assert lib.nsl_gptq_matmul_cuda(C.addressof(xs), C.addressof(pw), gs, 4, C.addressof(ys)) != 0
        lib.nsl_quant_forget_cuda(C.addressof(pw))


@pytest.mark.parametrize("dtype,gran,axis,gs", [(0, 0, 0, 0), (0, 1, 0, 0), (0, 1, 1, 0), (1, 0, 0, 0), (1, 2, 0, 4), (1, 2, 1, 4)])
def test_qtensor_matmul_mixed_cuda(lib, oracle, dtype, gran, axis, gs):
    """Every dtype/granularity nsl_qtensor_quantize produces, on the m16_test.nsl shapes."""
    rng = np.random.default_rng(16 + dtype * 7 + gran * 3 + axis)
    x, w = rng.standard_normal((4, 8)), rng.standard_normal((8, 16))
    data, scale, zp = oracle.qtensor_quantize(w, dtype, gran, axis, gs)
    shape = (C.c_int64 * 2)(8, 16)
    keep = (np.ascontiguousarray(data), np.ascontiguousarray(scale), np.ascontiguousarray(zp))
    qt = QuantizedTensor(keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data, shape, 2, dtype, gran, axis, gs,
                         scale.size, 1)
    xt = torch.from_numpy(x.astype(np.float32)).cuda()
    yt = torch.empty(4, 16, device="cuda")
    xs, ys = nsl_tensor(xt), nsl_tensor(yt)
    assert lib.nsl_qtensor_matmul_mixed_cuda(C.addressof(xs), C.addressof(qt), C.addressof(ys)) == C.addressof(ys)
    torch.cuda.synchronize()
    want = oracle.qtensor_matmul_mixed(x.astype(np.float32).astype(np.float64), data, scale, zp, (8, 16), dtype, gran, axis, gs)
    assert np.allclose(yt.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    if dtype == 0 and gran == 1 and axis == 0:
        assert np.all(np.abs(yt.cpu().numpy() - x @ w) <= 0.15 + 1.0 * np.abs(x @ w))   # m16_test.nsl:44-51
    lib.nsl_quant_forget_cuda(C.addressof(qt))


@pytest.mark.parametrize("gran,axis,gs", [(2, 0, 128), (0, 0, 0), (1, 1, 0)])
@pytest.mark.parametrize("xdt", [torch.float32, torch.bfloat16])
def test_qtensor_int4_reaches_the_streaming_kernels(lib, oracle, gran, axis, gs, xdt):
    """INT4 QuantizedTensors [K,N] whose scale is constant along k inside a group are re-laid out once and
    multiplied by the W4A16 kernels (fp32 x split into three bf16 parts); same answer as the reference's
    dequantise-then-matmul, on a non-default stream set through nsl_quant_set_stream_cuda."""
    rng = np.random.default_rng(40 + gran + axis)
    K, N = 256, 192
    w = rng.standard_normal((K, N)) * 0.05
    data, scale, zp = oracle.qtensor_quantize(w, 1, gran, axis, gs)
    shape = (C.c_int64 * 2)(K, N)
    keep = (np.ascontiguousarray(data), np.ascontiguousarray(scale), np.ascontiguousarray(zp))
    qt = QuantizedTensor(keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data, shape, 2, 1, gran, axis, gs, scale.size, 1)
    st = torch.cuda.Stream()
    lib.nsl_quant_set_stream_cuda(st.cuda_stream)
    assert lib.nsl_quant_reserve_cuda(1 << 20) == 1 << 20
    try:
        for M in (1, 3, 12, 40):                 # 3 M stacked rows for fp32 x: decode kernel up to M = 5, tensor-core GEMM beyond
            x = rng.standard_normal((M, K)).astype(np.float32)
            xt = torch.from_numpy(x).cuda().to(xdt)
            yt = torch.empty(M, N, device="cuda")
            torch.cuda.synchronize()
            xs, ys = nsl_tensor(xt), nsl_tensor(yt)
            assert lib.nsl_qtensor_matmul_mixed_cuda(C.addressof(xs), C.addressof(qt), C.addressof(ys)) == C.addressof(ys)
            st.synchronize()
            want = oracle.qtensor_matmul_mixed(xt.float().cpu().numpy().astype(np.float64), data, scale, zp, (K, N), 1, gran, axis, gs)
            got = yt.cpu().numpy()
            rms = np.sqrt((want ** 2).mean())
            assert np.all(np.abs(got - want) <= 1e-3 * np.maximum(np.abs(want), rms)), (M, np.abs(got - want).max(), rms)
    finally:
        lib.nsl_quant_set_stream_cuda(0)
        lib.nsl_quant_forget_cuda(C.addressof(qt))


def test_awq_pre_scale_weight_cuda_is_the_reference_bit_for_bit(lib, oracle):
    rng = np.random.default_rng(9)
    K, N = 48, 40
    w = rng.standard_normal((K, N)).astype(np.float32)
    scales = (np.abs(rng.standard_normal(N)) + 0.1).astype(np.float32)
    wt, yt = torch.from_numpy(w).cuda(), torch.empty(K, N, device="cuda")
    ws, ys = nsl_tensor(wt), nsl_tensor(yt)
    for alpha in (0.5, 0.25, 1.0):
        assert lib.nsl_awq_pre_scale_weight_cuda(C.addressof(ws), scales.ctypes.data, N, alpha, C.addressof(ys)) == C.addressof(ys)
        torch.cuda.synchronize()
        want = oracle.awq_pre_scale_weight(w, scales, alpha)
        assert np.array_equal(yt.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # no scales (or a wrong length): a copy, as the original does
    assert lib.nsl_awq_pre_scale_weight_cuda(C.addressof(ws), 0, 0, 0.5, C.addressof(ys)) != 0
    torch.cuda.synchronize()
    assert torch.equal(yt, wt)
    assert lib.nsl_awq_pre_scale_weight_cuda(0, 0, 0, 0.5, C.addressof(ys)) == 0


def test_reserved_code_is_rejected(lib, oracle, kat):
    """Bytes with a 2-bit field 0b11 are not trits (bitnet_packed_repr.rs: 0xFF, 0xC0): the pack shim
    refuses them on the host copy, and nslq_bitlinear_validate counts them on the device."""
    from nsl_b200 import NslqError, ops
    good = oracle.np_pack_trits_nk(np.random.default_rng(1).integers(-1, 2, size=(16, 64)).astype(np.int8))
    for bad_byte in kat["pack"]["invalid_bytes"]:
        bad = good.copy()
        bad[3, 5] = bad_byte
        assert lib.nsl_bitlinear_pack(bad.ctypes.data, 16, 64, 1.0) == 0
        layer = ops.BitLinear(torch.from_numpy(bad).cuda(), 1.0)
        with pytest.raises(NslqError):
            layer.validate()
        assert layer.invalid_bytes() == 1
    h = lib.nsl_bitlinear_pack(good.ctypes.data, 16, 64, 1.0)
    assert h != 0
    lib.nsl_bitlinear_free(h)
    layer = ops.BitLinear(torch.from_numpy(good).cuda(), 1.0)
    layer.validate()
    assert layer.invalid_bytes() == 0


def _empty_qtensor(oracle, shape, dtype, gran, axis, gs):
    """A QuantizedTensor as nsl_qtensor_quantize allocates it: host buffers sized by compute_num_scales."""
    total = int(np.prod(shape))
    ns = int(oracle.qtensor_num_scales(tuple(shape), gran, axis, gs))
    keep = (np.zeros((total + 1) // 2 if dtype == 1 else total, np.uint8), np.zeros(ns, np.float32), np.zeros(ns, np.uint8),
            (C.c_int64 * len(shape))(*shape))
    q = QuantizedTensor(keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data, keep[3], len(shape), dtype, gran, axis, gs, ns, 1)
    q._keep = keep
    return q, keep


@pytest.mark.parametrize("src_dt", [torch.float64, torch.float32])
def test_load_time_quantisers_fill_host_objects_with_the_reference_bytes(lib, oracle, src_dt):
    rng = np.random.default_rng(8)
    for shape, dtype, gran, axis, gs in [((64, 48), 1, 2, 0, 16), ((33, 40), 0, 1, 1, 0), ((6, 10, 4), 0, 0, 0, 0), ((128, 24), 1, 2, 1, 8)]:
        w = (rng.standard_normal(shape) * 2).astype(np.float32 if src_dt == torch.float32 else np.float64)
        wt = torch.from_numpy(w).cuda()
        ws = nsl_tensor(wt)
        q, (data, scale, zp, _) = _empty_qtensor(oracle, shape, dtype, gran, axis, gs)
        assert lib.nsl_qtensor_quantize_cuda(C.addressof(ws), C.addressof(q)) == C.addressof(q)
        want = oracle.qtensor_quantize(w.astype(np.float64), dtype, gran, axis, gs)
        used = 1 if gran == 0 else (shape[axis] if gran == 1 else int(np.prod(shape[:axis], dtype=np.int64)) * ((shape[axis] + gs - 1) // gs))
        assert np.array_equal(data, want[0]) and np.array_equal(zp, want[2])
        assert np.array_equal(scale[:used].view(np.uint32), want[1][:used].view(np.uint32))
        # and back, into a device tensor of the type the original returns
        out = torch.empty(shape, device="cuda", dtype=torch.float64)
        os_ = nsl_tensor(out)
        assert lib.nsl_qtensor_dequantize_cuda(C.addressof(q), C.addressof(os_)) == C.addressof(os_)
        ref = oracle.qtensor_dequantize(*want, shape, dtype, gran, axis, gs)
        assert np.array_equal(out.cpu().numpy().view(np.uint64), ref.view(np.uint64))
    # AWQ packing of a [K,N] weight
    K, N, gs = 96, 40, 32
    w = (rng.standard_normal((K, N)) * 0.05).astype(np.float32 if src_dt == torch.float32 else np.float64)
    wt = torch.from_numpy(w).cuda()
    ws = nsl_tensor(wt)
    G = (K + gs - 1) // gs
    keep = (np.zeros((K * N + 1) // 2, np.uint8), np.zeros(G * N, np.float64), np.zeros(G * N, np.float64))
    pw = AwqPackedWeight(keep[0].ctypes.data, keep[1].ctypes.data, keep[2].ctypes.data, K, N, gs, G, 1)
    assert lib.nsl_awq_quantize_cuda(C.addressof(ws), gs, C.addressof(pw)) == C.addressof(pw)
    data, scales, zeros = oracle.awq_quantize(w.astype(np.float64), gs)
    assert np.array_equal(keep[0], np.asarray(data).ravel())
    assert np.array_equal(keep[1].view(np.uint64), np.asarray(scales, np.float64).ravel().view(np.uint64))
    assert np.array_equal(keep[2].view(np.uint64), np.asarray(zeros, np.float64).ravel().view(np.uint64))
    # refusals: a CPU tensor, a QuantizedTensor allocated for another shape
    cpu = nsl_tensor(wt)
    cpu.device = 0
    assert lib.nsl_awq_quantize_cuda(C.addressof(cpu), gs, C.addressof(pw)) == 0
    q, _ = _empty_qtensor(oracle, (K, N + 1), 0, 0, 0, 0)
    assert lib.nsl_qtensor_quantize_cuda(C.addressof(ws), C.addressof(q)) == 0
