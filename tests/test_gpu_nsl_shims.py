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


TAG = {torch.float32: 1, torch.float16: 2, torch.bfloat16: 3}


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
        assert np.allclose(yt.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
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
