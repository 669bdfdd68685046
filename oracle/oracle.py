"""ctypes front end of the CPU checker (oracle/nslq_oracle.c) plus a numpy mirror.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's baseline legs (the CPU port; the reference's GPU kernel design restated).  The product package never imports this module.

The numpy mirror (`np_*`) restates the BitLinear arithmetic a second time, so
the C restatement is not its own only witness; both are pinned to the NSL
golden vectors in tests/test_oracle_golden.py.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnslq_oracle.so")
_PRIOR_SO = os.path.join(_HERE, "libnslq_prior_art.so")
_lib = None
_prior = None

i64, f32p, f64p = C.c_int64, C.POINTER(C.c_float), C.POINTER(C.c_double)
i8p, u8p, i32p, i64p = (C.POINTER(C.c_int8), C.POINTER(C.c_uint8), C.POINTER(C.c_int32),
                        C.POINTER(C.c_int64))


def build(force=False):
    """Compile the C checker (gcc) and the GPU prior-art baseline kernel (nvcc) with the Makefile beside them."""
    stale = False
    for so, src in ((_SO, "nslq_oracle.c"), (_PRIOR_SO, "gpu_prior_art.cu")):
        src = os.path.join(_HERE, src)
        stale = stale or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


def _load_prior():
    global _prior
    build()
    _prior = C.CDLL(_PRIOR_SO)
    _prior.nslo_gpu_prior_art_bitlinear.argtypes = [C.c_void_p] * 4 + [C.c_int64] * 3 + [C.c_float] + [C.c_void_p] * 3
    _prior.nslo_gpu_prior_art_w4_dequant.argtypes = [C.c_void_p] * 4 + [C.c_int64] * 3 + [C.c_void_p]


def gpu_prior_art_bitlinear(x, packed, weight_scale, return_acc=False, bias=None, residual=None):
    """The reference's GPU kernel design restated (oracle/gpu_prior_art.cu) on torch CUDA tensors: x [rows, hidden]
    f32, packed [out_dim, hidden/4] u8.  A baseline to time and to check, never part of the product."""
    import torch
    if _prior is None:
        _load_prior()
    rows, hidden = x.shape
    out_dim = packed.shape[0]
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and packed.is_contiguous() and packed.dtype == torch.uint8
    y = torch.empty(rows, out_dim, dtype=torch.float32, device=x.device)
    acc = torch.empty(rows, out_dim, dtype=torch.int32, device=x.device) if return_acc else None
    ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
    rc = _prior.nslo_gpu_prior_art_bitlinear(ptr(x), ptr(packed), ptr(y), ptr(acc), rows, hidden, out_dim, float(weight_scale),
                                             ptr(bias), ptr(residual), torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError("nslo_gpu_prior_art_bitlinear returned %d" % rc)
    return (y, acc) if return_acc else y


def gpu_prior_art_w4_dequant(codes, scale, zp, group):
    """The dequantisation half of the reference's route for a weight-only INT4 linear (oracle/gpu_prior_art.cu): codes
    [N, K/2] u8, scale [N, G] f32, zp [N, G] u8 on the GPU -> dense f32 [N, K], (q - zp) * scale in f64 rounded once."""
    import torch
    if _prior is None:
        _load_prior()
    N, K = codes.shape[0], codes.shape[1] * 2
    assert codes.is_cuda and codes.dtype == torch.uint8 and scale.dtype == torch.float32 and zp.dtype == torch.uint8
    assert codes.is_contiguous() and scale.is_contiguous() and zp.is_contiguous()
    w = torch.empty(N, K, dtype=torch.float32, device=codes.device)
    rc = _prior.nslo_gpu_prior_art_w4_dequant(codes.data_ptr(), scale.data_ptr(), zp.data_ptr(), w.data_ptr(), N, K, int(group),
                                              torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError("nslo_gpu_prior_art_w4_dequant returned %d" % rc)
    return w


def gpu_prior_art_w4_matmul(x, codes, scale, zp, group):
    """The reference's route for a weight-only INT4 linear -- dequantise the whole weight on every call, then a dense
    matmul (crates/nsl-runtime/src/quantize.rs:547-585) -- on torch CUDA tensors; the matmul is the BLAS library's f32
    tensor-core GEMM (TF32).  x [M, K] in any float dtype; returns f32 [M, N]."""
    import torch
    w = gpu_prior_art_w4_dequant(codes, scale, zp, group)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        return x.float() @ w.t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.nslo_absmax_scale_row.restype = C.c_float
        _lib.nslo_ternary_gemm_element.restype = C.c_float
        _lib.nslo_awq_dequantize_int4.restype = C.c_double
        _lib.nslo_dequantize_val.restype = C.c_double
        _lib.nslo_lcg_next.restype = C.c_uint64
        _lib.nslo_qtensor_num_scales.restype = C.c_int64
        _lib.nslo_awq_quantize_int4.restype = C.c_uint8
        _lib.nslo_awq_quantize_int4.argtypes = [C.c_double] * 3
        _lib.nslo_awq_dequantize_int4.argtypes = [C.c_uint8, C.c_double, C.c_double]
        _lib.nslo_dequantize_val.argtypes = [C.c_uint8, C.c_float, C.c_uint8]
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def max_threads():
    return int(lib().nslo_max_threads())


# --------------------------------------------------------------------------- RMSNorm (prologue of the fused quantiser)
def rmsnorm_f32(x, w, eps=1e-5):
    """nsl_tensor_rmsnorm on f32 rows: sequential f64 sum of squares, one rounding to f32."""
    x, w = _c(x, np.float32), _c(w, np.float32)
    rows, n = x.shape
    out = np.empty_like(x)
    lib().nslo_rmsnorm_f32(_p(x, C.POINTER(C.c_float)), _p(w, C.POINTER(C.c_float)), C.c_double(eps),
                           C.c_int64(rows), C.c_int64(n), _p(out, C.POINTER(C.c_float)))
    return out


# --------------------------------------------------------------------------- BitLinear
def absmax_scale_row(row):
    row = _c(row, np.float32)
    return float(lib().nslo_absmax_scale_row(_p(row, f32p), i64(row.size)))


def quantize_row_int8(row, scale):
    row = _c(row, np.float32)
    q = np.empty(row.size, np.int8)
    lib().nslo_quantize_row_int8(_p(row, f32p), i64(row.size), C.c_float(scale), _p(q, i8p))
    return q


def forward_reference(x, w_kn):
    """x [rows,hidden] f32, w_kn [hidden,out] trits -> (scales, q, acc, y)."""
    x, w_kn = _c(x, np.float32), _c(w_kn, np.int8)
    rows, hidden = x.shape
    out = w_kn.shape[1]
    assert w_kn.shape[0] == hidden
    scales = np.empty(rows, np.float32)
    q = np.empty((rows, hidden), np.int8)
    acc = np.empty((rows, out), np.int32)
    y = np.empty((rows, out), np.float32)
    lib().nslo_forward_reference(_p(x, f32p), i64(rows), i64(hidden), _p(w_kn, i8p), i64(out),
                                 _p(scales, f32p), _p(q, i8p), _p(acc, i32p), _p(y, f32p))
    return scales, q, acc, y


def bitlinear_forward_packed(x, packed, out_dim, weight_scale=1.0, threads=1):
    """x [rows,hidden] f32, packed [out_dim, hidden/4] u8 -> (scales, q, acc, y)."""
    x, packed = _c(x, np.float32), _c(packed, np.uint8)
    rows, hidden = x.shape
    assert packed.size == out_dim * hidden // 4
    scales = np.empty(rows, np.float32)
    q = np.empty((rows, hidden), np.int8)
    acc = np.empty((rows, out_dim), np.int32)
    y = np.empty((rows, out_dim), np.float32)
    rc = lib().nslo_bitlinear_forward_packed(
        _p(x, f32p), i64(rows), i64(hidden), _p(packed, u8p), i64(out_dim),
        C.c_float(weight_scale), C.c_int(threads),
        _p(scales, f32p), _p(q, i8p), _p(acc, i32p), _p(y, f32p))
    if rc:
        raise ValueError("nslo_bitlinear_forward_packed rc=%d" % rc)
    return scales, q, acc, y


def pack_trit_slice(trits):
    trits = _c(trits, np.int8).ravel()
    out = np.empty(trits.size // 4, np.uint8)
    rc = lib().nslo_pack_trit_slice(_p(trits, i8p), i64(trits.size), _p(out, u8p))
    if rc:
        raise ValueError("pack_trit_slice rc=%d" % rc)
    return out


def unpack_byte_slice(b):
    b = _c(b, np.uint8).ravel()
    out = np.empty(b.size * 4, np.int8)
    rc = lib().nslo_unpack_byte_slice(_p(b, u8p), i64(b.size), _p(out, i8p))
    if rc:
        raise ValueError("invalid 0b11 trit code")
    return out


def try_unpack_byte(byte):
    out = np.empty(4, np.int8)
    rc = lib().nslo_try_unpack_byte(C.c_uint8(byte), _p(out, i8p))
    return None if rc else out


def quantize_float_to_ternary(w):
    w = _c(w, np.float32).ravel()
    packed = np.empty(w.size // 4, np.uint8)
    trits = np.empty(w.size, np.int8)
    scale = C.c_float()
    rc = lib().nslo_quantize_float_to_ternary(_p(w, f32p), i64(w.size), _p(packed, u8p),
                                              _p(trits, i8p), C.byref(scale))
    if rc:
        raise ValueError("quantize_float_to_ternary rc=%d" % rc)
    return packed, trits, scale.value


def make_f10_inputs():
    acts = np.empty(128, np.float32)
    w = np.empty((128, 4), np.int8)
    lib().nslo_make_f10_inputs(_p(acts, f32p), _p(w, i8p))
    return acts, w


def make_gpu_random_case(rows, hidden, out_dim):
    acts = np.empty((rows, hidden), np.float32)
    w = np.empty((hidden, out_dim), np.int8)
    lib().nslo_make_gpu_random_case(i64(rows), i64(hidden), i64(out_dim), _p(acts, f32p),
                                    _p(w, i8p))
    return acts, w


def pack_weight_kn(w_kn):
    """[hidden,out] trits (reference test orientation) -> packed [out, hidden/4]."""
    w_nk = np.ascontiguousarray(np.asarray(w_kn, np.int8).T)
    return pack_trit_slice(w_nk).reshape(w_nk.shape[0], w_nk.shape[1] // 4)


# --------------------------------------------------------------------------- QuantizedTensor
def qtensor_num_scales(shape, gran, axis, gs):
    sh = np.asarray(shape, np.int64)
    return int(lib().nslo_qtensor_num_scales(_p(sh, i64p), i64(sh.size), i64(gran), i64(axis),
                                             i64(max(gs, 1))))


def qtensor_quantize(src, dtype, gran, axis=0, gs=0):
    src = _c(src, np.float64)
    sh = np.asarray(src.shape, np.int64)
    total = src.size
    ns = qtensor_num_scales(src.shape, gran, axis, gs)
    data = np.zeros((total + 1) // 2 if dtype == 1 else total, np.uint8)
    scale = np.empty(ns, np.float32)
    zp = np.zeros(ns, np.uint8)
    rc = lib().nslo_qtensor_quantize(_p(src, f64p), _p(sh, i64p), i64(sh.size), i64(dtype),
                                     i64(gran), i64(axis), i64(max(gs, 1)),
                                     _p(data, u8p), _p(scale, f32p), _p(zp, u8p))
    if rc:
        raise ValueError("qtensor_quantize rc=%d" % rc)
    return data, scale, zp


def qtensor_dequantize(data, scale, zp, shape, dtype, gran, axis=0, gs=0):
    sh = np.asarray(shape, np.int64)
    out = np.empty(int(np.prod(sh)), np.float64)
    data, scale, zp = _c(data, np.uint8), _c(scale, np.float32), _c(zp, np.uint8)
    rc = lib().nslo_qtensor_dequantize(_p(data, u8p), _p(scale, f32p), _p(zp, u8p), _p(sh, i64p),
                                       i64(sh.size), i64(dtype), i64(gran), i64(axis),
                                       i64(max(gs, 1)), _p(out, f64p))
    if rc:
        raise ValueError("qtensor_dequantize rc=%d" % rc)
    return out.reshape(tuple(int(s) for s in sh))


def qtensor_matmul_mixed(x, data, scale, zp, shape, dtype, gran, axis=0, gs=0):
    x = _c(x, np.float64)
    m = x.size // x.shape[-1]
    sh = np.asarray(shape, np.int64)
    out = np.empty((m, int(sh[1])), np.float64)
    data, scale, zp = _c(data, np.uint8), _c(scale, np.float32), _c(zp, np.uint8)
    rc = lib().nslo_qtensor_matmul_mixed(_p(x, f64p), i64(m), i64(x.shape[-1]), _p(data, u8p),
                                         _p(scale, f32p), _p(zp, u8p), _p(sh, i64p), i64(dtype),
                                         i64(gran), i64(axis), i64(max(gs, 1)), _p(out, f64p))
    if rc:
        raise ValueError("qtensor_matmul_mixed rc=%d" % rc)
    return out.reshape(x.shape[:-1] + (int(sh[1]),))


def compute_scale_zp(values, qmin, qmax):
    v = _c(values, np.float64)
    s, z = C.c_float(), C.c_uint8()
    lib().nslo_compute_scale_zp(_p(v, f64p), i64(v.size), C.c_double(qmin), C.c_double(qmax),
                                C.byref(s), C.byref(z))
    return s.value, z.value


# --------------------------------------------------------------------------- AWQ
def awq_group_params(group):
    g = _c(group, np.float64)
    s, z = C.c_double(), C.c_double()
    lib().nslo_awq_group_params(_p(g, f64p), i64(g.size), C.byref(s), C.byref(z))
    return s.value, z.value


def awq_quantize_int4(v, s, z):
    return int(lib().nslo_awq_quantize_int4(v, s, z))


def awq_dequantize_int4(q, s, z):
    return float(lib().nslo_awq_dequantize_int4(q, s, z))


def awq_quantize(w, gs):
    w = _c(w, np.float64)
    k, n = w.shape
    ng = (k + gs - 1) // gs
    data = np.zeros((k * n + 1) // 2, np.uint8)
    scales = np.empty(ng * n, np.float64)
    zeros = np.empty(ng * n, np.float64)
    lib().nslo_awq_quantize(_p(w, f64p), i64(k), i64(n), i64(gs), _p(data, u8p), _p(scales, f64p),
                            _p(zeros, f64p))
    return data, scales, zeros


def awq_dequantize(data, scales, zeros, k, n, gs):
    out = np.empty((k, n), np.float64)
    lib().nslo_awq_dequantize(_p(_c(data, np.uint8), u8p), _p(_c(scales, np.float64), f64p),
                              _p(_c(zeros, np.float64), f64p), i64(k), i64(n), i64(gs),
                              _p(out, f64p))
    return out


def awq_matmul(x, data, scales, zeros, k, n, gs, threads=1):
    x = _c(x, np.float64)
    m = x.shape[0]
    out = np.empty((m, n), np.float64)
    lib().nslo_awq_matmul(_p(x, f64p), i64(m), _p(_c(data, np.uint8), u8p),
                          _p(_c(scales, np.float64), f64p), _p(_c(zeros, np.float64), f64p),
                          i64(k), i64(n), i64(gs), C.c_int(threads), _p(out, f64p))
    return out


def awq_pre_scale_weight(w, scales, alpha):
    w, scales = _c(w, np.float32), _c(scales, np.float32)
    out = np.empty_like(w)
    lib().nslo_awq_pre_scale_weight(_p(w, f32p), i64(w.shape[0]), i64(w.shape[1]),
                                    _p(scales, f32p), C.c_float(alpha), _p(out, f32p))
    return out


def w4a16_matmul_nk(x_f32, codes, scale_f32, zp_u8, n, k, gs, threads=1):
    """x [M,K] f32 (widened bf16), codes [N,K/2] u8, scale [N,G] f32, zp [N,G] u8 -> f64 [M,N]."""
    x = _c(x_f32, np.float32)
    m = x.shape[0]
    out = np.empty((m, n), np.float64)
    lib().nslo_w4a16_matmul_nk(_p(x, f32p), i64(m), _p(_c(codes, np.uint8), u8p),
                               _p(_c(scale_f32, np.float32), f32p), _p(_c(zp_u8, np.uint8), u8p),
                               i64(n), i64(k), i64(gs), C.c_int(threads), _p(out, f64p))
    return out


# --------------------------------------------------------------------------- numpy mirror
def np_round_half_away(v):
    """Round half away from zero in the dtype of v (np.round is half-even: not used)."""
    t = np.trunc(v)
    return np.where(np.abs(v - t) >= v.dtype.type(0.5), t + np.copysign(v.dtype.type(1), v), t)


def np_act_quant(x):
    """Per-token absmax int8 (bitnet_reference_impl.rs:46-70) in float32 numpy."""
    x = np.asarray(x, np.float32)
    ax = np.abs(x)
    scale = np.where(np.isnan(ax), np.float32(0), ax).max(axis=-1).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = (np.float32(127.0) / scale).astype(np.float32)
        scaled = (x * inv[..., None]).astype(np.float32)
    nan = np.isnan(scaled)
    clipped = np.where(scaled < -127, np.float32(-127), np.where(scaled > 127, np.float32(127),
                                                                  scaled)).astype(np.float32)
    r = np_round_half_away(np.where(nan, np.float32(0), clipped).astype(np.float32))
    q = r.astype(np.int8)
    q[scale == 0] = 0
    return scale, q


def np_bitlinear(x, trits_nk, weight_scale=1.0):
    """(scale, q, acc, y) with trits [out,hidden]; int64 matmul then exact cast to int32."""
    scale, q = np_act_quant(x)
    acc = (q.astype(np.int64) @ np.asarray(trits_nk, np.int64).T).astype(np.int32)
    y = ((scale / np.float32(127.0)).astype(np.float32)[:, None] * acc.astype(np.float32))
    y = (y.astype(np.float32) * np.float32(weight_scale)).astype(np.float32)
    return scale, q, acc, y


def np_pack_trits_nk(trits_nk):
    """[out,hidden] trits -> [out,hidden/4] bytes, HIGH-BITS-FIRST (pack.rs:38-43)."""
    c = (np.asarray(trits_nk, np.int8) + 1).astype(np.uint8)
    c = c.reshape(c.shape[0], -1, 4)
    return ((c[..., 0] << 6) | (c[..., 1] << 4) | (c[..., 2] << 2) | c[..., 3]).astype(np.uint8)
