"""Loads libnslq_b200.so (the C ABI declared in include/nslq_b200.h) with ctypes.

There is no fallback: if the shared library is missing, loading raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnslq_b200.so")

vp, i64, i32, f32, f64 = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_double

# name -> (restype, argtypes); every symbol include/nslq_b200.h declares.
SIGNATURES = {
    "nslq_version": (i32, []),
    "nslq_last_error": (C.c_char_p, []),
    "nslq_set_dependent_launch": (None, [i32]),
    "nslq_device_status": (i32, [C.POINTER(i32)]),
    "nslq_act_quant_i8": (i32, [vp, i32, i64, i64, vp, vp, vp, vp, vp]),
    "nslq_swiglu_act_quant_i8": (i32, [vp, vp, i32, i64, i64, i64, i64, vp, vp, vp, vp, vp, vp]),
    "nslq_decode_attention": (i32, [vp, vp, vp, i64, i64, i64, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, vp, vp]),
    "nslq_rmsnorm_act_quant_i8": (i32, [vp, i32, vp, f64, i64, i64, vp, vp, vp, vp, vp, vp]),
    "nslq_bitlinear_create": (i32, [vp, i64, i64, f32, C.POINTER(vp)]),
    "nslq_bitlinear_destroy": (None, [vp]),
    "nslq_bitlinear_validate": (i32, [vp, C.POINTER(i64), vp]),
    "nslq_bitlinear_workspace_bytes": (i64, [i64, i64]),
    "nslq_bitlinear_forward": (i32, [vp, vp, i32, i64, vp, i32, vp, vp, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_quantized": (i32, [vp, vp, vp, vp, i64, vp, i32, vp, vp, vp, vp]),
    "nslq_bitlinear_forward_rmsnorm": (i32, [vp, vp, i32, i64, vp, C.c_double, vp, i32, vp, vp, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_swiglu": (i32, [vp, vp, vp, i32, i64, vp, i32, vp, vp, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_multi": (i32, [vp, i32, vp, i32, i64, vp, C.c_double, vp, i32, vp, i64, vp]),
    "nslq_bitlinear_forward_noalloc": (i32, [vp, vp, i32, i64, vp, i32, vp]),
    "nslq_noalloc_scratch_bytes": (i64, []),
    "nslq_w4a16_create_nk": (i32, [vp, vp, i32, vp, i32, i64, i64, i64, C.POINTER(vp)]),
    "nslq_w4a16_create_awq_kn": (i32, [vp, vp, vp, i64, i64, i64, C.POINTER(vp)]),
    "nslq_w4a16_create_qtensor_kn": (i32, [vp, vp, vp, i64, i64, i32, i32, i64, C.POINTER(vp)]),
    "nslq_w4a16_destroy": (None, [vp]),
    "nslq_w4a16_f32x_scratch_bytes": (i64, [vp, i64]),
    "nslq_w4a16_forward_f32x": (i32, [vp, vp, i64, vp, i32, vp, i64, vp]),
    "nslq_w4a16_forward": (i32, [vp, vp, i32, i64, vp, i32, vp]),
    "nslq_ternary_quantize_pack": (i32, [vp, i32, i64, vp, vp, vp]),
    "nslq_int4_quantize_nk": (i32, [vp, i32, i64, i64, i64, vp, vp, vp, vp]),
    "nslq_embed_gather": (i32, [vp, i32, i64, i64, vp, i64, vp, vp]),
    "nslq_rmsnorm_rows": (i32, [vp, vp, C.c_double, i64, i64, vp, i32, vp]),
    "nslq_rope_kv_prefill": (i32, [vp, vp, vp, i64, i64, i64, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, vp]),
    "nslq_argmax_rows": (i32, [vp, i32, i64, i64, i64, vp, vp, vp]),
    "nslq_bitnet_load_safetensors": (i32, [C.c_char_p, vp, C.POINTER(vp)]),
    "nslq_ternary_set_size": (i64, [vp]),
    "nslq_ternary_set_entry": (i32, [vp, i64, C.POINTER(C.c_char_p), C.POINTER(vp), C.POINTER(i64), C.POINTER(C.POINTER(i64)),
                                     C.POINTER(i32), C.POINTER(C.c_float)]),
    "nslq_ternary_set_destroy": (None, [vp]),
    "nslq_qtensor_num_scales": (i64, [C.POINTER(i64), i32, i32, i32, i64]),
    "nslq_qtensor_quantize": (i32, [vp, i32, C.POINTER(i64), i32, i32, i32, i32, i64, vp, vp, vp, vp]),
    "nslq_qtensor_dequantize": (i32, [vp, vp, vp, C.POINTER(i64), i32, i32, i32, i32, i64, vp, i32, vp]),
    "nslq_awq_quantize_kn": (i32, [vp, i32, i64, i64, i64, vp, vp, vp, vp]),
    "nslq_shard_rows": (i32, [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]),
    "nslq_shard_unique_id": (i32, [vp]),
    "nslq_shard_init": (i32, [vp, i32, i32, C.POINTER(vp)]),
    "nslq_shard_destroy": (None, [vp]),
    "nslq_shard_info": (i32, [vp, C.POINTER(i32), C.POINTER(i32)]),
    "nslq_allgather_cols": (i32, [vp, vp, i32, i64, i64, vp, vp, vp]),
    "nslq_shard_wait": (i32, [vp, vp, i64]),
    "nslq_symm_alloc": (i32, [vp, i64, C.POINTER(vp)]),
    "nslq_symm_free": (i32, [vp, vp]),
    "nslq_peer_barrier": (i32, [vp, vp]),
    "nslq_shard_status": (i32, [vp, C.POINTER(i32)]),
    "nslq_peer_allgather_cols": (i32, [vp, vp, i32, i64, i64, vp, vp]),
    "nslq_peer_push_cols_async": (i32, [vp, vp, i32, i64, i64, vp]),
    "nslq_bitlinear_gathered_workspace_bytes": (i64, [i64, i64, i64]),
    "nslq_bitlinear_forward_cols": (i32, [vp, vp, i32, i64, C.POINTER(vp), i32, i64, i64, i32, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_quantized_cols": (i32, [vp, vp, vp, vp, i64, C.POINTER(vp), i32, i64, i64, i32, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_gathered": (i32, [vp, vp, vp, i32, i64, vp, i32, vp, vp, i64, vp]),
    "nslq_bitlinear_forward_quantized_gathered": (i32, [vp, vp, vp, vp, vp, i64, vp, i32, vp, vp, i64, vp]),
}

# Entry points with NSL's own calling convention (include/nsl_shims.h): i64 handles in, i64 out.
SHIM_SIGNATURES = {
    "nsl_awq_matmul_cuda": (i64, [i64, i64, i64, i64]),
    "nsl_gptq_matmul_cuda": (i64, [i64, i64, i64, i64, i64]),
    "nsl_qtensor_matmul_mixed_cuda": (i64, [i64, i64, i64]),
    "nsl_quant_forget_cuda": (None, [i64]),
    "nsl_quant_set_stream_cuda": (None, [i64]),
    "nsl_quant_reserve_cuda": (i64, [i64]),
    "nsl_awq_pre_scale_weight_cuda": (i64, [i64, i64, i64, C.c_double, i64]),
    "nsl_qtensor_quantize_cuda": (i64, [i64, i64]),
    "nsl_qtensor_dequantize_cuda": (i64, [i64, i64]),
    "nsl_awq_quantize_cuda": (i64, [i64, i64, i64]),
    "nsl_bitlinear_pack": (i64, [i64, i64, i64, C.c_double]),
    "nsl_bitlinear_forward": (i64, [i64, i64, i64]),
    "nsl_bitlinear_free": (None, [i64]),
}

_lib = None


class NslqError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("nslq error %d: %s" % (code, text))
        self.code = code


def lib():
    """The loaded library.  Raises if it has not been built (python -m nsl_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libnslq_b200.so is missing (%s): build it with `python -m nsl_b200.build`; "
                "this package has no CPU or PyTorch fallback" % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in list(SIGNATURES.items()) + list(SHIM_SIGNATURES.items()):
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(rc):
    if rc != 0:
        raise NslqError(rc, lib().nslq_last_error().decode("utf-8", "replace"))
