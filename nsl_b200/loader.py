"""load_bitnet_b158_safetensors (crates/nsl-codegen/src/bitnet/loader.rs:200-220) over the C ABI: the
file is parsed and its BitLinear projection weights are quantised to packed ternary on the GPU by
nslq_bitnet_load_safetensors; this module only hands the entries over as PyTorch tensors."""
import ctypes as C
from dataclasses import dataclass

import torch

from . import ops
from ._lib import lib
from .ops import check


@dataclass
class LoadedTernaryWeight:
    """The reference's LoadedTernaryWeight (loader.rs:47-56), packed bytes on the device."""
    name: str
    packed: torch.Tensor        # uint8; [shape[0], shape[1] / 4] for a matrix, flat otherwise
    shape: tuple
    scale: float

    def bitlinear(self):
        """The layer this weight belongs to: y = BitLinear(x) with weight_scale = scale."""
        if len(self.shape) != 2:
            raise ValueError("%s is not a matrix" % self.name)
        return ops.BitLinear(self.packed, self.scale)


class _DeviceBytes:
    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def load_bitnet_b158_safetensors(path):
    """Every `*.self_attn.{q,k,v,o}_proj.weight` / `*.mlp.{gate,up,down}_proj.weight` tensor of the file,
    quantised on the current CUDA device.  Raises NslqError with the reference's LoaderError texts."""
    if not torch.cuda.is_available():
        raise RuntimeError("nsl_b200 quantises on the GPU; there is no CPU path")
    L = lib()
    handle = C.c_void_p()
    check(L.nslq_bitnet_load_safetensors(str(path).encode(), C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(handle)))
    out = []
    try:
        for i in range(int(L.nslq_ternary_set_size(handle))):
            name, ptr, nbytes = C.c_char_p(), C.c_void_p(), C.c_int64()
            shape, ndim, scale = C.POINTER(C.c_int64)(), C.c_int32(), C.c_float()
            check(L.nslq_ternary_set_entry(handle, i, C.byref(name), C.byref(ptr), C.byref(nbytes), C.byref(shape), C.byref(ndim),
                                           C.byref(scale)))
            shp = tuple(int(shape[d]) for d in range(ndim.value))
            packed = torch.as_tensor(_DeviceBytes(ptr.value, nbytes.value), device="cuda").clone()    # the set owns its bytes
            if len(shp) == 2 and shp[1] % 4 == 0:
                packed = packed.view(shp[0], shp[1] // 4)
            out.append(LoadedTernaryWeight(name.value.decode(), packed, shp, float(scale.value)))
    finally:
        L.nslq_ternary_set_destroy(handle)
    return out
