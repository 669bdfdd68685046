"""Host-side operators over torch CUDA tensors, one per entry point of the C ABI.

torch is used for device memory and streams only; all arithmetic runs in the
CUDA kernels of libnslq_b200.so.  Names follow NSL: BitLinear forward
(crates/nsl-codegen/src/bitnet/mod.rs:133), nsl_qtensor_matmul_mixed
(crates/nsl-runtime/src/quantize.rs:547), nsl_awq_matmul
(crates/nsl-runtime/src/awq.rs:261).
"""
import ctypes as C

import torch

from ._lib import check, lib

F64, F32, FP16, BF16, INT8, I32 = 0, 1, 2, 3, 4, 9
_TAG = {torch.float64: F64, torch.float32: F32, torch.float16: FP16, torch.bfloat16: BF16, torch.int8: INT8,
        torch.int32: I32}


def _tag(dtype):
    if dtype not in _TAG:
        raise TypeError("dtype %s has no NSL tensor tag on this path" % dtype)
    return _TAG[dtype]


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda2d(x, what):
    if not x.is_cuda:
        raise ValueError("%s must be a CUDA tensor (there is no CPU path)" % what)
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("%s must be a contiguous 2-D tensor" % what)
    return x


def act_quant_i8(x, plain=True, perm=True):
    """Per-token absmax int8 quantisation.  Returns dict(scale, rowsum, q_plain, q_perm)."""
    _cuda2d(x, "x")
    M, K = x.shape
    dev = x.device
    out = {
        "scale": torch.empty(M, dtype=torch.float32, device=dev),
        "rowsum": torch.empty(M, dtype=torch.int32, device=dev),
        "q_plain": torch.empty(M, K, dtype=torch.int8, device=dev) if plain else None,
        "q_perm": torch.empty(M, K, dtype=torch.int8, device=dev) if perm else None,
    }
    check(lib().nslq_act_quant_i8(_ptr(x), _tag(x.dtype), M, K, _ptr(out["q_plain"]), _ptr(out["q_perm"]),
                                  _ptr(out["scale"]), _ptr(out["rowsum"]), _stream()))
    return out


def rmsnorm_act_quant_i8(x, weight, eps=1e-5, plain=False, perm=True, return_h=False):
    """RMSNorm (NSL's f64 arithmetic, rounded once to f32) fused in front of act_quant_i8.
    Returns the dict of act_quant_i8, plus "h" (the normalised rows, f32) when return_h."""
    _cuda2d(x, "x")
    M, K = x.shape
    dev = x.device
    if weight.dtype != torch.float32 or weight.numel() != K or not weight.is_cuda:
        raise ValueError("weight must be a CUDA float32 tensor of K elements")
    out = {
        "scale": torch.empty(M, dtype=torch.float32, device=dev),
        "rowsum": torch.empty(M, dtype=torch.int32, device=dev),
        "q_plain": torch.empty(M, K, dtype=torch.int8, device=dev) if plain else None,
        "q_perm": torch.empty(M, K, dtype=torch.int8, device=dev) if perm else None,
        "h": torch.empty(M, K, dtype=torch.float32, device=dev) if return_h else None,
    }
    check(lib().nslq_rmsnorm_act_quant_i8(_ptr(x), _tag(x.dtype), _ptr(weight), float(eps), M, K, _ptr(out["h"]),
                                          _ptr(out["q_plain"]), _ptr(out["q_perm"]), _ptr(out["scale"]),
                                          _ptr(out["rowsum"]), _stream()))
    return out


def swiglu_act_quant_i8(gate, up, plain=False, perm=True, return_h=False):
    """SiLU(gate) * up (fp32 arithmetic) fused in front of act_quant_i8; gate, up [M,K] of one dtype."""
    for t, name in ((gate, "gate"), (up, "up")):      # rows may be column slices of a wider tensor
        if not (t.is_cuda and t.dim() == 2 and t.stride(1) == 1):
            raise ValueError("%s must be a 2-D CUDA tensor with contiguous rows" % name)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must have the same shape and dtype")
    M, K = gate.shape
    dev = gate.device
    out = {
        "scale": torch.empty(M, dtype=torch.float32, device=dev),
        "rowsum": torch.empty(M, dtype=torch.int32, device=dev),
        "q_plain": torch.empty(M, K, dtype=torch.int8, device=dev) if plain else None,
        "q_perm": torch.empty(M, K, dtype=torch.int8, device=dev) if perm else None,
        "h": torch.empty(M, K, dtype=torch.float32, device=dev) if return_h else None,
    }
    check(lib().nslq_swiglu_act_quant_i8(_ptr(gate), _ptr(up), _tag(gate.dtype), M, K, gate.stride(0), up.stride(0),
                                         _ptr(out["h"]), _ptr(out["q_plain"]),
                                         _ptr(out["q_perm"]), _ptr(out["scale"]), _ptr(out["rowsum"]), _stream()))
    return out


def decode_attention(q, k_new, v_new, k_cache, v_cache, cos_table, sin_table, pos, sm_scale, out=None):
    """RoPE at *pos, KV-cache append and causal single-query attention in one launch.
    q [B,H,D] (or [B,H*D]), k_new/v_new [B,Hkv,D] bf16; caches [B,Hkv,max_ctx,D] bf16 (row pos is
    written); cos/sin [max_ctx,D/2] f32; pos: int64 device tensor of one element.  Returns [B,H*D] bf16."""
    B, Hkv, max_ctx, D = k_cache.shape
    q, k_new, v_new = q.reshape(B, -1) if q.dim() != 2 else q, k_new.reshape(B, -1) if k_new.dim() != 2 else k_new, \
        v_new.reshape(B, -1) if v_new.dim() != 2 else v_new
    H = q.shape[1] // D
    for t in (q, k_new, v_new):                      # [B, heads*D] rows, possibly column slices of a fused projection
        if t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(1) != 1:
            raise ValueError("decode_attention: q, k, v must be CUDA bfloat16 with contiguous rows")
    for t in (k_cache, v_cache):
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("decode_attention: the caches must be contiguous CUDA bfloat16 tensors")
    if pos.dtype != torch.int64 or pos.numel() != 1 or not pos.is_cuda:
        raise ValueError("decode_attention: pos must be a one-element int64 CUDA tensor")
    if out is None:
        out = torch.empty(B, H * D, dtype=torch.bfloat16, device=q.device)
    check(lib().nslq_decode_attention(_ptr(q), _ptr(k_new), _ptr(v_new), q.stride(0), k_new.stride(0), v_new.stride(0),
                                      _ptr(k_cache), _ptr(v_cache), _ptr(cos_table),
                                      _ptr(sin_table), _ptr(pos), B, H, Hkv, D, max_ctx, float(sm_scale), _ptr(out),
                                      _stream()))
    return out


def embed_gather(table, tokens, out=None):
    """fp32 rows of `table` [V, H] for int64 `tokens` [B] (nslq_embed_gather)."""
    if not (table.is_cuda and table.is_contiguous() and table.dim() == 2 and tokens.dtype == torch.int64 and tokens.is_contiguous()):
        raise ValueError("table: contiguous CUDA [V, H]; tokens: contiguous int64")
    B = tokens.numel()
    out = out if out is not None else torch.empty(B, table.shape[1], dtype=torch.float32, device=table.device)
    check(lib().nslq_embed_gather(_ptr(table), _tag(table.dtype), table.shape[0], table.shape[1], _ptr(tokens), B, _ptr(out), _stream()))
    return out


def rmsnorm_rows(x, weight, eps=1e-5, out_dtype=torch.float32, out=None):
    """RMSNorm of fp32 rows with NSL's arithmetic, rounded to out_dtype (nslq_rmsnorm_rows)."""
    _cuda2d(x, "x")
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != x.shape[1]:
        raise ValueError("x fp32 [M, K] and an fp32 weight of K elements expected")
    out = out if out is not None else torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(lib().nslq_rmsnorm_rows(_ptr(x), _ptr(weight), float(eps), x.shape[0], x.shape[1], _ptr(out), _tag(out.dtype), _stream()))
    return out


def rope_kv_prefill(q, k, v, k_cache, v_cache, cos_table, sin_table, T, pos0=0):
    """Rotary embedding of a prompt in one launch (nslq_rope_kv_prefill): q [B*T, H*D] bf16 is rotated in place, k is
    rotated into k_cache[:, :, pos0:pos0+T] and v copied into v_cache ([B, Hkv, max_ctx, D] bf16)."""
    B, Hkv, max_ctx, D = k_cache.shape
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != B * T:
            raise ValueError("rope_kv_prefill: q, k, v must be CUDA bfloat16 [B*T, heads*D] with contiguous rows")
    for t in (k_cache, v_cache):
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous() or t.shape != k_cache.shape:
            raise ValueError("rope_kv_prefill: caches must be contiguous CUDA bfloat16 [B, Hkv, max_ctx, D]")
    if k.shape[1] != Hkv * D or v.shape[1] != Hkv * D or q.shape[1] % D != 0:
        raise ValueError("rope_kv_prefill: k, v rows must hold Hkv*D elements and q rows a multiple of D")
    for t in (cos_table, sin_table):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape[0] < max_ctx or t.shape[1] != D // 2:
            raise ValueError("rope_kv_prefill: cos/sin must be contiguous fp32 [max_ctx, D/2]")
    check(lib().nslq_rope_kv_prefill(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(k_cache), _ptr(v_cache),
                                     _ptr(cos_table), _ptr(sin_table), B, T, pos0, q.shape[1] // D, Hkv, D, max_ctx, _stream()))


def argmax_rows(x, out=None, counter=None):
    """Lowest index of each row's maximum as int64 (nslq_argmax_rows); `counter` (int64 tensor) is incremented."""
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a CUDA [M, V] tensor with unit column stride")
    out = out if out is not None else torch.empty(x.shape[0], dtype=torch.int64, device=x.device)
    check(lib().nslq_argmax_rows(_ptr(x), _tag(x.dtype), x.shape[0], x.shape[1], x.stride(0), _ptr(out), _ptr(counter), _stream()))
    return out


class BitLinear:
    """A ternary weight in NSL's packed layout ([out_dim, hidden_dim/4] uint8) on the GPU."""

    def __init__(self, packed, weight_scale=1.0):
        if not packed.is_cuda or packed.dtype != torch.uint8 or packed.dim() != 2 or not packed.is_contiguous():
            raise ValueError("packed must be a contiguous CUDA uint8 tensor [out_dim, hidden_dim/4]")
        self.packed = packed                    # keeps the borrowed buffer alive
        self.N, self.K = packed.shape[0], packed.shape[1] * 4
        self.weight_scale = float(weight_scale)
        h = C.c_void_p()
        check(lib().nslq_bitlinear_create(_ptr(packed), self.N, self.K, self.weight_scale, C.byref(h)))
        self._h = h
        self._ws = None

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:              # module globals are already gone at interpreter shutdown
            lib().nslq_bitlinear_destroy(h)

    def invalid_bytes(self):
        """Number of packed bytes that hold the reserved 2-bit code 0b11 (0 for a well-formed weight)."""
        n = C.c_int64()
        lib().nslq_bitlinear_validate(self._h, C.byref(n), _stream())
        return n.value

    def validate(self):
        """Raises NslqError if the weight holds the reserved code (nslq_bitlinear_validate)."""
        check(lib().nslq_bitlinear_validate(self._h, None, _stream()))

    def workspace(self, M):
        need = int(lib().nslq_bitlinear_workspace_bytes(M, self.K))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.packed.device)
        return self._ws

    def forward(self, x, out_dtype=torch.float32, return_acc=False, bias=None, residual=None, out=None,
                workspace=None):
        _cuda2d(x, "x")
        M = x.shape[0]
        if x.shape[1] != self.K:
            raise ValueError("x has hidden dim %d, weight expects %d" % (x.shape[1], self.K))
        y = out if out is not None else torch.empty(M, self.N, dtype=out_dtype, device=x.device)
        acc = torch.empty(M, self.N, dtype=torch.int32, device=x.device) if return_acc else None
        ws = workspace if workspace is not None else self.workspace(M)
        check(lib().nslq_bitlinear_forward(self._h, _ptr(x), _tag(x.dtype), M, _ptr(y), _tag(y.dtype), _ptr(acc),
                                           _ptr(bias), _ptr(residual), _ptr(ws), ws.numel(), _stream()))
        return (y, acc) if return_acc else y

    def forward_rmsnorm(self, x, norm_weight, eps=1e-5, out_dtype=torch.float32, return_acc=False, bias=None, residual=None,
                        out=None):
        """BitLinear(RMSNorm(x)): one launch for one token (nslq_bitlinear_forward_rmsnorm)."""
        _cuda2d(x, "x")
        M = x.shape[0]
        if x.shape[1] != self.K or norm_weight.numel() != self.K or norm_weight.dtype != torch.float32:
            raise ValueError("x [M, %d] and an fp32 norm weight of %d elements expected" % (self.K, self.K))
        y = out if out is not None else torch.empty(M, self.N, dtype=out_dtype, device=x.device)
        acc = torch.empty(M, self.N, dtype=torch.int32, device=x.device) if return_acc else None
        ws = self.workspace(M)            # used when the one-launch form does not take the call (more than one token, very wide rows)
        check(lib().nslq_bitlinear_forward_rmsnorm(self._h, _ptr(x), _tag(x.dtype), M, _ptr(norm_weight), float(eps), _ptr(y),
                                                   _tag(y.dtype), _ptr(acc), _ptr(bias), _ptr(residual), _ptr(ws),
                                                   ws.numel(), _stream()))
        return (y, acc) if return_acc else y

    def forward_swiglu(self, gate, up, out_dtype=torch.float32, return_acc=False, bias=None, residual=None, out=None):
        """BitLinear(SiLU(gate) * up): one launch for one token (nslq_bitlinear_forward_swiglu)."""
        _cuda2d(gate, "gate")
        _cuda2d(up, "up")
        M = gate.shape[0]
        if gate.shape != up.shape or gate.dtype != up.dtype or gate.shape[1] != self.K:
            raise ValueError("gate and up must both be [M, %d] of one dtype" % self.K)
        y = out if out is not None else torch.empty(M, self.N, dtype=out_dtype, device=gate.device)
        acc = torch.empty(M, self.N, dtype=torch.int32, device=gate.device) if return_acc else None
        ws = self.workspace(M)            # used when the one-launch form does not take the call (more than one token, very wide rows)
        check(lib().nslq_bitlinear_forward_swiglu(self._h, _ptr(gate), _ptr(up), _tag(gate.dtype), M, _ptr(y), _tag(y.dtype),
                                                  _ptr(acc), _ptr(bias), _ptr(residual), _ptr(ws),
                                                  ws.numel(), _stream()))
        return (y, acc) if return_acc else y

    @staticmethod
    def forward_multi(layers, x, norm_weight=None, eps=1e-5, out_dtype=torch.float32):
        """Sibling projections (q/k/v, gate/up) of the same rows, optionally behind an RMSNorm, as one call
        (nslq_bitlinear_forward_multi): one launch for one token.  Returns one [M, N_i] tensor per layer."""
        import ctypes as C
        _cuda2d(x, "x")
        M, K = x.shape
        if not 1 <= len(layers) <= 4 or any(l.K != K for l in layers):
            raise ValueError("1 to 4 layers with K = %d expected" % K)
        if norm_weight is not None and (norm_weight.numel() != K or norm_weight.dtype != torch.float32):
            raise ValueError("an fp32 norm weight of %d elements expected" % K)
        ys = [torch.empty(M, l.N, dtype=out_dtype, device=x.device) for l in layers]
        ws = layers[0].workspace(M)
        hs = (C.c_void_p * len(layers))(*[l._h for l in layers])
        ps = (C.c_void_p * len(layers))(*[y.data_ptr() for y in ys])
        check(lib().nslq_bitlinear_forward_multi(hs, len(layers), _ptr(x), _tag(x.dtype), M, _ptr(norm_weight), float(eps), ps,
                                                 _tag(out_dtype), _ptr(ws), ws.numel(), _stream()))
        return ys

    def forward_noalloc(self, x, out):
        """nslq_bitlinear_forward_noalloc: the scratch is the library's built-in area, so the
        call itself allocates nothing (x and out are the caller's)."""
        _cuda2d(x, "x")
        if x.shape[1] != self.K or tuple(out.shape) != (x.shape[0], self.N):
            raise ValueError("shape mismatch")
        check(lib().nslq_bitlinear_forward_noalloc(self._h, _ptr(x), _tag(x.dtype), x.shape[0], _ptr(out),
                                                   _tag(out.dtype), _stream()))
        return out

    def gathered_workspace(self, M):
        need = int(lib().nslq_bitlinear_gathered_workspace_bytes(M, self.K, self.N))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.packed.device)
        return self._ws

    def forward_gathered(self, comm, x, y_full, bias=None, workspace=None):
        """This rank's row shard of W applied to the replicated x; the result lands in columns
        [rank*N, (rank+1)*N) of y_full ([M, world*N], from comm.symm_empty) on EVERY rank.
        Bracket a group of these calls with comm.barrier() (nslq_bitlinear_forward_gathered)."""
        _cuda2d(x, "x")
        M = x.shape[0]
        if tuple(y_full.shape) != (M, comm.world * self.N):
            raise ValueError("y_full must be [M, world*N_shard]")
        ws = workspace if workspace is not None else self.gathered_workspace(M)
        check(lib().nslq_bitlinear_forward_gathered(comm._h, self._h, _ptr(x), _tag(x.dtype), M, _ptr(y_full),
                                                    _tag(y_full.dtype), _ptr(bias), _ptr(ws), ws.numel(), _stream()))
        return y_full

    def forward_quantized_gathered(self, comm, qa, y_full, bias=None, scratch=None):
        M = qa["scale"].shape[0]
        if scratch is None and M <= 16:
            scratch = self.gathered_workspace(M)
        check(lib().nslq_bitlinear_forward_quantized_gathered(
            comm._h, self._h, _ptr(qa["q_perm"]), _ptr(qa["scale"]), _ptr(qa["rowsum"]), M, _ptr(y_full),
            _tag(y_full.dtype), _ptr(bias), _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()))
        return y_full

    def forward_cols(self, x, copies, col0, bias=None, workspace=None):
        """Quantises x and writes the [M, N] result as columns [col0, col0+N) of every tensor in `copies`
        (each [M, ld]): nslq_bitlinear_forward_cols."""
        _cuda2d(x, "x")
        M, ld = x.shape[0], copies[0].shape[1]
        arr = (C.c_void_p * len(copies))(*[t.data_ptr() for t in copies])
        ws = workspace if workspace is not None else self.gathered_workspace(M)
        check(lib().nslq_bitlinear_forward_cols(self._h, _ptr(x), _tag(x.dtype), M, arr, len(copies), ld, col0,
                                                _tag(copies[0].dtype), _ptr(bias), _ptr(ws), ws.numel(), _stream()))

    def forward_quantized_cols(self, qa, copies, col0, bias=None):
        """Writes the [M, N] result as columns [col0, col0+N) of every tensor in `copies`
        (each [M, ld], same ld and dtype): nslq_bitlinear_forward_quantized_cols."""
        M = qa["scale"].shape[0]
        ld = copies[0].shape[1]
        for t in copies:
            if tuple(t.shape) != (M, ld) or t.dtype != copies[0].dtype or not t.is_contiguous():
                raise ValueError("copies must be contiguous [M, ld] tensors of one dtype")
        arr = (C.c_void_p * len(copies))(*[t.data_ptr() for t in copies])
        scratch = self.gathered_workspace(M) if M <= 16 else None
        check(lib().nslq_bitlinear_forward_quantized_cols(
            self._h, _ptr(qa["q_perm"]), _ptr(qa["scale"]), _ptr(qa["rowsum"]), M, arr, len(copies), ld, col0,
            _tag(copies[0].dtype), _ptr(bias), _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()))

    def forward_quantized(self, qa, out_dtype=torch.float32, return_acc=False, bias=None, residual=None, out=None):
        """qa: the dict act_quant_i8 returns (uses q_perm, scale, rowsum)."""
        M = qa["scale"].shape[0]
        dev = qa["scale"].device
        y = out if out is not None else torch.empty(M, self.N, dtype=out_dtype, device=dev)
        acc = torch.empty(M, self.N, dtype=torch.int32, device=dev) if return_acc else None
        check(lib().nslq_bitlinear_forward_quantized(self._h, _ptr(qa["q_perm"]), _ptr(qa["scale"]),
                                                     _ptr(qa["rowsum"]), M, _ptr(y), _tag(y.dtype), _ptr(acc),
                                                     _ptr(bias), _ptr(residual), _stream()))
        return (y, acc) if return_acc else y


class W4A16:
    """A uint4 group-quantised weight; see nslq_w4a16_create_nk / _awq_kn in the header."""

    def __init__(self, handle, keep, N, K, group_size):
        self._h, self._keep, self.N, self.K, self.group_size = handle, keep, N, K, group_size

    @classmethod
    def from_nk(cls, codes, scales, zero_points, group_size, zp_packed=False):
        N, K = codes.shape[0], codes.shape[1] * 2
        h = C.c_void_p()
        check(lib().nslq_w4a16_create_nk(_ptr(codes), _ptr(scales), _tag(scales.dtype), _ptr(zero_points),
                                         1 if zp_packed else 0, N, K, group_size, C.byref(h)))
        return cls(h, (codes,), N, K, group_size)

    @classmethod
    def from_awq_kn(cls, data, scales, zeros, K, N, group_size):
        h = C.c_void_p()
        check(lib().nslq_w4a16_create_awq_kn(_ptr(data), _ptr(scales), _ptr(zeros), K, N, group_size, C.byref(h)))
        return cls(h, (), N, K, group_size)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:
            lib().nslq_w4a16_destroy(h)

    def forward(self, x, out_dtype=None, out=None):
        _cuda2d(x, "x")
        M = x.shape[0]
        if x.shape[1] != self.K:
            raise ValueError("x has K=%d, weight expects %d" % (x.shape[1], self.K))
        y = out if out is not None else torch.empty(M, self.N, dtype=out_dtype or x.dtype, device=x.device)
        check(lib().nslq_w4a16_forward(self._h, _ptr(x), _tag(x.dtype), M, _ptr(y), _tag(y.dtype), _stream()))
        return y


def ternary_quantize_pack(w):
    """Float weight [out, in] -> (packed uint8 [out, in/4], scale tensor[1]) with the reference loader's arithmetic."""
    if not w.is_cuda or not w.is_contiguous():
        raise ValueError("w must be a contiguous CUDA tensor")
    packed = torch.empty(w.shape[0], w.shape[1] // 4, dtype=torch.uint8, device=w.device)
    scale = torch.empty(1, dtype=torch.float32, device=w.device)
    check(lib().nslq_ternary_quantize_pack(_ptr(w), _tag(w.dtype), w.numel(), _ptr(packed), _ptr(scale), _stream()))
    return packed, scale


def int4_quantize_nk(w, group_size):
    """[N,K] f32/f64 -> (codes [N,K/2], scale f32 [N,G], zero_point u8 [N,G]), the QuantizedTensor form."""
    N, K = w.shape
    G = (K + group_size - 1) // group_size
    codes = torch.empty(N, K // 2, dtype=torch.uint8, device=w.device)
    scale = torch.empty(N, G, dtype=torch.float32, device=w.device)
    zp = torch.empty(N, G, dtype=torch.uint8, device=w.device)
    check(lib().nslq_int4_quantize_nk(_ptr(w), _tag(w.dtype), N, K, group_size, _ptr(codes), _ptr(scale), _ptr(zp),
                                      _stream()))
    return codes, scale, zp


def qtensor_quantize(src, dtype, gran, axis=0, group_size=0):
    """nsl_qtensor_quantize on the GPU: src f32/f64 CUDA tensor -> (data u8, scale f32, zero_point u8) flat tensors."""
    if not src.is_cuda or not src.is_contiguous():
        raise ValueError("src must be a contiguous CUDA tensor")
    shape = (C.c_int64 * src.dim())(*src.shape)
    ns = int(lib().nslq_qtensor_num_scales(shape, src.dim(), gran, axis, group_size))
    if ns < 0:
        raise ValueError(lib().nslq_last_error().decode())
    total = src.numel()
    data = torch.empty((total + 1) // 2 if dtype == 1 else total, dtype=torch.uint8, device=src.device)
    scale = torch.empty(ns, dtype=torch.float32, device=src.device)
    zp = torch.empty(ns, dtype=torch.uint8, device=src.device)
    check(lib().nslq_qtensor_quantize(_ptr(src), _tag(src.dtype), shape, src.dim(), dtype, gran, axis, group_size,
                                      _ptr(data), _ptr(scale), _ptr(zp), _stream()))
    return data, scale, zp


def qtensor_dequantize(data, scale, zp, shape, dtype, gran, axis=0, group_size=0, out_dtype=torch.float64):
    sh = (C.c_int64 * len(shape))(*shape)
    out = torch.empty(*shape, dtype=out_dtype, device=data.device)
    check(lib().nslq_qtensor_dequantize(_ptr(data), _ptr(scale), _ptr(zp), sh, len(shape), dtype, gran, axis, group_size,
                                        _ptr(out), _tag(out_dtype), _stream()))
    return out


def awq_quantize_kn(w, group_size):
    """[K,N] f32/f64 -> (data [K*N/2], scales f64 [G*N], zeros f64 [G*N]), the AwqPackedWeight form."""
    K, N = w.shape
    G = (K + group_size - 1) // group_size
    data = torch.empty(K * N // 2, dtype=torch.uint8, device=w.device)
    scales = torch.empty(G * N, dtype=torch.float64, device=w.device)
    zeros = torch.empty(G * N, dtype=torch.float64, device=w.device)
    check(lib().nslq_awq_quantize_kn(_ptr(w), _tag(w.dtype), K, N, group_size, _ptr(data), _ptr(scales), _ptr(zeros),
                                     _stream()))
    return data, scales, zeros


def device_status():
    """Nonzero if a bounded wait inside a kernel expired since the last call (then cleared)."""
    torch.cuda.synchronize()      # torch's side streams are non-blocking: the library's read does not wait for them
    v = C.c_int()
    check(lib().nslq_device_status(C.byref(v)))
    return v.value


def shard_rows(N, world, rank):
    """(row0, rows) of the output rows rank `rank` owns under column-parallel sharding."""
    r0, n = C.c_int64(), C.c_int64()
    check(lib().nslq_shard_rows(N, world, rank, C.byref(r0), C.byref(n)))
    return r0.value, n.value
