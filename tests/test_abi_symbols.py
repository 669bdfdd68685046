"""CPU checks of the boundary: the shared library loads, exports every symbol the
header declares, and the argument checks that need no GPU behave."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from nsl_b200 import build
    return build.build()


def declared_symbols(header="nslq_b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nslq?_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(built):
    names = declared_symbols()
    assert "nslq_bitlinear_forward" in names and "nslq_w4a16_forward" in names
    l = C.CDLL(built)
    missing = [n for n in names if not hasattr(l, n)]
    assert not missing, missing


def test_ctypes_table_matches_header(built):
    from nsl_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert sorted(_lib.SHIM_SIGNATURES) == declared_symbols("nsl_shims.h")
    l = C.CDLL(built)
    assert not [n for n in declared_symbols("nsl_shims.h") if not hasattr(l, n)]


def test_shim_null_handling_without_gpu(built):
    """awq family: message + 0 on null, as the reference does (awq.rs:266)."""
    from nsl_b200 import _lib
    l = _lib.lib()
    assert l.nsl_awq_matmul_cuda(0, 0, 128, 0) == 0
    assert l.nsl_bitlinear_pack(0, 16, 64, 1.0) == 0
    assert l.nsl_bitlinear_forward(0, 0, 0) == 0
    l.nsl_bitlinear_free(0)
    l.nsl_quant_forget_cuda(12345)


def test_argument_checks_without_gpu(built):
    from nsl_b200 import _lib
    l = _lib.lib()
    assert l.nslq_version() >= 100
    r0, n = C.c_int64(), C.c_int64()
    assert l.nslq_shard_rows(8640, 8, 7, C.byref(r0), C.byref(n)) == 0 and (r0.value, n.value) == (7560, 1080)
    assert l.nslq_shard_rows(10, 4, 0, C.byref(r0), C.byref(n)) == -2
    assert b"divisible" in l.nslq_last_error()
    assert l.nslq_shard_rows(16, 4, 4, C.byref(r0), C.byref(n)) == -1
    h = C.c_void_p()
    assert l.nslq_bitlinear_create(None, 16, 64, 1.0, C.byref(h)) == -1
    assert l.nslq_bitlinear_create(C.c_void_p(256), 16, 62, 1.0, C.byref(h)) == -2     # K % 4
    assert l.nslq_bitlinear_create(C.c_void_p(256), 16, 64, 1.0, C.byref(h)) == 0
    assert l.nslq_bitlinear_workspace_bytes(16, 3200) >= 16 * 3200 + 128
    # missing workspace is refused before anything is launched
    assert l.nslq_bitlinear_forward(h, C.c_void_p(256), 1, 1, C.c_void_p(512), 1, None, None, None, None, 0, None) == -5
    l.nslq_bitlinear_destroy(h)
    assert l.nslq_act_quant_i8(None, 1, 1, 16, None, None, None, None, None) == -1
    assert l.nslq_w4a16_forward(None, None, 3, 1, None, 3, None) == -1


def test_no_oracle_in_product():
    """The package must not import or reference the CPU checker."""
    pkg = os.path.join(ROOT, "nsl_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)


def test_sharding_argument_checks_without_gpu(built):
    """nslq_shard_* refuse bad ranks, null communicators and null buffers before touching a device."""
    from nsl_b200 import _lib
    l = _lib.lib()
    h = C.c_void_p()
    assert l.nslq_shard_init(None, 3, 2, C.byref(h)) == -1 and b"rank 3 of 2" in l.nslq_last_error()
    assert l.nslq_shard_init(None, 0, 9, C.byref(h)) == -1              # more than NSLQ_MAX_RANKS
    assert l.nslq_shard_init(None, 0, 2, C.byref(h)) == -1 and b"unique id" in l.nslq_last_error()
    assert l.nslq_shard_init(None, 0, 1, None) == -1
    assert l.nslq_shard_unique_id(None) == -1
    assert l.nslq_allgather_cols(None, None, 1, 1, 16, None, None, None) == -1
    assert l.nslq_peer_barrier(None, None) == -1
    assert l.nslq_symm_alloc(None, 1024, C.byref(h)) == -1
    assert l.nslq_shard_wait(None, None, 10) == -1
    assert l.nslq_bitlinear_gathered_workspace_bytes(8, 3200, 1080) == l.nslq_bitlinear_workspace_bytes(8, 3200) + 34560
    assert l.nslq_bitlinear_gathered_workspace_bytes(256, 4096, 512) == l.nslq_bitlinear_workspace_bytes(256, 4096)
    w = C.c_void_p()
    assert l.nslq_bitlinear_create(C.c_void_p(256), 16, 64, 1.0, C.byref(w)) == 0
    arr = (C.c_void_p * 1)(C.c_void_p(4096))
    # columns [8, 24) do not fit rows of 16
    assert l.nslq_bitlinear_forward_quantized_cols(w, C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), 4, arr, 1, 16, 8, 1,
                                                   None, None, 0, None) == -2
    assert l.nslq_bitlinear_forward_quantized_cols(w, C.c_void_p(256), C.c_void_p(256), C.c_void_p(256), 4, arr, 9, 16, 0, 1,
                                                   None, None, 0, None) == -1
    l.nslq_bitlinear_destroy(w)
