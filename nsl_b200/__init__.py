"""B200 (sm_100a) kernels for NSL's quantized-linear path behind a C ABI.

`nsl_b200.ops` needs torch; `nsl_b200._lib` and `nsl_b200.build` do not.
"""
from ._lib import LIB_PATH, NslqError, lib  # noqa: F401
