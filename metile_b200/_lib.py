"""ctypes binding of csrc/libmetile_b200.so (C ABI declared in include/metile_b200.h).

The shared object is built in-tree by `python -m metile_b200.build`.  If it is missing the
import of any operator fails loudly: there is no CPU or PyTorch fallback on this path.
"""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(HERE, "csrc", "libmetile_b200.so")

FLAG_FORCE_GEMV = 0x1
FLAG_FORCE_UMMA = 0x2
FLAG_MLP_FUSED = 0x20
FLAG_HOST_PAIR = 0x40
FLAG_MLP_FUSED_MMA = 0x80
FLAG_GELU = 0x10

_VALUE_ERRORS = {-1, -2, -3, -6, -7}

_p = ctypes.c_void_p
_i = ctypes.c_int
_u = ctypes.c_uint
_z = ctypes.c_size_t
_f = ctypes.c_float

SIGNATURES = {
    "mt_version": (_i, []),
    "mt_status_string": (ctypes.c_char_p, [_i]),
    "mt_device_check": (_i, []),
    "mt_device_status": (_i, [ctypes.POINTER(ctypes.c_uint), _i]),
    "mt_selftest_bounded_wait": (_i, [_i, _u, _p]),
    "mt_affine_qmv": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _u, _p]),
    "mt_affine_swiglu": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _u, _p]),
    "mt_affine_mlp_workspace_bytes": (_z, [_i, _i, _i]),
    "mt_affine_mlp": (_i, [_p] * 12 + [_z, _p, _i, _i, _i, _i, _i, _u, _p]),
    "mt_affine_mlp_host": (_i, [_p] * 16 + [_z, _i, _i, _i, _i, _i, _u, _p]),
    "mt_affine_mlp_launches": (_i, [_i, _i, _i, _u]),
    "mt_affine_mlp_static_max_bytes": (_z, []),
    "mt_affine_mlp_static": (_i, [_p] * 12 + [_i, _i, _i, _i, _i, _u, _p]),
    "mt_add_rmsnorm": (_i, [_p, _p, _p, _p, _p, _i, _i, _f, _p]),
    "mt_rmsnorm": (_i, [_p, _p, _p, _i, _i, _f, _p]),
    "mt_attention_decode_workspace_bytes": (_z, [_i, _i, _i, _i]),
    "mt_attention_decode": (_i, [_p, _p, _p, _p, _p, _p, _z, _i, _i, _i, _i, _i, _i, _f, _p]),
    "mt_rope_kv_append": (_i, [_p, _p, _p, ctypes.c_longlong, _p, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p]),
    "mt_peer_group_create": (_i, [_i, _i, _z, ctypes.POINTER(ctypes.c_void_p), _p]),
    "mt_peer_group_connect": (_i, [_p, _p]),
    "mt_peer_group_set_mode": (_i, [_p, _i]),
    "mt_peer_all_reduce": (_i, [_p, _p, _p, _z, _u, _p]),
    "mt_peer_group_destroy": (_i, [_p]),
    "mt_dense_rows": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "mt_dense_swiglu": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "mt_dense_act": (_i, [_p, _p, _p, _i, _i, _i, _u, _p]),
}

_lib = None


def load():
    """Load the shared library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise ImportError(
            f"{LIBRARY_PATH} is missing. Build it with `python -m metile_b200.build` "
            "(needs nvcc); this package has no fallback path."
        )
    lib = ctypes.CDLL(LIBRARY_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(lib, name)
        function.restype = restype
        function.argtypes = argtypes
    _lib = lib
    return lib


def status_string(code):
    return load().mt_status_string(int(code)).decode()


def check(code, what):
    """Raise the exception the reference's operators raise for the same class of error."""
    if code == 0:
        return
    message = f"{what}: {status_string(code)} (status {code})"
    if code in _VALUE_ERRORS:
        raise ValueError(message)
    raise RuntimeError(message)


def device_status(reset=True):
    """(ok, words) -- words[0] != 0 means a bounded device-side wait gave up."""
    words = (ctypes.c_uint * 4)()
    code = load().mt_device_status(words, 1 if reset else 0)
    return code == 0, tuple(int(v) for v in words)
