"""ctypes wrapper around oracle/liboracle_affine.so (the C + OpenMP restatement).

TEST INFRASTRUCTURE ONLY.  Inputs and outputs are numpy arrays; bf16 data is uint16 bit
patterns.  See oracle/affine_c.c for the reference lines each routine follows.
"""

from __future__ import annotations

import ctypes

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(array):
    return None if array is None else array.ctypes.data_as(ctypes.c_void_p)


def _u16(array):
    return None if array is None else np.ascontiguousarray(array, dtype=np.uint16)


def num_threads():
    return int(lib().oracle_num_threads())


def set_threads(threads):
    """Use `threads` OpenMP threads from now on (a launcher may have exported OMP_NUM_THREADS=1)."""
    lib().oracle_set_threads(int(threads))
    return num_threads()


def qmm(x_bits, packed, scale_bits, bias_bits, residual_bits=None):
    x = _u16(x_bits)
    m, k = x.shape
    w = np.ascontiguousarray(packed, dtype=np.uint32)
    n = w.shape[0]
    out = np.empty((m, n), dtype=np.uint16)
    rc = lib().oracle_qmm_bf16(_p(x), _p(w), _p(_u16(scale_bits)), _p(_u16(bias_bits)),
                               _p(_u16(residual_bits)), _p(out), m, k, n)
    if rc:
        raise ValueError("oracle_qmm_bf16 rejected the shapes")
    return out


def swiglu(x_bits, gate, up):
    x = _u16(x_bits)
    m, k = x.shape
    gw, gs, gb = (np.ascontiguousarray(gate[0], dtype=np.uint32), _u16(gate[1]), _u16(gate[2]))
    uw, us, ub = (np.ascontiguousarray(up[0], dtype=np.uint32), _u16(up[1]), _u16(up[2]))
    n = gw.shape[0]
    out = np.empty((m, n), dtype=np.uint16)
    rc = lib().oracle_swiglu_bf16(_p(x), _p(gw), _p(gs), _p(gb), _p(uw), _p(us), _p(ub), _p(out),
                                  m, k, n)
    if rc:
        raise ValueError("oracle_swiglu_bf16 rejected the shapes")
    return out


def mlp(x_bits, gate, up, down, residual_bits=None):
    x = _u16(x_bits)
    m, h = x.shape
    gw, gs, gb = (np.ascontiguousarray(gate[0], dtype=np.uint32), _u16(gate[1]), _u16(gate[2]))
    uw, us, ub = (np.ascontiguousarray(up[0], dtype=np.uint32), _u16(up[1]), _u16(up[2]))
    dw, ds, db = (np.ascontiguousarray(down[0], dtype=np.uint32), _u16(down[1]), _u16(down[2]))
    inter = gw.shape[0]
    hidden = np.empty((m, inter), dtype=np.uint16)
    out = np.empty((m, h), dtype=np.uint16)
    rc = lib().oracle_mlp_bf16(_p(x), _p(gw), _p(gs), _p(gb), _p(uw), _p(us), _p(ub), _p(dw),
                               _p(ds), _p(db), _p(_u16(residual_bits)), _p(hidden), _p(out),
                               m, h, inter)
    if rc:
        raise ValueError("oracle_mlp_bf16 rejected the shapes")
    return out


def add_rmsnorm(x_bits, residual_bits, weight_bits, eps):
    x = _u16(x_bits)
    rows, h = x.shape
    total = np.empty((rows, h), dtype=np.uint16)
    norm = np.empty((rows, h), dtype=np.uint16)
    lib().oracle_add_rmsnorm_bf16(_p(x), _p(_u16(residual_bits)), _p(_u16(weight_bits)), _p(total),
                                  _p(norm), rows, h, ctypes.c_float(eps))
    return total, norm
