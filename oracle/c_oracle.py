"""ctypes front end of oracle/splat_oracle.c (the C restatement of the reference kernels).

TEST INFRASTRUCTURE ONLY.  Operates on fp32 numpy arrays / CPU torch tensors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from .acsr_oracle import affine_ints

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libsplat_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "splat_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "libsplat_oracle.so"], check=True,
                       capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(x):
    if hasattr(x, "detach"):
        x = x.detach().float().cpu().numpy()
    return np.asarray(x, dtype=np.float32)


def num_threads() -> int:
    return lib().oracle_num_threads()


def attention(q, k, v, meta: dict, trailing_dim: int, scale: float = 1.0, return_parts=False):
    """q, k, v: (BH, L, d) (k row-major: the transposed view of the reference's K^T).
    Runs SDDMM -> softmax -> SpMM with S and P materialised, like the reference's forward."""
    q, k, v = (np.ascontiguousarray(_f32(t)) for t in (q, k, v))
    BH, L, d = q.shape
    start, stride, nnz = (np.ascontiguousarray(a.astype(np.int32)) for a in affine_ints(meta))
    T = int(trailing_dim)
    s = np.empty((BH, L, T), dtype=np.float32)
    p = np.empty((BH, L, T), dtype=np.float32)
    o = np.empty((BH, L, d), dtype=np.float32)
    i64 = ctypes.c_int64
    lib().oracle_attention(_p(q), _p(k), i64(L * d), i64(d), i64(1), _p(v), _p(o), _p(s), _p(p),
                           _p(start), _p(stride), _p(nnz), i64(BH), i64(L), i64(d), i64(T),
                           ctypes.c_float(scale))
    return (o, s, p) if return_parts else o
