"""ctypes binding of the plain-C oracle (``windowed_oracle.c``).  TEST INFRASTRUCTURE ONLY."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    """Compile ``liboracle_c.so`` beside this file (no-op when up to date)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    return os.path.join(_HERE, "liboracle_c.so")


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle_c.so")
        if not os.path.exists(path):
            build()
        lib = ctypes.CDLL(path)
        lib.tmw_oracle_row_count.restype = ctypes.c_long
        lib.tmw_oracle_row_count.argtypes = [ctypes.c_long] * 4
        fp = ctypes.POINTER(ctypes.c_float)
        lib.tmw_oracle_attention_f32.restype = ctypes.c_int
        lib.tmw_oracle_attention_f32.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 7 + [
            ctypes.c_long,
            ctypes.c_long,
            ctypes.c_float,
        ]
        _LIB = lib
    return _LIB


def row_count(p: int, length: int, window: int, n_persistent: int) -> int:
    return int(_lib().tmw_oracle_row_count(p, length, window, n_persistent))


def attention(q, k, v, window: int, n_persistent: int, q_pos0: int = 0, k_pos0=None, scale: float = 0.0):
    """q ``[B,H,Rq,dh]``, k/v ``[B,H,Rk,dh]`` (numpy or torch CPU, any float) → float32 numpy."""
    q, k, v = (np.ascontiguousarray(np.asarray(t, dtype=np.float32)) for t in (q, k, v))
    B, H, rq, dh = q.shape
    rk = k.shape[2]
    if k_pos0 is None:
        k_pos0 = n_persistent
    o = np.empty_like(q)
    fp = ctypes.POINTER(ctypes.c_float)
    rc = _lib().tmw_oracle_attention_f32(
        q.ctypes.data_as(fp), k.ctypes.data_as(fp), v.ctypes.data_as(fp), o.ctypes.data_as(fp),
        B, H, rq, rk, dh, window, n_persistent, q_pos0, k_pos0, scale,
    )
    if rc != 0:
        raise ValueError("tmw_oracle_attention_f32: bad arguments")
    return o
