"""ctypes front end of the C oracle in ``attn_ref.c`` (test infrastructure).

The shipped library never imports this module: it exists so that tests, the
smoke check and the benchmark's CPU-baseline leg can run the reference math on
host arrays.  All tensors are compact ``[B, H, T, D]`` float32 numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libattn_ref.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``attn_ref.c`` with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "attn_ref.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "_build/libattn_ref.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        L.ref_num_threads.restype = ctypes.c_int
        L.ref_causal_mask.argtypes = [ctypes.c_int] * 3 + [fp]
        L.ref_causal_mask.restype = None
        L.ref_attn_fwd.argtypes = [fp, fp, fp] + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int, fp, fp]
        L.ref_attn_fwd.restype = ctypes.c_int
        L.ref_attn_fwd_bwd.argtypes = ([fp, fp, fp, fp] + [ctypes.c_int] * 4 +
                                       [ctypes.c_float, ctypes.c_int] + [fp] * 5)
        L.ref_attn_fwd_bwd.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) if a is not None else None


def _c(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    assert a.ndim == 4, "expected [B, H, T, D]"
    return a


def num_threads() -> int:
    return int(lib().ref_num_threads())


def causal_mask(batch: int, tgt_len: int, offset: int = 0) -> np.ndarray:
    out = np.empty((batch, 1, tgt_len, tgt_len + offset), np.float32)
    lib().ref_causal_mask(batch, tgt_len, offset, _p(out))
    return out


def default_scale(D: int) -> float:
    """The module's scale: 1/sqrt(head_dim) in f64, cast to f32 (gpt.rs:139, storage.rs:115-117)."""
    return float(np.float32(1.0 / np.sqrt(np.float64(D))))


def attn_fwd(q, k, v, scale=None, causal=True):
    q, k, v = _c(q), _c(k), _c(v)
    B, H, T, D = q.shape
    scale = default_scale(D) if scale is None else scale
    o = np.empty_like(q)
    lse = np.empty((B, H, T), np.float32)
    rc = lib().ref_attn_fwd(_p(q), _p(k), _p(v), B, H, T, D, scale, int(causal), _p(o), _p(lse))
    if rc:
        raise MemoryError("oracle: allocation failed")
    return o, lse


def attn_fwd_bwd(q, k, v, d_o, scale=None, causal=True):
    """Returns (o, lse, dq, dk, dv)."""
    q, k, v, d_o = _c(q), _c(k), _c(v), _c(d_o)
    B, H, T, D = q.shape
    scale = default_scale(D) if scale is None else scale
    o = np.empty_like(q)
    lse = np.empty((B, H, T), np.float32)
    dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(q)
    rc = lib().ref_attn_fwd_bwd(_p(q), _p(k), _p(v), _p(d_o), B, H, T, D, scale, int(causal),
                                _p(o), _p(lse), _p(dq), _p(dk), _p(dv))
    if rc:
        raise MemoryError("oracle: allocation failed")
    return o, lse, dq, dk, dv
