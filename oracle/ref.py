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
        L.ref_adamw_step.argtypes = [fp, fp, fp, fp, ctypes.c_longlong] + [ctypes.c_double] * 5 + [ctypes.c_int]
        L.ref_adamw_step.restype = None
        L.ref_grad_sq_sum.argtypes = [fp, ctypes.c_longlong]
        L.ref_grad_sq_sum.restype = ctypes.c_float
        L.ref_rmsnorm.argtypes = [fp, ctypes.c_longlong, ctypes.c_int, ctypes.c_double, fp, fp, fp]
        L.ref_rmsnorm.restype = None
        L.ref_rope_pack.argtypes = [fp, fp, fp] + [ctypes.c_int] * 5 + [fp]
        L.ref_rope_pack.restype = None
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


def precompute_rotary_embeddings(seq_len: int, head_dim: int, base: float = 10000.0):
    """cos / sin cache [T, D/2] in f32, the arithmetic of gpt.rs:12-46: inv_freq = 1 / base^(2i/D)
    in f32, angle = t * inv_freq in f32, then cos / sin.  (The reference keeps the cache as
    [1, T, 1, D/2]; the two unit axes only serve broadcasting.)"""
    assert head_dim % 2 == 0, "RoPE requires an even head dimension"
    half = head_dim // 2
    channel = (2 * np.arange(half)).astype(np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base), channel / np.float32(head_dim))).astype(np.float32)
    freqs = (np.arange(seq_len, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)


def rope_pack(x, cos, sin, inverse: bool = False):
    """f32: [B,T,H,D] -> rotated [B,H,T,D]; inverse: gradient [B,H,T,D] -> [B,T,H,D] (C restatement)."""
    x = _c(x)
    cos = np.ascontiguousarray(cos, dtype=np.float32)
    sin = np.ascontiguousarray(sin, dtype=np.float32)
    if inverse:
        B, H, T, D = x.shape
        y = np.empty((B, T, H, D), np.float32)
    else:
        B, T, H, D = x.shape
        y = np.empty((B, H, T, D), np.float32)
    assert cos.shape == (T, D // 2) and sin.shape == (T, D // 2)
    lib().ref_rope_pack(_p(x), _p(cos), _p(sin), B, T, H, D, int(inverse), _p(y))
    return y


def rope_pack_f16(x, cos, sin, inverse: bool = False):
    """f16 storage: the same op chain with every multiply and add rounded to f16, as the reference's
    f16 element-wise ops do (numpy float16 arithmetic rounds each operation once)."""
    x = np.asarray(x, np.float16)
    cos = np.asarray(cos, np.float16)
    sin = np.asarray(sin, np.float16)
    if inverse:
        src = np.transpose(x, (0, 2, 1, 3))                     # [B,H,T,D] -> [B,T,H,D]
        s = (sin * np.float16(-1.0))[None, :, None, :]
    else:
        src = x
        s = sin[None, :, None, :]
    c = cos[None, :, None, :]
    half = src.shape[3] // 2
    a, b = src[..., :half], src[..., half:]
    y1 = a * c + b * s
    y2 = a * (s * np.float16(-1.0)) + b * c
    y = np.concatenate([y1, y2], axis=3).astype(np.float16)     # [B,T,H,D]
    return y if inverse else np.ascontiguousarray(np.transpose(y, (0, 2, 1, 3)))


def adamw_step(w, g, m, v, step: int, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
    """One AdamW step on one parameter, in place on contiguous f32 arrays w, m, v (optim.rs:214-251)."""
    for a in (w, g, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    lib().ref_adamw_step(_p(w), _p(g), _p(m), _p(v), w.size, lr, betas[0], betas[1], eps, weight_decay, step)


def clip_grad_norm(grads, max_norm: float):
    """clip_grad_norm (optim.rs:257-297) on a list of contiguous f32 gradient arrays, scaled in place when
    the norm exceeds max_norm; returns the norm before clipping as a Python float (f32 value)."""
    assert max_norm > 0.0, "max_norm must be positive"
    if not grads:
        return 0.0
    total = np.float32(0.0)
    for g in grads:
        assert g.dtype == np.float32 and g.flags.c_contiguous
        total = np.float32(total + np.float32(lib().ref_grad_sq_sum(_p(g), g.size)))
    norm = np.float32(np.sqrt(total))
    if not np.isfinite(norm) or norm <= np.float32(max_norm):
        return float(norm)
    scale = np.float32(max_norm / (float(norm) + 1e-6))
    for g in grads:
        g *= scale
    return float(norm)


def rmsnorm(x, eps: float, dy=None):
    """RMSNorm over the last axis of a contiguous f32 array (nn.rs:244-251); returns y, or (y, dx) with dy."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    C = x.shape[-1]
    rows = x.size // C
    y = np.empty_like(x)
    if dy is None:
        lib().ref_rmsnorm(_p(x), rows, C, eps, None, _p(y), None)
        return y
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    dx = np.empty_like(x)
    lib().ref_rmsnorm(_p(x), rows, C, eps, _p(dy), _p(y), _p(dx))
    return y, dx


def attn_decode(q, k, v, scale=None, causal=True):
    """Tq query rows against Tk >= Tq key / value rows, f32, the op chain of gpt.rs:139-144 with the additive
    mask of functional.rs:12-55 at seqlen_offset = Tk - Tq (the pinned ref_causal_mask); returns (o, lse)."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.float32) for a in (q, k, v))
    B, H, Tq, D = q.shape
    Tk = k.shape[2]
    scale = default_scale(D) if scale is None else scale
    s = np.einsum("bhid,bhjd->bhij", q, k).astype(np.float32) * np.float32(scale)
    if causal:
        s = s + causal_mask(B, Tq, Tk - Tq)
    m = s.max(axis=3, keepdims=True)
    e = np.exp(s - m)
    lse = (np.log(e.sum(axis=3, keepdims=True, dtype=np.float32)) + m).astype(np.float32)
    p = np.exp(s - lse).astype(np.float32)
    return np.einsum("bhij,bhjd->bhid", p, v).astype(np.float32), lse[..., 0]
