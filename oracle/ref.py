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
    """Compile ``attn_ref.c`` and ``gpt_ref.c`` with the Makefile beside them; returns the .so path."""
    srcs = [os.path.join(_HERE, f) for f in ("attn_ref.c", "gpt_ref.c")]
    stale = (not os.path.exists(_SO)) or any(os.path.getmtime(_SO) < os.path.getmtime(s) for s in srcs)
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
        ll, lp = ctypes.c_longlong, ctypes.POINTER(ctypes.c_longlong)
        for name in ("ref_matmul_nn", "ref_matmul_nt", "ref_matmul_tn"):
            getattr(L, name).argtypes = [fp, fp, fp, ll, ll, ll]
            getattr(L, name).restype = None
        L.ref_set_num_threads.argtypes = [ctypes.c_int]
        L.ref_set_num_threads.restype = ctypes.c_int
        L.ref_embedding_fwd.argtypes = [fp, lp, ll, ctypes.c_int, fp]
        L.ref_embedding_fwd.restype = None
        L.ref_embedding_bwd.argtypes = [fp, lp, ll, ctypes.c_int, ll, fp]
        L.ref_embedding_bwd.restype = None
        L.ref_cross_entropy_fwd.argtypes = [fp, lp, ll, ll, fp, fp]
        L.ref_cross_entropy_fwd.restype = ctypes.c_float
        L.ref_nll_loss.argtypes = [fp, lp, ll, ll, fp]
        L.ref_nll_loss.restype = ctypes.c_float
        L.ref_cross_entropy_bwd.argtypes = [fp, lp, ll, ll, fp]
        L.ref_cross_entropy_bwd.restype = None
        L.ref_rotary_cache.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_float, fp, fp]
        L.ref_rotary_cache.restype = None
        L.ref_gpt_step.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_double, ctypes.c_float, ctypes.c_int,
                                   ctypes.c_int, lp, lp, ctypes.POINTER(fp), fp, fp, ctypes.POINTER(fp)]
        L.ref_gpt_step.restype = ctypes.c_int
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


def set_num_threads(n: int | None = None) -> int:
    """Makes the oracle's OpenMP loops use ``n`` threads (default: every core this process may run on,
    whatever OMP_NUM_THREADS says: launchers such as torchrun export OMP_NUM_THREADS=1).  Returns n."""
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return int(lib().ref_set_num_threads(int(n)))


def _ids(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))


def matmul(a, b, kind: str = "nn"):
    """f32 matmul with k-sequential sums: nn: a[M,K] @ b[K,N]; nt: a[M,K] @ b[N,K]^T; tn: a[K,M]^T @ b[K,N]."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if kind == "nn":
        (M, K), N = a.shape, b.shape[1]
    elif kind == "nt":
        (M, K), N = a.shape, b.shape[0]
    else:
        (K, M), N = a.shape, b.shape[1]
    c = np.empty((M, N), np.float32)
    getattr(lib(), f"ref_matmul_{kind}")(_p(a), _p(b), _p(c), M, N, K)
    return c


def embedding_fwd(weight, ids):
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    ids_a, ids_p = _ids(ids)
    out = np.empty((ids_a.size, weight.shape[1]), np.float32)
    lib().ref_embedding_fwd(_p(weight), ids_p, ids_a.size, weight.shape[1], _p(out))
    return out


def embedding_bwd(dout, ids, vocab: int):
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    ids_a, ids_p = _ids(ids)
    dw = np.empty((vocab, dout.shape[1]), np.float32)
    lib().ref_embedding_bwd(_p(dout), ids_p, ids_a.size, dout.shape[1], vocab, _p(dw))
    return dw


def nll_loss(log_probs, targets, with_grad: bool = False):
    """nll_loss (loss.rs:11-15); with_grad also returns d loss / d log_probs."""
    lp = np.ascontiguousarray(log_probs, dtype=np.float32)
    t_a, t_p = _ids(targets)
    g = np.empty_like(lp) if with_grad else None
    loss = float(lib().ref_nll_loss(_p(lp), t_p, lp.shape[0], lp.shape[1], _p(g)))
    return (loss, g) if with_grad else loss


def cross_entropy(logits, targets, with_grad: bool = False):
    """cross_entropy (loss.rs:21-24): returns loss, or (loss, lse, dlogits)."""
    x = np.ascontiguousarray(logits, dtype=np.float32)
    t_a, t_p = _ids(targets)
    lse = np.empty(x.shape[0], np.float32)
    loss = float(lib().ref_cross_entropy_fwd(_p(x), t_p, x.shape[0], x.shape[1], None, _p(lse)))
    if not with_grad:
        return loss
    d = np.empty_like(x)
    lib().ref_cross_entropy_bwd(_p(x), t_p, x.shape[0], x.shape[1], _p(d))
    return loss, lse, d


def rotary_cache(T: int, D: int, base: float = 10000.0):
    cos = np.empty((T, D // 2), np.float32)
    sin = np.empty((T, D // 2), np.float32)
    lib().ref_rotary_cache(T, D, base, _p(cos), _p(sin))
    return cos, sin


def gpt_param_shapes(vocab: int, n_layer: int, n_head: int, n_embd: int, mlp_hidden: int):
    """(name, shape) of every parameter in the order of GPT::parameters (gpt.rs:358-365)."""
    out = [("wte.weight", (vocab, n_embd))]
    for i in range(n_layer):
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            out.append((f"blocks.{i}.attn.{n}.weight", (n_embd, n_embd)))
        out.append((f"blocks.{i}.mlp.up_proj.weight", (n_embd, mlp_hidden)))
        out.append((f"blocks.{i}.mlp.down_proj.weight", (mlp_hidden, n_embd)))
    out.append(("lm_head.weight", (n_embd, vocab)))
    return out


def gpt_init_params(cfg, seed: int = 0):
    """Random-init weights with the reference's distributions (nn.rs:166-176: uniform [-k, k], k = 1/sqrt(in);
    nn.rs:209-212: standard normal embedding) from a numpy seed (the reference's RNG is unseeded)."""
    rng = np.random.default_rng(seed)
    params = []
    for name, shape in gpt_param_shapes(*cfg):
        if name == "wte.weight":
            params.append(rng.standard_normal(shape).astype(np.float32))
        else:
            k = 1.0 / np.sqrt(shape[0])
            params.append((rng.random(shape, dtype=np.float32) * np.float32(2.0 * k) - np.float32(k)).astype(np.float32))
    return params


def gpt_step(cfg, params, ids, targets=None, B=None, T=None, eps: float = 1e-5, rope_base: float = 10000.0,
             want_logits: bool = True, want_grads: bool = True):
    """One forward (+ cross-entropy + backward) of the reference GPT on the CPU.  cfg = (vocab, n_layer, n_head,
    n_embd, mlp_hidden); params as from gpt_init_params; ids [B, T].  Returns dict(logits, loss, grads)."""
    ids = np.asarray(ids)
    if B is None:
        B, T = ids.shape
    ids_a, ids_p = _ids(ids.reshape(-1))
    V = cfg[0]
    fpp = ctypes.POINTER(ctypes.c_float)
    params = [np.ascontiguousarray(p, dtype=np.float32) for p in params]
    parr = (fpp * len(params))(*[_p(p) for p in params])
    logits = np.empty((B * T, V), np.float32) if want_logits else None
    loss = np.zeros(1, np.float32)
    tgt_p = None
    grads = garr = None
    if targets is not None:
        t_a, tgt_p = _ids(np.asarray(targets).reshape(-1))
        if want_grads:
            grads = [np.empty_like(p) for p in params]
            garr = (fpp * len(grads))(*[_p(g) for g in grads])
    ccfg = (ctypes.c_int * 5)(*cfg)
    rc = lib().ref_gpt_step(ccfg, eps, rope_base, B, T, ids_p, tgt_p, parr, _p(logits), _p(loss), garr)
    if rc:
        raise MemoryError("oracle: allocation failed")
    return {"logits": logits, "loss": float(loss[0]) if targets is not None else None, "grads": grads}
