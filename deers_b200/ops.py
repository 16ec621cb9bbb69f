"""Host-side mirror of the deers operator interface for the fused attention op.

deers builds its graph from ``TensorOp`` objects (src/ops.rs:82-97): ``forward``
consumes the op and returns the output tensor with the op stored in it,
``backward(grads, out_grad)`` accumulates input gradients into a
``GradientStore`` (src/backprop.rs:74-128) and ``dependencies`` lists the inputs.
``CausalAttention`` is that op for the chain of src/models/gpt.rs:139-144; the
storage-level pair ``attention_fwd`` / ``attention_bwd`` is what a new
``BackendStorage::attention_fwd/bwd`` (added like ``log_softmax_fwd/bwd``,
src/storage.rs:284-302) would call through the C ABI.

torch tensors stand in for ``CudaStorage`` + ``Layout`` (device memory, strides,
stream); all arithmetic happens in ``libdeers_b200.so``.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional, Tuple

import torch

from . import _lib
from .errors import DeviceMismatch, DTypeMismatch, LayoutMismatch

_DTYPES = {torch.float16: _lib.F16, torch.float32: _lib.F32}


class Context:
    """One library context per (device, stream): the analogue of deers' global CudaRuntime
    (src/storage/cuda.rs:455-521).  Work is enqueued on torch's current stream."""

    _cache: Dict[Tuple[int, int], "Context"] = {}

    def __init__(self, device: int, stream_ptr: int):
        self.handle = ctypes.c_void_p()
        self.device = device
        # torch's default stream is the legacy NULL stream; the C ABI reads NULL as "create
        # your own stream", so name the legacy stream by its CUDA handle value 1.
        stream_ptr = stream_ptr or 1
        _lib.check(_lib.lib().deers_b200_init(device, ctypes.c_void_p(stream_ptr), ctypes.byref(self.handle)))

    @classmethod
    def current(cls, device: torch.device) -> "Context":
        if device.type != "cuda":
            raise DeviceMismatch("the fused attention op only exists on the CUDA device (no CPU fallback)")
        idx = device.index if device.index is not None else torch.cuda.current_device()
        stream_obj = torch.cuda.current_stream(idx)
        stream = stream_obj.cuda_stream
        key = (idx, stream)
        ctx = cls._cache.get(key)
        if ctx is None:
            ctx = cls(idx, stream)
            ctx._stream_obj = stream_obj     # keeps the stream alive: its handle value cannot be reused by another
            cls._cache[key] = ctx
        return ctx

    def sync(self) -> None:
        """Device::synchronize (src/device.rs:66-72); raises if a kernel reported an error."""
        _lib.check(_lib.lib().deers_b200_sync(self.handle), self.handle)

    def launch_count(self) -> int:
        return int(_lib.lib().deers_b200_launch_count(self.handle))

    def kernel_timing(self, enable: bool) -> None:
        _lib.check(_lib.lib().deers_b200_kernel_timing(self.handle, int(enable)), self.handle)

    def kernel_time(self, kind: int, reset: bool = False):
        """(total milliseconds, launches) of one kernel kind since timing was enabled."""
        ms, n = ctypes.c_double(), ctypes.c_uint64()
        _lib.check(_lib.lib().deers_b200_kernel_time(self.handle, kind, int(reset), ctypes.byref(ms),
                                                     ctypes.byref(n)), self.handle)
        return ms.value, int(n.value)

    def selftest_wait(self, limit_ms: int = 5) -> List[int]:
        """Runs the give-up path of the bounded device waits (deers_b200_selftest_wait): returns
        [first wait gave up, second wait saw the abort flag, microseconds of each]."""
        res = (ctypes.c_int32 * 4)()
        _lib.check(_lib.lib().deers_b200_selftest_wait(self.handle, limit_ms, res), self.handle)
        return [int(v) for v in res]

    def selftest_umma(self) -> List[float]:
        errs = (ctypes.c_float * 6)()
        _lib.check(_lib.lib().deers_b200_selftest_umma(self.handle, errs), self.handle)
        return [float(e) for e in errs]


def _strides(t: torch.Tensor):
    return (ctypes.c_int64 * 4)(*t.stride())


def _check_inputs(name: str, tensors) -> None:
    q = tensors[0]
    if q.dim() != 4:
        raise LayoutMismatch(f"{name}: expected [B, H, T, D], got {tuple(q.shape)}")
    for t in tensors[1:]:
        if t.shape != q.shape:
            raise LayoutMismatch(f"{name}: {tuple(t.shape)} vs {tuple(q.shape)}")
        if t.dtype != q.dtype:
            raise DTypeMismatch(f"{name}: {t.dtype} vs {q.dtype}")
        if t.device != q.device:
            raise DeviceMismatch(f"{name}: {t.device} vs {q.device}")
    if q.dtype not in _DTYPES:
        raise DTypeMismatch(f"{name}: unsupported dtype {q.dtype}")


def _usable(t: torch.Tensor) -> bool:
    """True if the kernels can read `t` in place: inner stride 1 and aligned rows."""
    if t.stride(3) != 1:                 # the C ABI wants inner stride 1 even for a head_dim of 1
        return False
    esize = t.element_size()
    align = 16 if t.dtype == torch.float16 else 4
    if t.data_ptr() % align:
        return False
    return all((t.stride(i) * esize) % align == 0 or t.shape[i] == 1 for i in range(3))


def _compact(t: torch.Tensor) -> torch.Tensor:
    # Inputs that need contiguity are compacted by the op, as in src/ops.rs:1330,1405,1494.
    return t if _usable(t) else t.contiguous()


def _desc(q, k, v, o, d_o=None, dq=None, dk=None, dv=None, scale=1.0, causal=True) -> _lib.AttnDesc:
    B, H, T, D = q.shape
    d = _lib.AttnDesc()
    _lib.lib().deers_b200_attn_desc_compact(ctypes.byref(d), B, H, T, D, _DTYPES[q.dtype], int(causal), scale)
    d.q_strides, d.k_strides, d.v_strides, d.o_strides = _strides(q), _strides(k), _strides(v), _strides(o)
    if d_o is not None:
        d.do_strides, d.dq_strides, d.dk_strides, d.dv_strides = (_strides(d_o), _strides(dq), _strides(dk),
                                                                 _strides(dv))
    return d


def default_scale(head_dim: int) -> float:
    """1/sqrt(head_dim) computed in f64 as the module does (src/models/gpt.rs:139)."""
    return 1.0 / math.sqrt(float(head_dim))


def attention_fwd(q, k, v, scale: float, causal: bool = True, token_major_out: bool = False,
                  out: Optional[torch.Tensor] = None):
    """Storage-level forward: returns (o [B,H,T,D], lse [B,H,T] float32).

    ``out`` (same shape and dtype as q, inner stride 1) receives O in place, e.g. this rank's slices of
    the buffer an all-gather of O pushes from.

    o is compact by default.  With ``token_major_out`` its memory is a compact [B,T,H,D] buffer
    and the returned tensor is the [B,H,T,D] view of it, so the module's
    ``permute([0,2,1,3]).reshape([B,T,C])`` (src/models/gpt.rs:144) is a free view instead of the
    compaction copy of src/ops.rs:913: the kernels write through the view's strides."""
    _check_inputs("attention_fwd", (q, k, v))
    q, k, v = _compact(q), _compact(k), _compact(v)
    ctx = Context.current(q.device)
    if out is not None:
        if out.shape != q.shape or out.dtype != q.dtype or out.device != q.device or not _usable(out):
            raise LayoutMismatch(f"attention_fwd: out must match q ({tuple(q.shape)}, {q.dtype}) with unit inner stride")
        o = out
    elif token_major_out:
        B, H, T, D = q.shape
        o = torch.empty((B, T, H, D), dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    else:
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    d = _desc(q, k, v, o, scale=scale, causal=causal)
    # The forward needs scratch only for f16 head dims other than 64 / 128 (zero-padded copies of Q, K, V, O).
    need = int(_lib.lib().deers_b200_attn_workspace_bytes(ctypes.byref(d), 0))
    ws = torch.empty(need, dtype=torch.uint8, device=q.device) if need else None
    _lib.check(_lib.lib().deers_b200_attn_fwd(ctx.handle, ctypes.byref(d), q.data_ptr(), k.data_ptr(),
                                              v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                              ws.data_ptr() if need else None, need), ctx.handle)
    return o, lse


def workspace_bytes(q, scale: float = 1.0, causal: bool = True, pass_: int = 1) -> int:
    d = _desc(q, q, q, q, scale=scale, causal=causal)
    return int(_lib.lib().deers_b200_attn_workspace_bytes(ctypes.byref(d), pass_))


def attention_bwd(q, k, v, o, lse, d_o, scale: float, causal: bool = True, workspace: Optional[torch.Tensor] = None,
                  dv_out: Optional[torch.Tensor] = None):
    """Storage-level backward: returns (dq, dk, dv), each compact [B,H,T,D].  `workspace` (uint8, 256-byte
    aligned) of `workspace_bytes(q, pass_=2)` bytes selects the f16 backward that keeps dS tiles, of
    `pass_=1` bytes the recomputing one; without it the function allocates.  `dv_out` (a [B,H,T,D] view
    with inner stride 1, e.g. the v slice of a fused dqkv buffer seen head-major) receives dV in place
    instead: the kernels write through its strides."""
    _check_inputs("attention_bwd", (q, k, v, o, d_o))
    q, k, v, o, d_o = _compact(q), _compact(k), _compact(v), _compact(o), _compact(d_o)
    ctx = Context.current(q.device)
    dq, dk = (torch.empty(q.shape, dtype=q.dtype, device=q.device) for _ in range(2))
    if dv_out is not None:
        if tuple(dv_out.shape) != tuple(q.shape) or dv_out.dtype != q.dtype or not _usable(dv_out):
            raise LayoutMismatch("attention_bwd: dv_out must be a [B,H,T,D] view with inner stride 1 and aligned rows")
        dv = dv_out
    else:
        dv = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    d = _desc(q, k, v, o, d_o, dq, dk, dv, scale=scale, causal=causal)
    need = int(_lib.lib().deers_b200_attn_workspace_bytes(ctypes.byref(d), 1))
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        # The larger size lets the f16 backward keep its dS tiles (two tile products fewer); taken when it is
        # a small part of what the device has free, else the backward recomputes.
        fast = int(_lib.lib().deers_b200_attn_workspace_bytes(ctypes.byref(d), 2))
        if fast > need and fast <= torch.cuda.mem_get_info(q.device)[0] // 4:
            need = fast
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    _lib.check(_lib.lib().deers_b200_attn_bwd(ctx.handle, ctypes.byref(d), q.data_ptr(), k.data_ptr(),
                                              v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
                                              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), workspace.data_ptr(),
                                              workspace.numel() * workspace.element_size()), ctx.handle)
    return dq, dk, dv


def precompute_rotary_embeddings(seq_len: int, head_dim: int, base: float = 10000.0,
                                 dtype: torch.dtype = torch.float32, device="cpu"):
    """cos / sin cache shaped [1, T, 1, D/2] like the reference's (src/models/gpt.rs:12-46): host
    arithmetic in f32 (inv_freq = 1 / base^(2i/D), angle = t * inv_freq), rounded to f16 when asked."""
    if head_dim % 2:
        raise LayoutMismatch("RoPE requires an even head dimension")
    if dtype not in _DTYPES:
        raise DTypeMismatch("RoPE requires a floating-point dtype")
    half = head_dim // 2
    channel = (2 * torch.arange(half, dtype=torch.float32))
    inv_freq = 1.0 / torch.pow(torch.tensor(base, dtype=torch.float32), channel / float(head_dim))
    freqs = torch.arange(seq_len, dtype=torch.float32)[:, None] * inv_freq[None, :]
    shape = (1, seq_len, 1, half)
    return (freqs.cos().to(dtype).reshape(shape).to(device), freqs.sin().to(dtype).reshape(shape).to(device))


def _rope_call(src, cos, sin, dst, src_strides, dst_strides, B, T, H, D, inverse: bool) -> None:
    ctx = Context.current(src.device)
    d = _lib.RopeDesc()
    d.B, d.T, d.H, d.D = B, T, H, D
    d.dtype, d.inverse = _DTYPES[src.dtype], int(inverse)
    d.src_strides = (ctypes.c_int64 * 4)(*src_strides)
    d.dst_strides = (ctypes.c_int64 * 4)(*dst_strides)
    _lib.check(_lib.lib().deers_b200_rope_pack(ctx.handle, ctypes.byref(d), src.data_ptr(), cos.data_ptr(),
                                               sin.data_ptr(), dst.data_ptr()), ctx.handle)


def _check_rope(name: str, x, cos, sin, T: int, D: int):
    if x.dim() != 4:
        raise LayoutMismatch(f"{name}: RoPE expects a 4D attention tensor, got {tuple(x.shape)}")
    if D % 2:
        raise LayoutMismatch(f"{name}: RoPE requires an even head dimension")
    if x.dtype not in _DTYPES:
        raise DTypeMismatch(f"{name}: unsupported dtype {x.dtype}")
    if x.device.type != "cuda":
        raise DeviceMismatch(f"{name}: the fused op runs on the CUDA device only")
    if cos.shape != sin.shape:
        raise LayoutMismatch(f"{name}: RoPE cos/sin shapes must match")
    if cos.numel() != T * (D // 2) or cos.shape[-1] != D // 2:
        raise LayoutMismatch(f"{name}: RoPE cache must be [1, T, 1, D/2] for T={T}, D={D}, got {tuple(cos.shape)}")
    for c in (cos, sin):
        if c.dtype != x.dtype:
            raise DTypeMismatch(f"{name}: cache {c.dtype} vs tensor {x.dtype}")
        if c.device != x.device:
            raise DeviceMismatch(f"{name}: cache on {c.device}, tensor on {x.device}")
    return cos.contiguous(), sin.contiguous()


class RotaryPack:
    """``apply_rotary_emb(x, cos, sin).permute([0,2,1,3])`` (src/models/gpt.rs:49-73,135-136) as ONE op:
    x is the [B,T,H,D] projection output (any strides with inner stride 1), the result is a compact
    [B,H,T,D] tensor ready for ``CausalAttention``; backward rotates the incoming [B,H,T,D] gradient
    back and accumulates it as a [B,T,H,D] tensor.  Same life cycle as the other deers ops."""

    def __init__(self, x, cos, sin):
        self.x, self.cos, self.sin = x, cos, sin

    @classmethod
    def new(cls, x, cos, sin) -> "RotaryPack":
        if x.dim() == 4:
            cos, sin = _check_rope("RotaryPack", x, cos, sin, x.shape[1], x.shape[3])
        else:
            _check_rope("RotaryPack", x, cos, sin, 0, 0)
        if x.stride(3) != 1:
            x = x.contiguous()                      # inputs that need contiguity are compacted by the op
        return cls(x, cos, sin)

    def forward(self) -> torch.Tensor:
        B, T, H, D = self.x.shape
        y = torch.empty((B, H, T, D), dtype=self.x.dtype, device=self.x.device)
        ys = y.stride()
        _rope_call(self.x, self.cos, self.sin, y, self.x.stride(), (ys[0], ys[2], ys[1], ys[3]), B, T, H, D, False)
        return y

    def backward(self, grads: "GradientStore", out_grad: torch.Tensor, dx_out: Optional[torch.Tensor] = None) -> None:
        """`dx_out` (a [B,T,H,D] view with inner stride 1, e.g. the q slice of a fused dqkv buffer) receives
        the gradient in place instead of a fresh tensor."""
        B, T, H, D = self.x.shape
        if tuple(out_grad.shape) != (B, H, T, D):
            raise LayoutMismatch(f"RotaryPack.backward: gradient {tuple(out_grad.shape)} vs {(B, H, T, D)}")
        if out_grad.dtype != self.x.dtype:
            raise DTypeMismatch(f"RotaryPack.backward: {out_grad.dtype} vs {self.x.dtype}")
        g = out_grad if out_grad.stride(3) == 1 else out_grad.contiguous()
        if dx_out is not None:
            if tuple(dx_out.shape) != (B, T, H, D) or dx_out.dtype != self.x.dtype or dx_out.stride(3) != 1:
                raise LayoutMismatch("RotaryPack.backward: dx_out must be a [B,T,H,D] view with inner stride 1")
            dx = dx_out
        else:
            dx = torch.empty((B, T, H, D), dtype=self.x.dtype, device=self.x.device)
        gs = g.stride()
        _rope_call(g, self.cos, self.sin, dx, (gs[0], gs[2], gs[1], gs[3]), dx.stride(), B, T, H, D, True)
        grads.accumulate(self.x, dx)

    def dependencies(self) -> List[torch.Tensor]:
        return [self.x]

    def name(self) -> str:
        return "RotaryPack"


def rotary_pack(x, cos, sin) -> torch.Tensor:
    """Tensor-method form: RotaryPack.new(..).forward()."""
    return RotaryPack.new(x, cos, sin).forward()


class GradientStore:
    """Insert-or-add gradient map keyed by tensor identity (src/backprop.rs:74-128)."""

    def __init__(self):
        # id -> (tensor, gradient): holding the tensor keeps its id from being reused while the entry lives
        self._grads: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}

    def accumulate(self, tensor: torch.Tensor, grad: torch.Tensor) -> None:
        key = id(tensor)
        if key in self._grads:
            self._grads[key] = (tensor, self._grads[key][1] + grad)
        else:
            self._grads[key] = (tensor, grad)

    def get(self, tensor: torch.Tensor) -> Optional[torch.Tensor]:
        entry = self._grads.get(id(tensor))
        return entry[1] if entry is not None and entry[0] is tensor else None

    def insert(self, tensor: torch.Tensor, grad: torch.Tensor) -> None:
        self._grads[id(tensor)] = (tensor, grad)


class CausalAttention:
    """The fused op: ``softmax(scale * q @ k^T + causal_mask) @ v`` on ``[B, H, T, D]`` tensors.

    Same life cycle as deers ops: ``CausalAttention.new(...)`` validates (raising
    LayoutMismatch / DTypeMismatch / DeviceMismatch), ``forward()`` returns the
    output and keeps what the backward needs (O and the row lse) in ``self``, the
    pattern of LogSumExp / FusedLogSoftmax (src/ops.rs:1152-1159, 1214-1220).
    """

    def __init__(self, q, k, v, scale: float, causal: bool = True, token_major_out: bool = False):
        self.q, self.k, self.v = q, k, v
        self.scale, self.causal = float(scale), bool(causal)
        self.token_major_out = bool(token_major_out)
        self.o: Optional[torch.Tensor] = None
        self.lse: Optional[torch.Tensor] = None

    @classmethod
    def new(cls, q, k, v, scale: Optional[float] = None, causal: bool = True,
            token_major_out: bool = False) -> "CausalAttention":
        _check_inputs("CausalAttention", (q, k, v))
        if q.device.type != "cuda":
            raise DeviceMismatch("CausalAttention: the fused op runs on the CUDA device only")
        return cls(q, k, v, default_scale(q.shape[3]) if scale is None else scale, causal, token_major_out)

    def forward(self) -> torch.Tensor:
        self.o, self.lse = attention_fwd(self.q, self.k, self.v, self.scale, self.causal, self.token_major_out)
        return self.o

    def backward(self, grads: GradientStore, out_grad: torch.Tensor) -> None:
        if self.o is None:
            raise RuntimeError("CausalAttention.backward before forward")
        dq, dk, dv = attention_bwd(self.q, self.k, self.v, self.o, self.lse, out_grad, self.scale, self.causal)
        grads.accumulate(self.q, dq)
        grads.accumulate(self.k, dk)
        grads.accumulate(self.v, dv)

    def dependencies(self) -> List[torch.Tensor]:
        return [self.q, self.k, self.v]

    def name(self) -> str:
        return "CausalAttention"


def causal_attention(q, k, v, scale: Optional[float] = None) -> torch.Tensor:
    """Tensor-method form (house style of src/tensor.rs:379-381): new(..).forward()."""
    return CausalAttention.new(q, k, v, scale).forward()


def attention_fwd_bwd_host(q, k, v, d_o, scale: float, causal: bool = True, chunk_slices: int = 64,
                           device: Optional[torch.device] = None, scratch: Optional[torch.Tensor] = None,
                           out=None):
    """Forward + backward on HOST tensors (compact [B,H,T,D], ideally pinned) through the pipelined
    C-ABI call: returns (o, dq, dk, dv, lse) as host tensors.  `scratch` is device memory the caller
    may keep between calls; `out` optional preallocated (o, dq, dk, dv, lse) host tensors."""
    _check_inputs("attention_fwd_bwd_host", (q, k, v, d_o))
    for t in (q, k, v, d_o):
        if t.device.type != "cpu" or not t.is_contiguous():
            raise LayoutMismatch("attention_fwd_bwd_host: expected compact host tensors")
    device = device or torch.device("cuda", torch.cuda.current_device())
    ctx = Context.current(device)
    B, H, T, D = q.shape
    d = _lib.AttnDesc()
    _lib.lib().deers_b200_attn_desc_compact(ctypes.byref(d), B, H, T, D, _DTYPES[q.dtype], int(causal), scale)
    need = int(_lib.lib().deers_b200_attn_host_scratch_bytes(ctypes.byref(d), chunk_slices))
    if scratch is None or scratch.numel() * scratch.element_size() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=device)
    if out is None:
        pin = q.is_pinned()
        out = tuple(torch.empty(q.shape, dtype=q.dtype, pin_memory=pin) for _ in range(4)) + \
              (torch.empty((B, H, T), dtype=torch.float32, pin_memory=pin),)
    o, dq, dk, dv, lse = out
    _lib.check(_lib.lib().deers_b200_attn_fwd_bwd_host(
        ctx.handle, ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(), o.data_ptr(),
        lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), chunk_slices, scratch.data_ptr(),
        scratch.numel() * scratch.element_size()), ctx.handle)
    return o, dq, dk, dv, lse


# ---------------------------------------------------------------------------------------------
# Optimizer: multi-tensor AdamW with the gradient-norm clip folded in (f32)
# ---------------------------------------------------------------------------------------------
def _optim_table(parameters, grads: GradientStore, moments=None):
    """The C array of deers_optim_tensor for the parameters that have a gradient (optim.rs:221-225
    skips the others), plus the objects that must stay alive during the call."""
    rows, keep = [], []
    for p in parameters:
        g = grads.get(p)
        if g is None:
            continue
        if p.dtype != torch.float32 or g.dtype != torch.float32:
            raise DTypeMismatch(f"optimizer: f32 parameters and gradients only, got {p.dtype} / {g.dtype}")
        if p.device.type != "cuda" or g.device != p.device:
            raise DeviceMismatch("optimizer: parameters and gradients must live on the CUDA device")
        if tuple(g.shape) != tuple(p.shape):
            raise LayoutMismatch(f"optimizer: gradient {tuple(g.shape)} vs parameter {tuple(p.shape)}")
        if not p.is_contiguous():
            raise LayoutMismatch("optimizer: parameters must be compact")
        if not g.is_contiguous():
            g = g.contiguous()
            grads.insert(p, g)
        m, v = moments(p) if moments is not None else (None, None)
        rows.append((p, g, m, v))
        keep.extend((p, g, m, v))
    table = (_lib.OptimTensor * max(len(rows), 1))()
    for i, (p, g, m, v) in enumerate(rows):
        table[i].w, table[i].g = p.data_ptr(), g.data_ptr()
        table[i].m = m.data_ptr() if m is not None else None
        table[i].v = v.data_ptr() if v is not None else None
        table[i].n = p.numel()
    return table, len(rows), keep


def grad_norm_device(parameters, grads: GradientStore) -> Optional[torch.Tensor]:
    """sqrt(sum of squares of every gradient) as a one-element f32 tensor ON THE DEVICE (no host
    synchronisation): what `AdamW.step_with_grads(..., clip_norm=...)` consumes."""
    table, n, keep = _optim_table(parameters, grads)
    if n == 0:
        return None
    dev = keep[0].device
    ctx = Context.current(dev)
    norm = torch.empty(1, dtype=torch.float32, device=dev)
    nbytes = int(_lib.lib().deers_b200_optim_scratch_bytes())
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.check(_lib.lib().deers_b200_grad_norm(ctx.handle, n, table, norm.data_ptr(), scratch.data_ptr(), nbytes),
               ctx.handle)
    return norm


def clip_grad_norm(parameters, grads: GradientStore, max_norm: float) -> float:
    """`clip_grad_norm` (src/optim.rs:257-297): clips the global gradient norm to max_norm, scaling the
    stored gradients in place, and returns the norm before clipping (one host read, like the reference)."""
    assert max_norm > 0.0, "max_norm must be positive"
    if len(parameters) == 0:
        return 0.0
    norm = grad_norm_device(parameters, grads)
    if norm is None:
        return 0.0
    table, n, keep = _optim_table(parameters, grads)
    ctx = Context.current(norm.device)
    _lib.check(_lib.lib().deers_b200_grad_clip(ctx.handle, n, table, norm.data_ptr(), float(max_norm)), ctx.handle)
    return float(norm.item())


class AdamW:
    """`AdamWConfig::new(lr).betas(..).eps(..).weight_decay(..).build(parameters)` and the optimizer it
    builds (src/optim.rs:49-251), with every parameter updated by one fused launch.  Parameters are
    compact f32 CUDA tensors updated in place; moments are created as zeros on first use."""

    def __init__(self, parameters, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        self.parameters = list(parameters)
        self._lr, self.betas, self.eps, self.weight_decay = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(weight_decay)
        self._m: Dict[int, torch.Tensor] = {}
        self._v: Dict[int, torch.Tensor] = {}
        self._step = 0

    def set_lr(self, lr: float) -> None:
        self._lr = float(lr)

    def lr(self) -> float:
        return self._lr

    def step_count(self) -> int:
        return self._step

    def set_step_count(self, step: int) -> None:
        self._step = int(step)

    def state_for(self, parameter):
        if id(parameter) not in self._m:
            return None
        return self._m[id(parameter)], self._v[id(parameter)]

    def load_state_for(self, parameter, m, v) -> None:
        self._m[id(parameter)], self._v[id(parameter)] = m.detach().contiguous(), v.detach().contiguous()

    def _moments(self, p):
        if id(p) not in self._m:
            self._m[id(p)] = torch.zeros_like(p)
            self._v[id(p)] = torch.zeros_like(p)
        return self._m[id(p)], self._v[id(p)]

    def step_with_grads(self, grads: GradientStore, clip_norm: Optional[torch.Tensor] = None,
                        max_norm: float = 0.0) -> None:
        """One AdamW step (optim.rs:214-251).  With `clip_norm` (the device tensor of
        `grad_norm_device`) and `max_norm`, the clip of clip_grad_norm is applied to the gradients on
        the fly inside the same launch, without a host round trip."""
        self._step += 1
        table, n, keep = _optim_table(self.parameters, grads, self._moments)
        if n == 0:
            return
        ctx = Context.current(keep[0].device)
        h = _lib.AdamWHyper(self._lr, self.betas[0], self.betas[1], self.eps, self.weight_decay, self._step)
        _lib.check(_lib.lib().deers_b200_adamw_step(ctx.handle, n, table, ctypes.byref(h),
                                                    clip_norm.data_ptr() if clip_norm is not None else None,
                                                    float(max_norm)), ctx.handle)


# ---------------------------------------------------------------------------------------------
# RMSNorm (f32), one fused launch each way
# ---------------------------------------------------------------------------------------------
class RMSNorm:
    """`RMSNorm::forward` (src/nn.rs:244-251) as one op with the TensorOp life cycle: ``new`` validates,
    ``forward`` returns y and keeps the per-row inverse norm for ``backward``."""

    def __init__(self, x, eps: float):
        self.x, self.eps = x, float(eps)
        self.inv: Optional[torch.Tensor] = None

    @classmethod
    def new(cls, x, eps: float) -> "RMSNorm":
        if x.dim() < 1:
            raise LayoutMismatch("RMSNorm: needs at least one axis")
        if x.dtype != torch.float32:
            raise DTypeMismatch(f"RMSNorm: f32 only, got {x.dtype}")
        if x.device.type != "cuda":
            raise DeviceMismatch("RMSNorm: the fused op runs on the CUDA device only")
        return cls(x if x.is_contiguous() else x.contiguous(), eps)

    def forward(self) -> torch.Tensor:
        C = self.x.shape[-1]
        rows = self.x.numel() // C
        ctx = Context.current(self.x.device)
        y = torch.empty_like(self.x)
        self.inv = torch.empty(max(rows, 1), dtype=torch.float32, device=self.x.device)
        _lib.check(_lib.lib().deers_b200_rmsnorm_fwd(ctx.handle, rows, C, self.eps, self.x.data_ptr(), y.data_ptr(),
                                                     self.inv.data_ptr()), ctx.handle)
        return y

    def backward(self, grads: GradientStore, out_grad: torch.Tensor) -> None:
        if self.inv is None:
            raise RuntimeError("RMSNorm.backward before forward")
        if tuple(out_grad.shape) != tuple(self.x.shape):
            raise LayoutMismatch(f"RMSNorm.backward: gradient {tuple(out_grad.shape)} vs {tuple(self.x.shape)}")
        if out_grad.dtype != torch.float32:
            raise DTypeMismatch(f"RMSNorm.backward: {out_grad.dtype}")
        g = out_grad if out_grad.is_contiguous() else out_grad.contiguous()
        C = self.x.shape[-1]
        rows = self.x.numel() // C
        ctx = Context.current(self.x.device)
        dx = torch.empty_like(self.x)
        _lib.check(_lib.lib().deers_b200_rmsnorm_bwd(ctx.handle, rows, C, self.x.data_ptr(), self.inv.data_ptr(),
                                                     g.data_ptr(), dx.data_ptr()), ctx.handle)
        grads.accumulate(self.x, dx)

    def dependencies(self) -> List[torch.Tensor]:
        return [self.x]

    def name(self) -> str:
        return "RMSNorm"


def rms_norm(x, eps: float) -> torch.Tensor:
    """Module form: RMSNorm.new(x, eps).forward()."""
    return RMSNorm.new(x, eps).forward()


# ---------------------------------------------------------------------------------------------
# Decode-time attention against a key / value cache
# ---------------------------------------------------------------------------------------------
def attention_decode(q, k_cache, v_cache, scale: Optional[float] = None, causal: bool = True, want_lse: bool = False):
    """``softmax(scale * q @ k^T + causal_mask(B, Tq, Tk - Tq)) @ v`` for Tq new rows against Tk cached rows
    (the mask of src/nn/functional.rs:12-55 with seqlen_offset = Tk - Tq).  q: [B,H,Tq,D]; caches:
    [B,H,Tk,D] (views of a larger cache are read in place).  Returns o [B,H,Tq,D] (and lse [B,H,Tq])."""
    if q.dim() != 4 or k_cache.dim() != 4 or v_cache.dim() != 4:
        raise LayoutMismatch("attention_decode: expected [B, H, T, D] tensors")
    B, H, Tq, D = q.shape
    Tk = k_cache.shape[2]
    if tuple(k_cache.shape) != (B, H, Tk, D) or tuple(v_cache.shape) != (B, H, Tk, D) or Tk < Tq:
        raise LayoutMismatch(f"attention_decode: q {tuple(q.shape)}, k {tuple(k_cache.shape)}, v {tuple(v_cache.shape)}")
    for t in (k_cache, v_cache):
        if t.dtype != q.dtype:
            raise DTypeMismatch(f"attention_decode: {t.dtype} vs {q.dtype}")
        if t.device != q.device:
            raise DeviceMismatch(f"attention_decode: {t.device} vs {q.device}")
    if q.dtype not in _DTYPES:
        raise DTypeMismatch(f"attention_decode: unsupported dtype {q.dtype}")
    if q.device.type != "cuda":
        raise DeviceMismatch("attention_decode: the op runs on the CUDA device only")
    q, k_cache, v_cache = (t if t.stride(3) == 1 else t.contiguous() for t in (q, k_cache, v_cache))
    ctx = Context.current(q.device)
    o = torch.empty_like(q, memory_format=torch.contiguous_format)
    lse = torch.empty((B, H, Tq), dtype=torch.float32, device=q.device) if want_lse else None
    d = _lib.DecodeDesc()
    d.B, d.H, d.Tq, d.Tk, d.D = B, H, Tq, Tk, D
    d.dtype, d.causal, d.scale = _DTYPES[q.dtype], int(causal), default_scale(D) if scale is None else float(scale)
    d.q_strides, d.k_strides, d.v_strides, d.o_strides = _strides(q), _strides(k_cache), _strides(v_cache), _strides(o)
    need = int(_lib.lib().deers_b200_attn_decode_workspace_bytes(ctypes.byref(d)))
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    _lib.check(_lib.lib().deers_b200_attn_decode(ctx.handle, ctypes.byref(d), q.data_ptr(), k_cache.data_ptr(),
                                                 v_cache.data_ptr(), o.data_ptr(),
                                                 lse.data_ptr() if lse is not None else None, ws.data_ptr(), need),
               ctx.handle)
    return (o, lse) if want_lse else o


# ---------------------------------------------------------------------------------------------
# Linear projections (f16): forward and the two backward products on the tcgen05 GEMM
# ---------------------------------------------------------------------------------------------
def _gemm(M, N, K, a, a_mn, b, b_mn, dev, dtype):
    ctx = Context.current(dev)
    c = torch.empty((M, N), dtype=dtype, device=dev)
    _lib.check(_lib.lib().deers_b200_gemm_f16(ctx.handle, M, N, K, a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(),
                                              b.stride(0), int(b_mn), c.data_ptr(), c.stride(0)), ctx.handle)
    return c


class Linear:
    """``x.matmul(weight)`` of `Linear::forward` (src/nn.rs:184-190; weight is [in_features, out_features])
    as a TensorOp-style node whose backward accumulates dx = dy @ W^T and dW = x^T @ dy
    (src/ops.rs:1089-1101).  f16 tensors on the CUDA device; x is [..., in_features]."""

    def __init__(self, x, weight):
        self.x, self.weight = x, weight

    @classmethod
    def new(cls, x, weight) -> "Linear":
        if weight.dim() != 2 or x.dim() < 1 or x.shape[-1] != weight.shape[0]:
            raise LayoutMismatch(f"Linear: x {tuple(x.shape)} vs weight {tuple(weight.shape)}")
        if x.dtype != torch.float16 or weight.dtype != torch.float16:
            raise DTypeMismatch(f"Linear: f16 only on this path, got {x.dtype} / {weight.dtype}")
        if x.device.type != "cuda" or weight.device != x.device:
            raise DeviceMismatch("Linear: tensors must live on the same CUDA device")
        if weight.shape[0] % 8 or weight.shape[1] % 8:
            raise LayoutMismatch("Linear: in_features and out_features must be multiples of 8 (16-byte rows)")
        return cls(x if x.is_contiguous() else x.contiguous(), weight if weight.is_contiguous() else weight.contiguous())

    def forward(self) -> torch.Tensor:
        K, N = self.weight.shape
        x2 = self.x.reshape(-1, K)
        y = _gemm(x2.shape[0], N, K, x2, False, self.weight, True, self.x.device, self.x.dtype)
        return y.reshape(*self.x.shape[:-1], N)

    def backward(self, grads: GradientStore, out_grad: torch.Tensor) -> None:
        K, N = self.weight.shape
        x2 = self.x.reshape(-1, K)
        g2 = out_grad.reshape(-1, N)
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        rows = x2.shape[0]
        dx = _gemm(rows, K, N, g2, False, self.weight, False, self.x.device, self.x.dtype)
        dw = _gemm(K, N, rows, x2, True, g2, True, self.x.device, self.x.dtype)
        grads.accumulate(self.x, dx.reshape(self.x.shape))
        grads.accumulate(self.weight, dw)

    def dependencies(self) -> List[torch.Tensor]:
        return [self.x, self.weight]

    def name(self) -> str:
        return "Linear"
