"""Host-side mirror of the deers GPT model and its training step on the device-resident model object.

Mirrors `models::gpt::{GPTConfig, GPT}` (src/models/gpt.rs:259-378), `loss::cross_entropy`
(src/loss.rs:21-24) and the loop body of the trainer (examples/tinystories_train.rs:188-218) above the
C ABI: every kernel runs in ``libdeers_b200.so``; torch tensors only hold device memory for ids, logits
and read-backs.  Also the storage-level wrappers of the f32 building blocks (`linear_f32`, `embedding`,
`cross_entropy`) that the parity tests call one at a time.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from .errors import DeviceMismatch, DTypeMismatch, LayoutMismatch
from .ops import Context


@dataclass
class GPTConfig:
    """`GPTConfig` (src/models/gpt.rs:259-285)."""
    vocab_size: int
    sequence_len: int
    n_layer: int
    n_head: int
    n_embd: int
    mlp_hidden_dim: int
    rms_norm_eps: float = 1e-5
    rope_base: float = 10000.0

    def head_dim(self) -> int:
        return self.n_embd // self.n_head


class GPT:
    """The model of src/models/gpt.rs living in device memory (weights, gradients, AdamW moments,
    activations).  Parameters are addressed by index in the order of `GPT::parameters`
    (gpt.rs:358-365) or by their checkpoint key."""

    def __init__(self, config: GPTConfig, device: torch.device, max_batch: int):
        if device.type != "cuda":
            raise DeviceMismatch("the model step only exists on the CUDA device (no CPU fallback)")
        self.config = config
        # The step is replayed from a CUDA graph, and the legacy default stream cannot be captured: the model
        # enqueues on a stream of its own.  Calls order it after the caller's current stream and the caller's
        # stream after it, so tensors passed in and handed back behave as on one stream.
        self.stream = torch.cuda.Stream(device=device)
        with torch.cuda.stream(self.stream):
            self.ctx = Context.current(device)
        self.device = device
        self.handle = ctypes.c_void_p()
        c = _lib.GptConfig(config.vocab_size, config.sequence_len, config.n_layer, config.n_head, config.n_embd,
                           config.mlp_hidden_dim, config.rms_norm_eps, config.rope_base)
        _lib.check(_lib.lib().deers_b200_gpt_create(self.ctx.handle, ctypes.byref(c), max_batch,
                                                    ctypes.byref(self.handle)), self.ctx.handle)
        self.step_count = 0

    def __del__(self):
        try:
            if self.handle:
                _lib.lib().deers_b200_gpt_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # -- parameters -------------------------------------------------------------------------------
    def num_parameters(self) -> int:
        return int(_lib.lib().deers_b200_gpt_num_params(self.handle))

    def parameter_info(self, index: int) -> Tuple[str, Tuple[int, int]]:
        name = ctypes.create_string_buffer(96)
        rows, cols = ctypes.c_int64(), ctypes.c_int64()
        _lib.check(_lib.lib().deers_b200_gpt_param_info(self.handle, index, name, 96, ctypes.byref(rows),
                                                        ctypes.byref(cols)), self.ctx.handle)
        return name.value.decode(), (int(rows.value), int(cols.value))

    def named_parameters(self) -> List[Tuple[str, Tuple[int, int]]]:
        return [self.parameter_info(i) for i in range(self.num_parameters())]

    def _set(self, index: int, what: int, array) -> None:
        name, shape = self.parameter_info(index)
        a = np.ascontiguousarray(array, dtype=np.float32)
        if a.shape != shape:
            raise LayoutMismatch(f"{name}: expected {shape}, got {a.shape}")
        _lib.check(_lib.lib().deers_b200_gpt_param_set(self.handle, index, what, a.ctypes.data_as(ctypes.c_void_p)),
                   self.ctx.handle)

    def _get(self, index: int, what: int) -> np.ndarray:
        _, shape = self.parameter_info(index)
        a = np.empty(shape, np.float32)
        _lib.check(_lib.lib().deers_b200_gpt_param_get(self.handle, index, what, a.ctypes.data_as(ctypes.c_void_p)),
                   self.ctx.handle)
        return a

    def load_parameters(self, arrays) -> None:
        """`ParamStore::load`-style upload (src/nn.rs:62-81): one [rows, cols] f32 array per parameter."""
        arrays = list(arrays)
        if len(arrays) != self.num_parameters():
            raise LayoutMismatch(f"expected {self.num_parameters()} tensors, got {len(arrays)}")
        for i, a in enumerate(arrays):
            self._set(i, 0, a)

    def parameter(self, index: int) -> np.ndarray:
        return self._get(index, 0)

    def grad(self, index: int) -> np.ndarray:
        return self._get(index, 1)

    def moments(self, index: int) -> Tuple[np.ndarray, np.ndarray]:
        """AdamW state of one parameter (`AdamW::state_dict`, src/optim.rs:162-205)."""
        return self._get(index, 2), self._get(index, 3)

    def load_moments(self, index: int, m, v) -> None:
        self._set(index, 2, m)
        self._set(index, 3, v)

    def graph_active(self) -> bool:
        """True once steps are replayed from a captured CUDA graph."""
        return bool(_lib.lib().deers_b200_gpt_graph_active(self.handle))

    def set_graph(self, enable: bool) -> None:
        _lib.check(_lib.lib().deers_b200_gpt_set_graph(self.handle, int(enable)), self.ctx.handle)

    # -- forward / training -----------------------------------------------------------------------
    def _ids(self, name: str, t: torch.Tensor, n: Optional[int] = None) -> torch.Tensor:
        if t.device != self.device:
            raise DeviceMismatch(f"{name}: {t.device} vs {self.device}")
        if t.dtype != torch.int64:
            raise DTypeMismatch(f"{name}: token ids are int64 (DType::I64), got {t.dtype}")
        t = t.contiguous()
        if n is not None and t.numel() != n:
            raise LayoutMismatch(f"{name}: expected {n} ids, got {t.numel()}")
        return t

    class _Ordered:
        """Orders the model's stream after the caller's current stream on entry and the caller's after the
        model's on exit (two event waits, no host synchronisation; nothing when they are the same stream)."""

        def __init__(self, model):
            self.model = model

        def __enter__(self):
            self.outer = torch.cuda.current_stream(self.model.device)
            if self.outer != self.model.stream:
                self.model.stream.wait_stream(self.outer)
            self.guard = torch.cuda.stream(self.model.stream)
            self.guard.__enter__()

        def __exit__(self, *exc):
            self.guard.__exit__(*exc)
            if self.outer != self.model.stream:
                self.outer.wait_stream(self.model.stream)
            return False

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        """`GPT::forward` (gpt.rs:329-355): ids [B, T] -> logits [B, T, vocab]."""
        if idx.dim() != 2:
            raise LayoutMismatch("GPT expects token ids with shape [B, T]")
        idx = self._ids("idx", idx)
        B, T = idx.shape
        with GPT._Ordered(self):
            logits = torch.empty((B, T, self.config.vocab_size), dtype=torch.float32, device=self.device)
            _lib.check(_lib.lib().deers_b200_gpt_forward(self.handle, idx.data_ptr(), B, T, logits.data_ptr()),
                       self.ctx.handle)
        return logits

    def forward_backward(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """forward, `cross_entropy` and `loss.backward()`: returns the loss (1-element device tensor);
        the gradients are read with `grad(index)`."""
        idx = self._ids("idx", idx)
        B, T = idx.shape
        targets = self._ids("targets", targets, B * T)
        with GPT._Ordered(self):
            loss = torch.empty(1, dtype=torch.float32, device=self.device)
            _lib.check(_lib.lib().deers_b200_gpt_forward_backward(self.handle, idx.data_ptr(), targets.data_ptr(), B, T,
                                                                  loss.data_ptr()), self.ctx.handle)
        return loss

    def _hyper(self, lr, betas, eps, weight_decay) -> _lib.AdamWHyper:
        self.step_count += 1                                    # optim.rs:215
        return _lib.AdamWHyper(lr, betas[0], betas[1], eps, weight_decay, self.step_count)

    def train_step(self, idx: torch.Tensor, targets: torch.Tensor, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                   weight_decay: float = 0.0, max_grad_norm: float = 0.0):
        """One step of the trainer loop (tinystories_train.rs:188-218, one micro-batch) on device ids:
        returns (loss, grad_norm) as 1-element device tensors, nothing synchronises."""
        idx = self._ids("idx", idx)
        B, T = idx.shape
        targets = self._ids("targets", targets, B * T)
        h = self._hyper(lr, betas, eps, weight_decay)
        with GPT._Ordered(self):
            out = torch.empty(2, dtype=torch.float32, device=self.device)
            _lib.check(_lib.lib().deers_b200_gpt_train_step(self.handle, idx.data_ptr(), targets.data_ptr(), B, T,
                                                            ctypes.byref(h), max_grad_norm, out.data_ptr(),
                                                            out.data_ptr() + 4), self.ctx.handle)
        return out[0:1], out[1:2]

    def train_step_host(self, idx: np.ndarray, targets: np.ndarray, lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                        weight_decay: float = 0.0, max_grad_norm: float = 0.0) -> Tuple[float, float]:
        """The same step with ids and targets in host memory (what `sample_batch` + `from_vec` do in the
        trainer) and the loss read back: returns (loss, grad_norm) as floats."""
        idx = np.ascontiguousarray(idx, dtype=np.int64)
        targets = np.ascontiguousarray(targets, dtype=np.int64)
        if idx.ndim != 2 or targets.size != idx.size:
            raise LayoutMismatch("expected ids [B, T] and B*T targets")
        B, T = idx.shape
        loss, norm = ctypes.c_float(), ctypes.c_float()
        h = self._hyper(lr, betas, eps, weight_decay)
        torch.cuda.set_device(self.device)
        _lib.check(_lib.lib().deers_b200_gpt_train_step_host(self.handle, idx.ctypes.data_as(ctypes.c_void_p),
                                                             targets.ctypes.data_as(ctypes.c_void_p), B, T,
                                                             ctypes.byref(h), max_grad_norm, ctypes.byref(loss),
                                                             ctypes.byref(norm)), self.ctx.handle)
        return float(loss.value), float(norm.value)


# ---- storage-level wrappers of the f32 building blocks ----------------------------------------------

def _f32(name: str, t: torch.Tensor) -> torch.Tensor:
    if t.device.type != "cuda":
        raise DeviceMismatch(f"{name}: no CPU fallback")
    if t.dtype != torch.float32:
        raise DTypeMismatch(f"{name}: expected float32, got {t.dtype}")
    return t


def gemm_f32(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool = False, b_mn_major: bool = True,
             epilogue: int = _lib.EPI_NONE, residual: Optional[torch.Tensor] = None, aux: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A * B through deers_b200_gemm_f32.  `a` is [M,K] (or [K,M] when a_mn_major), `b` is [K,N] when
    b_mn_major (the layout of a Linear weight) or [N,K]; 2-D tensors with unit inner stride, any row stride."""
    _f32("a", a), _f32("b", b)
    for t in (a, b):
        if t.dim() != 2 or t.stride(1) != 1:
            raise LayoutMismatch("gemm_f32 operands are 2-D with unit inner stride")
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    Kb, N = b.shape if b_mn_major else (b.shape[1], b.shape[0])
    if K != Kb:
        raise LayoutMismatch(f"inner dimensions differ: {K} vs {Kb}")
    ctx = Context.current(a.device)
    c = out if out is not None else torch.empty((M, N), dtype=torch.float32, device=a.device)
    ep = _lib.GemmEpilogue(epilogue, residual.data_ptr() if residual is not None else None,
                           residual.stride(0) if residual is not None else 0,
                           aux.data_ptr() if aux is not None else None)
    L = _lib.lib()
    nbytes = int(L.deers_b200_gemm_f32_workspace_bytes(ctx.handle, M, N, K))
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=a.device)
    _lib.check(L.deers_b200_gemm_f32(ctx.handle, M, N, K, a.data_ptr(), a.stride(0), int(a_mn_major), b.data_ptr(),
                                     b.stride(0), int(b_mn_major), c.data_ptr(), c.stride(0), ctypes.byref(ep),
                                     ws.data_ptr(), ws.numel()), ctx.handle)
    return c


def split_f16x3(x: torch.Tensor, scale: float = 1.0):
    """The f16 pair (hi, lo) of a 2-D f32 tensor: x * scale = hi + lo * 2^-11 (deers_b200_split_f16x3).  The pair
    is returned as [rows, cols] views of buffers whose rows are padded to a multiple of 8 elements."""
    _f32("x", x)
    if x.dim() != 2 or x.stride(1) != 1:
        raise LayoutMismatch("split_f16x3 wants a 2-D tensor with unit inner stride")
    rows, cols = x.shape
    ld = (cols + 7) // 8 * 8
    ctx = Context.current(x.device)
    hi = torch.zeros((rows, ld), dtype=torch.float16, device=x.device)
    lo = torch.zeros((rows, ld), dtype=torch.float16, device=x.device)
    _lib.check(_lib.lib().deers_b200_split_f16x3(ctx.handle, rows, cols, x.data_ptr(), x.stride(0), scale, hi.data_ptr(),
                                                 lo.data_ptr(), ld), ctx.handle)
    return hi[:, :cols], lo[:, :cols]


def gemm_f16x3(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool = False, b_mn_major: bool = True,
               scale_a: float = 1.0, scale_b: float = 1.0) -> torch.Tensor:
    """C = A * B in f32 through the tensor core on split f16 operands (deers_b200_gemm_f16x3); operand
    conventions as gemm_f32."""
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    Kb, N = b.shape if b_mn_major else (b.shape[1], b.shape[0])
    if K != Kb:
        raise LayoutMismatch(f"inner dimensions differ: {K} vs {Kb}")
    a_hi, a_lo = split_f16x3(a, scale_a)
    b_hi, b_lo = split_f16x3(b, scale_b)
    ctx = Context.current(a.device)
    L = _lib.lib()
    ldc = (N + 3) // 4 * 4
    c = torch.full((M, ldc), float("nan"), dtype=torch.float32, device=a.device)
    nbytes = int(L.deers_b200_gemm_f16x3_workspace_bytes(ctx.handle, M, N, K))
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=a.device)
    _lib.check(L.deers_b200_gemm_f16x3(ctx.handle, M, N, K, a_hi.data_ptr(), a_lo.data_ptr(), a_hi.stride(0), int(a_mn_major),
                                       b_hi.data_ptr(), b_lo.data_ptr(), b_hi.stride(0), int(b_mn_major), c.data_ptr(), ldc,
                                       1.0 / (scale_a * scale_b), ws.data_ptr(), ws.numel()), ctx.handle)
    return c[:, :N]


def embedding(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """`Embedding::forward` (src/nn.rs:214-221)."""
    _f32("weight", weight)
    ctx = Context.current(weight.device)
    flat = ids.reshape(-1).contiguous()
    out = torch.empty((flat.numel(), weight.shape[1]), dtype=torch.float32, device=weight.device)
    _lib.check(_lib.lib().deers_b200_embedding_fwd(ctx.handle, weight.data_ptr(), flat.data_ptr(), flat.numel(),
                                                   weight.shape[1], weight.shape[0], out.data_ptr()), ctx.handle)
    return out.reshape(*ids.shape, weight.shape[1])


def embedding_backward(dout: torch.Tensor, ids: torch.Tensor, vocab: int) -> torch.Tensor:
    _f32("dout", dout)
    ctx = Context.current(dout.device)
    flat = ids.reshape(-1).contiguous()
    d2 = dout.reshape(flat.numel(), -1).contiguous()
    dw = torch.empty((vocab, d2.shape[1]), dtype=torch.float32, device=dout.device)
    _lib.check(_lib.lib().deers_b200_embedding_bwd(ctx.handle, d2.data_ptr(), flat.data_ptr(), flat.numel(),
                                                   d2.shape[1], vocab, dw.data_ptr()), ctx.handle)
    return dw


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, with_grad: bool = False):
    """`loss::cross_entropy` (src/loss.rs:21-24) on [rows, vocab] logits: returns loss (1-element tensor) or
    (loss, lse, dlogits)."""
    _f32("logits", logits)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise LayoutMismatch("logits are [rows, vocab] with unit inner stride")
    ctx = Context.current(logits.device)
    rows, V = logits.shape
    targets = targets.reshape(-1).contiguous()
    L = _lib.lib()
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss = torch.empty(1, dtype=torch.float32, device=logits.device)
    scratch = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _lib.check(L.deers_b200_cross_entropy_fwd(ctx.handle, rows, V, logits.data_ptr(), logits.stride(0), targets.data_ptr(),
                                              lse.data_ptr(), loss.data_ptr(), scratch.data_ptr(), rows * 4), ctx.handle)
    if not with_grad:
        return loss
    d = torch.empty((rows, V), dtype=torch.float32, device=logits.device)
    _lib.check(L.deers_b200_cross_entropy_bwd(ctx.handle, rows, V, logits.data_ptr(), logits.stride(0), targets.data_ptr(),
                                              lse.data_ptr(), 1.0, d.data_ptr(), d.stride(0)), ctx.handle)
    return loss, lse, d
