"""CPU tests of the C-ABI boundary: the library loads, exports every declared
symbol, and its host-side helpers behave (no compute calls: there is no GPU here)."""
import ctypes
import os
import re

import pytest

from deers_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "deers_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(deers_b200_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.SYMBOLS)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    for name in declared_symbols():
        assert hasattr(L, name), name


def test_status_strings():
    assert _lib.status_string(_lib.OK) == "ok"
    for code in range(1, 10):
        assert _lib.status_string(code) not in ("", "ok", "unknown status")
    assert _lib.status_string(99) == "unknown status"
    assert _lib.status_string(-1) == "unknown status"


def test_desc_compact_strides():
    d = _lib.AttnDesc()
    _lib.lib().deers_b200_attn_desc_compact(ctypes.byref(d), 4, 6, 256, 32, _lib.F32, 1, 0.5)
    assert (d.B, d.H, d.T, d.D, d.dtype, d.causal) == (4, 6, 256, 32, _lib.F32, 1)
    want = [6 * 256 * 32, 256 * 32, 32, 1]
    for f in ("q", "k", "v", "o", "do", "dq", "dk", "dv"):
        assert list(getattr(d, f + "_strides")) == want
    assert abs(d.scale - 0.5) < 1e-9


def test_workspace_bytes():
    L = _lib.lib()
    d = _lib.AttnDesc()
    L.deers_b200_attn_desc_compact(ctypes.byref(d), 4, 6, 256, 32, _lib.F32, 1, 0.5)
    assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 0) == 0
    assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 1) >= 4 * 6 * 256 * 4
    L.deers_b200_attn_desc_compact(ctypes.byref(d), 8, 12, 1024, 64, _lib.F16, 1, 0.125)
    assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 1) >= 8 * 12 * 1024 * 4
    # f16 head dims other than 64 / 128 (multiples of 8) run zero-padded: the forward needs four padded tensors,
    # the backward eight more bytes-wise plus its own scratch.
    L.deers_b200_attn_desc_compact(ctypes.byref(d), 1, 1, 16, 48, _lib.F16, 1, 1.0)
    padded = 1 * 1 * 16 * 64 * 2
    assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 0) >= 4 * padded
    assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 1) >= 8 * padded
    # Unsupported requests need no workspace because they are rejected.
    for bad in (20, 136):
        L.deers_b200_attn_desc_compact(ctypes.byref(d), 1, 1, 16, bad, _lib.F16, 1, 1.0)
        assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 0) == 0
        assert L.deers_b200_attn_workspace_bytes(ctypes.byref(d), 1) == 0


def test_null_arguments_are_rejected_not_crashed():
    L = _lib.lib()
    assert L.deers_b200_init(0, None, None) == _lib.ERR_NULL
    assert L.deers_b200_sync(None) == _lib.ERR_NULL
    assert L.deers_b200_attn_fwd(None, None, None, None, None, None, None, None, 0) == _lib.ERR_NULL
    assert L.deers_b200_launch_count(None) == 0
    L.deers_b200_destroy(None)


def test_init_without_gpu_reports_an_error():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = ctypes.c_void_p()
    rc = _lib.lib().deers_b200_init(0, None, ctypes.byref(ctx))
    assert rc in (_lib.ERR_CUDA, _lib.ERR_DEVICE) and not ctx.value


def test_ops_refuse_cpu_tensors():
    import torch
    from deers_b200 import ops
    from deers_b200.errors import DeviceMismatch, DTypeMismatch, LayoutMismatch
    q = torch.zeros(1, 1, 4, 8)
    with pytest.raises(DeviceMismatch):
        ops.CausalAttention.new(q, q, q)
    with pytest.raises(LayoutMismatch):
        ops.CausalAttention.new(q, q[:, :, :2], q)
    with pytest.raises(DTypeMismatch):
        ops.CausalAttention.new(q, q.half(), q)
    with pytest.raises(LayoutMismatch):
        ops.CausalAttention.new(q[0], q[0], q[0])


def test_rotary_pack_validation_without_a_gpu():
    # Constructor errors follow the reference's conventions (src/error.rs:13-26; the asserts of
    # apply_rotary_emb, src/models/gpt.rs:49-66); no compute call is made.
    import pytest
    import torch
    from deers_b200 import ops
    from deers_b200.errors import DeviceMismatch, DTypeMismatch, LayoutMismatch
    cos, sin = ops.precompute_rotary_embeddings(5, 8)
    assert tuple(cos.shape) == (1, 5, 1, 4) and cos.dtype == torch.float32
    assert torch.equal(cos[0, 0, 0], torch.ones(4)) and torch.equal(sin[0, 0, 0], torch.zeros(4))
    x = torch.zeros(2, 5, 3, 8)
    with pytest.raises(DeviceMismatch):
        ops.RotaryPack.new(x, cos, sin)                       # CPU tensors: there is no CPU fallback
    with pytest.raises(LayoutMismatch):
        ops.RotaryPack.new(torch.zeros(5, 3, 8), cos, sin)    # not 4-D
    with pytest.raises(LayoutMismatch):
        ops.RotaryPack.new(torch.zeros(2, 5, 3, 7), cos, sin)  # odd head_dim
    with pytest.raises(DTypeMismatch):
        ops.RotaryPack.new(torch.zeros(2, 5, 3, 8, dtype=torch.int64), cos, sin)
    with pytest.raises(LayoutMismatch):
        ops.precompute_rotary_embeddings(5, 7)
