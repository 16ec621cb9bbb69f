"""The workspace-free f16 backward (deers_b200_attn_bwd_f16_static).

Some callers of this library are not allowed to allocate device memory at the moment they need a
backward pass (allocator callbacks, hosts with a frozen memory plan, latency-critical paths), so the
library also offers the f16 backward with its scratch in a fixed array inside the library image.
This test calls that entry point through the C ABI twice in a row, on two different problems, and
checks every gradient against the regular entry point (which takes a caller-provided workspace) on
the same inputs: both run the same kernels, so the results must be bitwise equal, and the second
call must not be disturbed by what the first one left in the shared array.  It also checks that a
problem too large for the built-in array is refused with a clear error instead of being run.

The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(ctx, q, k, v, o, lse, do, scale):
    from deers_b200 import _lib, ops
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    d = ops._desc(q, k, v, o, do, dq, dk, dv, scale=scale, causal=True)
    rc = _lib.lib().deers_b200_attn_bwd_f16_static(ctx.handle, ctypes.byref(d), q.data_ptr(), k.data_ptr(),
                                                   v.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(),
                                                   dq.data_ptr(), dk.data_ptr(), dv.data_ptr())
    return rc, (dq, dk, dv)


def test_static_scratch_backward_matches_workspace_backward_twice():
    from deers_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    ctx = ops.Context.current(dev)
    gen = torch.Generator(device=dev).manual_seed(77)
    # Two problems of different size back to back: the second reuses (part of) the first one's scratch.
    for shape in ((2, 3, 700, 128), (1, 5, 300, 64)):
        q, k, v, do = (torch.randn(shape, device=dev, dtype=torch.float16, generator=gen) for _ in range(4))
        scale = ops.default_scale(shape[3])
        o, lse = ops.attention_fwd(q, k, v, scale)
        # the static entry recomputes S and dP in its dQ kernel: compare with the same choice (pass-1 workspace)
        ws = torch.empty(ops.workspace_bytes(q, scale, True, pass_=1), dtype=torch.uint8, device=dev)
        want = ops.attention_bwd(q, k, v, o, lse, do, scale, workspace=ws)
        rc, got = _call_static(ctx, q, k, v, o, lse, do, scale)
        assert rc == _lib.OK, _lib.status_string(rc)
        ctx.sync()
        for name, g, w in zip(("dq", "dk", "dv"), got, want):
            assert torch.isfinite(g).all(), name
            assert torch.equal(g, w), f"{shape} {name}: max diff {(g.float() - w.float()).abs().max().item()}"


def test_static_scratch_rejects_oversized_problem():
    from deers_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    ctx = ops.Context.current(dev)
    # 1,048,576 rows is the limit; B*H*Tpad = 2 * 4100 * 128 exceeds it.  The tensors are never touched.
    t = torch.empty((2, 4100, 128, 64), device=dev, dtype=torch.float16)
    lse = torch.empty((2, 4100, 128), device=dev, dtype=torch.float32)
    rc, _ = _call_static(ctx, t, t, t, t, lse, t, 0.125)
    assert rc == _lib.ERR_WORKSPACE
    msg = _lib.lib().deers_b200_last_error(ctx.handle).decode()
    assert "built-in array" in msg and "deers_b200_attn_bwd" in msg
    ctx.sync()
