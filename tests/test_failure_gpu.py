"""Failure detection on the GPU without a fault or a hang: the give-up path of the bounded device-side waits, and
bitwise repeatability of the full-size kept-dS backward (a race would show as a bit difference)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_the_context_stays_usable():
    """A barrier nobody completes, waited on with a 5 ms limit: the kernel returns, the error word is set,
    kernels launched before the next sync leave their outputs alone, sync reports DEERS_ERR_KERNEL once, and
    after that everything runs normally."""
    from deers_b200 import _lib, ops
    from deers_b200.errors import CudaError
    from oracle import ref
    from tests.gpu_util import make_inputs, to_dev
    from tests.helpers import TOL_F16, assert_close
    ctx = ops.Context.current(torch.device("cuda", torch.cuda.current_device()))
    ctx.sync()
    gave_up, saw_abort, us_first, us_second = ctx.selftest_wait(5)
    assert gave_up == 1, "the wait must run out"
    assert saw_abort == 1, "a later wait of the CTA returns through the abort flag"
    assert 4000 <= us_first < 200000, us_first                  # about the limit, far from the default 2 s
    assert us_second < 2000, us_second
    # the error word is still set: a persistent f16 kernel started now returns without writing
    q, k, v, _ = make_inputs(1, 2, 256, 128, torch.float16, seed=3)
    tq, tk, tv = (to_dev(a, torch.float16) for a in (q, k, v))
    o = torch.full((1, 2, 256, 128), float("nan"), dtype=torch.float16, device="cuda")
    lse = torch.full((1, 2, 256), float("nan"), dtype=torch.float32, device="cuda")
    d = ops._desc(tq, tk, tv, o, scale=ops.default_scale(128), causal=True)
    _lib.check(_lib.lib().deers_b200_attn_fwd(ctx.handle, d, tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                                              o.data_ptr(), lse.data_ptr(), None, 0), ctx.handle)
    with pytest.raises(CudaError) as info:
        ctx.sync()
    assert info.value.status == _lib.ERR_KERNEL
    assert "0x37f" in str(info.value), str(info.value)          # self-test family 0x300, wait id 0x7f
    assert torch.isnan(o).all() and torch.isnan(lse).all(), "outputs untouched while the error was pending"
    ctx.sync()                                                   # cleared: a second sync is clean
    o2, lse2 = ops.attention_fwd(tq, tk, tv, ops.default_scale(128))
    ctx.sync()
    want_o, want_lse = ref.attn_fwd(q, k, v)
    assert_close(o2.float().cpu().numpy(), want_o, TOL_F16, "o after recovery")
    assert_close(lse2.cpu().numpy(), want_lse, TOL_F16, "lse after recovery")


def _repeat_backward(B, H, T, D, repeats, seed):
    from deers_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = (torch.randn(B, H, T, D, device="cuda", dtype=torch.float16, generator=g) for _ in range(4))
    scale = ops.default_scale(D)
    o, lse = ops.attention_fwd(q, k, v, scale, True)
    nbytes = ops.workspace_bytes(q, scale, True, pass_=2)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    first = None
    for it in range(repeats):
        ws.fill_(0xFF)                                           # NaN patterns: a tile read before written would show
        dq, dk, dv = ops.attention_bwd(q, k, v, o, lse, do, scale, True, workspace=ws)
        ops.Context.current(q.device).sync()
        if first is None:
            first = (dq.clone(), dk.clone(), dv.clone())
            for t in first:
                assert torch.isfinite(t).all()
        else:
            for name, a, b in zip(("dq", "dk", "dv"), first, (dq, dk, dv)):
                assert torch.equal(a, b), f"run {it}: {name} differs from run 0 ({(a != b).sum().item()} elements)"
        del dq, dk, dv


def test_cfg5_kept_ds_backward_is_bitwise_repeatable():
    """BASELINE cfg 5 at full size (B=64, T=2048, H=32, D=128), the backward that keeps its dS tiles, 20 runs on
    the same inputs with the workspace re-poisoned before each: dQ, dK, dV must be bit-identical."""
    _repeat_backward(64, 32, 2048, 128, repeats=20, seed=55)


def test_cfg4_kept_ds_backward_is_bitwise_repeatable():
    _repeat_backward(2, 16, 8192, 128, repeats=20, seed=44)
