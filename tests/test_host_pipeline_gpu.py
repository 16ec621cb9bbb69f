"""GPU test of the pipelined host-tensor call (deers_b200_attn_fwd_bwd_host): host in, host out,
chunks that do not divide the slice count, results equal to the device-resident path."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL_F16, TOL_F32, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,shape,chunk,tol", [
    (torch.float16, (3, 5, 200, 64), 4, TOL_F16),      # 15 slices in chunks of 4: ragged last chunk, 4 chunks > 3 buffer sets
    (torch.float16, (2, 2, 260, 128), 64, TOL_F16),    # one chunk
    (torch.float32, (2, 3, 70, 32), 2, TOL_F32),
])
def test_host_call_matches_oracle_and_device_path(dtype, shape, chunk, tol):
    from deers_b200 import ops
    from oracle import ref
    rng = np.random.default_rng(31)
    host = [rng.standard_normal(shape).astype(np.float32) for _ in range(4)]
    if dtype == torch.float16:
        host = [a.astype(np.float16).astype(np.float32) for a in host]
    want = ref.attn_fwd_bwd(*host)
    pinned = [torch.from_numpy(a).to(dtype).pin_memory() for a in host]
    scale = ops.default_scale(shape[3])
    o, dq, dk, dv, lse = ops.attention_fwd_bwd_host(*pinned, scale, True, chunk_slices=chunk)
    for name, g, w in zip(("o", "lse", "dq", "dk", "dv"), (o, lse, dq, dk, dv), want):
        assert_close(g.float().numpy(), w, tol, f"{shape}/{name}")
    # Bitwise equal to the device-resident path (same kernels, slices are independent).
    dev = [t.cuda() for t in pinned]
    o_dev, lse_dev = ops.attention_fwd(dev[0], dev[1], dev[2], scale, True)
    # the host call gives each chunk the small workspace (its dQ kernel recomputes): same choice here
    ws = torch.empty(max(ops.workspace_bytes(dev[0], scale, True, pass_=1), 256), dtype=torch.uint8, device="cuda")
    grads_dev = ops.attention_bwd(dev[0], dev[1], dev[2], o_dev, lse_dev, dev[3], scale, True, workspace=ws)
    assert torch.equal(o_dev.cpu(), o)
    for gd, g in zip(grads_dev, (dq, dk, dv)):
        assert torch.equal(gd.cpu(), g)


def test_host_call_rejects_small_scratch():
    import ctypes
    from deers_b200 import _lib, ops
    ctx = ops.Context.current(torch.device("cuda", 0))
    d = _lib.AttnDesc()
    _lib.lib().deers_b200_attn_desc_compact(ctypes.byref(d), 1, 2, 64, 64, _lib.F16, 1, 0.125)
    h = torch.zeros((1, 2, 64, 64), dtype=torch.float16)
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    rc = _lib.lib().deers_b200_attn_fwd_bwd_host(ctx.handle, ctypes.byref(d), *([h.data_ptr()] * 5), None,
                                                 *([h.data_ptr()] * 3), 2, small.data_ptr(), 1024)
    assert rc == _lib.ERR_WORKSPACE
