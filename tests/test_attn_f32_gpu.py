"""GPU parity of the f32 (FFMA) kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from tests.helpers import REF_ABS_TOL_ACCEL, TOL_F32, assert_close

pytestmark = pytest.mark.gpu


def test_cfg1_readme_gpt_shape():
    # BASELINE config 1: B=4, T=256, H=6, head_dim=32, scale 1/sqrt(32).
    from tests.gpu_util import check_case
    check_case(4, 6, 256, 32, torch.float32, TOL_F32, seed=0)


@pytest.mark.parametrize("shape", [
    (2, 2, 3, 2),      # the reference's own attention test shape (tests/gpt.rs:38-49)
    (1, 1, 1, 4),      # single token
    (1, 2, 17, 8),
    (2, 3, 64, 32),
    (1, 2, 65, 32),    # one row into the second tile
    (1, 2, 70, 20),    # D not a multiple of 16
    (1, 1, 130, 64),
    (1, 2, 200, 128),
    (1, 1, 77, 7),     # odd head_dim: scalar load path
    (2, 1, 128, 96),
])
def test_shapes(shape):
    from tests.gpu_util import check_case
    check_case(*shape, torch.float32, TOL_F32, seed=sum(shape))


def test_noncausal_and_custom_scale():
    from tests.gpu_util import check_case
    check_case(1, 2, 100, 32, torch.float32, TOL_F32, seed=4, causal=False)
    check_case(1, 2, 100, 32, torch.float32, TOL_F32, seed=5, scale=0.37)


def test_golden_vectors(golden):
    from tests.gpu_util import run_fwd_bwd
    for name, c in golden.items():
        got = run_fwd_bwd(c["q"], c["k"], c["v"], c["do"], torch.float32, None, bool(c["causal"]))
        for label, g in zip(("o", "lse", "dq", "dk", "dv"), got):
            assert_close(g, c[label], TOL_F32, f"{name}/{label}")
            # the reference's own accelerator tolerance, absolute (tests/gpt.rs:8-9)
            assert np.abs(g - c[label]).max() < REF_ABS_TOL_ACCEL


def test_strided_views_like_the_module():
    # v reaches the op as permute([0,2,1,3]) of [B,T,H,D] (src/models/gpt.rs:137): strides
    # [T*H*D, D, H*D, 1]; q/k arrive with D slowest and are compacted by the op.
    from deers_b200 import ops
    from oracle import ref
    B, H, T, D = 2, 3, 48, 32
    rng = np.random.default_rng(11)
    base = [rng.standard_normal((B, T, H, D)).astype(np.float32) for _ in range(4)]
    dev = [torch.from_numpy(a).cuda().permute(0, 2, 1, 3) for a in base]          # views, inner stride 1
    q_dslow = torch.from_numpy(base[0]).cuda().permute(3, 1, 2, 0).contiguous().permute(3, 2, 1, 0)
    assert q_dslow.stride(3) != 1
    host = [np.ascontiguousarray(a.transpose(0, 2, 1, 3)) for a in base]
    want = ref.attn_fwd_bwd(*host)
    op = ops.CausalAttention.new(q_dslow, dev[1], dev[2])
    o = op.forward()
    g = ops.GradientStore()
    op.backward(g, dev[3])
    got = [o, op.lse] + [g.get(t) for t in op.dependencies()]
    for name, a, w in zip(("o", "lse", "dq", "dk", "dv"), got, want):
        assert_close(a.cpu().numpy(), w, TOL_F32, name)


def test_backward_is_bitwise_reproducible():
    # dK/dV (and dQ) are accumulated without atomics: two runs must agree bit for bit.
    from tests.gpu_util import make_inputs, run_fwd_bwd
    args = make_inputs(2, 2, 300, 64, torch.float32, 9)
    a = run_fwd_bwd(*args, torch.float32)
    b = run_fwd_bwd(*args, torch.float32)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_properties_first_row_and_linearity():
    from deers_b200 import ops
    torch.manual_seed(0)
    q, k, v = (torch.randn(2, 2, 150, 32, device="cuda") for _ in range(3))
    o = ops.causal_attention(q, k, v)
    assert torch.allclose(o[:, :, 0], v[:, :, 0], atol=1e-6)
    o2 = ops.causal_attention(q, k, 3.0 * v)
    assert torch.allclose(o2, 3.0 * o, rtol=1e-5, atol=1e-5)


def test_layout_and_argument_errors():
    import ctypes
    from deers_b200 import _lib, ops
    ctx = ops.Context.current(torch.device("cuda", 0))
    L = _lib.lib()
    d = _lib.AttnDesc()
    L.deers_b200_attn_desc_compact(ctypes.byref(d), 1, 1, 16, 32, _lib.F32, 1, 1.0)
    buf = torch.zeros(4096, device="cuda")
    p = buf.data_ptr()
    assert L.deers_b200_attn_fwd(ctx.handle, ctypes.byref(d), None, p, p, p, p, None, 0) == _lib.ERR_NULL
    d.q_strides[3] = 2
    assert L.deers_b200_attn_fwd(ctx.handle, ctypes.byref(d), p, p, p, p, p, None, 0) == _lib.ERR_LAYOUT
    d.q_strides[3] = 1
    d.D = 300
    assert L.deers_b200_attn_fwd(ctx.handle, ctypes.byref(d), p, p, p, p, p, None, 0) == _lib.ERR_SHAPE
    d.D = 32
    d.dtype = 7
    assert L.deers_b200_attn_fwd(ctx.handle, ctypes.byref(d), p, p, p, p, p, None, 0) == _lib.ERR_DTYPE
    d.dtype = _lib.F32
    assert L.deers_b200_attn_bwd(ctx.handle, ctypes.byref(d), p, p, p, p, p, p, p, p, p, None, 0) == _lib.ERR_WORKSPACE
    ctx.sync()
