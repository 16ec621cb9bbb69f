"""GPU parity of the f16 (tcgen05 / TMEM / TMA) kernels against the f32 CPU oracle
evaluated on the f16-rounded inputs, through the C ABI.  Tolerance 2e-2 (max-abs
error over the reference tensor's max-abs) as the north star states."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL_F16, assert_close

pytestmark = pytest.mark.gpu


def test_umma_selftest_operand_layouts():
    # Inputs are multiples of 1/64 in [-2, 2): every product and partial sum is exact in f32.
    from deers_b200 import ops
    errs = ops.Context.current(torch.device("cuda", 0)).selftest_umma()
    assert errs == [0.0] * 6, errs


@pytest.mark.parametrize("shape", [
    (1, 1, 128, 64),
    (1, 1, 128, 128),
    (1, 2, 256, 128),
    (2, 3, 384, 64),
    (1, 2, 1, 64),       # single token
    (1, 2, 100, 128),    # T below one tile
    (1, 2, 130, 64),     # two rows into the second tile
    (1, 1, 777, 128),    # ragged last tile
])
def test_forward_shapes(shape):
    from deers_b200 import ops
    from oracle import ref
    from tests.gpu_util import make_inputs, to_dev
    q, k, v, _ = make_inputs(*shape, torch.float16, seed=sum(shape))
    want_o, want_lse = ref.attn_fwd(q, k, v)
    o, lse = ops.attention_fwd(*(to_dev(a, torch.float16) for a in (q, k, v)), ops.default_scale(shape[3]))
    ops.Context.current(o.device).sync()
    assert_close(o.float().cpu().numpy(), want_o, TOL_F16, f"{shape}/o")
    assert_close(lse.cpu().numpy(), want_lse, TOL_F16, f"{shape}/lse")


def test_forward_noncausal_and_scale():
    from deers_b200 import ops
    from oracle import ref
    from tests.gpu_util import make_inputs, to_dev
    q, k, v, _ = make_inputs(1, 2, 300, 64, torch.float16, seed=21)
    for scale, causal in ((0.2, True), (0.125, False)):
        want_o, want_lse = ref.attn_fwd(q, k, v, scale=scale, causal=causal)
        o, lse = ops.attention_fwd(*(to_dev(a, torch.float16) for a in (q, k, v)), scale, causal)
        assert_close(o.float().cpu().numpy(), want_o, TOL_F16, "o")
        assert_close(lse.cpu().numpy(), want_lse, TOL_F16, "lse")


def test_forward_rescale_path():
    # Keys whose scores grow along the sequence force the running max to jump by far
    # more than 2^8 between tiles, exercising the in-TMEM rescale of O.
    from deers_b200 import ops
    from oracle import ref
    from tests.gpu_util import to_dev
    B, H, T, D = 1, 1, 512, 64
    rng = np.random.default_rng(2)
    q = np.abs(rng.standard_normal((B, H, T, D))).astype(np.float16).astype(np.float32)
    k = np.abs(rng.standard_normal((B, H, T, D))).astype(np.float32)
    k *= (1.0 + 6.0 * (np.arange(T) // 128))[None, None, :, None]
    k = k.astype(np.float16).astype(np.float32)
    v = rng.standard_normal((B, H, T, D)).astype(np.float16).astype(np.float32)
    want_o, want_lse = ref.attn_fwd(q, k, v)
    o, lse = ops.attention_fwd(*(to_dev(a, torch.float16) for a in (q, k, v)), ops.default_scale(D))
    assert_close(o.float().cpu().numpy(), want_o, TOL_F16, "o")
    assert_close(lse.cpu().numpy(), want_lse, TOL_F16, "lse")


@pytest.mark.parametrize("shape", [
    (2, 3, 300, 32),     # the reference GPT's head_dim (n_embd 192 / 6 heads) in f16
    (1, 2, 130, 16),
    (1, 2, 257, 96),     # padded to 128
    (1, 1, 64, 8),
])
def test_head_dims_other_than_64_and_128(shape):
    """The reference derives head_dim = n_embd / n_head freely (src/models/gpt.rs:86-100).  f16 head dims that
    are not a tensor-core tile width run on zero-padded copies: forward and backward against the oracle, and
    the workspace sizes the padded path asks for."""
    from deers_b200 import ops
    from tests.gpu_util import check_case
    check_case(*shape, torch.float16, TOL_F16, seed=sum(shape))
    q = torch.empty(shape, dtype=torch.float16, device="cuda")
    rows_bytes = shape[0] * shape[1] * shape[2] * (64 if shape[3] <= 64 else 128) * 2
    assert ops.workspace_bytes(q, pass_=0) >= 4 * rows_bytes
    assert ops.workspace_bytes(q, pass_=1) >= 8 * rows_bytes
    assert ops.workspace_bytes(torch.empty((1, 1, 128, 64), dtype=torch.float16, device="cuda"), pass_=0) == 0


def test_head_dim_not_a_multiple_of_8_is_refused():
    from deers_b200 import ops
    from deers_b200.errors import DeersError
    q = torch.zeros((1, 1, 64, 20), dtype=torch.float16, device="cuda")
    with pytest.raises(DeersError):
        ops.attention_fwd(q, q, q, 0.2)


def test_cfg2_forward_backward():
    # BASELINE config 2: f16, B=8, T=1024, H=12, head_dim=64; every slice checked.
    from tests.gpu_util import check_case
    check_case(8, 12, 1024, 64, torch.float16, TOL_F16, seed=0)


@pytest.mark.parametrize("shape", [
    (1, 1, 128, 64), (1, 1, 128, 128), (1, 2, 256, 128), (2, 2, 384, 64), (1, 2, 100, 128),
    (1, 2, 130, 64), (1, 1, 777, 128), (1, 1, 1, 64),
])
def test_backward_shapes(shape):
    from tests.gpu_util import check_case
    check_case(*shape, torch.float16, TOL_F16, seed=sum(shape) + 1)


def test_backward_noncausal():
    from tests.gpu_util import check_case
    check_case(1, 2, 300, 64, torch.float16, TOL_F16, seed=8, causal=False)


def test_dk_dv_bitwise_reproducible():
    from tests.gpu_util import make_inputs, run_fwd_bwd
    args = make_inputs(2, 2, 640, 128, torch.float16, 9)
    a = run_fwd_bwd(*args, torch.float16)
    b = run_fwd_bwd(*args, torch.float16)
    for idx in (0, 1, 3, 4):      # o, lse, dk, dv: no atomics anywhere on their path
        assert np.array_equal(a[idx], b[idx])


def _sampled_slices(B, H, T, D, n_random, seed):
    """Full-size run on the device, oracle on a fixed sample of (b, h) slices."""
    from deers_b200 import ops
    from oracle import ref
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = (torch.randn(B, H, T, D, device="cuda", dtype=torch.float16, generator=g) for _ in range(4))
    op = ops.CausalAttention.new(q, k, v)
    o = op.forward()
    grads = ops.GradientStore()
    # The backward with room for its dS tiles; the workspace starts as all-ones bytes (NaN patterns), so a
    # tile that were read without having been written would show.
    ws = torch.full((ops.workspace_bytes(q, op.scale, True, pass_=2),), 0xFF, dtype=torch.uint8, device="cuda")
    for t, g in zip((q, k, v), ops.attention_bwd(q, k, v, o, op.lse, do, op.scale, True, workspace=ws)):
        grads.accumulate(t, g)
    ops.Context.current(q.device).sync()
    del ws
    rng = np.random.default_rng(seed)
    picks = {(0, 0), (B - 1, H - 1)} | {(int(rng.integers(B)), int(rng.integers(H))) for _ in range(n_random)}
    for b, h in sorted(picks):
        host = [t[b:b + 1, h:h + 1].float().cpu().numpy() for t in (q, k, v, do)]
        want = ref.attn_fwd_bwd(*host)
        got = [o, op.lse, grads.get(q), grads.get(k), grads.get(v)]
        for name, gt, w in zip(("o", "lse", "dq", "dk", "dv"), got, want):
            assert_close(gt[b:b + 1, h:h + 1].float().cpu().numpy(), w, TOL_F16, f"slice({b},{h})/{name}")
    # Size-independent properties over the whole tensor: finite everywhere, causal row 0 == v[0].
    for t in (o, grads.get(q), grads.get(k), grads.get(v)):
        assert torch.isfinite(t).all()
    assert torch.allclose(o[:, :, 0].float(), v[:, :, 0].float(), atol=2e-3)


def test_cfg4_long_context_sampled_slices():
    # BASELINE config 4: B=2, T=8192, H=16, head_dim=128.
    _sampled_slices(2, 16, 8192, 128, n_random=2, seed=4)


def test_cfg5_shape_sampled_slices():
    # BASELINE config 5 at full size on one GPU: B=64, T=2048, H=32, head_dim=128.
    _sampled_slices(64, 32, 2048, 128, n_random=6, seed=5)


@pytest.mark.parametrize("shape,causal", [((1, 2, 256, 128), True), ((2, 2, 384, 64), True), ((1, 2, 130, 64), True),
                                          ((1, 1, 777, 128), True), ((1, 2, 300, 64), False), ((1, 1, 1, 64), True),
                                          ((3, 8, 1100, 128), True), ((2, 5, 900, 64), False)])
def test_backward_workspace_selects_kept_ds_or_recompute(shape, causal):
    # The workspace size picks the backward: pass-2 bytes keep the dS tiles between the two main kernels,
    # pass-1 bytes make the dQ kernel recompute S and dP.  Both against the oracle, and against each other.
    from deers_b200 import ops
    from oracle import ref
    from tests.gpu_util import make_inputs, to_dev
    q, k, v, do = make_inputs(*shape, torch.float16, seed=sum(shape) + 31)
    want = ref.attn_fwd_bwd(q, k, v, do, causal=causal)
    tq, tk, tv, tdo = (to_dev(a, torch.float16) for a in (q, k, v, do))
    scale = ops.default_scale(shape[3])
    o, lse = ops.attention_fwd(tq, tk, tv, scale, causal)
    small, large = (ops.workspace_bytes(tq, scale, causal, pass_=p) for p in (1, 2))
    assert large > small
    got = {}
    for name, nbytes in (("recompute", small), ("kept", large)):
        ws = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")      # NaN patterns: nothing may be read unwritten
        got[name] = [t.float().cpu().numpy() for t in ops.attention_bwd(tq, tk, tv, o, lse, tdo, scale, causal, workspace=ws)]
        ops.Context.current(tq.device).sync()
        for label, g, w in zip(("dq", "dk", "dv"), got[name], want[2:]):
            assert_close(g, w, TOL_F16, f"{name}/{shape}/{label}")
    # dK and dV come from the same kernel and the same arithmetic either way
    assert np.array_equal(got["recompute"][1], got["kept"][1]) and np.array_equal(got["recompute"][2], got["kept"][2])
    again = [t.float().cpu().numpy() for t in ops.attention_bwd(tq, tk, tv, o, lse, tdo, scale, causal,
                                                                 workspace=torch.zeros(large, dtype=torch.uint8, device="cuda"))]
    assert np.array_equal(again[0], got["kept"][0])          # no atomics: bitwise repeatable
