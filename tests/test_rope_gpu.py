"""GPU parity of the fused rotary embedding + head-major pack (and of the [B,T,H,D]-direct
attention output) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL_F16, TOL_F32, assert_close

pytestmark = pytest.mark.gpu


def _golden():
    import os
    blob = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_golden.npz"))
    cases = {}
    for key in blob.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = blob[key]
    return cases


def _run(x, cos, sin, dy, dtype):
    """x [B,T,H,D], dy [B,H,T,D] host arrays -> (y, dx) through the TensorOp-style mirror."""
    from deers_b200 import ops
    tx = torch.from_numpy(x).to("cuda", dtype)
    tc = torch.from_numpy(cos).to("cuda", dtype).reshape(1, cos.shape[0], 1, cos.shape[1])
    ts = torch.from_numpy(sin).to("cuda", dtype).reshape(1, sin.shape[0], 1, sin.shape[1])
    op = ops.RotaryPack.new(tx, tc, ts)
    y = op.forward()
    grads = ops.GradientStore()
    op.backward(grads, torch.from_numpy(dy).to("cuda", dtype))
    ops.Context.current(tx.device).sync()
    assert y.is_contiguous() and tuple(y.shape) == (x.shape[0], x.shape[2], x.shape[1], x.shape[3])
    return y.cpu().numpy(), grads.get(op.dependencies()[0]).cpu().numpy()


def test_f32_is_bit_exact_against_the_oracle_and_matches_golden():
    from oracle import ref
    for name, c in _golden().items():
        y, dx = _run(c["x"], c["cos"], c["sin"], c["dy"], torch.float32)
        assert np.array_equal(y, ref.rope_pack(c["x"], c["cos"], c["sin"])), name
        assert np.array_equal(dx, ref.rope_pack(c["dy"], c["cos"], c["sin"], inverse=True)), name
        assert_close(y, c["y"], TOL_F32, f"{name}/y")
        assert_close(dx, c["dx"], TOL_F32, f"{name}/dx")


@pytest.mark.parametrize("shape", [
    (2, 3, 2, 2),        # the reference's own GPT test shape (tests/gpt.rs:38-49): scalar path
    (1, 7, 3, 6),        # half rows of 3 elements: scalar path
    (2, 33, 5, 16),      # f16: 16-byte pieces; f32: two pieces per half row
    (1, 130, 4, 64),
    (2, 64, 6, 128),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_shapes_bit_exact(shape, dtype):
    from oracle import ref
    B, T, H, D = shape
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal((B, T, H, D)).astype(np.float32)
    dy = rng.standard_normal((B, H, T, D)).astype(np.float32)
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    if dtype == torch.float16:
        x16, dy16 = x.astype(np.float16), dy.astype(np.float16)
        y, dx = _run(x16.astype(np.float32), cos, sin, dy16.astype(np.float32), dtype)
        want_y = ref.rope_pack_f16(x16, cos, sin)
        want_dx = ref.rope_pack_f16(dy16, cos, sin, inverse=True)
        # every multiply and add rounds to f16 on both sides: identical bits
        assert np.array_equal(y.view(np.uint16), want_y.view(np.uint16))
        assert np.array_equal(dx.view(np.uint16), want_dx.view(np.uint16))
        assert_close(y, ref.rope_pack(x16.astype(np.float32), cos, sin), TOL_F16, "y vs f32 oracle")
    else:
        y, dx = _run(x, cos, sin, dy, dtype)
        assert np.array_equal(y, ref.rope_pack(x, cos, sin))
        assert np.array_equal(dx, ref.rope_pack(dy, cos, sin, inverse=True))


def test_strided_and_misaligned_inputs():
    # The projection output may be a slice of a fused qkv buffer: row stride 3*D, and an offset that
    # breaks 16-byte alignment must fall back to the scalar path with the same bits.
    from deers_b200 import ops
    from oracle import ref
    B, T, H, D = 2, 20, 3, 32
    rng = np.random.default_rng(5)
    qkv = rng.standard_normal((B, T, H, 3 * D)).astype(np.float32)
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    tqkv = torch.from_numpy(qkv).cuda()
    tc = torch.from_numpy(cos).cuda().reshape(1, T, 1, D // 2)
    ts = torch.from_numpy(sin).cuda().reshape(1, T, 1, D // 2)
    for off in (0, D, 2 * D):
        y = ops.rotary_pack(tqkv[..., off:off + D], tc, ts)
        assert np.array_equal(y.cpu().numpy(), ref.rope_pack(qkv[..., off:off + D], cos, sin))
    flat = torch.zeros(B * T * H * D + 1, dtype=torch.float32, device="cuda")
    mis = flat[1:].view(B, T, H, D)                      # 4-byte aligned only
    mis.copy_(torch.from_numpy(qkv[..., :D]))
    y = ops.rotary_pack(mis, tc, ts)
    assert np.array_equal(y.cpu().numpy(), ref.rope_pack(qkv[..., :D], cos, sin))


def test_rope_then_attention_with_token_major_output():
    # The module's path (src/models/gpt.rs:135-144): rope(q), rope(k) -> [B,H,T,D]; v as a permuted view;
    # y leaves as [B,T,H,D] without a copy; gradients flow back through the inverse rotation.
    from deers_b200 import ops
    from oracle import ref
    B, T, H, D = 2, 96, 3, 32
    rng = np.random.default_rng(9)
    q, k, v = (rng.standard_normal((B, T, H, D)).astype(np.float32) for _ in range(3))
    dy = rng.standard_normal((B, T, H, D)).astype(np.float32)            # gradient of the [B,T,H*D] output
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    tq, tk, tv, tdy = (torch.from_numpy(a).cuda() for a in (q, k, v, dy))
    tc = torch.from_numpy(cos).cuda().reshape(1, T, 1, D // 2)
    ts = torch.from_numpy(sin).cuda().reshape(1, T, 1, D // 2)
    rq, rk = ops.RotaryPack.new(tq, tc, ts), ops.RotaryPack.new(tk, tc, ts)
    qh, kh = rq.forward(), rk.forward()
    vh_t = tv.permute(0, 2, 1, 3)                                         # a view, consumed in place
    att = ops.CausalAttention.new(qh, kh, vh_t, token_major_out=True)
    o = att.forward()                                                     # [B,H,T,D] view of [B,T,H,D] memory
    y = o.permute(0, 2, 1, 3)
    assert y.is_contiguous()                                              # the module's reshape is a free view
    grads = ops.GradientStore()
    att.backward(grads, tdy.permute(0, 2, 1, 3))
    rq.backward(grads, grads.get(qh))
    rk.backward(grads, grads.get(kh))
    ops.Context.current(tq.device).sync()

    qh_ref, kh_ref = ref.rope_pack(q, cos, sin), ref.rope_pack(k, cos, sin)
    vh = np.ascontiguousarray(v.transpose(0, 2, 1, 3))
    o_ref, _, dqh, dkh, dvh = ref.attn_fwd_bwd(qh_ref, kh_ref, vh, np.ascontiguousarray(dy.transpose(0, 2, 1, 3)))
    assert_close(y.cpu().numpy(), o_ref.transpose(0, 2, 1, 3), TOL_F32, "y")
    assert_close(grads.get(tq).cpu().numpy(), ref.rope_pack(dqh, cos, sin, inverse=True), TOL_F32, "dq")
    assert_close(grads.get(tk).cpu().numpy(), ref.rope_pack(dkh, cos, sin, inverse=True), TOL_F32, "dk")
    assert_close(grads.get(vh_t).cpu().numpy(), dvh, TOL_F32, "dv")


def test_full_size_rotation_properties():
    # B=64, T=2048, H=32, D=128 f16 (the q tensor of the headline workload): sampled rows against the
    # oracle bit for bit, and the size-independent property that rotating back returns x up to f16 rounding.
    from deers_b200 import ops
    from oracle import ref
    B, T, H, D = 64, 2048, 32, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((B, T, H, D), generator=g, device="cuda", dtype=torch.float32).to(torch.float16)
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    tc = torch.from_numpy(cos).to("cuda", torch.float16).reshape(1, T, 1, D // 2)
    ts = torch.from_numpy(sin).to("cuda", torch.float16).reshape(1, T, 1, D // 2)
    op = ops.RotaryPack.new(x, tc, ts)
    y = op.forward()
    grads = ops.GradientStore()
    op.backward(grads, y)                                   # rotate back
    back = grads.get(x)
    ops.Context.current(x.device).sync()
    err = (back.float() - x.float()).abs().max().item()
    assert err <= 3e-2 * x.float().abs().max().item()      # three f16 roundings each way
    for b, h in ((0, 0), (63, 31), (17, 5)):
        got = y[b, h].cpu().numpy()
        want = ref.rope_pack_f16(x[b:b + 1, :, h:h + 1, :].cpu().numpy(), cos, sin)[0, 0]
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    del back, grads, y, x
    torch.cuda.empty_cache()
