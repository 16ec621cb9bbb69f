"""The attention block of the reference's GPT (src/models/gpt.rs:118-147) on this library's kernels only, f16:
fused q/k/v projection (one GEMM), rotary pack read straight out of the fused buffer, fused attention with
token-major output, output projection; and the whole backward, with dQ / dK / dV written in place into one
fused gradient buffer.  Checked against the CPU oracle chain in f32."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL_F16, assert_close

pytestmark = pytest.mark.gpu


def test_attention_block_forward_and_backward():
    from deers_b200 import ops
    from oracle import ref
    B, T, H, D = 2, 160, 4, 64
    C = H * D
    rng = np.random.default_rng(21)
    f16 = lambda a: a.astype(np.float16)
    x = f16(rng.standard_normal((B, T, C)))
    wqkv = f16(rng.standard_normal((C, 3 * C)) / np.sqrt(C))            # [in, out]: q | k | v columns
    wo = f16(rng.standard_normal((C, C)) / np.sqrt(C))
    dy = f16(rng.standard_normal((B, T, C)))
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    tx, twqkv, two, tdy = (torch.from_numpy(a).cuda() for a in (x, wqkv, wo, dy))
    tc = torch.from_numpy(cos).to("cuda", torch.float16).reshape(1, T, 1, D // 2)
    ts = torch.from_numpy(sin).to("cuda", torch.float16).reshape(1, T, 1, D // 2)

    # ---- forward
    lin_qkv = ops.Linear.new(tx, twqkv)
    qkv = lin_qkv.forward()                                             # [B,T,3C]
    q4, k4, v4 = (qkv[..., i * C:(i + 1) * C].view(B, T, H, D) for i in range(3))     # views, no copies
    rq, rk = ops.RotaryPack.new(q4, tc, ts), ops.RotaryPack.new(k4, tc, ts)
    qh, kh = rq.forward(), rk.forward()                                 # [B,H,T,D]
    vh = v4.permute(0, 2, 1, 3)                                         # view with strides (T*3C, D, 3C, 1)
    att = ops.CausalAttention.new(qh, kh, vh, token_major_out=True)
    o = att.forward()
    y_att = o.permute(0, 2, 1, 3).reshape(B, T, C)                      # free view of the token-major buffer
    assert y_att.data_ptr() == o.data_ptr()
    lin_o = ops.Linear.new(y_att, two)
    y = lin_o.forward()

    # ---- backward, gradients of q, k, v land in one [B,T,3C] buffer
    grads = ops.GradientStore()
    lin_o.backward(grads, tdy)
    d_att = grads.get(y_att).view(B, T, H, D).permute(0, 2, 1, 3)      # dO as a strided [B,H,T,D] view
    dqkv = torch.empty_like(qkv)
    dq4, dk4, dv4 = (dqkv[..., i * C:(i + 1) * C].view(B, T, H, D) for i in range(3))
    dqh, dkh, _ = ops.attention_bwd(qh, kh, vh, att.o, att.lse, d_att, att.scale, True, dv_out=dv4.permute(0, 2, 1, 3))
    rq.backward(grads, dqh, dx_out=dq4)
    rk.backward(grads, dkh, dx_out=dk4)
    lin_qkv.backward(grads, dqkv)
    ops.Context.current(tx.device).sync()

    # ---- oracle chain in f32 on the same f16 values (intermediate tensors rounded to f16 like the device path)
    r16 = lambda a: a.astype(np.float16).astype(np.float32)
    x32, wqkv32, wo32, dy32 = (a.astype(np.float32) for a in (x, wqkv, wo, dy))
    c16, s16 = r16(cos), r16(sin)
    qkv_ref = r16(x32.reshape(-1, C) @ wqkv32).reshape(B, T, 3 * C)
    qr, kr, vr = (qkv_ref[..., i * C:(i + 1) * C].reshape(B, T, H, D) for i in range(3))
    qh_ref, kh_ref = r16(ref.rope_pack(qr, c16, s16)), r16(ref.rope_pack(kr, c16, s16))
    vh_ref = np.ascontiguousarray(vr.transpose(0, 2, 1, 3))
    datt_ref = r16(dy32.reshape(-1, C) @ wo32.T).reshape(B, T, H, D).transpose(0, 2, 1, 3)
    o_ref, _, dqh_ref, dkh_ref, dvh_ref = ref.attn_fwd_bwd(qh_ref, kh_ref, vh_ref, np.ascontiguousarray(datt_ref))
    yatt_ref = r16(o_ref.transpose(0, 2, 1, 3).reshape(B, T, C))
    y_ref = yatt_ref.reshape(-1, C) @ wo32
    dqkv_ref = np.concatenate([ref.rope_pack(r16(dqh_ref), c16, s16, inverse=True).reshape(B, T, C),
                               ref.rope_pack(r16(dkh_ref), c16, s16, inverse=True).reshape(B, T, C),
                               dvh_ref.transpose(0, 2, 1, 3).reshape(B, T, C)], axis=2)
    dx_ref = r16(dqkv_ref).reshape(-1, 3 * C) @ wqkv32.T
    dwqkv_ref = x32.reshape(-1, C).T @ r16(dqkv_ref).reshape(-1, 3 * C)
    dwo_ref = yatt_ref.reshape(-1, C).T @ dy32.reshape(-1, C)

    assert_close(y.float().cpu().numpy().reshape(-1, C), y_ref, TOL_F16, "y")
    assert_close(dqkv.float().cpu().numpy(), dqkv_ref, TOL_F16, "dqkv")
    assert_close(grads.get(tx).float().cpu().numpy().reshape(-1, C), dx_ref, TOL_F16, "dx")
    assert_close(grads.get(twqkv).float().cpu().numpy(), dwqkv_ref, TOL_F16, "dWqkv")
    assert_close(grads.get(two).float().cpu().numpy(), dwo_ref, TOL_F16, "dWo")
