"""CPU tests of the oracle: pinned mask values, golden vectors, and properties."""
import numpy as np

from oracle import ref
from tests.helpers import TOL_F32, assert_close

NEG = -np.inf


def test_causal_mask_known_answer():
    # Literal expected values of the reference's test (tests/nn.rs:194-218).
    want = [0.0, NEG, NEG, 0.0, 0.0, NEG, 0.0, 0.0, 0.0] * 2
    got = ref.causal_mask(2, 3, 0)
    assert got.shape == (2, 1, 3, 3)
    assert got.ravel().tolist() == want


def test_causal_mask_with_offset_known_answer():
    # tests/nn.rs:220-232
    got = ref.causal_mask(1, 2, 3)
    assert got.shape == (1, 1, 2, 5)
    assert got.ravel().tolist() == [0.0, 0.0, 0.0, 0.0, NEG, 0.0, 0.0, 0.0, 0.0, 0.0]


def test_oracle_matches_golden(golden):
    for name, c in golden.items():
        causal = bool(c["causal"])
        o, lse, dq, dk, dv = ref.attn_fwd_bwd(c["q"], c["k"], c["v"], c["do"], causal=causal)
        for label, got in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
            assert_close(got, c[label], TOL_F32, f"{name}/{label}")
        o2, lse2 = ref.attn_fwd(c["q"], c["k"], c["v"], causal=causal)
        assert np.array_equal(o2, o) and np.array_equal(lse2, lse)


def test_softmax_rows_known_inputs():
    # The literal rows the reference feeds its softmax / log_sum_exp tests
    # (tests/tensor.rs:296,1887,2119): with V = identity the op returns the softmax itself.
    x = np.array([[1.0, 2.0, 3.0], [1.5, 0.5, -1.0]], np.float32)
    T, D = 2, 3
    # Build q, k so that q @ k^T = x on a non-causal 2 x 3 problem padded to square T=3.
    q = np.zeros((1, 1, 3, 3), np.float32); q[0, 0, :2, :] = x
    k = np.eye(3, dtype=np.float32)[None, None]
    v = np.eye(3, dtype=np.float32)[None, None]
    o, lse = ref.attn_fwd(q, k, v, scale=1.0, causal=False)
    want = np.exp(x - x.max(1, keepdims=True)); want /= want.sum(1, keepdims=True)
    assert np.abs(o[0, 0, :2] - want).max() < 1e-6
    assert np.abs(lse[0, 0, :2] - np.log(np.exp(x.astype(np.float64)).sum(1))).max() < 1e-6


def test_first_row_is_v0_and_rows_sum():
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((2, 2, 9, 4)).astype(np.float32) for _ in range(3))
    o, lse = ref.attn_fwd(q, k, v)
    # Causal row 0 attends to key 0 only.
    assert np.allclose(o[:, :, 0], v[:, :, 0], atol=1e-6)
    # Linearity in V.
    o2, _ = ref.attn_fwd(q, k, 2.0 * v)
    assert np.allclose(o2, 2.0 * o, atol=1e-5)


def test_gradients_by_finite_differences():
    rng = np.random.default_rng(5)
    B, H, T, D = 1, 1, 5, 4
    q, k, v, do = (rng.standard_normal((B, H, T, D)) for _ in range(4))
    _, _, dq, dk, dv = ref.attn_fwd_bwd(q, k, v, do)

    def loss(q_, k_, v_):
        q64, k64, v64 = (np.asarray(x, np.float64)[0, 0] for x in (q_, k_, v_))
        s = q64 @ k64.T * ref.default_scale(D)
        s = np.where(np.triu(np.ones((T, T), bool), 1), -np.inf, s)
        p = np.exp(s - s.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
        return float(((p @ v64) * do[0, 0]).sum())

    eps = 1e-5
    for name, x, g in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        for idx in [(0, 0, 1, 2), (0, 0, 4, 0), (0, 0, 2, 3)]:
            xp, xm = x.copy(), x.copy()
            xp[idx] += eps; xm[idx] -= eps
            args_p = {"q": q, "k": k, "v": v}; args_m = dict(args_p)
            args_p[name] = xp; args_m[name] = xm
            fd = (loss(args_p["q"], args_p["k"], args_p["v"]) - loss(args_m["q"], args_m["k"], args_m["v"])) / (2 * eps)
            assert abs(fd - g[idx]) < 2e-3, (name, idx, fd, g[idx])


def _rope_golden():
    import os
    blob = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rope_golden.npz"))
    cases = {}
    for key in blob.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = blob[key]
    return cases


def test_rope_oracle_matches_golden():
    # float64 autograd over the reference's op chain (tests/golden/make_golden.py) vs the f32 restatement
    for name, c in _rope_golden().items():
        y = ref.rope_pack(c["x"], c["cos"], c["sin"])
        dx = ref.rope_pack(c["dy"], c["cos"], c["sin"], inverse=True)
        assert np.abs(y - c["y"]).max() <= 1e-6 * max(np.abs(c["y"]).max(), 1.0), name
        assert np.abs(dx - c["dx"]).max() <= 1e-6 * max(np.abs(c["dx"]).max(), 1.0), name
        cos, sin = ref.precompute_rotary_embeddings(c["x"].shape[1], c["x"].shape[3])
        assert np.array_equal(cos, c["cos"]) and np.array_equal(sin, c["sin"])


def test_rope_oracle_op_order_and_f16_emulation():
    rng = np.random.default_rng(1)
    B, T, H, D = 2, 9, 3, 16
    x = rng.standard_normal((B, T, H, D)).astype(np.float32)
    cos, sin = ref.precompute_rotary_embeddings(T, D)
    # numpy f32 evaluates the same chain with one rounding per op: identical bits
    a, b = x[..., :D // 2], x[..., D // 2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    want = np.concatenate([a * c + b * s, a * (s * np.float32(-1)) + b * c], 3).transpose(0, 2, 1, 3)
    assert np.array_equal(ref.rope_pack(x, cos, sin), want)
    # position 0 is the identity rotation; rotating back restores x up to rounding
    assert np.array_equal(ref.rope_pack(x, cos, sin)[:, :, 0, :], x[:, 0].transpose(0, 1, 2))
    back = ref.rope_pack(ref.rope_pack(x, cos, sin), cos, sin, inverse=True)
    assert np.abs(back - x).max() < 1e-6
    y16 = ref.rope_pack_f16(x, cos, sin)
    assert y16.dtype == np.float16 and np.abs(y16.astype(np.float32) - ref.rope_pack(x, cos, sin)).max() < 1e-2


def test_clip_grad_norm_oracle_known_answer():
    # Literal values of the reference's own test (src/optim.rs:556-570).
    g = [np.array([3.0, 4.0], np.float32)]
    norm = ref.clip_grad_norm(g, 1.0)
    assert abs(norm - 5.0) < 1e-5 and abs(g[0][0] - 0.6) < 1e-4 and abs(g[0][1] - 0.8) < 1e-4
    g = [np.array([0.3, 0.4], np.float32)]
    assert abs(ref.clip_grad_norm(g, 1.0) - 0.5) < 1e-6 and g[0].tolist() == [np.float32(0.3), np.float32(0.4)]


def test_adamw_oracle_op_order_and_reference_unit_tests():
    rng = np.random.default_rng(0)
    n = 1000
    w, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v = (0.1 * rng.standard_normal(n)).astype(np.float32), (0.01 * np.abs(rng.standard_normal(n))).astype(np.float32)
    w2, m2, v2 = w.copy(), m.copy(), v.copy()
    ref.adamw_step(w2, g, m2, v2, 7, 1e-3, (0.9, 0.95), 1e-8, 0.1)
    f = np.float32                                           # numpy f32: one rounding per op, like the reference
    mm = m * f(0.9) + g * f(1 - 0.9)
    vv = v * f(0.95) + (g * g) * f(1 - 0.95)
    mh, vh = mm * f(1 / (1 - 0.9 ** 7)), vv * f(1 / (1 - 0.95 ** 7))
    ww = w * f(1 - 1e-3 * 0.1) - (mh / (np.sqrt(vh) + f(1e-8))) * f(1e-3)
    assert np.array_equal(mm, m2) and np.array_equal(vv, v2) and np.array_equal(ww, w2)
    # src/optim.rs:417-432: minimise (x-3)^2 from x = 0 with lr 0.1: x moves toward 3
    x, mx, vx = np.zeros(1, np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32)
    ref.adamw_step(x, np.array([-6.0], np.float32), mx, vx, 1, 0.1)
    assert x[0] > 0.0
    # src/optim.rs:535-553: x^2 + y^2 converges to the origin in 100 steps
    p, pm, pv = np.array([5.0, -3.0], np.float32), np.zeros(2, np.float32), np.zeros(2, np.float32)
    for step in range(1, 101):
        ref.adamw_step(p, (2 * p).astype(np.float32), pm, pv, step, 0.1)
    assert np.abs(p).max() < 0.1


def _npz(name):
    import os
    blob = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))
    cases = {}
    for key in blob.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = blob[key]
    return cases


def test_rmsnorm_oracle_matches_golden():
    for name, c in _npz("rmsnorm_golden.npz").items():
        y, dx = ref.rmsnorm(c["x"], float(c["eps"]), c["dy"])
        assert_close(y, c["y"], 1e-5, f"{name}/y")
        # at C = 1 the gradient cancels to ~eps: an absolute floor stands in for the missing scale
        assert np.abs(dx - c["dx"]).max() <= 1e-5 * np.abs(c["dx"]).max() + 1e-6, name
        # every output row has mean square 1 (up to eps)
        if c["x"].shape[1] > 1:
            assert np.allclose((y.astype(np.float64) ** 2).mean(1), 1.0, atol=1e-3)


def test_decode_oracle_agrees_with_the_square_oracle():
    # Tq == Tk reduces to the causal forward; with Tq < Tk the rows equal the last rows of the square case.
    rng = np.random.default_rng(2)
    B, H, T, D = 1, 2, 12, 8
    q, k, v = (rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(3))
    o_sq, lse_sq = ref.attn_fwd(q, k, v)
    o_d, lse_d = ref.attn_decode(q, k, v)
    assert_close(o_d, o_sq, TOL_F32, "square o")
    assert_close(lse_d, lse_sq, TOL_F32, "square lse")
    o_tail, lse_tail = ref.attn_decode(q[:, :, -3:], k, v)
    assert_close(o_tail, o_sq[:, :, -3:], TOL_F32, "tail o")
    assert_close(lse_tail, lse_sq[:, :, -3:], TOL_F32, "tail lse")
