"""CPU tests of the GPT-step oracle: the literal values the reference's own tests hold, and the float64
autograd golden vectors of the whole model."""
import os

import numpy as np
import pytest

from oracle import ref

HERE = os.path.dirname(os.path.abspath(__file__))


def gpt_golden():
    blob = np.load(os.path.join(HERE, "golden", "gpt_golden.npz"))
    cases = {}
    for key in blob.files:
        name, field = key.split("/")
        cases.setdefault(name, {})[field] = blob[key]
    return cases


def test_nll_loss_forward_literal():
    # src/loss.rs:31-46
    lp = np.array([[-0.9076, -1.2076, -2.4076], [-0.4076, -1.9076, -1.5076]], np.float32)
    assert abs(ref.nll_loss(lp, [0, 2]) - 1.2076) < 1e-4


def test_nll_loss_backward_literal():
    # src/loss.rs:48-65: exact equality in the reference's test
    lp = np.array([[-0.9, -1.2, -2.4], [-0.4, -1.9, -1.5]], np.float32)
    _, g = ref.nll_loss(lp, [1, 0], with_grad=True)
    assert g.reshape(-1).tolist() == [0.0, -0.5, 0.0, -0.5, 0.0, 0.0]


def test_cross_entropy_rows_sum_to_zero():
    # src/loss.rs:67-84
    logits = np.array([[1.0, 2.0, 3.0], [1.0, -1.0, 0.0]], np.float32)
    loss, lse, d = ref.cross_entropy(logits, [2, 0], with_grad=True)
    assert d.shape == (2, 3)
    assert np.abs(d.sum(axis=1)).max() < 1e-4
    # value of log-softmax + nll by hand in float64
    x = logits.astype(np.float64)
    lsm = x - np.log(np.exp(x).sum(1, keepdims=True))
    assert abs(loss - (-(lsm[0, 2] + lsm[1, 0]) / 2)) < 1e-6


def test_rmsnorm_literal():
    # tests/nn.rs:172-186: RMSNorm of [1,2,3], eps 1e-5 -> [1,2,3] / sqrt(14/3) within 1e-4
    y = ref.rmsnorm(np.array([[1.0, 2.0, 3.0]], np.float32), 1e-5)
    rms = np.float32(np.sqrt(np.float32(14.0) / np.float32(3.0)))
    assert np.abs(y[0] - np.array([1.0, 2.0, 3.0], np.float32) / rms).max() < 1e-4


def test_matmul_kinds_agree_with_numpy():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((7, 5)).astype(np.float32)
    b = rng.standard_normal((5, 9)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(ref.matmul(a, b, "nn") - want).max() < 1e-5
    assert np.abs(ref.matmul(a, np.ascontiguousarray(b.T), "nt") - want).max() < 1e-5
    assert np.abs(ref.matmul(np.ascontiguousarray(a.T), b, "tn") - want).max() < 1e-5


def test_embedding_backward_adds_repeated_tokens_in_order():
    rng = np.random.default_rng(1)
    d = rng.standard_normal((6, 4)).astype(np.float32)
    ids = np.array([3, 1, 3, 0, 3, 1])
    dw = ref.embedding_bwd(d, ids, 5)
    assert np.array_equal(dw[3], (d[0] + d[2]) + d[4])
    assert np.array_equal(dw[1], d[1] + d[5])
    assert np.array_equal(dw[0], d[3])
    assert not dw[2].any() and not dw[4].any()
    assert np.array_equal(ref.embedding_fwd(rng.standard_normal((5, 4)).astype(np.float32), ids).shape, (6, 4))


@pytest.mark.parametrize("name", ["tests_gpt_rs", "two_layer_V37"])
def test_gpt_step_matches_float64_autograd(name):
    """Logits, loss and every parameter gradient at the shape and token ids of the reference's model test
    (tests/gpt.rs:38-66) against float64 autograd; tolerance = the reference's CPU tolerance 1e-4 (tests/gpt.rs:8)."""
    g = gpt_golden()[name]
    V, L, H, C, Hm, B, T = (int(v) for v in g["cfg"])
    n = 2 + 6 * L
    params = [g[f"param{i}"] for i in range(n)]
    r = ref.gpt_step((V, L, H, C, Hm), params, g["ids"].reshape(B, T), g["targets"])
    assert np.abs(r["logits"] - g["logits"]).max() < 1e-4
    assert abs(r["loss"] - float(g["loss"])) < 1e-4
    for i in range(n):
        assert np.abs(r["grads"][i] - g[f"grad{i}"]).max() < 1e-4, i


def test_gpt_param_shapes_order():
    shapes = ref.gpt_param_shapes(8, 1, 2, 4, 8)
    assert [s[0] for s in shapes] == ["wte.weight", "blocks.0.attn.q_proj.weight", "blocks.0.attn.k_proj.weight",
                                      "blocks.0.attn.v_proj.weight", "blocks.0.attn.out_proj.weight",
                                      "blocks.0.mlp.up_proj.weight", "blocks.0.mlp.down_proj.weight", "lm_head.weight"]
    total = sum(int(np.prod(s)) for _, s in ref.gpt_param_shapes(50257, 6, 6, 192, 768))
    assert total == 21952896          # the parameter count of BASELINE cfg 3
