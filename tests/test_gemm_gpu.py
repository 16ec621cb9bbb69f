"""GPU parity of the tcgen05 f16 GEMM (the three products of a Linear layer) against a float32 product of
the same f16 inputs, through the C ABI."""
import numpy as np
import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
TOL = 2e-3          # f16 output of an f32-accumulated product: half an f16 ulp is 4.9e-4 of the value


def _rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float16)


@pytest.mark.parametrize("mnk", [(128, 128, 128), (256, 384, 512), (1024, 192, 192), (1000, 200, 72), (8, 8, 8),
                                 (130, 136, 264), (4096, 768, 192)])
def test_linear_forward_and_backward(mnk):
    from deers_b200 import ops
    M, N, K = mnk
    x, w, dy = _rand((M, K), 1), (_rand((K, N), 2).astype(np.float32) / np.sqrt(K)).astype(np.float16), _rand((M, N), 3)
    tx, tw, tdy = (torch.from_numpy(a).cuda() for a in (x, w, dy))
    op = ops.Linear.new(tx, tw)
    y = op.forward()
    grads = ops.GradientStore()
    op.backward(grads, tdy)
    ops.Context.current(tx.device).sync()
    x32, w32, dy32 = (a.astype(np.float32) for a in (x, w, dy))
    assert_close(y.float().cpu().numpy(), x32 @ w32, TOL, f"y {mnk}")                 # nn.rs:184-190
    assert_close(grads.get(tx).float().cpu().numpy(), dy32 @ w32.T, TOL, f"dx {mnk}")  # ops.rs:1089-1101
    assert_close(grads.get(tw).float().cpu().numpy(), x32.T @ dy32, TOL, f"dw {mnk}")


def test_exact_on_small_integers_and_repeatable():
    # products of small integers are exact in f16 / f32: the result must equal the integer product bit for bit
    from deers_b200 import ops
    rng = np.random.default_rng(7)
    M, N, K = 384, 256, 320
    x = rng.integers(-3, 4, (M, K)).astype(np.float16)
    w = rng.integers(-2, 3, (K, N)).astype(np.float16)
    tx, tw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y1 = ops.Linear.new(tx, tw).forward()
    y2 = ops.Linear.new(tx, tw).forward()
    ops.Context.current(tx.device).sync()
    want = (x.astype(np.int64) @ w.astype(np.int64)).astype(np.float32)
    assert np.array_equal(y1.float().cpu().numpy(), want)
    assert torch.equal(y1, y2)


def test_batched_input_and_errors():
    from deers_b200 import ops
    from deers_b200.errors import DTypeMismatch, LayoutMismatch
    x, w = _rand((2, 24, 64), 4), _rand((64, 96), 5)
    tx, tw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = ops.Linear.new(tx, tw).forward()
    assert tuple(y.shape) == (2, 24, 96)
    assert_close(y.float().cpu().numpy(), x.astype(np.float32) @ w.astype(np.float32), TOL, "batched")
    with pytest.raises(LayoutMismatch):
        ops.Linear.new(tx, torch.zeros(60, 96, dtype=torch.float16, device="cuda"))
    with pytest.raises(DTypeMismatch):
        ops.Linear.new(tx.float(), tw.float())
