"""GPU parity of the fused RMSNorm forward / backward against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu
TOL = 1e-5      # f32, sums in a different order than the reference's left-to-right sum


def _run(x, dy, eps):
    from deers_b200 import ops
    tx = torch.from_numpy(x).cuda()
    op = ops.RMSNorm.new(tx, eps)
    y = op.forward()
    grads = ops.GradientStore()
    op.backward(grads, torch.from_numpy(dy).cuda())
    ops.Context.current(tx.device).sync()
    return y.cpu().numpy(), grads.get(op.dependencies()[0]).cpu().numpy()


def test_golden_vectors():
    import os
    blob = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rmsnorm_golden.npz"))
    for name in sorted({k.split("/")[0] for k in blob.files}):
        x, dy, eps = blob[f"{name}/x"], blob[f"{name}/dy"], float(blob[f"{name}/eps"])
        y, dx = _run(x, dy, eps)
        assert_close(y, blob[f"{name}/y"], TOL, f"{name}/y")
        assert np.abs(dx - blob[f"{name}/dx"]).max() <= TOL * np.abs(blob[f"{name}/dx"]).max() + 1e-6, name


@pytest.mark.parametrize("shape", [(4, 256, 192), (3, 5, 7), (2, 1024), (33, 1028), (5, 8192), (2, 8196), (1, 4100 * 4), (6, 1), (3, 1026)])
def test_shapes_against_the_oracle(shape):
    from oracle import ref
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    dy = rng.standard_normal(shape).astype(np.float32)
    want_y, want_dx = ref.rmsnorm(x, 1e-6, dy)
    y, dx = _run(x, dy, 1e-6)
    assert_close(y, want_y, TOL, "y")
    assert np.abs(dx - want_dx).max() <= TOL * np.abs(want_dx).max() + 1e-6


def test_model_sized_rows_and_properties():
    # cfg 5's token count with the headline width: 131072 rows of 4096 (2 GiB in, 2 GiB out): rows have unit
    # mean square, the gradient is orthogonal to x in every row (d/dx of a scale-invariant map), sampled rows
    # match the oracle.
    from deers_b200 import ops
    from oracle import ref
    rows, C = 64 * 2048, 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(rows, C, device="cuda", generator=g)
    dy = torch.randn(rows, C, device="cuda", generator=g)
    op = ops.RMSNorm.new(x, 1e-6)
    y = op.forward()
    grads = ops.GradientStore()
    op.backward(grads, dy)
    dx = grads.get(x)
    ops.Context.current(x.device).sync()
    ms = (y.double() ** 2).mean(1)
    assert (ms - 1.0).abs().max().item() < 1e-4
    assert ((dx.double() * x.double()).sum(1).abs().max().item()) < 1e-2 * C ** 0.5
    for r in (0, rows - 1, 77777):
        wy, wdx = ref.rmsnorm(x[r:r + 1].cpu().numpy(), 1e-6, dy[r:r + 1].cpu().numpy())
        assert_close(y[r:r + 1].cpu().numpy(), wy, TOL, "y row")
        assert_close(dx[r:r + 1].cpu().numpy(), wdx, TOL, "dx row")
