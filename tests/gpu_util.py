"""Helpers for the GPU parity tests: run the library through the C ABI on seeded
inputs and compare with the CPU oracle."""
import numpy as np
import torch

from deers_b200 import ops
from oracle import ref
from tests.helpers import assert_close


def make_inputs(B, H, T, D, dtype, seed):
    """Q, K, V, dO ~ N(0,1) from a seed; f16 cases round the f32 draws once."""
    rng = np.random.default_rng(seed)
    arrs = [rng.standard_normal((B, H, T, D)).astype(np.float32) for _ in range(4)]
    if dtype == torch.float16:
        arrs = [a.astype(np.float16).astype(np.float32) for a in arrs]
    return arrs


def to_dev(a, dtype):
    return torch.from_numpy(a).to(device="cuda", dtype=dtype)


def run_fwd_bwd(q, k, v, do, dtype, scale=None, causal=True):
    """Runs the op through the TensorOp-style mirror; returns host float32 arrays."""
    tq, tk, tv, tdo = (to_dev(a, dtype) for a in (q, k, v, do))
    op = ops.CausalAttention.new(tq, tk, tv, scale, causal)
    o = op.forward()
    lse = op.lse
    grads = ops.GradientStore()
    op.backward(grads, tdo)
    ops.Context.current(tq.device).sync()
    out = [o, lse] + [grads.get(t) for t in op.dependencies()]
    return [t.float().cpu().numpy() for t in out]


def check_case(B, H, T, D, dtype, tol, seed=0, scale=None, causal=True, label=""):
    q, k, v, do = make_inputs(B, H, T, D, dtype, seed)
    want = ref.attn_fwd_bwd(q, k, v, do, scale=scale, causal=causal)
    got = run_fwd_bwd(q, k, v, do, dtype, scale, causal)
    errs = {}
    for name, g, w in zip(("o", "lse", "dq", "dk", "dv"), got, want):
        errs[name] = assert_close(g, w, tol, f"{label or (B, H, T, D)}/{name}")
    return errs
