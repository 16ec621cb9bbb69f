"""Generates tests/golden/attn_golden.npz.

The reference (deers) is Rust and cannot run in the build image, and its own
attention test computes expected values with candle at test time, so there is no
stored reference vector to copy.  These vectors come from an independent
implementation instead: float64 torch autograd over the exact op chain of
src/models/gpt.rs:139-144 (matmul, scale, additive -inf mask, softmax, matmul),
seeded, at small shapes including the shape of the reference's own attention
test (tests/gpt.rs:38-49: B=2, T=3, 2 heads, head_dim 2).

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

CASES = {  # name: (B, H, T, D, causal)
    "gpt_rs_shape": (2, 2, 3, 2, True),
    "odd_T17_D8": (1, 2, 17, 8, True),
    "tile_T64_D32": (1, 2, 64, 32, True),
    "ragged_T70_D32": (1, 1, 70, 32, True),
    "T130_D32": (1, 1, 130, 32, True),
    "noncausal_T33_D16": (1, 2, 33, 16, False),
}


def run(B, H, T, D, causal, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = (torch.randn(B, H, T, D, generator=g, dtype=torch.float32) for _ in range(4))
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    scale = float(np.float32(1.0 / np.sqrt(np.float64(D))))
    scores = (q64 @ k64.transpose(2, 3)) * scale
    if causal:
        i = torch.arange(T)
        mask = torch.where(i[None, :] > i[:, None], float("-inf"), 0.0).double()
        scores = scores + mask
    lse = torch.logsumexp(scores, dim=3)
    y = scores.softmax(3) @ v64
    y.backward(do.double())
    out = dict(q=q, k=k, v=v, do=do, o=y.detach(), lse=lse.detach(), dq=q64.grad, dk=k64.grad, dv=v64.grad)
    return {n: t.detach().to(torch.float32).numpy() for n, t in out.items()}


def main():
    blob = {}
    for idx, (name, (B, H, T, D, causal)) in enumerate(CASES.items()):
        for key, arr in run(B, H, T, D, causal, 1000 + idx).items():
            blob[f"{name}/{key}"] = arr
        blob[f"{name}/causal"] = np.array(int(causal))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(path, **blob)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
