"""Generates tests/golden/attn_golden.npz, rope_golden.npz, rmsnorm_golden.npz and gpt_golden.npz.

The reference (deers) is Rust and cannot run in the build image, and its own
attention test computes expected values with candle at test time, so there is no
stored reference vector to copy.  These vectors come from an independent
implementation instead: float64 torch autograd over the exact op chain of
src/models/gpt.rs:139-144 (matmul, scale, additive -inf mask, softmax, matmul),
seeded, at small shapes including the shape of the reference's own attention
test (tests/gpt.rs:38-49: B=2, T=3, 2 heads, head_dim 2).

rope_golden.npz holds the rotary embedding + head-major permute of src/models/gpt.rs:49-73,135-136
(x [B,T,H,D] -> y [B,H,T,D]) and its gradient, again as float64 torch autograd over the reference's op
chain (narrow, mul, add, cat, permute), with the cos / sin cache of gpt.rs:12-46 computed in f32.

gpt_golden.npz holds logits, loss and every parameter gradient of the whole model of src/models/gpt.rs
(embedding, blocks of RMSNorm / attention with RoPE / relu^2 MLP with residuals, final norm, lm_head) under
cross_entropy (src/loss.rs:21-24), as float64 torch autograd over the same op chain, at the shape and token ids of
the reference's own model test (tests/gpt.rs:38-66: vocab 8, 1 layer, 2 heads, n_embd 4, mlp 8, B=2, T=3) and at
a second, larger shape; the weights are seeded draws from the reference's init distributions.

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


ROPE_CASES = {  # name: (B, T, H, D)
    "gpt_rs_shape": (2, 3, 2, 2),
    "odd_T17_D8": (1, 17, 3, 8),
    "T64_D32": (2, 64, 4, 32),
    "T5_D64": (1, 5, 2, 64),
}


def rope_cache(T, D, base=10000.0):
    half = D // 2
    channel = (2 * np.arange(half)).astype(np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base), channel / np.float32(D))).astype(np.float32)
    freqs = (np.arange(T, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)


def run_rope(B, T, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, H, D, generator=g, dtype=torch.float32)
    dy = torch.randn(B, H, T, D, generator=g, dtype=torch.float32)
    cos, sin = rope_cache(T, D)
    c = torch.from_numpy(cos).double()[None, :, None, :]
    s = torch.from_numpy(sin).double()[None, :, None, :]
    x64 = x.double().requires_grad_(True)
    x1, x2 = x64.narrow(3, 0, D // 2), x64.narrow(3, D // 2, D // 2)
    y = torch.cat([x1 * c + x2 * s, x1 * (s * -1.0) + x2 * c], 3).permute(0, 2, 1, 3)
    y.backward(dy.double())
    out = dict(x=x, dy=dy, y=y.detach().contiguous(), dx=x64.grad)
    res = {n: t.detach().to(torch.float32).numpy() for n, t in out.items()}
    res["cos"], res["sin"] = cos, sin
    return res


NORM_CASES = {"gpt_rows": (8, 192, 1e-6), "odd_C7": (5, 7, 1e-5), "wide_C1024": (3, 1024, 1e-6), "C1": (4, 1, 1e-6)}


def run_rmsnorm(rows, C, eps, seed):
    """RMSNorm (src/nn.rs:244-251) and its gradient as float64 torch autograd over the reference's op chain."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, C, generator=g, dtype=torch.float32)
    dy = torch.randn(rows, C, generator=g, dtype=torch.float32)
    x64 = x.double().requires_grad_(True)
    y = x64 * ((x64 * x64).mean(1, keepdim=True) + eps).pow(-0.5)
    y.backward(dy.double())
    return dict(x=x.numpy(), dy=dy.numpy(), y=y.detach().float().numpy(), dx=x64.grad.float().numpy(),
                eps=np.array(eps))


GPT_CASES = {  # name: (vocab, n_layer, n_head, n_embd, mlp_hidden, B, T)
    "tests_gpt_rs": (8, 1, 2, 4, 8, 2, 3),
    "two_layer_V37": (37, 2, 3, 24, 40, 2, 9),
}


def run_gpt(V, L, H, C, Hm, B, T, seed, eps=1e-5, base=10000.0):
    rng = np.random.default_rng(seed)
    shapes = [("wte", (V, C))]
    for i in range(L):
        shapes += [(f"b{i}.q", (C, C)), (f"b{i}.k", (C, C)), (f"b{i}.v", (C, C)), (f"b{i}.out", (C, C)),
                   (f"b{i}.up", (C, Hm)), (f"b{i}.down", (Hm, C))]
    shapes.append(("lm_head", (C, V)))
    params = []
    for name, shape in shapes:
        if name == "wte":
            params.append(rng.standard_normal(shape).astype(np.float32))
        else:
            k = 1.0 / np.sqrt(shape[0])
            params.append((rng.random(shape, dtype=np.float32) * np.float32(2 * k) - np.float32(k)).astype(np.float32))
    if (V, B, T) == (8, 2, 3):
        ids = np.array([1, 2, 3, 4, 3, 2], np.int64)          # tests/gpt.rs:51-66
        targets = np.array([2, 3, 4, 3, 2, 1], np.int64)
    else:
        ids = rng.integers(0, V, B * T).astype(np.int64)
        ids[1] = ids[0]                                        # a repeated token: its embedding rows add up
        targets = rng.integers(0, V, B * T).astype(np.int64)
    D = C // H
    cos, sin = rope_cache(T, D, base)
    c = torch.from_numpy(cos).double()[None, :, None, :]
    s = torch.from_numpy(sin).double()[None, :, None, :]
    W = [torch.from_numpy(p).double().requires_grad_(True) for p in params]

    def norm(x):
        return x * ((x * x).mean(-1, keepdim=True) + eps).pow(-0.5)

    def rope(x):
        x1, x2 = x.narrow(3, 0, D // 2), x.narrow(3, D // 2, D // 2)
        return torch.cat([x1 * c + x2 * s, x1 * (s * -1.0) + x2 * c], 3)

    x = W[0][torch.from_numpy(ids)].reshape(B, T, C)
    i = torch.arange(T)
    mask = torch.where(i[None, :] > i[:, None], float("-inf"), 0.0).double()
    scale = float(np.float32(1.0 / np.sqrt(np.float64(D))))
    for l in range(L):
        wq, wk, wv, wo, wu, wd = W[1 + 6 * l: 7 + 6 * l]
        n1 = norm(x).reshape(B * T, C)
        q = rope((n1 @ wq).reshape(B, T, H, D)).permute(0, 2, 1, 3)
        k = rope((n1 @ wk).reshape(B, T, H, D)).permute(0, 2, 1, 3)
        v = (n1 @ wv).reshape(B, T, H, D).permute(0, 2, 1, 3)
        att = ((q @ k.transpose(2, 3)) * scale + mask).softmax(3)
        y = (att @ v).permute(0, 2, 1, 3).reshape(B * T, C)
        x = x + (y @ wo).reshape(B, T, C)
        n2 = norm(x).reshape(B * T, C)
        r = torch.relu(n2 @ wu)
        x = x + ((r * r) @ wd).reshape(B, T, C)
    logits = norm(x).reshape(B * T, C) @ W[-1]
    loss = torch.nn.functional.cross_entropy(logits, torch.from_numpy(targets))
    loss.backward()
    out = {"cfg": np.array([V, L, H, C, Hm, B, T]), "ids": ids, "targets": targets,
           "logits": logits.detach().float().numpy(), "loss": np.array(loss.item(), np.float32)}
    for idx, (p, w) in enumerate(zip(params, W)):
        out[f"param{idx}"] = p
        out[f"grad{idx}"] = w.grad.float().numpy()
    return out


def main_gpt():
    blob = {}
    for idx, (name, cfg) in enumerate(GPT_CASES.items()):
        for key, arr in run_gpt(*cfg, seed=4000 + idx).items():
            blob[f"{name}/{key}"] = arr
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gpt_golden.npz")
    np.savez_compressed(path, **blob)
    print(path, os.path.getsize(path), "bytes")


def main():
    nblob = {}
    for idx, (name, (rows, C, eps)) in enumerate(NORM_CASES.items()):
        for key, arr in run_rmsnorm(rows, C, eps, 3000 + idx).items():
            nblob[f"{name}/{key}"] = arr
    npath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rmsnorm_golden.npz")
    np.savez_compressed(npath, **nblob)
    print(npath, os.path.getsize(npath), "bytes")
    rblob = {}
    for idx, (name, (B, T, H, D)) in enumerate(ROPE_CASES.items()):
        for key, arr in run_rope(B, T, H, D, 2000 + idx).items():
            rblob[f"{name}/{key}"] = arr
    rpath = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rope_golden.npz")
    np.savez_compressed(rpath, **rblob)
    print(rpath, os.path.getsize(rpath), "bytes")
    blob = {}
    for idx, (name, (B, H, T, D, causal)) in enumerate(CASES.items()):
        for key, arr in run(B, H, T, D, causal, 1000 + idx).items():
            blob[f"{name}/{key}"] = arr
        blob[f"{name}/causal"] = np.array(int(causal))
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(path, **blob)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    import sys
    if "--gpt-only" in sys.argv:        # leaves the other fixtures untouched
        main_gpt()
    else:
        main()
        main_gpt()
