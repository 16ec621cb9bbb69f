"""GPU parity of decode-time attention (a few query rows against a key / value cache) against the CPU oracle."""
import numpy as np
import pytest
import torch

from tests.helpers import TOL_F16, TOL_F32, assert_close

pytestmark = pytest.mark.gpu


def _case(B, H, Tq, Tk, D, dtype, seed, causal=True, scale=None):
    from deers_b200 import ops
    from oracle import ref
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, H, Tq, D)).astype(np.float32)
    k = rng.standard_normal((B, H, Tk, D)).astype(np.float32)
    v = rng.standard_normal((B, H, Tk, D)).astype(np.float32)
    if dtype == torch.float16:
        q, k, v = (a.astype(np.float16).astype(np.float32) for a in (q, k, v))
    want_o, want_lse = ref.attn_decode(q, k, v, scale, causal)
    tq, tk, tv = (torch.from_numpy(a).to("cuda", dtype) for a in (q, k, v))
    o, lse = ops.attention_decode(tq, tk, tv, scale, causal, want_lse=True)
    ops.Context.current(tq.device).sync()
    tol = TOL_F16 if dtype == torch.float16 else TOL_F32
    assert_close(o.float().cpu().numpy(), want_o, tol, f"o {B,H,Tq,Tk,D}")
    assert_close(lse.cpu().numpy(), want_lse, tol, f"lse {B,H,Tq,Tk,D}")


@pytest.mark.parametrize("shape", [
    (2, 3, 1, 1, 8),          # the very first token
    (2, 2, 1, 17, 2),         # the reference's GPT test head_dim
    (1, 6, 1, 256, 32),       # README GPT: one new token against the full context
    (2, 4, 1, 1000, 64),
    (1, 2, 5, 300, 128),      # a few rows at once (speculative / chunked prefill tail)
    (1, 1, 7, 7, 20),         # Tq == Tk: plain causal attention
    (1, 2, 3, 4099, 96),      # many splits, ragged last chunk
    (1, 1, 1, 33, 200),       # head_dim not a multiple of 32
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_shapes(shape, dtype):
    _case(*shape, dtype, seed=sum(shape))


def test_noncausal_scale_and_cache_views():
    from deers_b200 import ops
    from oracle import ref
    _case(1, 2, 4, 100, 32, torch.float32, 3, causal=False)
    _case(1, 2, 2, 100, 32, torch.float32, 4, scale=0.3)
    # the cache is allocated for 512 rows; only the first Tk are valid: a view is read in place
    B, H, Tmax, Tk, D = 2, 3, 512, 200, 64
    rng = np.random.default_rng(6)
    kc = rng.standard_normal((B, H, Tmax, D)).astype(np.float32)
    vc = rng.standard_normal((B, H, Tmax, D)).astype(np.float32)
    q = rng.standard_normal((B, H, 1, D)).astype(np.float32)
    tk, tv = torch.from_numpy(kc).cuda(), torch.from_numpy(vc).cuda()
    o = ops.attention_decode(torch.from_numpy(q).cuda(), tk[:, :, :Tk], tv[:, :, :Tk])
    want, _ = ref.attn_decode(q, kc[:, :, :Tk], vc[:, :, :Tk])
    assert_close(o.cpu().numpy(), want, TOL_F32, "cache view")


def test_step_by_step_decoding_equals_the_full_forward():
    # Size-independent property: feeding the rows one at a time against a growing cache reproduces the
    # fused causal forward over the whole sequence (the reference recomputes that forward for every token).
    from deers_b200 import ops
    B, H, T, D = 1, 4, 160, 64
    g = torch.Generator(device="cuda").manual_seed(12)
    q, k, v = (torch.randn(B, H, T, D, device="cuda", generator=g) for _ in range(3))
    full = ops.causal_attention(q, k, v)
    rows = [ops.attention_decode(q[:, :, t:t + 1], k[:, :, :t + 1], v[:, :, :t + 1]) for t in range(T)]
    ops.Context.current(q.device).sync()
    got = torch.cat(rows, dim=2)
    assert (got - full).abs().max().item() <= 1e-4 * full.abs().max().item()


def test_long_cache_f16():
    # 64 slices x 32768 cached rows x 128 (1 GB of K and V): sampled slices against the oracle.
    from deers_b200 import ops
    from oracle import ref
    B, H, Tk, D = 2, 32, 32768, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    k = torch.randn(B, H, Tk, D, device="cuda", generator=g).to(torch.float16)
    v = torch.randn(B, H, Tk, D, device="cuda", generator=g).to(torch.float16)
    q = torch.randn(B, H, 1, D, device="cuda", generator=g).to(torch.float16)
    o = ops.attention_decode(q, k, v)
    ops.Context.current(q.device).sync()
    for b, h in ((0, 0), (1, 31), (1, 7)):
        want, _ = ref.attn_decode(q[b:b + 1, h:h + 1].float().cpu().numpy(), k[b:b + 1, h:h + 1].float().cpu().numpy(),
                                  v[b:b + 1, h:h + 1].float().cpu().numpy())
        assert_close(o[b:b + 1, h:h + 1].float().cpu().numpy(), want, TOL_F16, f"slice {b},{h}")
