"""Shared helpers of the parity tests: tolerances and oracle-side reference values."""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import composite, philox

# Parity bar for fp16 results against the fp32 composite on the same inputs.
ATOL, RTOL = 1e-3, 2e-3


def assert_close(got: torch.Tensor, ref: torch.Tensor, what: str, dtype=torch.float16, atol=ATOL, rtol=RTOL):
    """fp16: every element within atol + rtol*|ref|.
    bf16: one ulp (2^-8 relative) is coarser than rtol, so the roundings of P, dS and of the result
    alone can exceed the bar; require 99.5 % of the elements inside it and none further than
    8*atol + 2 ulp of the reference value."""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    tol = atol + rtol * ref.abs()
    if dtype == torch.bfloat16:
        inside = (err <= tol).float().mean().item()
        assert inside >= 0.995, f"{what}: only {inside:.5f} of elements within tolerance"
        hard = 8.0 * atol + 2.0 * ref.abs() * 2.0 ** -8
        assert (err <= hard).all(), f"{what}: max abs err {err.max().item():.3e} beyond 2 ulp"
    else:
        bad = err > tol
        assert not bad.any(), (f"{what}: {int(bad.sum())} elements out of tolerance, max abs err "
                               f"{err.max().item():.3e} at ref {ref.flatten()[err.argmax()].item():.3e}")


def keep_mask(seed, offset, bh_offset, B, H, S_q, S_k, p):
    m = philox.dropout_keep_mask(seed, offset, bh_offset, B * H, S_q, S_k, p)
    return torch.from_numpy(m.reshape(B, H, S_q, S_k).astype(np.float32))


def oracle_forward(q, k, v, *, lens=None, add_mask=None, p_drop=0.0, seed=0, offset=0, bh_offset=0, scale=None):
    """CPU oracle on CPU copies of the inputs. Returns dict(o, lse, ...) float32."""
    q, k, v = q.cpu(), k.cpu(), v.cpu()
    B, H, S_q, _ = q.shape
    S_k = k.shape[2]
    add = None
    if lens is not None:
        eff = torch.where(lens.cpu() <= 0, torch.full_like(lens.cpu(), S_k), lens.cpu())
        add = composite.padding_add_mask(eff, S_k)
    if add_mask is not None:
        add = add_mask.cpu().reshape(B, 1, 1, S_k)
    keep, ks = None, 1.0
    if p_drop > 0:
        keep = keep_mask(seed, offset, bh_offset, B, H, S_q, S_k, p_drop)
        ks = philox.keep_scale(p_drop)
    return composite.attention_fp32(q, k, v, add_mask=add, keep=keep, keep_scale=ks, scale=scale), add, keep, ks


def oracle_backward(q, k, v, d_o, *, add, keep, ks, scale=None):
    return composite.attention_grads_fp32(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), add_mask=add, keep=keep, keep_scale=ks,
                                          scale=scale)


def randn_like_config(B, H, S_q, S_k, D, dtype, seed, device):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S_q, D, generator=g).to(dtype)
    k = torch.randn(B, H, S_k, D, generator=g).to(dtype)
    v = torch.randn(B, H, S_k, D, generator=g).to(dtype)
    d_o = torch.randn(B, H, S_q, D, generator=g).to(dtype)
    lens = torch.randint(max(1, S_k // 2), S_k + 1, (B,), generator=g, dtype=torch.int32)
    return tuple(t.to(device) for t in (q, k, v, d_o, lens))
