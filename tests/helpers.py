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
    8*atol + 2 ulp of the reference value.  (With fewer than ~128 keys or query rows the sums are too
    short for that to hold in bf16: see assert_no_worse_than_eager.)"""
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


def eager_16bit(q, k, v, d_o, *, add, keep, ks, scale=None):
    """The eager composite evaluated the way the reference's scripts run it (perf_measurement_train.py:
    every operator in the tensors' own 16-bit dtype), with autograd: (o, dq, dk, dv) on the CPU.  It is the
    yardstick for how much error the 16-bit roundings of P, dS and the results cost by themselves."""
    q, k, v = (t.detach().cpu().clone().requires_grad_(True) for t in (q, k, v))
    dt = q.dtype
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    t = torch.matmul(q, k.transpose(-1, -2)) * sc
    if add is not None:
        t = t + add.to(dt)
    p = torch.softmax(t, -1)
    if keep is not None:
        p = p * (keep * ks).to(dt)
    o = torch.matmul(p, v)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), d_o.cpu())
    return o.detach(), dq, dk, dv


def assert_no_worse_than_eager(got, ref, eager, what: str, atol=ATOL):
    """For 16-bit cases in which rounding alone breaks the elementwise bar (bf16, short sums): the error
    against the fp32 composite may be at most twice that of the 16-bit eager composite (+ atol), in
    the maximum and in the mean."""
    got, ref, eager = (t.detach().float().cpu() for t in (got, ref, eager))
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    e_got, e_eager = (got - ref).abs(), (eager - ref).abs()
    assert e_got.max() <= 2.0 * e_eager.max() + atol, f"{what}: max err {e_got.max():.3e}, eager 16-bit {e_eager.max():.3e}"
    assert e_got.mean() <= 2.0 * e_eager.mean() + 0.1 * atol, f"{what}: mean err {e_got.mean():.3e}, eager 16-bit {e_eager.mean():.3e}"


def randn_like_config(B, H, S_q, S_k, D, dtype, seed, device):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S_q, D, generator=g).to(dtype)
    k = torch.randn(B, H, S_k, D, generator=g).to(dtype)
    v = torch.randn(B, H, S_k, D, generator=g).to(dtype)
    d_o = torch.randn(B, H, S_q, D, generator=g).to(dtype)
    lens = torch.randint(max(1, S_k // 2), S_k + 1, (B,), generator=g, dtype=torch.int32)
    return tuple(t.to(device) for t in (q, k, v, d_o, lens))
