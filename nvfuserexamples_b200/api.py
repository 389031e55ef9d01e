"""Host-side mirror of the reference's operator interface, on top of the C ABI.

The three legacy functions have the names, argument order and meaning of the reference's
torch operators (shmsong/NvFuserExamples fmha/fmha_manual.cpp:1218-1238; called at
test.py:25 and test_train_mha.py:32-33).  They and the new functions go straight to
libfmha_sm100.so through ctypes — the same calls `torch.ops.mha_manual.*` makes from C++ —
and raise if the library is missing, the device is not a B200 or a call fails.
"""
from __future__ import annotations

from typing import Optional, Tuple

from . import capi


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("mha_manual operators need CUDA tensors: there is no CPU implementation")


def _dense(t, like, n):
    if t.dtype != like.dtype:
        raise TypeError("dense masks must have the dtype of q")
    if t.numel() != n:
        raise ValueError("dense masks must have B*H*S_q*S_k elements")
    return t.contiguous()


def fmha_nvfuser(input, qk, v, amask):
    """ctx = softmax(Q K^T / sqrt(D) + (1 - amask) * -10000) V   (fmha_manual.cpp:1218-1222).
    input/qk/v: [B*H, S, D] fp16 or bf16; amask: [B*H, S_q, S_k], 1 = keep."""
    _require_cuda(input, qk, v, amask)
    n = input.shape[0] * input.shape[1] * qk.shape[1]
    return capi.fwd(input, qk, v, mask_kind=capi.MASK_DENSE_KEEP, mask=_dense(amask, input, n), want_lse=False)["o"]


def fmha_train_nvfuser(input, qk, v, pad_mask, dropout_mask):
    """ctx = (softmax(Q K^T / sqrt(D) + pad_mask) * dropout_mask / 0.5) V   (fmha_manual.cpp:1224-1229)."""
    _require_cuda(input, qk, v, pad_mask, dropout_mask)
    n = input.shape[0] * input.shape[1] * qk.shape[1]
    return capi.fwd(input, qk, v, mask_kind=capi.MASK_DENSE_ADDITIVE, mask=_dense(pad_mask, input, n),
                    dropout_kind=capi.DROPOUT_DENSE, dropout_mask=_dense(dropout_mask, input, n), dropout_scale=2.0,
                    want_lse=False)["o"]


def fmha_train_saveim_nvfuser(input, qk, v, pad_mask, dropout_mask):
    """[ctx, softmax, softmax * dropout_mask / 0.5]   (fmha_manual.cpp:1231-1238)."""
    _require_cuda(input, qk, v, pad_mask, dropout_mask)
    n = input.shape[0] * input.shape[1] * qk.shape[1]
    r = capi.fwd(input, qk, v, mask_kind=capi.MASK_DENSE_ADDITIVE, mask=_dense(pad_mask, input, n),
                 dropout_kind=capi.DROPOUT_DENSE, dropout_mask=_dense(dropout_mask, input, n), dropout_scale=2.0,
                 want_lse=False, save_softmax=True, save_dropout=True)
    return [r["o"], r["softmax"], r["dropout_out"]]


def _mask_args(mask, seqlens, B, S_k):
    import torch
    if mask is not None and seqlens is not None:
        raise ValueError("give either mask or seqlens, not both")
    if mask is not None:
        if mask.numel() != B * S_k:
            raise ValueError("mask must be an additive [B,S_k] (or [B,1,1,S_k]) tensor")
        return capi.MASK_KEY_ADDITIVE, mask.reshape(B, S_k).to(torch.float32).contiguous()
    if seqlens is not None:
        if seqlens.numel() != B:
            raise ValueError("seqlens must be [B]")
        return capi.MASK_SEQLEN, seqlens.reshape(B).to(torch.int32).contiguous()
    return capi.MASK_NONE, None


def fmha_forward(q, k, v, *, mask=None, seqlens=None, p_drop: float = 0.0, seed: int = 0, offset: int = 0,
                 scale: Optional[float] = None, bh_offset: int = 0, out=None, status=None) -> Tuple[object, object]:
    """O, LSE = attention(q, k, v) with a compact padding mask (additive float [B,S_k]) or valid
    key lengths (int [B]) and Philox dropout keyed by (seed, offset).  q/k/v: [B,H,S,D]."""
    _require_cuda(q, k, v, mask, seqlens)
    kind, m = _mask_args(mask, seqlens, q.shape[0], k.shape[-2])
    r = capi.fwd(q, k, v, mask_kind=kind, mask=m, dropout_kind=capi.DROPOUT_PHILOX if p_drop > 0 else capi.DROPOUT_NONE,
                 p_drop=p_drop, seed=seed, offset=offset, bh_offset=bh_offset, scale=scale, out=out, status=status)
    return r["o"], r["lse"]


def fmha_backward(d_o, q, k, v, o, lse, *, mask=None, seqlens=None, p_drop: float = 0.0, seed: int = 0, offset: int = 0,
                  scale: Optional[float] = None, bh_offset: int = 0, workspace=None, status=None, out=None):
    """dQ, dK, dV of fmha_forward; the probabilities are recomputed from `lse`.  `out` = (dq, dk, dv) tensors to
    write into, e.g. three views of one [B,S,3,H,D] gradient buffer of a fused QKV projection."""
    _require_cuda(d_o, q, k, v, o, lse, mask, seqlens)
    if out is not None:
        _require_cuda(*out)
    kind, m = _mask_args(mask, seqlens, q.shape[0], k.shape[-2])
    return capi.bwd(d_o, q, k, v, o, lse, mask_kind=kind, mask=m, p_drop=p_drop, seed=seed, offset=offset,
                    bh_offset=bh_offset, scale=scale, workspace=workspace, status=status, out=out)


def philox_dropout_mask(B: int, H: int, S_q: int, S_k: int, p: float, seed: int, offset: int, bh_offset: int = 0,
                        device=None):
    """Dense keep mask [B,H,S_q,S_k] (uint8) the kernels apply for (seed, offset): generated by
    the library on the host (device=None, returns a numpy array) or on a CUDA device."""
    if device is None:
        return capi.philox_mask_host(seed, offset, bh_offset, B * H, S_q, S_k, p).reshape(B, H, S_q, S_k)
    return capi.philox_mask_device(seed, offset, bh_offset, B * H, S_q, S_k, p, device).view(B, H, S_q, S_k)
