"""CPU oracle for the fused attention path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py may
import this module; the library under nvfuserexamples_b200/ never does.

It restates, operation by operation, the eager composites the reference checks its fused
kernels against (paths inside shmsong/NvFuserExamples):

  * inference form  test.py:12-18           fp32 math on fp16 inputs, keep-mask converted as
                                             (1 - amask) * -10000, scale 1/8, output cast to half
  * train form      test_train_mha.py:14-21  native-dtype math, additive pad mask, explicit 0/1
                                             dropout mask, division by dropout_prob (0.5)

and generalises them to [B,H,S,D], a compact padding mask and Philox dropout, which is what
the new entry points compute.  Backward values come from torch.autograd through the fp32
composite (the reference has no backward pass, README.md:1).

Pinned against the reference: tests/golden/make_golden.py executes the reference's own
`reference_mha` functions (source read from the reference checkout) and stores their
outputs; tests/test_oracle.py checks this module against those files bit for bit.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

# ----------------------------------------------------------------------------------------
# the two reference composites, restated
# ----------------------------------------------------------------------------------------

def reference_mha_inference(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, amask: torch.Tensor) -> torch.Tensor:
    """test.py:12-18.  q,k,v [BH,S,D]; amask [BH,S_q,S_k] with 1 = keep, 0 = masked."""
    p = q.to(torch.float).matmul(k.permute((0, 2, 1)).to(torch.float))          # test.py:13
    p_masked = p / 8 + (1.0 - amask.to(torch.float)) * -10000.0                   # test.py:15
    s = torch.softmax(p_masked, -1)                                               # test.py:16
    ctx = torch.matmul(s, v.to(torch.float)).to(torch.half)                       # test.py:17
    return ctx


def reference_mha_train(q, k, v, pad_mask, dropout_mask, dropout_prob: float = 0.5, scale: float = 1.0 / 8):
    """test_train_mha.py:14-21.  Returns (softmax, dropout_out, ctx), all in the input dtype."""
    out1 = q.matmul(k.permute((0, 2, 1)))                                         # :15
    out2 = out1 * scale                                                           # :16
    out3 = out2 + pad_mask                                                        # :17
    out4 = torch.softmax(out3, -1)                                                # :18
    out5 = (out4 / dropout_prob) * dropout_mask                                   # :19
    out6 = torch.matmul(out5, v)                                                  # :20
    return out4, out5, out6


# ----------------------------------------------------------------------------------------
# generalised fp32 composite (the comparison target of the parity tests)
# ----------------------------------------------------------------------------------------

def attention_fp32(q, k, v, *, add_mask: Optional[torch.Tensor] = None, keep: Optional[torch.Tensor] = None,
                   keep_scale: float = 1.0, scale: Optional[float] = None):
    """fp32 composite on low-precision inputs (the test.py:13-17 recipe: upcast, compute, no
    intermediate rounding).  q [.., S_q, D], k/v [.., S_k, D]; add_mask broadcastable to
    [.., S_q, S_k]; keep is a 0/1 tensor of that shape, kept entries are multiplied by keep_scale.
    Returns dict(scores, softmax, dropout_out, o, lse), all float32."""
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scores = torch.matmul(qf, kf.transpose(-1, -2))
    t = scores * scale
    if add_mask is not None:
        t = t + add_mask.to(torch.float32)
    lse = torch.logsumexp(t, -1)
    sm = torch.softmax(t, -1)
    dr = sm if keep is None else sm * (keep.to(torch.float32) * keep_scale)
    o = torch.matmul(dr, vf)
    return dict(scores=scores, softmax=sm, dropout_out=dr, o=o, lse=lse)


def attention_grads_fp32(q, k, v, d_o, **kw) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dQ, dK, dV of attention_fp32(...)['o'] contracted with d_o, by autograd in fp32."""
    qf = q.detach().to(torch.float32).requires_grad_(True)
    kf = k.detach().to(torch.float32).requires_grad_(True)
    vf = v.detach().to(torch.float32).requires_grad_(True)
    o = attention_fp32(qf, kf, vf, **kw)["o"]
    dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), d_o.to(torch.float32))
    return dq, dk, dv


def padding_add_mask(lens: torch.Tensor, S_k: int, value: float = -10000.0) -> torch.Tensor:
    """[B] valid lengths -> additive [B,1,1,S_k] mask: 0 for j < len, `value` otherwise."""
    j = torch.arange(S_k, device=lens.device).view(1, 1, 1, S_k)
    return torch.where(j < lens.view(-1, 1, 1, 1), 0.0, value).to(torch.float32)


# ----------------------------------------------------------------------------------------
# numpy restatement of the forward (independent of torch kernels; small sizes)
# ----------------------------------------------------------------------------------------

def attention_numpy(q: np.ndarray, k: np.ndarray, v: np.ndarray, add_mask=None, keep=None, keep_scale=1.0, scale=None):
    q64, k64, v64 = q.astype(np.float64), k.astype(np.float64), v.astype(np.float64)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    t = np.matmul(q64, np.swapaxes(k64, -1, -2)) * scale
    if add_mask is not None:
        t = t + add_mask
    m = t.max(-1, keepdims=True)
    e = np.exp(t - m)
    l = e.sum(-1, keepdims=True)
    sm = e / l
    if keep is not None:
        sm_d = sm * keep * keep_scale
    else:
        sm_d = sm
    return dict(o=np.matmul(sm_d, v64), lse=(m + np.log(l))[..., 0], softmax=sm)


# ----------------------------------------------------------------------------------------
# synthetic inputs of the benchmark configurations: the recipe (shapes, seeds, generators) lives with the
# library's workload definitions, which know nothing of this oracle; re-exported here for the tests
# ----------------------------------------------------------------------------------------
from nvfuserexamples_b200.workloads import CONFIG_SEEDS, CONFIGS, PHILOX_SEEDS, make_inputs  # noqa: E402,F401
