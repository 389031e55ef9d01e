"""The allocation-free backward entry point (fmha_sm100_bwd_static_scratch), through the C ABI.

It exists for hosts that cannot allocate device memory when they call: the scratch comes from an
array inside the library image.  This file is collected last on purpose, so that a run that stops
at the first failure has already run every other test; the test must pass both alone in a fresh
process and after the rest of the suite (the array is shared by all calls and keeps old contents).
"""
import ctypes as C

import pytest
import torch

from nvfuserexamples_b200 import capi
from tests import helpers


def _case(dev, B, H, S_q, S_k, D, dtype, p_drop, seed):
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S_q, S_k, D, dtype, seed=seed, device=dev)
    kw = dict(mask_kind=capi.MASK_SEQLEN, mask=lens, p_drop=p_drop, seed=31, offset=seed)
    fwd = capi.fwd(q, k, v, mask_kind=capi.MASK_SEQLEN, mask=lens, p_drop=p_drop, seed=31, offset=seed,
                   dropout_kind=capi.DROPOUT_PHILOX if p_drop > 0 else capi.DROPOUT_NONE)
    return (d_o, q, k, v, fwd["o"], fwd["lse"]), kw


@pytest.mark.gpu
def test_static_scratch_backward_matches_workspace_backward_twice(cuda_device):
    """Two calls in a row with different sizes: the second must not see what the first left."""
    cases = [(2, 2, 384, 256, 64, torch.float16, 0.1, 5), (1, 3, 200, 333, 128, torch.bfloat16, 0.0, 6)]
    for B, H, S_q, S_k, D, dtype, p_drop, seed in cases:
        args, kw = _case(cuda_device, B, H, S_q, S_k, D, dtype, p_drop, seed)
        ref = capi.bwd(*args, **kw)                       # existing entry point, caller workspace
        got = capi.bwd_static_scratch(*args, **kw)        # new entry point, built-in scratch
        torch.cuda.synchronize(cuda_device)
        # dK and dV have a fixed summation order: identical.  dQ is accumulated with atomics, whose
        # order varies between any two launches: same tolerance as the parity tests.
        assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
        helpers.assert_close(got[0], ref[0].float(), "dq", dtype)
        # ... and against the CPU oracle directly, at the parity tests' tolerance
        d_o, q, k, v = args[:4]
        oref, add, keep, ks = helpers.oracle_forward(q, k, v, lens=kw["mask"], p_drop=p_drop, seed=31, offset=seed)
        rdq, rdk, rdv = helpers.oracle_backward(q, k, v, d_o, add=add, keep=keep, ks=ks)
        for name, g, r in (("dq", got[0], rdq), ("dk", got[1], rdk), ("dv", got[2], rdv)):
            if dtype == torch.bfloat16 and min(S_q, S_k) < 256:   # short bf16 sums: the 16-bit eager composite is the yardstick
                eager = dict(zip(("o", "dq", "dk", "dv"), helpers.eager_16bit(q, k, v, d_o, add=add, keep=keep, ks=ks)))
                helpers.assert_no_worse_than_eager(g, r, eager[name], name)
            else:
                helpers.assert_close(g, r, name, dtype)


def test_static_scratch_rejects_sizes_beyond_the_array():
    lib = capi.load()
    p = capi.BwdParams()
    p.struct_bytes = C.sizeof(capi.BwdParams)
    p.dtype, p.B, p.H, p.S_q, p.S_k, p.D, p.scale = capi.DTYPE_F16, 32, 16, 512, 512, 64, 0.125
    assert capi.bwd_workspace_bytes(p) > capi.STATIC_SCRATCH_BYTES
    assert lib.fmha_sm100_bwd_static_scratch(C.byref(p), None) == capi.FMHA_ERR_TOO_LARGE


def test_static_scratch_validates_without_a_gpu():
    lib = capi.load()
    assert lib.fmha_sm100_bwd_static_scratch(None, None) == capi.FMHA_ERR_BAD_ARG
    p = capi.BwdParams()
    p.struct_bytes = 12
    assert lib.fmha_sm100_bwd_static_scratch(C.byref(p), None) == capi.FMHA_ERR_BAD_ARG
