"""CPU tests of the oracle: pinned against the reference's own composites (golden files
produced by tests/golden/make_golden.py) and against PyTorch's Philox engine."""
import ctypes as C
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import composite, philox
from tests.golden import make_golden

GOLD = Path(__file__).resolve().parent / "golden"
ROOT = GOLD.parent.parent


def test_inference_composite_matches_reference_output():
    g = np.load(GOLD / "ref_inference.npz")
    bh, s, d = (int(x) for x in g["shape"])
    q, k, v, amask = make_golden.inference_inputs(int(g["seed"]), bh, s, d)
    np.testing.assert_array_equal(make_golden.checksum(q, k, v, amask), g["input_checksum"])
    ctx = composite.reference_mha_inference(q, k, v, amask)
    assert ctx.dtype == torch.half
    np.testing.assert_array_equal(ctx.numpy(), g["ctx"])  # bit exact


def test_train_composite_matches_reference_output():
    g = np.load(GOLD / "ref_train.npz")
    bh, s, d = (int(x) for x in g["shape"])
    q, k, v, pad, dm = make_golden.train_inputs(int(g["seed"]), bh, s, d)
    np.testing.assert_array_equal(make_golden.checksum(q, k, v, pad, dm), g["input_checksum"])
    sm, dr, ctx = composite.reference_mha_train(q, k, v, pad, dm)
    np.testing.assert_array_equal(sm.numpy(), g["softmax"])
    np.testing.assert_array_equal(dr.numpy(), g["dropout_out"])
    np.testing.assert_array_equal(ctx.numpy(), g["ctx"])


def test_general_composite_reduces_to_reference_forms():
    g = np.load(GOLD / "ref_inference.npz")
    bh, s, d = (int(x) for x in g["shape"])
    q, k, v, amask = make_golden.inference_inputs(int(g["seed"]), bh, s, d)
    add = (1.0 - amask.float()) * -10000.0
    o = composite.attention_fp32(q, k, v, add_mask=add, scale=1.0 / 8)["o"]
    ref = torch.from_numpy(g["ctx"]).float()
    assert (o - ref).abs().max().item() < 2e-3  # only the final rounding to half differs


def test_numpy_restatement_agrees_with_torch_composite():
    x = composite.make_inputs(2, 2, 96, 64, torch.float32, (40, 96), seed=3)
    add = composite.padding_add_mask(x["lens"], 96)
    t = composite.attention_fp32(x["q"], x["k"], x["v"], add_mask=add)
    n = composite.attention_numpy(x["q"].numpy(), x["k"].numpy(), x["v"].numpy(), add_mask=add.numpy())
    np.testing.assert_allclose(t["o"].numpy(), n["o"], atol=2e-5)
    np.testing.assert_allclose(t["lse"].numpy(), n["lse"], atol=2e-4, rtol=1e-5)


def test_analytic_cases():
    torch.manual_seed(0)
    q = torch.randn(1, 1, 5, 64)
    v = torch.randn(1, 1, 7, 64)
    k = torch.randn(1, 1, 7, 64)
    # a single key: every output row is that key's value row
    o1 = composite.attention_fp32(q, k[:, :, :1], v[:, :, :1])["o"]
    np.testing.assert_allclose(o1.numpy(), v[:, :, :1].expand(1, 1, 5, 64).numpy(), atol=1e-6)
    # equal scores: the mean of the values
    o2 = composite.attention_fp32(torch.zeros_like(q), k, v)["o"]
    np.testing.assert_allclose(o2.numpy(), v.mean(2, keepdim=True).expand(1, 1, 5, 64).numpy(), atol=1e-6)
    # a fully masked row under the additive mask: the shift cancels (test.py:15 semantics)
    add = torch.full((1, 1, 1, 7), -10000.0)
    o3 = composite.attention_fp32(q, k, v, add_mask=add)["o"]
    o4 = composite.attention_fp32(q, k, v)["o"]
    np.testing.assert_allclose(o3.numpy(), o4.numpy(), atol=5e-3)


def test_autograd_oracle_matches_finite_differences():
    torch.manual_seed(1)
    q, k, v, d_o = (torch.randn(1, 1, 6, 64, dtype=torch.float64) for _ in range(4))
    dq, dk, dv = composite.attention_grads_fp32(q, k, v, d_o)
    eps = 1e-3
    f = lambda qq: (composite.attention_fp32(qq, k.float(), v.float())["o"].double() * d_o).sum().item()
    qe = q.float().clone()
    qe[0, 0, 2, 5] += eps
    qm = q.float().clone()
    qm[0, 0, 2, 5] -= eps
    fd = (f(qe) - f(qm)) / (2 * eps)
    assert abs(fd - dq[0, 0, 2, 5].item()) < 5e-2 * max(1.0, abs(fd))


# ---- Philox --------------------------------------------------------------------------------

def test_philox_numpy_matches_pytorch_engine_vectors():
    kat = np.load(GOLD / "philox_kat.npz")
    for seed, ctr, words in zip(kat["seeds"], kat["counters"], kat["words"]):
        seed = int(seed)
        w = philox.philox4x32_10(seed & 0xFFFFFFFF, seed >> 32, *[int(c) for c in ctr])
        assert [int(x) for x in w] == [int(x) for x in words]


def _c_lib():
    return C.CDLL(str(ROOT / "oracle" / "_build" / "libphilox_ref.so"))


def test_philox_c_matches_pytorch_engine_vectors():
    lib = _c_lib()
    kat = np.load(GOLD / "philox_kat.npz")
    out = (C.c_uint32 * 4)()
    for seed, ctr, words in zip(kat["seeds"], kat["counters"], kat["words"]):
        seed = int(seed)
        c = (C.c_uint32 * 4)(*[int(x) for x in ctr])
        lib.philox4x32_10_c(C.c_uint32(seed & 0xFFFFFFFF), C.c_uint32(seed >> 32), c, out)
        assert list(out) == [int(x) for x in words]


@pytest.mark.parametrize("p", [0.0, 0.1, 0.25, 0.5, 0.9])
def test_keep_mask_three_implementations_agree(p):
    from nvfuserexamples_b200 import capi
    seed, offset, bh0, n_bh, sq, sk = 0x5EED0001_0000_0042, 7, 5, 3, 37, 70
    a = philox.dropout_keep_mask(seed, offset, bh0, n_bh, sq, sk, p)
    lib = _c_lib()
    b = np.empty((n_bh, sq, sk), dtype=np.uint8)
    lib.dropout_keep_mask_c(C.c_uint64(seed), C.c_uint32(offset), C.c_int32(bh0), C.c_int32(n_bh), C.c_int32(sq),
                            C.c_int32(sk), C.c_float(p), b.ctypes.data_as(C.c_void_p))
    c = capi.philox_mask_host(seed, offset, bh0, n_bh, sq, sk, p)  # the product library's host generator
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(a, c)
    thr = philox.dropout_threshold(p)
    assert thr == capi.dropout_threshold(p) == lib.dropout_threshold_c(C.c_float(p))
    assert abs(a.mean() - (1 - thr / 128)) < 0.03


def test_keep_mask_sharding_invariance():
    full = philox.dropout_keep_mask(9, 1, 0, 8, 16, 48, 0.3)
    part = philox.dropout_keep_mask(9, 1, 3, 2, 16, 48, 0.3)
    np.testing.assert_array_equal(full[3:5], part)
    other = philox.dropout_keep_mask(9, 2, 0, 8, 16, 48, 0.3)
    assert (full != other).mean() > 0.2  # a different offset is a different stream
