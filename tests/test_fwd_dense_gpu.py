"""The persistent forward kernel of the reference's dense-mask operators (fmha_nvfuser, fmha_train_nvfuser:
fmha/fmha_manual.cpp:1218-1229 of shmsong/NvFuserExamples) against the fp32 composite of the oracle
(test.py:12-18 and test_train_mha.py:14-21 restated) and against the general kernel, which the flag
FLAG_P_VIA_SMEM selects for the same call.

Shapes: one item per CTA and several (more items than SMs, so that every buffer ring wraps), one key step and
several, ragged query tiles and ragged last key steps, fp16 and bf16, keep and additive masks, with and without
the dense dropout mask."""
import pytest
import torch

from nvfuserexamples_b200 import capi
from oracle import composite
from tests import helpers

pytestmark = pytest.mark.gpu

SHAPES = [          # (B*H, S_q, S_k)
    (4, 128, 128),     # one item per CTA, one key step: the reference's tile
    (3, 200, 136),     # ragged second query tile, 8 keys in the second step
    (5, 77, 384),      # three key steps
    (1, 1, 8),         # a single query row
    (300, 130, 264),   # 600 items over 148 CTAs, three steps each, ragged in both directions
    (700, 128, 128),   # 700 items: every ring wraps several times
]


def _inputs(bh, sq, sk, dt, dev):
    g = torch.Generator(device=dev).manual_seed(bh * 7 + sq + sk)
    q = torch.randn(1, bh, sq, 64, device=dev, generator=g).to(dt)
    k = torch.randn(1, bh, sk, 64, device=dev, generator=g).to(dt)
    v = torch.randn(1, bh, sk, 64, device=dev, generator=g).to(dt)
    am = torch.empty(bh, sq, sk, device=dev).random_(2, generator=g).to(dt)
    dm = torch.empty(bh, sq, sk, device=dev).random_(2, generator=g).to(dt)
    return q, k, v, am, dm


def _run(q, k, v, am, dm, keep, drop, general, save=False):
    mask = am if keep else ((1 - am) * -1000).to(am.dtype)
    kw = dict(mask_kind=capi.MASK_DENSE_KEEP if keep else capi.MASK_DENSE_ADDITIVE, mask=mask, scale=0.125)
    if drop:
        kw.update(dropout_kind=capi.DROPOUT_DENSE, dropout_mask=dm, dropout_scale=2.0)
    if save:
        kw.update(save_softmax=True, save_dropout=True)
    if general:
        kw["flags"] = capi.FLAG_P_VIA_SMEM
    st = torch.zeros(4, dtype=torch.int32, device=q.device)
    res = capi.fwd(q, k, v, status=st, **kw)
    capi.check_status(st)
    return res, (1.0 - am.float()) * -10000.0 if keep else mask.float()


@pytest.mark.parametrize("bh,sq,sk", SHAPES)
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_dense_kernel_matches_composite_and_general_kernel(cuda_device, bh, sq, sk, dt):
    q, k, v, am, dm = _inputs(bh, sq, sk, dt, cuda_device)
    for keep in (True, False):
        for drop in (False, True):
            res, add = _run(q, k, v, am, dm, keep, drop, general=False)
            gen, _ = _run(q, k, v, am, dm, keep, drop, general=True)
            ref = composite.attention_fp32(q[0], k[0], v[0], add_mask=add, keep=dm.float() if drop else None, keep_scale=2.0,
                                           scale=0.125)
            what = f"bh={bh} sq={sq} sk={sk} {dt} keep={keep} drop={drop}"
            o, og = res["o"][0].float(), gen["o"][0].float()
            # logsumexp: natural log, fp32; the two kernels differ by summation order only
            lse = res["lse"].reshape(bh, sq)
            assert torch.allclose(lse, ref["lse"], atol=1e-3, rtol=1e-4), what
            assert (lse - gen["lse"].reshape(bh, sq)).abs().max().item() < 1e-4, what
            # O: inside the parity bar where the sums are long enough for it (see helpers.assert_close), and in every
            # case no further from the fp32 composite than the general kernel is (both round P once to 16 bits)
            e_dense = (o - ref["o"]).abs().max().item()
            e_general = (og - ref["o"]).abs().max().item()
            assert e_dense <= max(1.5 * e_general, 1e-3), f"{what}: {e_dense:.3e} against {e_general:.3e}"
            if not drop and sk >= 128 and sq >= 128:
                helpers.assert_close(res["o"][0], ref["o"], what, dt)


def test_masks_that_tma_cannot_address_fall_back_to_the_general_kernel(cuda_device):
    """Mask rows that are no multiple of 16 bytes (S_k = 51) cannot be staged by TMA: same results through the
    general kernel, which reads them with plain loads."""
    q, k, v, am, dm = _inputs(6, 140, 51, torch.float16, cuda_device)
    for drop in (False, True):
        res, add = _run(q, k, v, am, dm, True, drop, general=False)
        gen, _ = _run(q, k, v, am, dm, True, drop, general=True)
        assert torch.equal(res["o"], gen["o"]) and torch.equal(res["lse"], gen["lse"])


def test_reference_shape_many_calls_are_deterministic(cuda_device):
    """B*H = 512, S = 128, D = 64 (test.py:22-25): repeated calls give bit-identical results (no dependence on the
    timing of the loads, the tensor core or the store warp)."""
    q, k, v, am, dm = _inputs(512, 128, 128, torch.float16, cuda_device)
    first, _ = _run(q, k, v, am, dm, False, True, general=False)
    for _ in range(10):
        again, _ = _run(q, k, v, am, dm, False, True, general=False)
        assert torch.equal(first["o"], again["o"]) and torch.equal(first["lse"], again["lse"])


@pytest.mark.parametrize("bh,sq,sk", [(4, 128, 128), (700, 128, 128), (3, 200, 120), (5, 77, 64), (150, 300, 128)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_save_intermediates_mode(cuda_device, bh, sq, sk, dt):
    """`fmha_train_saveim_nvfuser` (fmha/fmha_manual.cpp:1231-1238) with one key step: the softmax and dropout tensors
    and the context computed from the ROUNDED dropout tensor (:891-897), against the fp32 composite and the general
    kernel, on shapes whose last query tile and only key step are ragged (the tile stores are clipped per head)."""
    q, k, v, am, dm = _inputs(bh, sq, sk, dt, cuda_device)
    res, add = _run(q, k, v, am, dm, False, True, general=False, save=True)
    gen, _ = _run(q, k, v, am, dm, False, True, general=True, save=True)
    ref = composite.attention_fp32(q[0], k[0], v[0], add_mask=add, keep=dm.float(), keep_scale=2.0, scale=0.125)
    what = f"save bh={bh} sq={sq} sk={sk} {dt}"
    ulp = 2.0 ** -10 if dt == torch.float16 else 2.0 ** -7   # one rounding of values up to 1 (softmax) or 2 (dropout)
    for name, key, top in (("softmax", "softmax", 1.0), ("dropout_out", "dropout_out", 2.0)):
        got, want = res[name].float(), ref[key]
        assert got.shape == want.shape, what
        assert (got - want).abs().max().item() <= 1.5 * top * ulp + 1e-5, f"{what}: {name}"
        assert (got - gen[name].float()).abs().max().item() <= 2 * top * ulp, f"{what}: {name} against the general kernel"
    lse = res["lse"].reshape(bh, sq)
    assert torch.allclose(lse, ref["lse"], atol=1e-3, rtol=1e-4), what
    # the context: the second GEMM consumed the rounded dropout tensor, so compare with that product in fp32
    o_from_saved = torch.matmul(res["dropout_out"].float(), v[0].float())
    assert (res["o"][0].float() - o_from_saved).abs().max().item() <= (4e-3 if dt == torch.float16 else 3e-2), what
    e_dense = (res["o"][0].float() - ref["o"]).abs().max().item()
    e_general = (gen["o"][0].float() - ref["o"]).abs().max().item()
    assert e_dense <= max(1.5 * e_general, 1e-3), f"{what}: {e_dense:.3e} against {e_general:.3e}"
