"""Backward parity on the GPU against autograd through the fp32 composite (the reference has
no backward pass), through the C ABI."""
import pytest
import torch

from nvfuserexamples_b200 import api, capi, sharding
from oracle import composite
from tests import helpers

pytestmark = pytest.mark.gpu

SHAPES = [
    (2, 2, 128, 128, 64, torch.float16),
    (1, 2, 384, 256, 64, torch.float16),
    (2, 2, 512, 512, 64, torch.float16),     # BERT-large training sequence length
    (2, 2, 200, 333, 64, torch.float16),
    (1, 2, 256, 256, 128, torch.float16),
    (1, 2, 77, 300, 128, torch.bfloat16),
    (2, 2, 384, 384, 64, torch.bfloat16),
]


def _run(dev, B, H, S_q, S_k, D, dtype, mask, p_drop, seed=1):
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S_q, S_k, D, dtype, seed=seed, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    kw, okw = {}, {}
    if mask == "seqlen":
        kw["seqlens"], okw["lens"] = lens, lens
    elif mask == "key":
        add = composite.padding_add_mask(lens.cpu(), S_k).reshape(B, S_k).to(dev)
        kw["mask"], okw["add_mask"] = add, add
    o, lse = api.fmha_forward(q, k, v, p_drop=p_drop, seed=77, offset=2, status=status, **kw)
    dq, dk, dv = api.fmha_backward(d_o, q, k, v, o, lse, p_drop=p_drop, seed=77, offset=2, status=status, **kw)
    assert capi.check_status(status) == [0, 0, 0, 0]
    ref, add, keep, ks = helpers.oracle_forward(q, k, v, p_drop=p_drop, seed=77, offset=2, **okw)
    rdq, rdk, rdv = helpers.oracle_backward(q, k, v, d_o, add=add, keep=keep, ks=ks)
    if dtype == torch.bfloat16 and min(S_q, S_k) < 128:
        # sums too short for bf16's operand roundings to average out: measure against the 16-bit eager composite
        eo, edq, edk, edv = helpers.eager_16bit(q, k, v, d_o, add=add, keep=keep, ks=ks)
        for got, want, eager, name in ((o, ref["o"], eo, "o"), (dq, rdq, edq, "dq"), (dk, rdk, edk, "dk"), (dv, rdv, edv, "dv")):
            helpers.assert_no_worse_than_eager(got, want, eager, name)
        return
    helpers.assert_close(o, ref["o"], "o", dtype)
    helpers.assert_close(dq, rdq, "dq", dtype)
    helpers.assert_close(dk, rdk, "dk", dtype)
    helpers.assert_close(dv, rdv, "dv", dtype)


@pytest.mark.parametrize("B,H,S_q,S_k,D,dtype", SHAPES)
@pytest.mark.parametrize("mask", ["none", "seqlen", "key"])
def test_backward_matches_autograd_oracle(cuda_device, B, H, S_q, S_k, D, dtype, mask):
    _run(cuda_device, B, H, S_q, S_k, D, dtype, mask, 0.0)


@pytest.mark.parametrize("D,dtype,p", [(64, torch.float16, 0.1), (128, torch.bfloat16, 0.25), (64, torch.float16, 0.5)])
def test_backward_with_philox_dropout(cuda_device, D, dtype, p):
    _run(cuda_device, 2, 2, 384, 384, D, dtype, "seqlen", p)


def test_more_work_items_than_sms_spot_checked_against_the_oracle(cuda_device):
    """The persistent kernel draws (key tile, head, batch) items from a counter: with 16*16*4 = 1024 items every
    CTA processes several, including items whose key tile is wholly masked.  Three heads are checked against the
    oracle evaluated on those heads alone (the Philox counter uses the global head index)."""
    B, H, S, D, p = 16, 16, 512, 64, 0.1
    q, k, v, d_o, _ = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=31, device=cuda_device)
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(100, S + 1, (B,), generator=g, dtype=torch.int32).to(cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=9, offset=4, status=status)
    dq, dk, dv = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=9, offset=4, status=status)
    assert capi.check_status(status) == [0, 0, 0, 0]
    for b, h in ((0, 0), (7, 9), (15, 15)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        ref, add, keep, ks = helpers.oracle_forward(q[sl], k[sl], v[sl], lens=lens[b:b + 1], p_drop=p, seed=9, offset=4,
                                                    bh_offset=b * H + h)
        rdq, rdk, rdv = helpers.oracle_backward(q[sl], k[sl], v[sl], d_o[sl], add=add, keep=keep, ks=ks)
        helpers.assert_close(o[sl], ref["o"], f"o[{b},{h}]")
        helpers.assert_close(dq[sl], rdq, f"dq[{b},{h}]")
        helpers.assert_close(dk[sl], rdk, f"dk[{b},{h}]")
        helpers.assert_close(dv[sl], rdv, f"dv[{b},{h}]")
    # a second call on the same workspace-free path gives the same dK, dV bit for bit (work counter reset)
    dq2, dk2, dv2 = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=9, offset=4, status=status)
    assert torch.equal(dk2, dk) and torch.equal(dv2, dv)
    helpers.assert_close(dq2, dq.float(), "dq repeated")


@pytest.mark.parametrize("B,H,S_q,S_k,D", [(1, 1, 1, 1, 64), (1, 1, 5, 130, 64), (3, 1, 129, 1, 128), (1, 2, 1, 257, 128)])
def test_backward_tiny_and_ragged_shapes(cuda_device, B, H, S_q, S_k, D):
    _run(cuda_device, B, H, S_q, S_k, D, torch.float16, "none", 0.0, seed=14)
    if S_k > 1:
        # With a single key dQ is an exact cancellation (dS = dP - delta = 0); with dropout delta comes from O
        # rounded to 16 bits, so the kernel's dQ is |dP| * 2^-11 instead of 0: outside a bar anchored at ref = 0.
        _run(cuda_device, B, H, S_q, S_k, D, torch.float16, "seqlen", 0.25, seed=15)


def _random_case(i):
    g = torch.Generator().manual_seed(1000 + i)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    D = (64, 128)[r(0, 1)]
    dtype = (torch.float16, torch.bfloat16)[r(0, 1)]
    return dict(B=r(1, 3), H=r(1, 4), S_q=r(1, 450), S_k=r(4, 450), D=D, dtype=dtype, mask=("none", "seqlen", "key")[r(0, 2)],
                p_drop=(0.0, 0.1, 0.3)[r(0, 2)])


@pytest.mark.parametrize("i", range(24))
def test_forward_and_backward_on_random_shapes(cuda_device, i):
    """Seeded random shapes, head dimensions, dtypes, masks and dropout rates against the oracle."""
    c = _random_case(i)
    _run(cuda_device, c["B"], c["H"], c["S_q"], c["S_k"], c["D"], c["dtype"], c["mask"], c["p_drop"], seed=50 + i)


def test_masked_out_key_tiles_get_zero_gradients(cuda_device):
    B, H, S, D = 2, 2, 384, 64
    q, k, v, d_o, _ = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=3, device=cuda_device)
    lens = torch.tensor([100, 384], dtype=torch.int32, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens)
    dq, dk, dv = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens)
    assert (dk[0, :, 100:] == 0).all() and (dv[0, :, 100:] == 0).all()
    assert dk[1].abs().sum() > 0 and dv[0, :, :100].abs().sum() > 0


def test_backward_on_fused_qkv_projection_layout(cuda_device):
    """Q, K, V are views of one [B,S,3,H,D] projection output, dO and O are [B,S,H,D], and the gradients
    land in one [B,S,3,H,D] buffer: no permute or copy on either side of the operator."""
    dev = cuda_device
    B, S, H, D, p = 2, 320, 3, 64, 0.1
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(B, S, 3, H, D, generator=g).half().to(dev)
    d_o = (torch.randn(B, S, H, D, generator=g).half().to(dev)).permute(0, 2, 1, 3)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    lens = torch.tensor([320, 190], dtype=torch.int32, device=dev)
    out = torch.empty(B, S, H, D, dtype=torch.half, device=dev).permute(0, 2, 1, 3)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=3, offset=1, out=out)
    assert o.data_ptr() == out.data_ptr()
    dqkv = torch.full((B, S, 3, H, D), float("nan"), dtype=torch.half, device=dev)
    dq, dk, dv = (dqkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    got = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=3, offset=1, out=(dq, dk, dv))
    assert [t.data_ptr() for t in got] == [dq.data_ptr(), dk.data_ptr(), dv.data_ptr()]
    torch.cuda.synchronize()
    assert not torch.isnan(dqkv).any()
    qc, kc, vc, doc = q.contiguous(), k.contiguous(), v.contiguous(), d_o.contiguous()
    ref, add, keep, ks = helpers.oracle_forward(qc, kc, vc, p_drop=p, seed=3, offset=1, lens=lens)
    rdq, rdk, rdv = helpers.oracle_backward(qc, kc, vc, doc, add=add, keep=keep, ks=ks)
    helpers.assert_close(o, ref["o"], "o")
    helpers.assert_close(dq, rdq, "dq")
    helpers.assert_close(dk, rdk, "dk")
    helpers.assert_close(dv, rdv, "dv")


def test_sharded_backward_equals_unsharded(cuda_device):
    B, H, S, D, p = 4, 2, 256, 64, 0.1
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=4, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=5, offset=0)
    full = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=5, offset=0)
    parts = [[], [], []]
    for r in range(4):
        sh = sharding.make_shard(B, H, 4, r)
        f = lambda t: sharding.shard_tensor(t, sh).contiguous()
        ls = sharding.shard_per_batch(lens, sh)
        got = api.fmha_backward(f(d_o), f(q), f(k), f(v), f(o), lse.reshape(B * H, S)[sh.bh_start:sh.bh_start + sh.bh_count].contiguous(),
                                seqlens=ls, p_drop=p, seed=5, offset=0, bh_offset=sh.bh_offset)
        for acc, t in zip(parts, got):
            acc.append(t.reshape(sh.bh_count, S, D))
    # dK and dV have a fixed summation order; dQ is summed by atomics over key tiles
    assert torch.equal(torch.cat(parts[1]), full[1].reshape(B * H, S, D))
    assert torch.equal(torch.cat(parts[2]), full[2].reshape(B * H, S, D))
    assert (torch.cat(parts[0]).float() - full[0].reshape(B * H, S, D).float()).abs().max().item() <= 2e-3


def test_full_size_linearity_in_d_o(cuda_device):
    """BERT-large training shape: gradients are linear in dO, so bwd(2 dO) == 2 bwd(dO) to rounding.
    One (batch, head) slice is also checked against the oracle."""
    name = "bert_large_train"
    B, H, S, D, dtype, lr, p, _ = composite.CONFIGS[name]
    x = composite.make_inputs(B, H, S, D, dtype, lr, composite.CONFIG_SEEDS[name], with_do=True)
    q, k, v, d_o, lens = (x[n].to(cuda_device) for n in ("q", "k", "v", "d_o", "lens"))
    seed = composite.PHILOX_SEEDS[name]
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=seed, offset=0)
    g1 = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=seed, offset=0)
    g2 = api.fmha_backward(d_o * 2, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=seed, offset=0)
    for a2, a1 in zip(g2, g1):  # exact up to fp16 subnormal rounding of tiny dS entries and the final rounding
        assert (a2.float() - 2 * a1.float()).abs().max().item() <= 4e-3
    b, h = 3, 5
    sl = lambda t: t[b:b + 1, h:h + 1]
    ref, add, keep, ks = helpers.oracle_forward(sl(q), sl(k), sl(v), lens=lens[b:b + 1], p_drop=p, seed=seed, offset=0,
                                                bh_offset=b * H + h)
    rdq, rdk, rdv = helpers.oracle_backward(sl(q), sl(k), sl(v), sl(d_o), add=add, keep=keep, ks=ks)
    helpers.assert_close(sl(g1[0]), rdq, "dq slice")
    helpers.assert_close(sl(g1[1]), rdk, "dk slice")
    helpers.assert_close(sl(g1[2]), rdv, "dv slice")


@pytest.mark.parametrize("seed", [1004, 1005])
def test_bench_batch_many_slices_against_oracle(cuda_device, seed):
    """The benchmark's own batches (bench.py: B=32, H=16, S=512, D=64 fp16, input seeds 1004 and 1005, Philox seed
    0x5EED0004, offset = input set) through forward + backward at full size; 16 (batch, head) slices spread over the
    batch - first and last heads of a batch element, neighbours in the order the persistent backward CTAs draw their
    work items - are each compared with the oracle (about 0.1 s of CPU per slice)."""
    from nvfuserexamples_b200 import workloads
    B, H, S, D, p = 32, 16, 512, 64, 0.1
    x = workloads.make_inputs(B, H, S, D, torch.float16, (256, 512), seed, with_do=True)
    q, k, v, d_o, lens = (x[n].to(cuda_device) for n in ("q", "k", "v", "d_o", "lens"))
    pseed, off = 0x5EED0004, seed - 1004
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=pseed, offset=off, status=status)
    dq, dk, dv = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, p_drop=p, seed=pseed, offset=off, status=status)
    assert capi.check_status(status) == [0, 0, 0, 0]
    g = torch.Generator().manual_seed(seed)
    picks = {(0, 0), (0, H - 1), (B - 1, H - 1), (B - 1, 0), (9, 3), (9, 4)}   # boundaries and neighbours ...
    while len(picks) < 16:                                                      # ... and random ones
        picks.add((int(torch.randint(0, B, (1,), generator=g)), int(torch.randint(0, H, (1,), generator=g))))
    for b, h in sorted(picks):
        sl = lambda t: t[b:b + 1, h:h + 1]
        ref, add, keep, ks = helpers.oracle_forward(sl(q), sl(k), sl(v), lens=lens[b:b + 1], p_drop=p, seed=pseed, offset=off,
                                                    bh_offset=b * H + h)
        rdq, rdk, rdv = helpers.oracle_backward(sl(q), sl(k), sl(v), sl(d_o), add=add, keep=keep, ks=ks)
        helpers.assert_close(sl(o), ref["o"], f"o[{b},{h}]")
        helpers.assert_close(sl(lse), ref["lse"], f"lse[{b},{h}]", torch.float16, atol=1e-3, rtol=1e-4)
        helpers.assert_close(sl(dq), rdq, f"dq[{b},{h}]")
        helpers.assert_close(sl(dk), rdk, f"dk[{b},{h}]")
        helpers.assert_close(sl(dv), rdv, f"dv[{b},{h}]")


def test_long_sequence_head_dim_128_bf16(cuda_device):
    """The long-sequence training shape (S = 2048, D = 128, bf16, no dropout) on two heads."""
    _run(cuda_device, 1, 2, 2048, 2048, 128, torch.bfloat16, "seqlen", 0.0, seed=8)


def test_long_sequence_many_heads_cross_work_item_boundaries(cuda_device):
    """The long-sequence shape on 2 x 8 heads of 16 key tiles each: 256 backward work items on 148 persistent CTAs, so
    most CTAs hand over from one item to the next (other head, other valid length) in the middle of the run.  Three
    heads - the first, one whose items straddle the first wave, the last - are compared with the oracle."""
    B, H, S, D, dtype = 2, 8, 2048, 128, torch.bfloat16
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, dtype, seed=12, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, status=status)
    dq, dk, dv = api.fmha_backward(d_o, q, k, v, o, lse, seqlens=lens, status=status)
    assert capi.check_status(status) == [0, 0, 0, 0]
    for b, h in [(0, 0), (1, 1), (1, 7)]:
        sl = lambda t: t[b:b + 1, h:h + 1]
        ref, add, keep, ks = helpers.oracle_forward(sl(q), sl(k), sl(v), lens=lens[b:b + 1])
        rdq, rdk, rdv = helpers.oracle_backward(sl(q), sl(k), sl(v), sl(d_o), add=add, keep=keep, ks=ks)
        helpers.assert_close(sl(o), ref["o"], f"o[{b},{h}]", dtype)
        helpers.assert_close(sl(dq), rdq, f"dq[{b},{h}]", dtype)
        helpers.assert_close(sl(dk), rdk, f"dk[{b},{h}]", dtype)
        helpers.assert_close(sl(dv), rdv, f"dv[{b},{h}]", dtype)


def test_backward_accepts_a_broadcast_gradient(cuda_device):
    """A loss like (o * w).sum() with w of shape [D] makes autograd hand the operator an EXPANDED gradient (strides
    0,0,0,1): the operator must copy it to a dense tensor, not reject it."""
    import mha_manual  # noqa: F401
    B, H, S, D = 2, 2, 128, 64
    q, k, v, _, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=14, device=cuda_device)
    w = torch.linspace(-1, 1, D, device=cuda_device, dtype=torch.float16)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = torch.ops.mha_manual.fmha(qg, kg, vg, None, lens)
    (out * w).sum().backward()
    d_o = w.expand(B, H, S, D).contiguous()
    ref, add, keep, ks = helpers.oracle_forward(q, k, v, lens=lens)
    rdq, rdk, rdv = helpers.oracle_backward(q, k, v, d_o, add=add, keep=keep, ks=ks)
    helpers.assert_close(qg.grad, rdq, "dq")
    helpers.assert_close(kg.grad, rdk, "dk")
    helpers.assert_close(vg.grad, rdv, "dv")
