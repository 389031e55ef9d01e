"""Packed variable-length batches (FMHA_MASK_CU_SEQLENS) against the fp32 oracle, sequence by sequence.

The reference lists padded / irregular shapes as open work (fmha/fmha_manual.cpp:110, :178 of
shmsong/NvFuserExamples); here a batch is one [total_rows, H, D] tensor per operand plus row offsets."""
import pytest
import torch

from nvfuserexamples_b200 import capi
from tests import helpers

pytestmark = pytest.mark.gpu


def packed_batch(lens, H, D, dtype, seed, device):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    q, k, v, d_o = (torch.randn(total, H, D, generator=g).to(dtype).to(device) for _ in range(4))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=device)
    return q, k, v, d_o, cu


def per_sequence_oracle(q, k, v, d_o, lens, p_drop, seed, offset, max_len):
    """Runs the composite (and its autograd backward) on every sequence alone.  The dropout mask of
    sequence b is rows/columns [0, len_b) of the mask the padded batch would draw."""
    H = q.shape[1]
    outs = {n: [] for n in ("o", "lse", "dq", "dk", "dv")}
    keep_all = helpers.keep_mask(seed, offset, 0, len(lens), H, max_len, max_len, p_drop) if p_drop > 0 else None
    ks = helpers.philox.keep_scale(p_drop) if p_drop > 0 else 1.0
    r0 = 0
    for b, n in enumerate(lens):
        if n == 0:
            continue
        sl = slice(r0, r0 + n)
        qb, kb, vb, dob = (x[sl].permute(1, 0, 2).unsqueeze(0).cpu() for x in (q, k, v, d_o))   # [1,H,n,D]
        keep = keep_all[b:b + 1, :, :n, :n] if keep_all is not None else None
        ref = helpers.composite.attention_fp32(qb, kb, vb, add_mask=None, keep=keep, keep_scale=ks)
        dq, dk, dv = helpers.composite.attention_grads_fp32(qb, kb, vb, dob, add_mask=None, keep=keep, keep_scale=ks)
        outs["o"].append(ref["o"][0].permute(1, 0, 2))
        outs["lse"].append(ref["lse"][0])                     # [H, n]
        for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            outs[name].append(t[0].permute(1, 0, 2))
        r0 += n
    return {"o": torch.cat(outs["o"]), "lse": torch.cat(outs["lse"], dim=1), "dq": torch.cat(outs["dq"]),
            "dk": torch.cat(outs["dk"]), "dv": torch.cat(outs["dv"])}


@pytest.mark.parametrize("D,dtype,p_drop", [(64, torch.float16, 0.0), (64, torch.float16, 0.1),
                                            (128, torch.bfloat16, 0.0), (128, torch.float16, 0.1)])
def test_packed_batch_matches_the_oracle_per_sequence(cuda_device, D, dtype, p_drop):
    lens = [200, 77, 128, 1, 333, 256]      # partial tiles, an exact tile, a single row, multiples of the tile
    H, max_len = 3, 384
    q, k, v, d_o, cu = packed_batch(lens, H, D, dtype, seed=21, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    canary = 7.0
    o = torch.full_like(q, canary)
    res = capi.fwd_varlen(q, k, v, cu, max_len, p_drop=p_drop, seed=5, offset=2, status=status, out=o)
    dq, dk, dv = capi.bwd_varlen(d_o, q, k, v, res["o"], res["lse"], cu, max_len, p_drop=p_drop, seed=5, offset=2,
                                 status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = per_sequence_oracle(q, k, v, d_o, lens, p_drop, 5, 2, max_len)
    helpers.assert_close(res["o"], ref["o"], "o", dtype)
    helpers.assert_close(res["lse"], ref["lse"], "lse", torch.float16, atol=2e-3)
    helpers.assert_close(dq, ref["dq"], "dq", dtype)
    helpers.assert_close(dk, ref["dk"], "dk", dtype)
    helpers.assert_close(dv, ref["dv"], "dv", dtype)


@pytest.mark.parametrize("i", range(10))
def test_packed_batches_of_random_composition(cuda_device, i):
    """Seeded random numbers of sequences, lengths (empty ones included), heads, head dimension and dropout."""
    g = torch.Generator().manual_seed(2000 + i)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    lens = [r(0, 400) if r(0, 5) else 0 for _ in range(r(1, 7))]
    if sum(lens) == 0:
        lens[0] = 37
    H, D, p_drop = r(1, 4), (64, 128)[r(0, 1)], (0.0, 0.1, 0.3)[r(0, 2)]
    max_len = max(lens)
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=300 + i, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    res = capi.fwd_varlen(q, k, v, cu, max_len, p_drop=p_drop, seed=9, offset=i, status=status)
    dq, dk, dv = capi.bwd_varlen(d_o, q, k, v, res["o"], res["lse"], cu, max_len, p_drop=p_drop, seed=9, offset=i,
                                 status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = per_sequence_oracle(q, k, v, d_o, lens, p_drop, 9, i, max_len)
    for name, got in (("o", res["o"]), ("dq", dq), ("dk", dk), ("dv", dv)):
        # a sequence of one row: dS cancels exactly and dQ is the rounding of delta (see the single-key note of the backward tests)
        helpers.assert_close(got, ref[name], f"{name} lens={lens}", atol=4e-3 if (name == "dq" and 1 in lens and p_drop > 0) else helpers.ATOL)


def test_packed_batch_with_more_work_items_than_sms(cuda_device):
    """48 sequences x 8 heads x up to 3 key tiles: every persistent CTA handles several items of different
    lengths; two sequences are checked against the oracle on their own."""
    g = torch.Generator().manual_seed(17)
    lens = torch.randint(1, 385, (48,), generator=g).tolist()
    H, D = 8, 64
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=23, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    res = capi.fwd_varlen(q, k, v, cu, 384, status=status)
    dq, dk, dv = capi.bwd_varlen(d_o, q, k, v, res["o"], res["lse"], cu, 384, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    for b in (0, 29, 47):
        sl = slice(starts[b], starts[b + 1])
        ref = per_sequence_oracle(q[sl], k[sl], v[sl], d_o[sl], [lens[b]], 0.0, 0, 0, 384)
        helpers.assert_close(res["o"][sl], ref["o"], f"o[{b}]")
        helpers.assert_close(dq[sl], ref["dq"], f"dq[{b}]")
        helpers.assert_close(dk[sl], ref["dk"], f"dk[{b}]")
        helpers.assert_close(dv[sl], ref["dv"], f"dv[{b}]")


def test_packed_batch_equals_the_padded_batch_on_its_valid_rows(cuda_device):
    """Forward outputs of the packed call are bit-identical to the padded call with valid lengths:
    same tiles, same arithmetic, same Philox bits."""
    lens = [130, 64, 255]
    H, D, S = 2, 64, 256
    q, k, v, _, cu = packed_batch(lens, H, D, torch.float16, seed=3, device=cuda_device)
    res = capi.fwd_varlen(q, k, v, cu, S, p_drop=0.1, seed=9, offset=1)
    qp, kp, vp = (torch.zeros(len(lens), H, S, D, dtype=torch.float16, device=cuda_device) for _ in range(3))
    r0 = 0
    for b, n in enumerate(lens):
        for dst, src in ((qp, q), (kp, k), (vp, v)):
            dst[b, :, :n] = src[r0:r0 + n].permute(1, 0, 2)
        r0 += n
    lens_t = torch.tensor(lens, dtype=torch.int32, device=cuda_device)
    pad = capi.fwd(qp, kp, vp, mask_kind=capi.MASK_SEQLEN, mask=lens_t, dropout_kind=capi.DROPOUT_PHILOX, p_drop=0.1,
                   seed=9, offset=1)
    r0 = 0
    for b, n in enumerate(lens):
        assert torch.equal(res["o"][r0:r0 + n].permute(1, 0, 2), pad["o"][b, :, :n])
        assert torch.equal(res["lse"][:, r0:r0 + n], pad["lse"][b, :, :n])
        r0 += n


def test_packed_batch_with_empty_sequences(cuda_device):
    """Sequences of length zero own no rows and produce nothing; their neighbours are unaffected."""
    lens = [0, 130, 0, 0, 40, 0]
    H, D = 2, 64
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=8, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    res = capi.fwd_varlen(q, k, v, cu, 256, p_drop=0.1, seed=2, offset=1, status=status)
    dq, dk, dv = capi.bwd_varlen(d_o, q, k, v, res["o"], res["lse"], cu, 256, p_drop=0.1, seed=2, offset=1, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    ref = per_sequence_oracle(q, k, v, d_o, lens, 0.1, 2, 1, 256)
    helpers.assert_close(res["o"], ref["o"], "o")
    helpers.assert_close(dq, ref["dq"], "dq")
    helpers.assert_close(dk, ref["dk"], "dk")
    helpers.assert_close(dv, ref["dv"], "dv")


def test_packed_batch_leaves_neighbouring_rows_alone(cuda_device):
    """A sequence's last, partial tile must not write into the next sequence (or past the end)."""
    lens = [5, 300, 60]
    H, D = 2, 64
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=4, device=cuda_device)
    total = sum(lens)
    # outputs with guard rows behind the packed rows
    o = torch.full((total + 64, H, D), 3.0, dtype=torch.float16, device=cuda_device)
    res = capi.fwd_varlen(q, k, v, cu, 384, out=o[:total])
    torch.cuda.synchronize()
    assert (o[total:] == 3.0).all()
    ref = per_sequence_oracle(q, k, v, d_o, lens, 0.0, 0, 0, 384)
    helpers.assert_close(res["o"], ref["o"], "o")


def test_packed_autograd_operator(cuda_device):
    import mha_manual  # noqa: F401
    ops = torch.ops.mha_manual
    lens = [150, 40, 257]
    H, D = 2, 64
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=12, device=cuda_device)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    o = ops.fmha_varlen(q, k, v, cu, 384, 0.1, 77, 4)
    o.backward(d_o)
    ref = per_sequence_oracle(q.detach(), k.detach(), v.detach(), d_o, lens, 0.1, 77, 4, 384)
    helpers.assert_close(o, ref["o"], "o")
    helpers.assert_close(q.grad, ref["dq"], "dq")
    helpers.assert_close(k.grad, ref["dk"], "dk")
    helpers.assert_close(v.grad, ref["dv"], "dv")
    # the device-resident offset is added to the launch parameter: 1 + 3 draws the bits of offset 4
    off = torch.full((1,), 3, dtype=torch.int64, device=cuda_device)
    o2, _ = ops.fmha_varlen_fwd(q.detach(), k.detach(), v.detach(), cu, 384, 0.1, 77, 1, None, off)
    assert torch.equal(o2, o.detach())
    ops.check_status()


def test_packed_batch_on_the_fused_projection_layout(cuda_device):
    """qkv [total_rows,3,H,D] in, o [total_rows,H,D] out, one [total_rows,3,H,D] gradient back; sequences that
    end inside a tile exercise the row-wise edge stores through the strided layout."""
    import mha_manual  # noqa: F401
    ops = torch.ops.mha_manual
    lens = [150, 0, 40, 257, 128]
    H, D, p = 3, 64, 0.1
    q, k, v, d_o, cu = packed_batch(lens, H, D, torch.float16, seed=31, device=cuda_device)
    qkv = torch.stack((q, k, v), dim=1).contiguous().requires_grad_()     # [total, 3, H, D]
    o = ops.fmha_varlen_qkvpacked(qkv, cu, 384, p, 77, 4)
    assert o.shape == q.shape and o.is_contiguous()
    (dqkv,) = torch.autograd.grad(o, (qkv,), d_o)
    assert dqkv.shape == qkv.shape and dqkv.is_contiguous()
    ops.check_status()
    ref = per_sequence_oracle(q, k, v, d_o, lens, p, 77, 4, 384)
    helpers.assert_close(o, ref["o"], "o")
    for i, name in enumerate(("dq", "dk", "dv")):
        helpers.assert_close(dqkv[:, i], ref[name], name)
    # the same bits as the three-tensor operator
    o2, _ = ops.fmha_varlen_fwd(q, k, v, cu, 384, p, 77, 4)
    assert torch.equal(o2, o.detach())


def test_sequence_longer_than_max_seqlen_is_cut_not_spilled(cuda_device):
    """A sequence longer than the stated max_seqlen is processed up to max_seqlen (queries and keys alike) and its
    rows past that are left alone; above all, nothing of it lands in its neighbours' outputs or gradients (the dQ
    accumulator and delta rows of the next head lie right behind max_seqlen)."""
    import mha_manual  # noqa: F401
    lens, max_len, H, D, dtype = [150, 300, 90], 256, 2, 64, torch.float16
    q, k, v, d_o, cu = packed_batch(lens, H, D, dtype, seed=33, device=cuda_device)
    # what it must equal: the same batch with the long sequence cut to its first max_seqlen rows
    keep_rows = torch.cat([torch.arange(0, 150), torch.arange(150, 150 + 256), torch.arange(450, 540)]).to(cuda_device)
    cut = [150, 256, 90]
    qc, kc, vc, doc = (x[keep_rows].contiguous() for x in (q, k, v, d_o))
    ref = per_sequence_oracle(qc, kc, vc, doc, cut, 0.0, 0, 0, max_len)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    canary = 7.0
    o = torch.full_like(q, canary)
    res = capi.fwd_varlen(q, k, v, cu, max_len, status=status, out=o)
    dq, dk, dv = capi.bwd_varlen(d_o, q, k, v, res["o"], res["lse"], cu, max_len, status=status)
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0, 0, 0]
    helpers.assert_close(res["o"][keep_rows], ref["o"], "o", dtype)
    assert (res["o"][406:450] == canary).all(), "rows past max_seqlen were written"
    helpers.assert_close(dq[keep_rows], ref["dq"], "dq", dtype)
    helpers.assert_close(dk[keep_rows], ref["dk"], "dk", dtype)
    helpers.assert_close(dv[keep_rows], ref["dv"], "dv", dtype)
    # the torch operators hand back zeros for the rows that are not computed
    ops = torch.ops.mha_manual
    o2, lse2 = ops.fmha_varlen_fwd(q, k, v, cu, max_len)
    g = ops.fmha_varlen_bwd(d_o, q, k, v, o2, lse2, cu, max_len)
    assert (o2[406:450] == 0).all() and all((t[406:450] == 0).all() for t in g)
    helpers.assert_close(g[0][keep_rows], ref["dq"], "dq (operator)", dtype)
