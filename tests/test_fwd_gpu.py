"""Forward parity on the GPU: the CUDA path, called through the C ABI, against the CPU oracle
on the same seeded inputs.  Tolerance: |got - ref| <= 1e-3 + 2e-3 |ref| (see helpers.assert_close)."""
import numpy as np
import pytest
import torch

from nvfuserexamples_b200 import api, capi, sharding
from oracle import composite, philox
from tests import helpers

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, H, S_q, S_k, D, dtype
    (2, 4, 128, 128, 64, torch.float16),     # the reference's own sequence length and head size
    (2, 3, 384, 384, 64, torch.float16),     # BERT-large forward shape, fewer heads
    (1, 2, 512, 512, 64, torch.bfloat16),
    (2, 2, 200, 333, 64, torch.float16),     # ragged: neither length is a tile multiple
    (1, 2, 77, 1000, 128, torch.bfloat16),
    (1, 2, 256, 384, 128, torch.float16),
    (3, 1, 1, 5, 64, torch.float16),         # a single query row, five keys
]


@pytest.mark.parametrize("B,H,S_q,S_k,D,dtype", SHAPES)
@pytest.mark.parametrize("mask", ["none", "seqlen", "key"])
def test_forward_matches_oracle(cuda_device, B, H, S_q, S_k, D, dtype, mask):
    q, k, v, _, lens = helpers.randn_like_config(B, H, S_q, S_k, D, dtype, seed=100 + S_q + S_k, device=cuda_device)
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    kw, okw = {}, {}
    if mask == "seqlen":
        kw["seqlens"], okw["lens"] = lens, lens
    elif mask == "key":
        add = composite.padding_add_mask(lens.cpu(), S_k).reshape(B, S_k).to(cuda_device)
        kw["mask"], okw["add_mask"] = add, add
    o, lse = api.fmha_forward(q, k, v, status=status, **kw)
    assert capi.check_status(status) == [0, 0, 0, 0]
    ref, *_ = helpers.oracle_forward(q, k, v, **okw)
    helpers.assert_close(o, ref["o"], "o", dtype)
    helpers.assert_close(lse, ref["lse"], "lse", torch.float16, atol=1e-3, rtol=1e-4)


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
@pytest.mark.parametrize("p_drop", [0.1, 0.5])
def test_forward_philox_dropout(cuda_device, D, dtype, p_drop):
    B, H, S = 2, 2, 384
    q, k, v, _, lens = helpers.randn_like_config(B, H, S, S, D, dtype, seed=7, device=cuda_device)
    o, lse = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p_drop, seed=0xABCDEF12345, offset=9)
    ref, *_ = helpers.oracle_forward(q, k, v, lens=lens, p_drop=p_drop, seed=0xABCDEF12345, offset=9)
    helpers.assert_close(o, ref["o"], "o", dtype)
    helpers.assert_close(lse, ref["lse"], "lse", torch.float16, atol=1e-3, rtol=1e-4)  # lse ignores dropout


def test_dropout_mask_bit_exact(cuda_device):
    """The keep decisions taken inside the kernel, the library's device and host generators and
    the numpy restatement are the same bits."""
    B, H, S_q, S_k, p, seed, off = 1, 3, 200, 333, 0.1, 0x5EED0003, 11
    q, k, v, _, _ = helpers.randn_like_config(B, H, S_q, S_k, 64, torch.float16, seed=1, device=cuda_device)
    res = capi.fwd(q, k, v, dropout_kind=capi.DROPOUT_PHILOX, p_drop=p, seed=seed, offset=off, keep_mask_out=True)
    kernel = res["keep_mask"].cpu().numpy()
    oracle = philox.dropout_keep_mask(seed, off, 0, B * H, S_q, S_k, p)
    np.testing.assert_array_equal(kernel, oracle)
    dev = api.philox_dropout_mask(B, H, S_q, S_k, p, seed, off, device=cuda_device).cpu().numpy().reshape(B * H, S_q, S_k)
    np.testing.assert_array_equal(dev, oracle)
    np.testing.assert_array_equal(api.philox_dropout_mask(B, H, S_q, S_k, p, seed, off).reshape(B * H, S_q, S_k), oracle)
    # and the production kernel (no debug outputs) dropped the same entries as the instrumented one:
    # the two differ only by rounding, a differing keep decision would show as an O(1) difference
    o_fast, _ = api.fmha_forward(q, k, v, p_drop=p, seed=seed, offset=off)
    assert (o_fast.float() - res["o"].float()).abs().max().item() <= 2e-3


def test_tensor_memory_and_shared_memory_paths_agree(cuda_device):
    q, k, v, _, lens = helpers.randn_like_config(2, 2, 256, 384, 64, torch.float16, seed=5, device=cuda_device)
    a = capi.fwd(q, k, v, mask_kind=capi.MASK_SEQLEN, mask=lens, debug_scores=True)  # general kernel, P in tensor memory
    b = capi.fwd(q, k, v, mask_kind=capi.MASK_SEQLEN, mask=lens, flags=capi.FLAG_P_VIA_SMEM)
    assert torch.equal(a["o"], b["o"]) and torch.equal(a["lse"], b["lse"])


def test_raw_scores_are_the_fp32_gemm(cuda_device):
    q, k, v, _, _ = helpers.randn_like_config(1, 2, 128, 256, 128, torch.float16, seed=2, device=cuda_device)
    res = capi.fwd(q, k, v, debug_scores=True)
    ref = torch.matmul(q.float().cpu(), k.float().cpu().transpose(-1, -2)).reshape(2, 128, 256)
    assert (res["scores"].cpu() - ref).abs().max().item() < 1e-3


def test_edge_cases(cuda_device):
    dev = cuda_device
    torch.manual_seed(0)
    # single key: output rows equal that key's value row exactly
    q = torch.randn(1, 1, 130, 64, device=dev).half()
    k = torch.randn(1, 1, 1, 64, device=dev).half()
    v = torch.randn(1, 1, 1, 64, device=dev).half()
    o, lse = api.fmha_forward(q, k, v)
    assert torch.equal(o, v.expand(1, 1, 130, 64))
    # equal scores: mean of the values
    k8 = torch.randn(1, 1, 8, 64, device=dev).half()
    v8 = torch.randn(1, 1, 8, 64, device=dev).half()
    o, _ = api.fmha_forward(torch.zeros_like(q), k8, v8)
    helpers.assert_close(o, v8.float().mean(2, keepdim=True).expand(1, 1, 130, 64), "mean")
    # valid length 0 == nothing masked; a fully masked additive row == unmasked row (test.py:15 semantics)
    q2, k2, v2, _, _ = helpers.randn_like_config(2, 1, 64, 200, 64, torch.float16, seed=3, device=dev)
    o_none, _ = api.fmha_forward(q2, k2, v2)
    o_len0, _ = api.fmha_forward(q2, k2, v2, seqlens=torch.zeros(2, dtype=torch.int32, device=dev))
    assert torch.equal(o_none, o_len0)
    o_all, _ = api.fmha_forward(q2, k2, v2, mask=torch.full((2, 200), -10000.0, device=dev))
    helpers.assert_close(o_all, o_none.float(), "fully masked", atol=4e-3)
    # empty batch is a no-op, zero keys is an error
    api.fmha_forward(q2[:0], k2[:0], v2[:0])
    with pytest.raises(capi.FmhaError):
        api.fmha_forward(q2, k2[:, :, :0], v2[:, :, :0])


def test_strided_views_bshd(cuda_device):
    """[B,S,3,H,D] packed projections viewed as [B,H,S,D] without a copy."""
    B, S, H, D = 2, 256, 3, 64
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(B, S, 3, H, D, generator=g).half().to(cuda_device)
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    out = torch.empty(B, S, H, D, dtype=torch.half, device=cuda_device).permute(0, 2, 1, 3)
    o, _ = api.fmha_forward(q, k, v, out=out)
    ref, *_ = helpers.oracle_forward(q.contiguous(), k.contiguous(), v.contiguous())
    helpers.assert_close(o, ref["o"], "o strided")


def test_sharded_equals_unsharded_bitwise(cuda_device):
    B, H, S, D, p = 4, 3, 256, 64, 0.1
    q, k, v, _, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=9, device=cuda_device)
    full, lse_full = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=3, offset=1)
    for world in (2, 8):
        parts = []
        for r in range(world):
            sh = sharding.make_shard(B, H, world, r)
            qs, ks, vs = (sharding.shard_tensor(t, sh).contiguous() for t in (q, k, v))
            o, _ = api.fmha_forward(qs, ks, vs, seqlens=sharding.shard_per_batch(lens, sh), p_drop=p, seed=3, offset=1,
                                    bh_offset=sh.bh_offset)
            parts.append(o.reshape(sh.bh_count, S, D))
        assert torch.equal(torch.cat(parts), full.reshape(B * H, S, D))


@pytest.mark.parametrize("D,dtype", [(64, torch.float16), (128, torch.bfloat16)])
def test_forward_is_bit_reproducible_across_calls(cuda_device, D, dtype):
    """More CTAs than resident slots, valid lengths and an additive key mask, with dropout: 40 calls give the same bits
    (nothing in the forward depends on the order in which CTAs, loads or MMAs complete)."""
    B, H, S = 8, 16, 512
    q, k, v, _, lens = helpers.randn_like_config(B, H, S, S, D, dtype, seed=12, device=cuda_device)
    add = composite.padding_add_mask(lens, S).reshape(B, S).contiguous()
    for kw in (dict(seqlens=lens), dict(mask=add)):
        first_o, first_lse = api.fmha_forward(q, k, v, p_drop=0.1, seed=4, offset=2, **kw)
        for _ in range(40):
            o, lse = api.fmha_forward(q, k, v, p_drop=0.1, seed=4, offset=2, **kw)
        assert torch.equal(o, first_o) and torch.equal(lse, first_lse)


@pytest.mark.parametrize("name", ["bert_base_fwd", "bert_large_fwd"])
def test_full_size_properties(cuda_device, name):
    """At the benchmark sizes the CPU oracle is too slow, so check size-independent properties:
    V = 1 gives O = 1 (probabilities sum to one), permuting the keys changes nothing, and one
    (batch, head) slice matches the oracle."""
    B, H, S, D, dtype, lr, p, _ = composite.CONFIGS[name]
    x = composite.make_inputs(B, H, S, D, dtype, lr, composite.CONFIG_SEEDS[name])
    q, k, v, lens = (x[n].to(cuda_device) for n in ("q", "k", "v", "lens"))
    ones = torch.ones_like(v)
    o1, lse = api.fmha_forward(q, k, ones, seqlens=lens)
    assert (o1.float() - 1).abs().max().item() <= 2e-3
    full = torch.full_like(lens, S)
    perm = torch.randperm(S, generator=torch.Generator().manual_seed(1)).to(cuda_device)
    o_a, lse_a = api.fmha_forward(q, k, v, seqlens=full)
    o_b, lse_b = api.fmha_forward(q, k[:, :, perm].contiguous(), v[:, :, perm].contiguous(), seqlens=full)
    assert (o_a.float() - o_b.float()).abs().max().item() <= 4e-3
    assert (lse_a - lse_b).abs().max().item() <= 1e-3
    b, h = B - 1, H // 2
    od, _ = api.fmha_forward(q, k, v, seqlens=lens, p_drop=p, seed=composite.PHILOX_SEEDS[name], offset=0)
    ref, *_ = helpers.oracle_forward(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], lens=lens[b:b + 1],
                                     p_drop=p, seed=composite.PHILOX_SEEDS[name], offset=0, bh_offset=b * H + h)
    helpers.assert_close(od[b:b + 1, h:h + 1], ref["o"], "slice o", dtype)


def test_bounded_wait_reports_instead_of_hanging(cuda_device):
    """Failure detection without faulting the GPU: a wait nothing satisfies runs out, the kernel
    returns, the status block names the site, and the context keeps working."""
    status = torch.zeros(4, dtype=torch.int32, device=cuda_device)
    capi.selftest_wait_timeout(status)
    with pytest.raises(capi.FmhaError) as e:
        capi.check_status(status)
    assert e.value.code == capi.FMHA_ERR_DEVICE_TIMEOUT and "900" in str(e.value)
    assert capi.check_status(status) == [0, 0, 0, 0]  # cleared by the failing check
    q, k, v, _, _ = helpers.randn_like_config(1, 1, 128, 128, 64, torch.float16, seed=1, device=cuda_device)
    o, _ = api.fmha_forward(q, k, v, status=status)
    ref, *_ = helpers.oracle_forward(q, k, v)
    helpers.assert_close(o, ref["o"], "o after timeout")
