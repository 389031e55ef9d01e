"""The torch operator layer on the GPU: the reference's own checks (test.py:20-29 and
test_train_mha.py:23-41 of shmsong/NvFuserExamples) restated with seeds, the golden outputs of
the reference composites, and the autograd operator."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import composite
from tests import helpers
from tests.golden import make_golden

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def ops():
    import mha_manual  # noqa: F401  (registers torch.ops.mha_manual)
    return torch.ops.mha_manual


def test_reference_inference_check(ops, cuda_device):
    """test.py with its sizes (B*H = 512, S = 128, D = 64) and its tolerance (atol 1e-2), plus ours."""
    torch.manual_seed(0)
    bh, s, d = 32 * 16, 128, 64
    q, k, v = (torch.randn(bh, s, d, dtype=torch.half, device=cuda_device) for _ in range(3))
    amask = torch.empty(bh, s, s, device=cuda_device).random_(2).to(torch.half)
    fused = ops.fmha_nvfuser(q, k, v, amask)
    ctx = composite.reference_mha_inference(q, k, v, amask)  # the composite itself, on the GPU as in test.py
    assert torch.allclose(ctx, fused, atol=1e-2)
    ref = composite.attention_fp32(q, k, v, add_mask=(1.0 - amask.float()) * -10000.0, scale=1 / 8)["o"]
    helpers.assert_close(fused, ref, "ctx")
    ops.check_status()


def test_reference_train_check(ops, cuda_device):
    torch.manual_seed(1)
    bh, s, d = 32 * 16, 128, 64
    q, k, v = (torch.randn(bh, s, d, dtype=torch.half, device=cuda_device) for _ in range(3))
    pad = torch.empty(bh, s, s, device=cuda_device).random_(2).to(torch.half) * (-1000)
    dm = torch.empty(bh, s, s, device=cuda_device).random_(2).to(torch.half)
    sm, dr, ctx = composite.reference_mha_train(q, k, v, pad, dm)
    ctx_fused = ops.fmha_train_nvfuser(q, k, v, pad, dm)
    saved = ops.fmha_train_saveim_nvfuser(q, k, v, pad, dm)
    assert torch.allclose(ctx_fused, ctx, atol=1e-2)            # test_train_mha.py:36
    assert torch.allclose(saved[0], ctx, atol=1e-2)             # test_train_mha.py:41
    r = composite.attention_fp32(q, k, v, add_mask=pad.float(), keep=dm.float(), keep_scale=2.0, scale=1 / 8)
    # These two operators round the NORMALISED, doubled probabilities (values up to 2) to 16 bits before the second
    # GEMM, exactly as fmha/fmha_manual.cpp:478-482 and :891-897 do, so their context carries that rounding: the
    # yardstick is the reference's own 16-bit eager composite (`ctx` above), whose error against the fp32
    # composite the fused result may not exceed by more than a factor of two (+ the 1e-3 bar).
    helpers.assert_no_worse_than_eager(ctx_fused, r["o"], ctx, "ctx")
    helpers.assert_no_worse_than_eager(saved[0], r["o"], ctx, "saved ctx")
    helpers.assert_close(saved[1], r["softmax"], "softmax")
    helpers.assert_close(saved[2], r["dropout_out"], "dropout_out")
    ops.check_status()


def test_against_golden_outputs_of_the_reference_composites(ops, cuda_device):
    g = np.load(GOLD / "ref_inference.npz")
    bh, s, d = (int(x) for x in g["shape"])
    q, k, v, amask = (t.to(cuda_device) for t in make_golden.inference_inputs(int(g["seed"]), bh, s, d))
    fused = ops.fmha_nvfuser(q, k, v, amask)
    assert torch.allclose(torch.from_numpy(g["ctx"]).float(), fused.cpu().float(), atol=2e-3)
    g = np.load(GOLD / "ref_train.npz")
    bh, s, d = (int(x) for x in g["shape"])
    q, k, v, pad, dm = (t.to(cuda_device) for t in make_golden.train_inputs(int(g["seed"]), bh, s, d))
    out = ops.fmha_train_saveim_nvfuser(q, k, v, pad, dm)
    # the golden train composite ran natively in fp16 (its own error is ~1e-3, hence the reference's 1e-2)
    assert torch.allclose(torch.from_numpy(g["ctx"]).float(), out[0].cpu().float(), atol=1e-2)
    assert torch.allclose(torch.from_numpy(g["softmax"]).float(), out[1].cpu().float(), atol=2e-3)
    assert torch.allclose(torch.from_numpy(g["dropout_out"]).float(), out[2].cpu().float(), atol=4e-3)


def test_legacy_ops_accept_other_shapes(ops, cuda_device):
    torch.manual_seed(2)
    for bh, sq, sk, d, dt in ((3, 200, 136, 64, torch.half), (2, 128, 384, 128, torch.bfloat16), (2, 77, 51, 64, torch.half)):
        q = torch.randn(bh, sq, d, device=cuda_device).to(dt)
        k = torch.randn(bh, sk, d, device=cuda_device).to(dt)
        v = torch.randn(bh, sk, d, device=cuda_device).to(dt)
        amask = torch.empty(bh, sq, sk, device=cuda_device).random_(2).to(dt)
        dm = torch.empty(bh, sq, sk, device=cuda_device).random_(2).to(dt)
        pad = (1 - amask) * -1000
        ref = composite.attention_fp32(q, k, v, add_mask=(1.0 - amask.float()) * -10000.0)
        helpers.assert_close(ops.fmha_nvfuser(q, k, v, amask), ref["o"], f"ctx {bh,sq,sk,d}", dt)
        r2 = composite.attention_fp32(q, k, v, add_mask=pad.float(), keep=dm.float(), keep_scale=2.0)
        out = ops.fmha_train_saveim_nvfuser(q, k, v, pad, dm)
        eager_ctx = composite.reference_mha_train(q, k, v, pad, dm, scale=1.0 / d ** 0.5)[2]   # 16-bit eager composite
        helpers.assert_no_worse_than_eager(out[0], r2["o"], eager_ctx, "saved ctx")
        helpers.assert_close(out[1], r2["softmax"], "softmax", dt)
        helpers.assert_close(out[2], r2["dropout_out"], "dropout", dt)
        helpers.assert_no_worse_than_eager(ops.fmha_train_nvfuser(q, k, v, pad, dm), r2["o"], eager_ctx, "train ctx")


def test_autograd_operator(ops, cuda_device):
    B, H, S, D = 2, 2, 256, 64
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=6, device=cuda_device)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
    o = ops.fmha(q, k, v, None, lens, 0.1, 42, 1, None)
    o.backward(d_o)
    ref, add, keep, ks = helpers.oracle_forward(q.detach(), k.detach(), v.detach(), lens=lens, p_drop=0.1, seed=42, offset=1)
    rdq, rdk, rdv = helpers.oracle_backward(q.detach(), k.detach(), v.detach(), d_o, add=add, keep=keep, ks=ks)
    helpers.assert_close(o, ref["o"], "o")
    helpers.assert_close(q.grad, rdq, "dq")
    helpers.assert_close(k.grad, rdk, "dk")
    helpers.assert_close(v.grad, rdv, "dv")


def test_operators_can_be_captured_in_a_cuda_graph(ops, cuda_device):
    """Forward and backward replayed from a CUDA graph give what the eager calls gave.  The Philox
    offset is a launch parameter, so a captured graph replays the same dropout pattern."""
    B, H, S, D = 4, 4, 384, 64
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=8, device=cuda_device)
    args = (None, lens, 0.1, 11, 3)
    o0, lse0 = ops.fmha_fwd(q, k, v, *args)                      # warm-up: one-time set-up happens outside the capture
    dq0, dk0, dv0 = ops.fmha_bwd(d_o, q, k, v, o0, lse0, *args)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            o1, lse1 = ops.fmha_fwd(q, k, v, *args)
            dq1, dk1, dv1 = ops.fmha_bwd(d_o, q, k, v, o1, lse1, *args)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o1, o0) and torch.equal(lse1, lse0)
    assert torch.equal(dk1, dk0) and torch.equal(dv1, dv0)
    helpers.assert_close(dq1, dq0.float(), "dq replayed")        # summed by atomics: equal up to the order of additions
    ops.check_status()


def test_device_resident_philox_offset_gives_new_masks_on_graph_replay(ops, cuda_device):
    """offset_tensor: the kernels add its value to `offset`, so one captured graph draws the bits of
    (seed, offset + value) for whatever value the tensor holds at replay time."""
    B, H, S, D = 2, 4, 256, 64
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=9, device=cuda_device)
    off = torch.zeros(1, dtype=torch.int64, device=cuda_device)
    eager = {}
    for value in (0, 5):   # what the graph must reproduce: plain calls with offset 10 + value
        o, lse = ops.fmha_fwd(q, k, v, None, lens, 0.25, 3, 10 + value)
        eager[value] = (o, lse) + tuple(ops.fmha_bwd(d_o, q, k, v, o, lse, None, lens, 0.25, 3, 10 + value))
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            o, lse = ops.fmha_fwd(q, k, v, None, lens, 0.25, 3, 10, None, 0, off)
            dq, dk, dv = ops.fmha_bwd(d_o, q, k, v, o, lse, None, lens, 0.25, 3, 10, None, 0, off)
    torch.cuda.current_stream().wait_stream(side)
    for value in (0, 5):
        off.fill_(value)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(o, eager[value][0]) and torch.equal(lse, eager[value][1])
        assert torch.equal(dk, eager[value][3]) and torch.equal(dv, eager[value][4])
        helpers.assert_close(dq, eager[value][2].float(), "dq")
    assert not torch.equal(eager[0][0], eager[5][0])   # the two offsets really drew different masks
    # the autograd operator keeps the forward's value for its backward pass
    qg = q.clone().requires_grad_(True)
    off.fill_(5)
    out = ops.fmha(qg, k, v, None, lens, 0.25, 3, 10, None, off)
    off.fill_(99)
    out.backward(d_o)
    torch.cuda.synchronize()
    assert torch.equal(out, eager[5][0])
    helpers.assert_close(qg.grad, eager[5][2].float(), "dq via autograd")


def test_fused_projection_layout_operator(ops, cuda_device):
    """qkv [B,S,3,H,D] -> o [B,S,H,D], and autograd returns one [B,S,3,H,D] gradient: the layouts on both sides
    of a fused QKV projection, with no permute or copy around the kernels."""
    dev = cuda_device
    B, S, H, D, p = 2, 200, 3, 64, 0.1
    g = torch.Generator().manual_seed(8)
    qkv = torch.randn(B, S, 3, H, D, generator=g).half().to(dev).requires_grad_()
    d_o = torch.randn(B, S, H, D, generator=g).half().to(dev)
    lens = torch.tensor([200, 131], dtype=torch.int32, device=dev)
    o = ops.fmha_qkvpacked(qkv, None, lens, p, 11, 4)
    assert o.shape == (B, S, H, D) and o.is_contiguous()
    (dqkv,) = torch.autograd.grad(o, (qkv,), d_o)
    assert dqkv.shape == qkv.shape and dqkv.is_contiguous()
    ops.check_status()
    q, k, v = (qkv.detach()[:, :, i].permute(0, 2, 1, 3).contiguous() for i in range(3))
    ref, add, keep, ks = helpers.oracle_forward(q, k, v, p_drop=p, seed=11, offset=4, lens=lens)
    rdq, rdk, rdv = helpers.oracle_backward(q, k, v, d_o.permute(0, 2, 1, 3).contiguous(), add=add, keep=keep, ks=ks)
    helpers.assert_close(o.permute(0, 2, 1, 3), ref["o"], "o")
    for i, (name, want) in enumerate((("dq", rdq), ("dk", rdk), ("dv", rdv))):
        helpers.assert_close(dqkv[:, :, i].permute(0, 2, 1, 3), want, name)
    # the same numbers as the [B,H,S,D] operator on permuted views, bit for bit in the forward direction
    o2, _ = ops.fmha_fwd(q, k, v, None, lens, p, 11, 4)
    assert torch.equal(o2, o.permute(0, 2, 1, 3))


def test_operator_errors(ops, cuda_device):
    x = torch.zeros(2, 128, 64, dtype=torch.half, device=cuda_device)
    with pytest.raises(RuntimeError):
        ops.fmha_nvfuser(x, x, x, torch.zeros(2, 128, 64, dtype=torch.half, device=cuda_device))   # wrong mask size
    with pytest.raises(RuntimeError):
        ops.fmha_nvfuser(x.float(), x.float(), x.float(), torch.zeros(2, 128, 128, device=cuda_device))  # fp32 unsupported
    y = torch.zeros(2, 128, 96, dtype=torch.half, device=cuda_device)
    with pytest.raises(RuntimeError):
        ops.fmha_nvfuser(y, y, y, torch.zeros(2, 128, 128, dtype=torch.half, device=cuda_device))  # head dim 96


def test_operator_under_inference_mode(ops, cuda_device):
    """torch.inference_mode() removes the autograd keys: the differentiable operators must still run (forward only)."""
    B, H, S, D = 2, 2, 256, 64
    q, k, v, _, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=16, device=cuda_device)
    with torch.inference_mode():
        o = ops.fmha(q, k, v, None, lens)
        qkv = torch.stack([q, k, v], 2).permute(0, 3, 2, 1, 4).contiguous()   # [B,S,3,H,D]
        o2 = ops.fmha_qkvpacked(qkv, None, lens)
    ref, *_ = helpers.oracle_forward(q, k, v, lens=lens)
    helpers.assert_close(o, ref["o"], "o")
    helpers.assert_close(o2.permute(0, 2, 1, 3), ref["o"], "o (fused projection layout)")


def test_torch_compile_fullgraph(ops, cuda_device):
    """A function calling torch.ops.mha_manual.fmha compiles as ONE graph (no graph break at the operator) and its
    forward and backward results equal the eager call's."""
    B, H, S, D = 2, 2, 256, 64
    q, k, v, d_o, lens = helpers.randn_like_config(B, H, S, S, D, torch.float16, seed=17, device=cuda_device)

    def f(q, k, v, lens):
        return ops.fmha(q * 1.0, k, v, None, lens, 0.1, 7, 2, None) * 2.0

    cf = torch.compile(f, fullgraph=True, backend="aot_eager")   # the tracing and autograd partitioning are what is under test
    outs = []
    for fn in (f, cf):
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = fn(qg, kg, vg, lens)
        o.backward(d_o)
        outs.append((o.detach(), qg.grad, kg.grad, vg.grad))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][2], outs[1][2]) and torch.equal(outs[0][3], outs[1][3])     # dK, dV: fixed summation order
    assert (outs[0][1].float() - outs[1][1].float()).abs().max().item() <= 2e-3             # dQ: atomics
