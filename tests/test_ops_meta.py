"""Shape-only (Meta) kernels of the torch operators: what fake-tensor tracing needs.  Runs without a GPU.

The reference registers its three operators for the CUDA key only (fmha/fmha_manual.cpp:1240-1250 of
shmsong/NvFuserExamples) and has no backward; the Meta kernels and the autograd operator are additions."""
import pytest
import torch


@pytest.fixture(scope="module")
def ops():
    import mha_manual  # noqa: F401  (registers torch.ops.mha_manual)
    return torch.ops.mha_manual


def meta(*shape, dtype=torch.float16):
    return torch.empty(*shape, dtype=dtype, device="meta")


def test_legacy_ops_infer_shapes(ops):
    q, k, v = meta(512, 128, 64), meta(512, 128, 64), meta(512, 128, 64)
    m = meta(512, 128, 128)
    assert ops.fmha_nvfuser(q, k, v, m).shape == (512, 128, 64)
    assert ops.fmha_train_nvfuser(q, k, v, m, m).shape == (512, 128, 64)
    outs = ops.fmha_train_saveim_nvfuser(q, k, v, m, m)
    assert [tuple(o.shape) for o in outs] == [(512, 128, 64), (512, 128, 128), (512, 128, 128)]
    assert all(o.device.type == "meta" and o.dtype == torch.float16 for o in outs)


def test_forward_backward_infer_shapes(ops):
    q, k, v = meta(2, 4, 200, 128, dtype=torch.bfloat16), meta(2, 4, 77, 128, dtype=torch.bfloat16), meta(2, 4, 77, 128, dtype=torch.bfloat16)
    lens = torch.empty(2, dtype=torch.int32, device="meta")
    o, lse = ops.fmha_fwd(q, k, v, None, lens, 0.1, 5, 9)
    assert o.shape == q.shape and o.dtype == torch.bfloat16
    assert lse.shape == (2, 4, 200) and lse.dtype == torch.float32
    dq, dk, dv = ops.fmha_bwd(torch.empty_like(o), q, k, v, o, lse, None, lens, 0.1, 5, 9)
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    # [B*H, S, D] inputs give a [B*H, S] logsumexp
    o3, lse3 = ops.fmha_fwd(meta(6, 50, 64), meta(6, 40, 64), meta(6, 40, 64))
    assert o3.shape == (6, 50, 64) and lse3.shape == (6, 50)


def test_autograd_operator_traces_on_meta_tensors(ops):
    q = meta(2, 3, 64, 64).requires_grad_()
    k = meta(2, 3, 96, 64).requires_grad_()
    v = meta(2, 3, 96, 64).requires_grad_()
    o = ops.fmha(q, k, v, None, None, 0.0, 0, 0)
    assert o.shape == q.shape and o.requires_grad
    gq, gk, gv = torch.autograd.grad(o, (q, k, v), torch.empty_like(o))
    assert gq.shape == q.shape and gk.shape == k.shape and gv.shape == v.shape


def test_packed_batch_operators_infer_shapes(ops):
    q, k, v = meta(1000, 4, 64), meta(1000, 4, 64), meta(1000, 4, 64)
    cu = torch.empty(9, dtype=torch.int32, device="meta")
    o, lse = ops.fmha_varlen_fwd(q, k, v, cu, 384, 0.1, 1, 2)
    assert o.shape == (1000, 4, 64) and lse.shape == (4, 1000) and lse.dtype == torch.float32
    dq, dk, dv = ops.fmha_varlen_bwd(torch.empty_like(o), q, k, v, o, lse, cu, 384, 0.1, 1, 2)
    assert dq.shape == dk.shape == dv.shape == (1000, 4, 64)
    qg = meta(1000, 4, 64).requires_grad_()
    out = ops.fmha_varlen(qg, k, v, cu, 384)
    (g,) = torch.autograd.grad(out, (qg,), torch.empty_like(out))
    assert g.shape == qg.shape
    with pytest.raises(RuntimeError, match="same \\[total_rows, H, D\\] shape"):
        ops.fmha_varlen_fwd(q, meta(999, 4, 64), v, cu, 384)


def test_shape_errors_are_raised_without_a_device(ops):
    with pytest.raises(RuntimeError, match="head dimension"):
        ops.fmha_fwd(meta(1, 1, 16, 32), meta(1, 1, 16, 32), meta(1, 1, 16, 32))
    with pytest.raises(RuntimeError, match="sequence lengths differ"):
        ops.fmha_fwd(meta(1, 1, 16, 64), meta(1, 1, 16, 64), meta(1, 1, 24, 64))
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        ops.fmha_fwd(meta(1, 1, 16, 64, dtype=torch.float32), meta(1, 1, 16, 64, dtype=torch.float32), meta(1, 1, 16, 64, dtype=torch.float32))
    with pytest.raises(RuntimeError, match="B\\*H\\*S_q\\*S_k"):
        ops.fmha_nvfuser(meta(4, 16, 64), meta(4, 16, 64), meta(4, 16, 64), meta(4, 16, 8))


def test_fused_projection_layout_operators_infer_shapes(ops):
    qkv = meta(2, 300, 3, 4, 64)
    lens = torch.empty(2, dtype=torch.int32, device="meta")
    o, lse = ops.fmha_qkvpacked_fwd(qkv, None, lens, 0.1, 1, 2)
    assert o.shape == (2, 300, 4, 64) and lse.shape == (2, 4, 300) and lse.dtype == torch.float32
    assert ops.fmha_qkvpacked_bwd(torch.empty_like(o), qkv, o, lse, None, lens, 0.1, 1, 2).shape == qkv.shape
    qg = meta(2, 300, 3, 4, 64).requires_grad_()
    out = ops.fmha_qkvpacked(qg, None, lens, 0.1, 1, 2)
    (g,) = torch.autograd.grad(out, (qg,), torch.empty_like(out))
    assert out.shape == (2, 300, 4, 64) and g.shape == qg.shape
    with pytest.raises(RuntimeError):
        ops.fmha_qkvpacked_fwd(meta(2, 300, 2, 4, 64))


def test_packed_fused_projection_operators_infer_shapes(ops):
    qkv = meta(1000, 3, 4, 128, dtype=torch.bfloat16)
    cu = torch.empty(9, dtype=torch.int32, device="meta")
    o, lse = ops.fmha_varlen_qkvpacked_fwd(qkv, cu, 384, 0.1, 1, 2)
    assert o.shape == (1000, 4, 128) and lse.shape == (4, 1000) and lse.dtype == torch.float32
    assert ops.fmha_varlen_qkvpacked_bwd(torch.empty_like(o), qkv, o, lse, cu, 384, 0.1, 1, 2).shape == qkv.shape
    qg = meta(1000, 3, 4, 128, dtype=torch.bfloat16).requires_grad_()
    out = ops.fmha_varlen_qkvpacked(qg, cu, 384)
    (g,) = torch.autograd.grad(out, (qg,), torch.empty_like(out))
    assert g.shape == qg.shape


def test_differentiable_operators_run_below_the_autograd_keys(ops):
    """torch.inference_mode() excludes the autograd keys; the four differentiable operators then reach kernels of their
    own (forward only) instead of failing with "could not run ... with arguments from the 'Meta' backend"."""
    q, k, v = meta(2, 3, 64, 64), meta(2, 3, 96, 64), meta(2, 3, 96, 64)
    cu = torch.empty(5, dtype=torch.int32, device="meta")
    with torch.inference_mode():
        assert ops.fmha(q, k, v).shape == (2, 3, 64, 64)
        assert ops.fmha_qkvpacked(meta(2, 96, 3, 4, 64)).shape == (2, 96, 4, 64)
        assert ops.fmha_varlen(meta(100, 4, 64), meta(100, 4, 64), meta(100, 4, 64), cu, 64).shape == (100, 4, 64)
        assert ops.fmha_varlen_qkvpacked(meta(100, 3, 4, 64), cu, 64).shape == (100, 4, 64)


def test_torch_compile_traces_the_operator_as_one_graph(ops):
    """fullgraph=True: no graph break at the operator, and the compiled backward yields the three gradients."""
    def f(q, k, v):
        return ops.fmha(q * 1.0, k, v, None, None, 0.1, 7, 2, None) * 2.0

    cf = torch.compile(f, fullgraph=True, backend="aot_eager")
    q, k, v = meta(2, 3, 64, 64).requires_grad_(), meta(2, 3, 96, 64).requires_grad_(), meta(2, 3, 96, 64).requires_grad_()
    o = cf(q, k, v)
    assert o.shape == q.shape and o.requires_grad
    gq, gk, gv = torch.autograd.grad(o, (q, k, v), torch.empty_like(o))
    assert gq.shape == q.shape and gk.shape == k.shape and gv.shape == v.shape
