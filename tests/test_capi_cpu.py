"""CPU-side checks of the drop-in boundary: the library loads, exports what the header
declares, validates its arguments and refuses to run without a B200 — no compute calls."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from nvfuserexamples_b200 import api, capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "fmha_sm100.h").read_text()


def test_library_exports_every_declared_symbol():
    lib = capi.load()
    declared = sorted(set(re.findall(r"\b(fmha_sm100_\w+)\s*\(", HEADER)))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/fmha_sm100.h but not exported"
    assert set(capi.EXPORTS) == set(declared)


def test_abi_version_and_strerror():
    lib = capi.load()
    assert lib.fmha_sm100_abi_version() == 3
    for code in range(0, 8):
        assert isinstance(capi.strerror(code), str) and capi.strerror(code)
    assert capi.strerror(capi.FMHA_OK) == "ok"


def _fwd_params(**over):
    p = capi.FwdParams()
    p.struct_bytes = C.sizeof(capi.FwdParams)
    p.dtype, p.B, p.H, p.S_q, p.S_k, p.D, p.scale = capi.DTYPE_F16, 1, 1, 128, 128, 64, 0.125
    for k, v in over.items():
        setattr(p, k, v)
    return p


def test_struct_layout_is_checked():
    lib = capi.load()
    assert lib.fmha_sm100_fwd(C.byref(_fwd_params(B=0)), None) == capi.FMHA_OK  # empty batch: nothing to do
    assert lib.fmha_sm100_fwd(C.byref(_fwd_params(B=0, struct_bytes=8)), None) == capi.FMHA_ERR_BAD_ARG
    b = capi.BwdParams()
    b.struct_bytes = C.sizeof(capi.BwdParams)
    b.dtype, b.B, b.H, b.S_q, b.S_k, b.D, b.scale = capi.DTYPE_BF16, 0, 4, 128, 128, 128, 0.1
    assert lib.fmha_sm100_bwd(C.byref(b), None) == capi.FMHA_OK
    b.struct_bytes -= 4
    assert lib.fmha_sm100_bwd(C.byref(b), None) == capi.FMHA_ERR_BAD_ARG


def test_argument_validation_codes():
    lib = capi.load()
    call = lambda **kw: lib.fmha_sm100_fwd(C.byref(_fwd_params(**kw)), None)
    assert lib.fmha_sm100_fwd(None, None) == capi.FMHA_ERR_BAD_ARG
    assert call(D=32) == capi.FMHA_ERR_UNSUPPORTED
    assert call(dtype=7) == capi.FMHA_ERR_UNSUPPORTED
    assert call(S_q=-1) == capi.FMHA_ERR_BAD_ARG
    assert call(scale=0.0) == capi.FMHA_ERR_BAD_ARG
    assert call(B=70000) == capi.FMHA_ERR_TOO_LARGE
    assert call(mask_kind=9) == capi.FMHA_ERR_UNSUPPORTED
    assert call(mask_kind=capi.MASK_SEQLEN) == capi.FMHA_ERR_BAD_ARG           # mask pointer missing
    assert call(dropout_kind=capi.DROPOUT_PHILOX, p_drop=1.5) == capi.FMHA_ERR_BAD_ARG
    assert call(dropout_kind=capi.DROPOUT_PHILOX, p_drop=0.1, philox_offset=1 << 32) == capi.FMHA_ERR_BAD_ARG
    assert call() == capi.FMHA_ERR_BAD_ARG                                        # null q/k/v/o
    assert call(S_k=0) == capi.FMHA_ERR_BAD_ARG


def test_misaligned_and_bad_strides_are_rejected():
    lib = capi.load()
    good = capi.Tensor4(0x1000, 128 * 64, 128 * 64, 64)
    odd_ptr = capi.Tensor4(0x1008, 128 * 64, 128 * 64, 64)
    odd_stride = capi.Tensor4(0x1000, 128 * 64, 128 * 64, 60)
    for bad in (odd_ptr, odd_stride):
        p = _fwd_params(q=bad, k=good, v=good, o=good)
        assert lib.fmha_sm100_fwd(C.byref(p), None) == capi.FMHA_ERR_BAD_ARG


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful on a machine without a GPU")
def test_refuses_to_run_without_a_b200():
    lib = capi.load()
    t = capi.Tensor4(0x1000, 128 * 64, 128 * 64, 64)  # never dereferenced: the device check comes first
    p = _fwd_params(q=t, k=t, v=t, o=t)
    assert lib.fmha_sm100_fwd(C.byref(p), None) == capi.FMHA_ERR_NO_DEVICE
    st = (C.c_int32 * 4)()
    assert lib.fmha_sm100_selftest_wait_timeout(st, None) == capi.FMHA_ERR_NO_DEVICE


def test_workspace_size_formula():
    b = capi.BwdParams()
    b.struct_bytes = C.sizeof(capi.BwdParams)
    b.dtype, b.B, b.H, b.S_q, b.S_k, b.D, b.scale = capi.DTYPE_F16, 2, 3, 200, 77, 64, 0.125
    n = capi.bwd_workspace_bytes(b)
    align = lambda x: (x + 255) // 256 * 256
    # fp32 dQ accumulator + delta + the work-item counter of the persistent backward kernel
    assert n == align(6 * 256 * 64 * 4) + align(6 * 200 * 4) + 256


def test_dropout_threshold():
    assert [capi.dropout_threshold(p) for p in (0.0, 0.1, 0.25, 0.5, 0.999)] == [0, 13, 32, 64, 127]


def test_extension_registers_the_reference_operator_names():
    import mha_manual  # noqa: F401
    ops = torch.ops.mha_manual
    for name in ("fmha_nvfuser", "fmha_train_nvfuser", "fmha_train_saveim_nvfuser", "fmha_fwd", "fmha_bwd", "fmha",
                 "philox_dropout_mask", "check_status"):
        assert hasattr(ops, name)
    s = str(ops.fmha_train_saveim_nvfuser.default._schema)
    assert "Tensor input, Tensor qk, Tensor v, Tensor pad_mask, Tensor dropout_mask" in s and "Tensor[]" in s
    assert str(ops.fmha_nvfuser.default._schema).count("Tensor") == 5  # four inputs, one output


def test_no_cpu_fallback():
    import mha_manual  # noqa: F401
    x = torch.zeros(2, 128, 64, dtype=torch.half)
    m = torch.zeros(2, 128, 128, dtype=torch.half)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.mha_manual.fmha_nvfuser(x, x, x, m)
    with pytest.raises(RuntimeError):
        api.fmha_nvfuser(x, x, x, m)
    with pytest.raises(RuntimeError):
        api.fmha_forward(x.view(2, 1, 128, 64), x.view(2, 1, 128, 64), x.view(2, 1, 128, 64))


def test_host_mask_op_matches_oracle():
    import mha_manual  # noqa: F401
    from oracle import philox
    m = torch.ops.mha_manual.philox_dropout_mask(2, 3, 9, 33, 0.2, 77, 4, 1, False)
    ref = philox.dropout_keep_mask(77, 4, 1, 6, 9, 33, 0.2).reshape(2, 3, 9, 33)
    assert (m.numpy() == ref).all()


def test_ctypes_layer_rejects_layouts_the_abi_cannot_describe():
    """The C ABI carries no stride for the head dimension and takes lse / masks as dense arrays: the ctypes helpers
    must raise rather than let the kernels read the wrong elements."""
    import torch
    x = torch.zeros(2, 2, 16, 64, dtype=torch.float16)
    capi._t4(x)                                  # dense: fine
    capi._t4(x[:, :, ::2])                       # strided rows: fine, the ABI has a row stride
    with pytest.raises(ValueError):
        capi._t4(x.transpose(-1, -2))            # head dimension not contiguous
    with pytest.raises(ValueError):
        capi._t4(x[..., ::2])                    # sliced inside the head dimension
    with pytest.raises(ValueError):
        capi._t4_packed(torch.zeros(8, 2, 64, dtype=torch.float16)[..., ::2])
    lse = torch.zeros(2, 2, 16)
    capi._lse_ok(lse, 64)
    with pytest.raises(ValueError):
        capi._lse_ok(lse.double(), 64)
    with pytest.raises(ValueError):
        capi._lse_ok(torch.zeros(2, 2, 32)[..., ::2], 64)
    with pytest.raises(ValueError):
        capi._dense_ok(torch.zeros(4, 8).t(), "mask")
