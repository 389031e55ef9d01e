"""ctypes binding of include/fmha_sm100.h.

This is the same boundary a cgo/JNI/FFI binding would attach to: plain structs, raw device
pointers and an int status.  The Python helpers here only fill the structs from torch
tensors (torch supplies device memory and streams); they add no arithmetic of their own and
raise if the library is missing or a call fails — there is no CPU path behind them.
"""
from __future__ import annotations

import ctypes as C
import math
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfmha_sm100.so"

FMHA_OK = 0
FMHA_ERR_BAD_ARG = 1
FMHA_ERR_UNSUPPORTED = 2
FMHA_ERR_LAUNCH = 3
FMHA_ERR_DEVICE_TIMEOUT = 4
FMHA_ERR_NO_DEVICE = 5
FMHA_ERR_TOO_LARGE = 6

DTYPE_F16, DTYPE_BF16 = 0, 1
MASK_NONE, MASK_DENSE_KEEP, MASK_DENSE_ADDITIVE, MASK_KEY_ADDITIVE, MASK_SEQLEN, MASK_CU_SEQLENS = 0, 1, 2, 3, 4, 5
DROPOUT_NONE, DROPOUT_DENSE, DROPOUT_PHILOX = 0, 1, 2
FLAG_P_VIA_SMEM = 1
FLAG_BWD_SKIP_PREPARE = 2
FLAG_BWD_SKIP_FINISH = 4
STATIC_SCRATCH_BYTES = 32 << 20

EXPORTS = [
    "fmha_sm100_fwd", "fmha_sm100_bwd", "fmha_sm100_bwd_workspace_bytes", "fmha_sm100_dropout_threshold",
    "fmha_sm100_philox_mask_host", "fmha_sm100_philox_mask_device", "fmha_sm100_check_status",
    "fmha_sm100_strerror", "fmha_sm100_last_cuda_error", "fmha_sm100_abi_version",
    "fmha_sm100_selftest_wait_timeout", "fmha_sm100_bwd_static_scratch",
]


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class FwdParams(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("S_q", C.c_int32), ("S_k", C.c_int32), ("D", C.c_int32),
        ("scale", C.c_float),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4),
        ("lse", C.c_void_p),
        ("mask_kind", C.c_int32), ("mask", C.c_void_p),
        ("dropout_kind", C.c_int32), ("dropout_mask", C.c_void_p),
        ("dropout_scale", C.c_float), ("p_drop", C.c_float),
        ("philox_seed", C.c_uint64), ("philox_offset", C.c_uint64), ("philox_bh_offset", C.c_int32),
        ("save_softmax", C.c_void_p), ("save_dropout", C.c_void_p),
        ("keep_mask_out", C.c_void_p), ("debug_scores", C.c_void_p),
        ("flags", C.c_int32), ("status", C.c_void_p),
        ("total_rows", C.c_int32),
        ("philox_offset_dev", C.c_void_p),
    ]


class BwdParams(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_int32), ("dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("S_q", C.c_int32), ("S_k", C.c_int32), ("D", C.c_int32),
        ("scale", C.c_float),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("o", Tensor4), ("d_o", Tensor4),
        ("lse", C.c_void_p),
        ("dq", Tensor4), ("dk", Tensor4), ("dv", Tensor4),
        ("mask_kind", C.c_int32), ("mask", C.c_void_p),
        ("dropout_kind", C.c_int32), ("p_drop", C.c_float),
        ("philox_seed", C.c_uint64), ("philox_offset", C.c_uint64), ("philox_bh_offset", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("flags", C.c_int32), ("status", C.c_void_p),
        ("total_rows", C.c_int32),
        ("philox_offset_dev", C.c_void_p),
    ]


class FmhaError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        super().__init__(f"{what}: status {code} ({detail})")


_lib = None


def load() -> C.CDLL:
    """Loads libfmha_sm100.so (built in-tree by nvfuserexamples_b200.build). Raises if absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m nvfuserexamples_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    lib.fmha_sm100_fwd.argtypes = [C.POINTER(FwdParams), C.c_void_p]
    lib.fmha_sm100_fwd.restype = C.c_int
    lib.fmha_sm100_bwd.argtypes = [C.POINTER(BwdParams), C.c_void_p]
    lib.fmha_sm100_bwd.restype = C.c_int
    lib.fmha_sm100_bwd_static_scratch.argtypes = [C.POINTER(BwdParams), C.c_void_p]
    lib.fmha_sm100_bwd_static_scratch.restype = C.c_int
    lib.fmha_sm100_bwd_workspace_bytes.argtypes = [C.POINTER(BwdParams), C.POINTER(C.c_size_t)]
    lib.fmha_sm100_bwd_workspace_bytes.restype = C.c_int
    lib.fmha_sm100_dropout_threshold.argtypes = [C.c_float]
    lib.fmha_sm100_dropout_threshold.restype = C.c_int32
    lib.fmha_sm100_philox_mask_host.argtypes = [C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_float, C.c_void_p]
    lib.fmha_sm100_philox_mask_host.restype = C.c_int
    lib.fmha_sm100_philox_mask_device.argtypes = [C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                  C.c_float, C.c_void_p, C.c_void_p]
    lib.fmha_sm100_philox_mask_device.restype = C.c_int
    lib.fmha_sm100_check_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    lib.fmha_sm100_check_status.restype = C.c_int
    lib.fmha_sm100_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_void_p]
    lib.fmha_sm100_selftest_wait_timeout.restype = C.c_int
    lib.fmha_sm100_strerror.argtypes = [C.c_int]
    lib.fmha_sm100_strerror.restype = C.c_char_p
    lib.fmha_sm100_last_cuda_error.restype = C.c_int
    lib.fmha_sm100_abi_version.restype = C.c_int
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().fmha_sm100_strerror(code).decode()


def _check(code: int, what: str) -> None:
    if code != FMHA_OK:
        raise FmhaError(code, what, f"{strerror(code)}; cuda error {load().fmha_sm100_last_cuda_error()}")


# ---------------------------------------------------------------------------------------
# helpers that fill the structs from torch tensors
# ---------------------------------------------------------------------------------------
def _inner_contiguous(x, what: str) -> None:
    """The C ABI cannot see the stride of the last axis: it must be 1 (raise instead of computing on the wrong elements)."""
    if x.dim() < 3 or x.stride(-1) != 1:
        raise ValueError(f"{what}: the head dimension must be the contiguous last axis (shape {tuple(x.shape)}, "
                         f"strides {tuple(x.stride())})")


def _lse_ok(lse, n: int) -> None:
    import torch
    if lse.dtype != torch.float32 or not lse.is_contiguous() or lse.numel() != n:
        raise ValueError(f"lse must be a contiguous float32 tensor of {n} elements, got {lse.dtype} {tuple(lse.shape)} "
                         f"strides {tuple(lse.stride())}")


def _dense_ok(t, what: str) -> None:
    if t is not None and hasattr(t, "is_contiguous") and not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous (strides {tuple(t.stride())})")


def _t4(x) -> Tensor4:
    """[B,H,S,D] or [B*H,S,D] torch tensor -> fmha_tensor4 (element strides)."""
    _inner_contiguous(x, "tensor operand")
    if x.dim() == 4:
        return Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))
    return Tensor4(x.data_ptr(), x.stride(0), x.stride(0), x.stride(1))


def _dims(x):
    if x.dim() == 4:
        return x.shape[0], x.shape[1], x.shape[2], x.shape[3]
    return x.shape[0], 1, x.shape[1], x.shape[2]


def _dtype_code(x) -> int:
    import torch
    if x.dtype == torch.float16:
        return DTYPE_F16
    if x.dtype == torch.bfloat16:
        return DTYPE_BF16
    raise TypeError(f"unsupported dtype {x.dtype}")


def _stream_ptr(device) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def fwd(q, k, v, *, mask_kind=MASK_NONE, mask=None, dropout_kind=DROPOUT_NONE, dropout_mask=None,
        dropout_scale=1.0, p_drop=0.0, seed=0, offset=0, bh_offset=0, scale=None, want_lse=True,
        save_softmax=False, save_dropout=False, keep_mask_out=False, debug_scores=False, flags=0,
        status=None, out=None):
    """Calls fmha_sm100_fwd on the current stream.  Returns a dict with 'o', 'lse' and any
    requested dense outputs.  Inputs are torch CUDA tensors; nothing is copied."""
    import torch
    lib = load()
    B, H, S_q, D = _dims(q)
    S_k = _dims(k)[2]
    o = out if out is not None else torch.empty_like(q)
    res = {"o": o}
    p = FwdParams()
    p.struct_bytes = C.sizeof(FwdParams)
    p.dtype = _dtype_code(q)
    p.B, p.H, p.S_q, p.S_k, p.D = B, H, S_q, S_k, D
    p.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    p.q, p.k, p.v, p.o = _t4(q), _t4(k), _t4(v), _t4(o)
    if want_lse:
        res["lse"] = torch.empty((B, H, S_q), dtype=torch.float32, device=q.device)
        p.lse = res["lse"].data_ptr()
    _dense_ok(mask, "mask")
    _dense_ok(dropout_mask, "dropout_mask")
    p.mask_kind = mask_kind
    p.mask = _ptr(mask)
    p.dropout_kind = dropout_kind
    p.dropout_mask = _ptr(dropout_mask)
    p.dropout_scale = dropout_scale
    p.p_drop = p_drop
    p.philox_seed, p.philox_offset, p.philox_bh_offset = seed, offset, bh_offset
    dense = (B * H, S_q, S_k)
    if save_softmax:
        res["softmax"] = torch.empty(dense, dtype=q.dtype, device=q.device)
        p.save_softmax = res["softmax"].data_ptr()
    if save_dropout:
        res["dropout_out"] = torch.empty(dense, dtype=q.dtype, device=q.device)
        p.save_dropout = res["dropout_out"].data_ptr()
    if keep_mask_out:
        res["keep_mask"] = torch.full(dense, 255, dtype=torch.uint8, device=q.device)
        p.keep_mask_out = res["keep_mask"].data_ptr()
    if debug_scores:
        res["scores"] = torch.zeros(dense, dtype=torch.float32, device=q.device)
        p.debug_scores = res["scores"].data_ptr()
    p.flags = flags
    p.status = _ptr(status)
    _check(lib.fmha_sm100_fwd(C.byref(p), _stream_ptr(q.device)), "fmha_sm100_fwd")
    return res


def bwd_params(d_o, q, k, v, o, lse, dq, dk, dv, *, mask_kind=MASK_NONE, mask=None, p_drop=0.0, seed=0, offset=0,
               bh_offset=0, scale=None, status=None, flags=0) -> BwdParams:
    B, H, S_q, D = _dims(q)
    S_k = _dims(k)[2]
    p = BwdParams()
    p.struct_bytes = C.sizeof(BwdParams)
    p.dtype = _dtype_code(q)
    p.B, p.H, p.S_q, p.S_k, p.D = B, H, S_q, S_k, D
    p.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    p.q, p.k, p.v, p.o, p.d_o = _t4(q), _t4(k), _t4(v), _t4(o), _t4(d_o)
    _lse_ok(lse, B * H * S_q)
    _dense_ok(mask, "mask")
    p.lse = lse.data_ptr()
    p.dq, p.dk, p.dv = _t4(dq), _t4(dk), _t4(dv)
    p.mask_kind = mask_kind
    p.mask = _ptr(mask)
    p.dropout_kind = DROPOUT_PHILOX if p_drop > 0 else DROPOUT_NONE
    p.p_drop = p_drop
    p.philox_seed, p.philox_offset, p.philox_bh_offset = seed, offset, bh_offset
    p.status = _ptr(status)
    p.flags = flags
    return p


def bwd_workspace_bytes(p: BwdParams) -> int:
    n = C.c_size_t(0)
    _check(load().fmha_sm100_bwd_workspace_bytes(C.byref(p), C.byref(n)), "fmha_sm100_bwd_workspace_bytes")
    return n.value


def bwd(d_o, q, k, v, o, lse, *, workspace=None, out=None, **kw):
    """Calls fmha_sm100_bwd on the current stream. Returns (dq, dk, dv); `out` = (dq, dk, dv) to write into
    (any strides with a contiguous last dimension, e.g. three views of one [B,S,3,H,D] buffer)."""
    import torch
    dq, dk, dv = out if out is not None else (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v))
    p = bwd_params(d_o, q, k, v, o, lse, dq, dk, dv, **kw)
    need = bwd_workspace_bytes(p)
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=q.device)
    p.workspace = workspace.data_ptr()
    p.workspace_bytes = workspace.numel()
    _check(load().fmha_sm100_bwd(C.byref(p), _stream_ptr(q.device)), "fmha_sm100_bwd")
    return dq, dk, dv


# ---------------------------------------------------------------------------------------
# packed variable-length batches: q, k, v are [total_rows, H, D]; cu_seqlens int32 [B+1] on the device
# ---------------------------------------------------------------------------------------
def _t4_packed(x) -> Tensor4:
    """[total, H, D] torch tensor -> fmha_tensor4 (the batch stride is not used)."""
    _inner_contiguous(x, "packed tensor operand")
    return Tensor4(x.data_ptr(), 0, x.stride(1), x.stride(0))


def fwd_varlen(q, k, v, cu_seqlens, max_seqlen, *, p_drop=0.0, seed=0, offset=0, bh_offset=0, scale=None, status=None,
               out=None):
    """Forward over a packed batch.  Returns {'o': [total,H,D], 'lse': [H,total]}."""
    import torch
    total, H, D = q.shape
    o = out if out is not None else torch.empty_like(q)
    lse = torch.empty((H, total), dtype=torch.float32, device=q.device)
    p = FwdParams()
    p.struct_bytes = C.sizeof(FwdParams)
    p.dtype = _dtype_code(q)
    p.B, p.H, p.S_q, p.S_k, p.D = cu_seqlens.numel() - 1, H, max_seqlen, max_seqlen, D
    p.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    p.q, p.k, p.v, p.o = _t4_packed(q), _t4_packed(k), _t4_packed(v), _t4_packed(o)
    p.lse = lse.data_ptr()
    p.mask_kind, p.mask, p.total_rows = MASK_CU_SEQLENS, cu_seqlens.data_ptr(), total
    if p_drop > 0:
        p.dropout_kind, p.p_drop = DROPOUT_PHILOX, p_drop
    p.philox_seed, p.philox_offset, p.philox_bh_offset = seed, offset, bh_offset
    p.status = _ptr(status)
    _check(load().fmha_sm100_fwd(C.byref(p), _stream_ptr(q.device)), "fmha_sm100_fwd")
    return {"o": o, "lse": lse}


def bwd_varlen(d_o, q, k, v, o, lse, cu_seqlens, max_seqlen, *, p_drop=0.0, seed=0, offset=0, bh_offset=0, scale=None,
               status=None, workspace=None):
    """Backward over a packed batch.  Returns (dq, dk, dv), each [total,H,D]."""
    import torch
    total, H, D = q.shape
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = BwdParams()
    p.struct_bytes = C.sizeof(BwdParams)
    p.dtype = _dtype_code(q)
    p.B, p.H, p.S_q, p.S_k, p.D = cu_seqlens.numel() - 1, H, max_seqlen, max_seqlen, D
    p.scale = float(scale) if scale is not None else 1.0 / math.sqrt(D)
    p.q, p.k, p.v, p.o, p.d_o = (_t4_packed(x) for x in (q, k, v, o, d_o))
    _lse_ok(lse, H * total)
    _dense_ok(cu_seqlens, "cu_seqlens")
    p.lse = lse.data_ptr()
    p.dq, p.dk, p.dv = _t4_packed(dq), _t4_packed(dk), _t4_packed(dv)
    p.mask_kind, p.mask, p.total_rows = MASK_CU_SEQLENS, cu_seqlens.data_ptr(), total
    p.dropout_kind = DROPOUT_PHILOX if p_drop > 0 else DROPOUT_NONE
    p.p_drop = p_drop
    p.philox_seed, p.philox_offset, p.philox_bh_offset = seed, offset, bh_offset
    p.status = _ptr(status)
    need = bwd_workspace_bytes(p)
    if workspace is None:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=q.device)
    p.workspace = workspace.data_ptr()
    p.workspace_bytes = workspace.numel()
    _check(load().fmha_sm100_bwd(C.byref(p), _stream_ptr(q.device)), "fmha_sm100_bwd")
    return dq, dk, dv


def philox_mask_host(seed: int, offset: int, bh_offset: int, n_bh: int, S_q: int, S_k: int, p_drop: float):
    """Dense keep mask [n_bh,S_q,S_k] (uint8 numpy array) from the library's host generator."""
    import numpy as np
    out = np.empty((n_bh, S_q, S_k), dtype=np.uint8)
    _check(load().fmha_sm100_philox_mask_host(seed, offset, bh_offset, n_bh, S_q, S_k, p_drop,
                                              out.ctypes.data_as(C.c_void_p)), "fmha_sm100_philox_mask_host")
    return out


def philox_mask_device(seed, offset, bh_offset, n_bh, S_q, S_k, p_drop, device):
    import torch
    out = torch.empty((n_bh, S_q, S_k), dtype=torch.uint8, device=device)
    _check(load().fmha_sm100_philox_mask_device(seed, offset, bh_offset, n_bh, S_q, S_k, p_drop, out.data_ptr(),
                                                _stream_ptr(device)), "fmha_sm100_philox_mask_device")
    return out


def dropout_threshold(p_drop: float) -> int:
    return int(load().fmha_sm100_dropout_threshold(p_drop))


def check_status(status) -> list:
    """Synchronises and returns the four status words; raises FmhaError if a wait ran out."""
    words = (C.c_int32 * 4)()
    code = load().fmha_sm100_check_status(status.data_ptr(), _stream_ptr(status.device), words)
    if code != FMHA_OK:
        raise FmhaError(code, "fmha_sm100_check_status", f"{strerror(code)}; words {list(words)}")
    return list(words)


def selftest_wait_timeout(status) -> None:
    """Launches the library's bounded-wait self test on the current stream (see the header)."""
    _check(load().fmha_sm100_selftest_wait_timeout(status.data_ptr(), _stream_ptr(status.device)),
           "fmha_sm100_selftest_wait_timeout")


def bwd_static_scratch(d_o, q, k, v, o, lse, **kw):
    """fmha_sm100_bwd_static_scratch on the current stream: the backward pass with the scratch
    taken from the library's built-in array (no workspace argument, nothing allocated by the
    library).  Raises FmhaError(FMHA_ERR_TOO_LARGE) when the sizes need more than
    STATIC_SCRATCH_BYTES.  Returns (dq, dk, dv); the outputs themselves are the caller's tensors."""
    import torch
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p = bwd_params(d_o, q, k, v, o, lse, dq, dk, dv, **kw)
    _check(load().fmha_sm100_bwd_static_scratch(C.byref(p), _stream_ptr(q.device)), "fmha_sm100_bwd_static_scratch")
    return dq, dk, dv
