"""B200-native fused multi-head attention behind the `mha_manual` operator boundary.

Layout of the package:
  csrc/        hand-written sm_100a kernels, the C ABI (include/fmha_sm100.h) and the torch
               operator layer (`import mha_manual` -> torch.ops.mha_manual.*)
  build.py     in-tree nvcc build of both shared objects
  capi.py      ctypes binding of the C ABI
  api.py       Python mirror of the reference's operator interface plus the new entry points
  sharding.py  batch x heads partitioning across the GPUs of one box (no collective)
  workloads.py the named benchmark configurations and their seeded synthetic inputs (bench.py, tests)
"""
from . import capi, sharding  # noqa: F401
from .api import (fmha_backward, fmha_forward, fmha_nvfuser, fmha_train_nvfuser,  # noqa: F401
                  fmha_train_saveim_nvfuser, philox_dropout_mask)

__all__ = ["capi", "sharding", "fmha_forward", "fmha_backward", "fmha_nvfuser", "fmha_train_nvfuser",
           "fmha_train_saveim_nvfuser", "philox_dropout_mask"]
