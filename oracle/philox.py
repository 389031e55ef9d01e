"""Philox4x32-10 and the dropout keep-mask rule, restated in numpy — TEST INFRASTRUCTURE.

Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this.  The reference
project has no random-number code at all (its train operators take a dense 0/1 dropout mask,
fmha/fmha_manual.cpp:433-449 of shmsong/NvFuserExamples); this file restates the published
algorithm (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11,
Philox-4x32 with 10 rounds) and the element mapping the kernels use, so that a mask can be
regenerated from (seed, offset) and compared bit for bit.

Pinned two ways (tests/test_oracle.py): against PyTorch's own host Philox engine
(ATen/core/PhiloxRNGEngine.h, through oracle/philox_check.cpp) and against the plain-C
restatement in oracle/philox_ref.c.
"""
from __future__ import annotations

import numpy as np

M0 = np.uint64(0xD2511F53)
M1 = np.uint64(0xCD9E8D57)
W0 = 0x9E3779B9
W1 = 0xBB67AE85
MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(key0, key1, c0, c1, c2, c3):
    """Vectorised Philox4x32-10.  All arguments broadcastable uint32 arrays / ints.
    Returns four uint32 arrays."""
    c0 = np.asarray(c0, dtype=np.uint64) & MASK32
    c1 = np.asarray(c1, dtype=np.uint64) & MASK32
    c2 = np.asarray(c2, dtype=np.uint64) & MASK32
    c3 = np.asarray(c3, dtype=np.uint64) & MASK32
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0 = int(key0) & 0xFFFFFFFF
    k1 = int(key1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c0           # 32x32 -> 64 bit products
        p1 = M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & MASK32
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return tuple(x.astype(np.uint32) for x in (c0, c1, c2, c3))


def dropout_threshold(p_drop: float) -> int:
    """T = round(128 p) clamped to [0,127]; an element is kept iff (byte & 0x7f) >= T."""
    t = int(np.float32(p_drop) * np.float32(128.0) + np.float32(0.5))
    return max(0, min(127, t))


def keep_scale(p_drop: float) -> float:
    return 128.0 / (128 - dropout_threshold(p_drop))


def dropout_keep_mask(seed: int, offset: int, bh_offset: int, n_bh: int, S_q: int, S_k: int, p_drop: float) -> np.ndarray:
    """uint8 [n_bh,S_q,S_k], 1 = kept.  Counter = (q_row, key // 16, bh_offset + bh, offset),
    key = (seed low word, seed high word); byte (key % 16) of the 128-bit draw decides."""
    thr = dropout_threshold(p_drop)
    n_kb = (S_k + 15) // 16
    bh = (np.arange(n_bh, dtype=np.uint64) + np.uint64(bh_offset)).reshape(n_bh, 1, 1)
    row = np.arange(S_q, dtype=np.uint64).reshape(1, S_q, 1)
    kb = np.arange(n_kb, dtype=np.uint64).reshape(1, 1, n_kb)
    w = philox4x32_10(seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, row, kb, bh, np.uint64(offset & 0xFFFFFFFF))
    words = np.stack(w, axis=-1)                                  # [n_bh,S_q,n_kb,4] uint32
    shifts = (np.arange(4, dtype=np.uint32) * np.uint32(8)).reshape(1, 1, 1, 1, 4)
    bytes_ = (words[..., None] >> shifts) & np.uint32(0xFF)       # [.., 4 words, 4 bytes], little endian
    bytes_ = bytes_.reshape(n_bh, S_q, n_kb * 16)[:, :, :S_k]
    return ((bytes_ & np.uint32(0x7F)) >= np.uint32(thr)).astype(np.uint8)
