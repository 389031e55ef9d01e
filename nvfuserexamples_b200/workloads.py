"""Named workloads of the attention path and their seeded synthetic inputs.

The configurations are the ones the benchmark contract names (BERT-base / BERT-large are shape labels: every
tensor is seeded N(0,1) noise of that shape, valid lengths are drawn uniformly from the stated range).  This
module is plain input generation: it imports neither the CUDA library nor the CPU oracle, so the benchmark,
the tests and the oracle can all share one recipe.
"""
from __future__ import annotations

import torch

# name: (B, H, S, D, dtype, (len_lo, len_hi), p_drop, mode)
CONFIGS = {
    "cpu_composite": (2, 4, 128, 64, torch.float32, (64, 128), 0.0, "fwd"),
    "bert_base_fwd": (32, 12, 512, 64, torch.float16, (256, 512), 0.1, "fwd"),
    "bert_large_fwd": (64, 16, 384, 64, torch.float16, (128, 384), 0.1, "fwd"),
    "bert_large_train": (32, 16, 512, 64, torch.float16, (256, 512), 0.1, "fwd+bwd"),
    "long_seq_train": (256, 16, 2048, 128, torch.bfloat16, (1024, 2048), 0.0, "fwd+bwd"),
}
CONFIG_SEEDS = {name: 1001 + i for i, name in enumerate(CONFIGS)}
PHILOX_SEEDS = {name: 0x5EED0001 + i for i, name in enumerate(CONFIGS)}


def make_inputs(B: int, H: int, S: int, D: int, dtype, len_range, seed: int, with_do: bool = False):
    """Seeded N(0,1) Q/K/V (generated in fp32 on the CPU, then cast) and per-batch valid lengths
    drawn uniformly from [len_lo, len_hi]."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, D, generator=g).to(dtype)
    k = torch.randn(B, H, S, D, generator=g).to(dtype)
    v = torch.randn(B, H, S, D, generator=g).to(dtype)
    lens = torch.randint(len_range[0], len_range[1] + 1, (B,), generator=g, dtype=torch.int32)
    out = dict(q=q, k=k, v=v, lens=lens)
    if with_do:
        out["d_o"] = torch.randn(B, H, S, D, generator=g).to(dtype)
    return out
