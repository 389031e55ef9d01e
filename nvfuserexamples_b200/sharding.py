"""Batch x heads partitioning of one attention call across the GPUs of a box.

Every (batch, head) pair is an independent attention problem (the reference already maps
B*H to blockIdx.y, shmsong/NvFuserExamples fmha/fmha_manual.cpp:279), so rank r of W takes a
contiguous slice of the flattened B*H axis and no data crosses NVLink: inputs live on the
shard's device and outputs stay sharded (gather_outputs() is there for a caller that wants them whole).  The only shared state is the Philox counter, which
uses the GLOBAL (b*H + h) index — `bh_offset` below — so a sharded run draws exactly the
bits of the unsharded one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    bh_start: int   # first flattened (b*H + h) index of this rank
    bh_count: int   # number of (b, h) pairs of this rank
    H: int

    @property
    def bh_offset(self) -> int:
        """Value to pass as `bh_offset` / philox_bh_offset."""
        return self.bh_start

    @property
    def whole_batches(self) -> bool:
        return self.bh_start % self.H == 0 and self.bh_count % self.H == 0


def shard_bounds(n_bh: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of range(n_bh): the first n_bh % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if n_bh < 0:
        raise ValueError("negative size")
    base, extra = divmod(n_bh, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def make_shard(B: int, H: int, world: int, rank: int) -> Shard:
    start, count = shard_bounds(B * H, world, rank)
    return Shard(rank, world, start, count, H)


def shard_tensor(x, shard: Shard):
    """[B,H,S,D] -> this rank's slice.  Whole batches keep the [b,H,S,D] form; a slice that cuts
    through a batch is returned as [bh_count,1,S,D] (heads folded into the batch axis)."""
    B, H = x.shape[0], x.shape[1]
    flat = x.reshape(B * H, 1, *x.shape[2:])
    part = flat[shard.bh_start:shard.bh_start + shard.bh_count]
    if shard.whole_batches:
        return part.reshape(shard.bh_count // H, H, *x.shape[2:])
    return part


def shard_per_batch(v, shard: Shard):
    """Per-batch metadata ([B] lengths or [B,S_k] mask rows) -> per local batch entry, matching
    the form shard_tensor() returned."""
    H = shard.H
    if shard.whole_batches:
        return v[shard.bh_start // H:(shard.bh_start + shard.bh_count) // H]
    import torch
    idx = torch.arange(shard.bh_start, shard.bh_start + shard.bh_count, device=v.device) // H
    return v.index_select(0, idx)


def gather_outputs(part, shard: Shard, B: int, group=None):
    """Optional: the sharded outputs of every rank (what shard_tensor() would slice from the full tensor)
    -> the full [B,H,...] tensor on every rank, by one all-gather over `group` (NCCL on GPUs, over
    NVLink/NVSwitch; gloo on CPU).  The attention path itself never needs this exchange.  Shards may
    differ by one (batch, head) pair, so every rank contributes a buffer padded to the largest shard."""
    import torch
    import torch.distributed as dist
    n = B * shard.H
    flat = part.reshape(shard.bh_count, *part.shape[2:])
    width = -(-n // shard.world)
    buf = flat.new_zeros((width,) + tuple(flat.shape[1:]))
    buf[:shard.bh_count] = flat
    bufs = [torch.empty_like(buf) for _ in range(shard.world)]
    dist.all_gather(bufs, buf, group=group)
    pieces = [b[:shard_bounds(n, shard.world, r)[1]] for r, b in enumerate(bufs)]
    return torch.cat(pieces).reshape(B, shard.H, *flat.shape[1:])
