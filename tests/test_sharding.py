"""Host-side logic of the batch x heads sharding, on CPU: bounds, slicing, and a world-size-2
gloo run in which each rank evaluates its shard with the oracle and the gathered result must
equal the unsharded one bit for bit (same Philox bits through the global bh offset)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nvfuserexamples_b200 import sharding
from oracle import composite, philox


@pytest.mark.parametrize("n,world", [(512, 8), (1024, 4), (7, 3), (5, 8), (0, 2)])
def test_bounds_partition_the_range(n, world):
    got = [sharding.shard_bounds(n, world, r) for r in range(world)]
    assert got[0][0] == 0 and sum(c for _, c in got) == n
    for (s0, c0), (s1, _) in zip(got, got[1:]):
        assert s0 + c0 == s1
    assert max(c for _, c in got) - min(c for _, c in got) <= 1


def test_bad_rank_raises():
    with pytest.raises(ValueError):
        sharding.shard_bounds(8, 2, 2)
    with pytest.raises(ValueError):
        sharding.shard_bounds(8, 0, 0)


def test_slices_whole_batches_and_ragged():
    x = torch.arange(4 * 3 * 2 * 8).reshape(4, 3, 2, 8)
    lens = torch.tensor([5, 6, 7, 8])
    sh = sharding.make_shard(4, 3, 2, 1)      # 6 of 12 pairs, aligned to H=3
    assert sh.whole_batches and sh.bh_offset == 6
    assert torch.equal(sharding.shard_tensor(x, sh), x[2:4])
    assert torch.equal(sharding.shard_per_batch(lens, sh), lens[2:4])
    sh = sharding.make_shard(4, 3, 8, 2)      # 12 pairs over 8 ranks: cuts through batches
    assert not sh.whole_batches
    part = sharding.shard_tensor(x, sh)
    assert part.shape == (sh.bh_count, 1, 2, 8)
    assert torch.equal(part[:, 0], x.reshape(12, 2, 8)[sh.bh_start:sh.bh_start + sh.bh_count])
    assert torch.equal(sharding.shard_per_batch(lens, sh), lens[torch.arange(sh.bh_start, sh.bh_start + sh.bh_count) // 3])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, ragged: bool, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, S, D = (3, 3, 48, 64) if ragged else (4, 2, 48, 64)
        x = composite.make_inputs(B, H, S, D, torch.float16, (20, 48), seed=21)
        sh = sharding.make_shard(B, H, world, rank)
        q, k, v = (sharding.shard_tensor(x[n], sh) for n in ("q", "k", "v"))
        lens = sharding.shard_per_batch(x["lens"], sh)
        keep = torch.from_numpy(philox.dropout_keep_mask(5, 2, sh.bh_offset, sh.bh_count, S, S, 0.2).astype(np.float32))
        keep = keep.reshape(q.shape[0], q.shape[1], S, S)
        o = composite.attention_fp32(q, k, v, add_mask=composite.padding_add_mask(lens, S), keep=keep,
                                     keep_scale=philox.keep_scale(0.2))["o"].reshape(sh.bh_count, S, D)
        # the only collective is the optional gather of results; the data path has none
        full = sharding.gather_outputs(o.reshape(sh.bh_count, 1, S, D), sh, B).reshape(B * H, S, D)
        if rank == 0:
            keep_all = torch.from_numpy(philox.dropout_keep_mask(5, 2, 0, B * H, S, S, 0.2).astype(np.float32)).reshape(B, H, S, S)
            ref = composite.attention_fp32(x["q"], x["k"], x["v"], add_mask=composite.padding_add_mask(x["lens"], S),
                                           keep=keep_all, keep_scale=philox.keep_scale(0.2))["o"].reshape(B * H, S, D)
            out_q.put(bool(torch.equal(full, ref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ragged", [False, True])
def test_two_rank_gloo_sharded_equals_unsharded(ragged):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, ragged, out_q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out_q.get(timeout=10) is True
