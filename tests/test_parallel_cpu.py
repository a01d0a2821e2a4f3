"""Multi-GPU host logic on CPU: head sharding, page-aligned sequence split, and the gather of
per-rank (o, lse) states over a world_size-2 gloo group; the merged result equals attention over
the whole context (merge math checked with the oracle, the CUDA merge kernel is GPU-only)."""
import math
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from foscar_b200 import parallel


def test_shard_kv_heads():
    q, kv = parallel.shard_kv_heads(64, 8, 3, 8)
    assert list(kv) == [3] and list(q) == list(range(24, 32))
    q, kv = parallel.shard_kv_heads(64, 8, 1, 2)
    assert list(kv) == [4, 5, 6, 7] and q == range(32, 64)
    with pytest.raises(ValueError):
        parallel.shard_kv_heads(64, 8, 0, 3)
    with pytest.raises(ValueError):
        parallel.shard_kv_heads(64, 8, 8, 8)


@pytest.mark.parametrize("seq,world", [(100352, 2), (100352, 8), (65, 4), (1, 8), (64 * 7 + 3, 3)])
def test_split_sequence_is_a_page_aligned_partition(seq, world):
    ranges = [parallel.split_sequence(seq, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == seq
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0 and a0 <= a1
    for a0, a1 in ranges:
        assert (a0 % 64 == 0 or a0 == seq) and (a1 % 64 == 0 or a1 == seq)
    sizes = [-(-(b - a) // 64) for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, seq, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)            # every rank builds the same context
        hq, d = 4, 32
        q = torch.randn(1, hq, d, generator=g)
        k = torch.randn(seq, d, generator=g)
        v = torch.randn(seq, d, generator=g)
        a, b = parallel.split_sequence(seq, rank, world)
        if b > a:
            s = torch.einsum("bhd,td->bht", q, k[a:b]) * 0.3
            lse = torch.logsumexp(s, -1)
            o = torch.softmax(s, -1) @ v[a:b]
        else:
            lse = torch.full((1, hq), -math.inf)
            o = torch.zeros(1, hq, d)
        o_all, l_all = parallel.gather_states(o, lse)
        assert o_all.shape == (world, 1, hq, d) and l_all.shape == (world, 1, hq)
        L = torch.logsumexp(l_all, 0)
        w = torch.exp(l_all - L)
        merged = (w.unsqueeze(-1) * o_all).sum(0)
        s = torch.einsum("bhd,td->bht", q, k) * 0.3
        want = torch.softmax(s, -1) @ v
        ok = torch.allclose(merged, want, atol=1e-5) and \
            torch.allclose(L, torch.logsumexp(s, -1), atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq", [1000, 40])
def test_sequence_split_gather_and_merge_over_gloo(seq):
    world = 2
    port = 29500 + (os.getpid() + seq) % 2000
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, seq, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_merge_states_has_no_cpu_fallback():
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        parallel.merge_states(torch.zeros(2, 1, 4, 8), torch.zeros(2, 1, 4))
