"""Multi-GPU decode: how the path shards across the GPUs of one NVLink box.

The reference is a single-GPU library (no collective anywhere in it); these are the two ways
its decode path partitions:

* KV-head tensor parallel (batched serving): rank r owns KV heads [r*HKV/N, (r+1)*HKV/N) and the
  matching query heads, with its own cache, workspace and wrapper. Units are independent, so
  there is NO communication on the data path.
* Sequence split (one very long context): rank r holds the pages of a page-aligned token range
  and decodes it to a normalised (o, lse) pair; one all_gather of [B, HQ, D] + [B, HQ] floats
  per rank over NCCL (NVLink/NVSwitch) brings the pairs into every rank's own memory, and a
  local kernel merges them: out = sum_r exp(lse_r - L) o_r, L = logsumexp_r lse_r.

One process per GPU; `torch.distributed` is the plumbing.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib, device as _dev
from .pool_format import PAGE_SIZE


def shard_kv_heads(num_qo_heads: int, num_kv_heads: int, rank: int, world: int
                   ) -> Tuple[range, range]:
    """(query heads, KV heads) owned by `rank` under KV-head tensor parallelism."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads do not shard over {world} GPUs")
    if num_qo_heads % num_kv_heads:
        raise ValueError(f"num_qo_heads ({num_qo_heads}) must be a multiple of num_kv_heads "
                         f"({num_kv_heads})")
    per = num_kv_heads // world
    ratio = num_qo_heads // num_kv_heads
    return range(rank * per * ratio, (rank + 1) * per * ratio), range(rank * per, (rank + 1) * per)


def split_sequence(seq_len: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the page-aligned token range `rank` decodes of a `seq_len`-token context:
    pages are dealt as evenly as possible, earlier ranks taking the remainder."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    pages = -(-int(seq_len) // PAGE_SIZE)
    base, extra = divmod(pages, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(first * PAGE_SIZE, seq_len), min((first + count) * PAGE_SIZE, seq_len)


def gather_states(out: torch.Tensor, lse: torch.Tensor, group=None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """all_gather of every rank's (out [B, HQ, D], lse [B, HQ]) as f32: returns
    (o_shards [N, B, HQ, D], lse_shards [N, B, HQ]) in this rank's own memory."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    o32 = out.to(torch.float32).contiguous()
    l32 = lse.to(torch.float32).contiguous()
    # rank-major concatenation along the first dimension, viewed as [N, ...]
    o_all = torch.empty((world * o32.shape[0], *o32.shape[1:]), dtype=torch.float32,
                        device=o32.device)
    l_all = torch.empty((world * l32.shape[0], *l32.shape[1:]), dtype=torch.float32,
                        device=l32.device)
    dist.all_gather_into_tensor(o_all, o32, group=group)
    dist.all_gather_into_tensor(l_all, l32, group=group)
    return o_all.view(world, *o32.shape), l_all.view(world, *l32.shape)


def merge_states(o_shards: torch.Tensor, lse_shards: torch.Tensor,
                 out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None
                 ) -> torch.Tensor:
    """Merge (o, lse) pairs [N, B, HQ, D] / [N, B, HQ] held in local device memory with the
    library's merge kernel; a shard with lse = -inf (an empty range) contributes nothing."""
    if o_shards.dtype != torch.float32 or lse_shards.dtype != torch.float32:
        raise ValueError("merge_states takes f32 shards")
    if o_shards.device.type != "cuda":
        raise RuntimeError("merge_states runs the CUDA merge kernel; there is no CPU fallback")
    n, b, hq, d = o_shards.shape
    if tuple(lse_shards.shape) != (n, b, hq):
        raise ValueError(f"lse_shards must be [{n}, {b}, {hq}]; got {tuple(lse_shards.shape)}")
    o_shards, lse_shards = o_shards.contiguous(), lse_shards.contiguous()
    if out is None:
        out = torch.empty(b, hq, d, dtype=torch.bfloat16, device=o_shards.device)
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out.dtype]
    with _dev.on_device(o_shards.device):
        _lib.check(_lib.load().fq_merge_states(
            o_shards.data_ptr(), lse_shards.data_ptr(), n, b, hq, d, out.data_ptr(), code,
            None if lse is None else lse.data_ptr(), 0, 0,
            _dev.current_stream_ptr(o_shards.device)), "merge_states")
    return out


def gather_and_merge(out: torch.Tensor, lse: torch.Tensor, group=None,
                     merged: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The exchange step of a sequence split in ONE collective: this rank's (out [B, HQ, D],
    lse [B, HQ]) are packed as rows of D + 1 floats, all_gathered into local memory, and merged
    in place by the library's kernel (strided reads; no unpacking)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    b, hq, d = out.shape
    pack = torch.empty(b, hq, d + 1, dtype=torch.float32, device=out.device)
    pack[..., :d].copy_(out)
    pack[..., d].copy_(lse)
    packed = torch.empty(world * b, hq, d + 1, dtype=torch.float32, device=out.device)
    dist.all_gather_into_tensor(packed, pack, group=group)
    if merged is None:
        merged = torch.empty(b, hq, d, dtype=torch.bfloat16, device=out.device)
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[merged.dtype]
    base = packed.data_ptr()
    with _dev.on_device(out.device):
        _lib.check(_lib.load().fq_merge_states(
            base, base + 4 * d, world, b, hq, d, merged.data_ptr(), code, None, d + 1, d + 1,
            _dev.current_stream_ptr(out.device)), "merge_states")
    return merged


def sequence_split_decode(wrapper, q, cache, group=None, out: Optional[torch.Tensor] = None
                          ) -> torch.Tensor:
    """One decode step of a sequence-split context: this rank's wrapper (planned over its own
    token range) produces (o, lse); the pairs are gathered and merged on every rank. Plan the
    wrapper with `o_data_type=torch.float32` so that the shards' outputs are not rounded to
    bf16 before the merge."""
    b, hq, d = wrapper._batch_size, wrapper._num_qo_heads, wrapper._head_dim
    local = torch.empty(b, hq, d, dtype=wrapper._o_data_type, device=q.device)
    lse = torch.empty(b, hq, dtype=torch.float32, device=q.device)
    wrapper.run(q, cache, out=local, lse=lse)
    return gather_and_merge(local, lse, group, merged=out)
