"""Multi-GPU decode: how the path shards across the GPUs of one NVLink box.

The reference is a single-GPU library (no collective anywhere in it); these are the two ways
its decode path partitions:

* KV-head tensor parallel (batched serving): rank r owns KV heads [r*HKV/N, (r+1)*HKV/N) and the
  matching query heads, with its own cache, workspace and wrapper. Units are independent, so
  there is NO communication on the data path.
* Sequence split (one very long context): rank r holds the pages of a page-aligned token range
  and decodes it to a normalised (o, lse) pair; the pairs reach every rank's own memory and are
  merged there: out = sum_r exp(lse_r - L) o_r, L = logsumexp_r lse_r. Two forms of that
  exchange: `SequenceSplitExchange` (ONE launch per rank: plain stores into every peer's staging
  buffer through peer-mapped pointers, a flag, a bounded wait and the merge, all in the
  library's own kernel) and `gather_and_merge` (one NCCL all_gather plus the merge kernel).

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


class SequenceSplitExchange:
    """The cross-GPU step of a sequence split as one kernel launch per rank.

    Construction is collective over `group`: every rank allocates a staging buffer in torch's
    symmetric memory (peer-mapped into every process of the group) and learns the others'
    addresses. `run()` then launches the library's exchange kernel on the current stream: this
    rank's (o, lse) rows go into its slot of every rank's buffer with plain stores, the step is
    posted on a flag, the peers' flags are waited for (bounded: a peer that never posts sets the
    time-out status bit and leaves `out` untouched) and the rows are merged from this rank's own
    memory. No NCCL call, no copy kernel, no multicast on the data path."""

    def __init__(self, batch: int, num_qo_heads: int, head_dim: int, group=None, device=None):
        import os
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        # plain peer mappings only: no NVLink multicast object is bound to the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.shape = (batch, num_qo_heads, head_dim)
        self.device = torch.device("cuda", _dev.cuda_index(device))
        lib = _lib.load()
        nbytes = int(lib.fq_exchange_bytes(self.world, batch, num_qo_heads, head_dim))
        if nbytes < 0:
            _lib.check(nbytes, "exchange_bytes")
        self.buffer = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        handle = symm.rendezvous(self.buffer, self.group)
        self._handle = handle
        self._ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # every rank's zeroed flags are in place before anyone posts a step
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def last_status(self) -> int:
        return int(self.status.item())

    def run(self, o_local: torch.Tensor, lse_local: torch.Tensor, out: torch.Tensor,
            lse: Optional[torch.Tensor] = None, wait_budget_cycles: int = 0) -> torch.Tensor:
        """o_local f32 [B, HQ, D] and lse_local f32 [B, HQ] of this rank; `out` receives the
        merged rows (bf16 / f16 / f32), `lse` (optional) the merged log-sum-exp."""
        b, hq, d = self.shape
        if o_local.dtype != torch.float32 or tuple(o_local.shape) != (b, hq, d) \
                or not o_local.is_contiguous():
            raise ValueError(f"o_local must be a contiguous f32 [{b}, {hq}, {d}] tensor (plan the "
                             f"wrapper with o_data_type=torch.float32)")
        if lse_local.dtype != torch.float32 or tuple(lse_local.shape) != (b, hq) \
                or not lse_local.is_contiguous():
            raise ValueError(f"lse_local must be a contiguous f32 [{b}, {hq}] tensor")
        if tuple(out.shape) != (b, hq, d) or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous [{b}, {hq}, {d}] tensor")
        code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out.dtype]
        # step 0: the kernel counts the steps itself, so the call can be captured in a CUDA graph
        # and replayed (every rank replays the same number of times)
        with _dev.on_device(self.device):
            _lib.check(_lib.load().fq_exchange_merge(
                self._ptrs, self.rank, self.world, o_local.data_ptr(), lse_local.data_ptr(), b,
                hq, d, 0, out.data_ptr(), code,
                None if lse is None else lse.data_ptr(), wait_budget_cycles,
                self.status.data_ptr(), _dev.current_stream_ptr(self.device)), "exchange_merge")
        return out


def sequence_split_decode(wrapper, q, cache, group=None, out: Optional[torch.Tensor] = None,
                          exchange: Optional[SequenceSplitExchange] = None,
                          scratch=None) -> torch.Tensor:
    """One decode step of a sequence-split context: this rank's wrapper (planned over its own
    token range, with `o_data_type=torch.float32` so that the shards' outputs are not rounded to
    bf16 before the merge) produces (o, lse); the pairs are exchanged and merged on every rank:
    by `exchange` (one launch) when given, else by one NCCL all_gather and the merge kernel.
    `scratch` = (o f32 [B, HQ, D], lse f32 [B, HQ]) reuses caller-owned buffers."""
    b, hq, d = wrapper._batch_size, wrapper._num_qo_heads, wrapper._head_dim
    if scratch is None:
        local = torch.empty(b, hq, d, dtype=wrapper._o_data_type, device=q.device)
        lse = torch.empty(b, hq, dtype=torch.float32, device=q.device)
    else:
        local, lse = scratch
    wrapper.run(q, cache, out=local, lse=lse)
    if exchange is not None:
        if out is None:
            out = torch.empty(b, hq, d, dtype=torch.bfloat16, device=q.device)
        return exchange.run(local, lse, out)
    return gather_and_merge(local, lse, group, merged=out)
