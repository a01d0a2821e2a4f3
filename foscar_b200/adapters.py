"""Block-table adapters: an engine's padded page table to the ragged form `plan()` takes.

Engines of the SGLang / vLLM family keep one row of physical page ids per request,
`block_table` int32 [batch, pages_per_row], plus the KV lengths in tokens. The decode plans on
the ragged pair (`indptr` [batch + 1], `indices` [pages in use]) of the reference's `plan()`
(docs/integration.md:41-76 gives the conversion as a host loop over the rows). The functions
here do it with device tensor ops only, so they can sit in a captured step:

  - `plan_inputs`        exact-size `indices` (one host read for the total page count);
  - `plan_inputs_padded` fixed-size `indices` [batch * pages_per_row] whose tail past
                         `indptr[-1]` is page 0 and is never read (no host read at all).

Nothing here touches the cache; `slot_mapping_of` is the matching helper for the writer.
"""
from __future__ import annotations

import torch

from .pool_format import PAGE_SIZE


def _page_counts(seq_lens: torch.Tensor, pages_per_row: int, page_size: int) -> torch.Tensor:
    if page_size != PAGE_SIZE:
        raise ValueError(f"the cache's pages hold {PAGE_SIZE} tokens; got page_size={page_size}")
    counts = (seq_lens.to(torch.int64) + (page_size - 1)) // page_size
    return counts.clamp_(0, pages_per_row)


def _check(block_table: torch.Tensor, seq_lens: torch.Tensor) -> None:
    if block_table.dim() != 2:
        raise ValueError(f"block_table must be [batch, pages_per_row]; got "
                         f"{tuple(block_table.shape)}")
    if seq_lens.dim() != 1 or seq_lens.shape[0] != block_table.shape[0]:
        raise ValueError(f"seq_lens must be [{block_table.shape[0]}]; got "
                         f"{tuple(seq_lens.shape)}")
    if seq_lens.device != block_table.device:
        raise ValueError(f"seq_lens is on {seq_lens.device}, block_table on "
                         f"{block_table.device}")


def plan_inputs_padded(block_table: torch.Tensor, seq_lens: torch.Tensor,
                       page_size: int = PAGE_SIZE):
    """(indptr int32 [B + 1], indices int32 [B * pages_per_row], seq_lens int32 [B]).

    Entry j < indptr[-1] of `indices` is page (j - indptr[b]) of request b, b found by a
    binary search of j in indptr; later entries are 0. No value is read on the host, every
    output has a shape fixed by the inputs' shapes. A length that needs more pages than the
    row holds is clipped to the row; `plan()` then refuses it (its lengths check)."""
    _check(block_table, seq_lens)
    batch, width = block_table.shape
    dev = block_table.device
    counts = _page_counts(seq_lens, width, page_size)
    indptr = torch.zeros(batch + 1, dtype=torch.int64, device=dev)
    torch.cumsum(counts, 0, out=indptr[1:])
    j = torch.arange(batch * width, device=dev, dtype=torch.int64)
    row = torch.searchsorted(indptr[1:], j, right=True).clamp_(max=max(batch - 1, 0))
    col = (j - indptr[row]).clamp_(0, max(width - 1, 0))
    live = j < indptr[-1]
    flat = block_table.reshape(-1).to(torch.int32)
    indices = torch.where(live, flat[row * width + col] if batch * width else flat,
                          torch.zeros((), dtype=torch.int32, device=dev))
    return indptr.to(torch.int32), indices, seq_lens.to(torch.int32)


def plan_inputs(block_table: torch.Tensor, seq_lens: torch.Tensor, page_size: int = PAGE_SIZE):
    """(indptr int32 [B + 1], indices int32 [pages in use], seq_lens int32 [B]): the padded
    form cut at the page count (one host read)."""
    indptr, indices, lens = plan_inputs_padded(block_table, seq_lens, page_size)
    return indptr, indices[:int(indptr[-1])], lens


def seq_lens_of_last_page(indptr: torch.Tensor, last_page_len: torch.Tensor,
                          page_size: int = PAGE_SIZE) -> torch.Tensor:
    """KV lengths in tokens for a scheduler that tracks each request's last page fill
    (in [1, page_size]) instead of a token count; a request without pages has length 0."""
    pages = (indptr[1:] - indptr[:-1]).to(torch.int64)
    lens = (pages - 1) * page_size + last_page_len.to(torch.int64)
    return torch.where(pages > 0, lens, torch.zeros_like(lens)).to(torch.int32)


def slot_mapping_of(block_table: torch.Tensor, positions: torch.Tensor,
                    page_size: int = PAGE_SIZE) -> torch.Tensor:
    """int64 [B] cache slots (`page * page_size + offset`) of token `positions[b]` of each
    request, the `slot_mapping` of `cache.append` for a decode step that adds one token per
    request. A position past the row's pages gives slot -1 (the writer skips negative slots)."""
    if page_size != PAGE_SIZE:
        raise ValueError(f"the cache's pages hold {PAGE_SIZE} tokens; got page_size={page_size}")
    pos = positions.to(torch.int64)
    col = pos // page_size
    inside = (pos >= 0) & (col < block_table.shape[1])
    page = block_table.to(torch.int64).gather(
        1, col.clamp(0, max(block_table.shape[1] - 1, 0)).view(-1, 1)).view(-1)
    return torch.where(inside, page * page_size + pos % page_size, torch.full_like(pos, -1))
