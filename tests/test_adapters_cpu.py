"""Block-table adapter: padded page table -> the ragged (indptr, indices) of plan(), against a
plain host loop over the rows (the conversion docs/integration.md:61-76 of the reference gives)."""
import numpy as np
import pytest
import torch

from foscar_b200.adapters import (plan_inputs, plan_inputs_padded, seq_lens_of_last_page,
                                  slot_mapping_of)

PAGE = 64


def _loop(block_table, seq_lens):
    counts = [-(-int(n) // PAGE) for n in seq_lens]
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    rows = [block_table[b, :n] for b, n in enumerate(counts)]
    return indptr, (np.concatenate(rows) if rows else np.zeros(0)).astype(np.int32)


@pytest.mark.parametrize("lens", [[1], [64, 65, 1, 640], [0, 5, 0, 200, 64], [640] * 7])
def test_plan_inputs_matches_row_loop(lens):
    rng = np.random.default_rng(len(lens))
    width = max(1, max(-(-n // PAGE) for n in lens))
    table = rng.permutation(len(lens) * width).astype(np.int32).reshape(len(lens), width)
    want_ptr, want_idx = _loop(table, lens)
    ptr, idx, sl = plan_inputs(torch.from_numpy(table), torch.tensor(lens, dtype=torch.int64))
    assert ptr.dtype == idx.dtype == sl.dtype == torch.int32
    assert np.array_equal(ptr.numpy(), want_ptr)
    assert np.array_equal(idx.numpy(), want_idx)
    assert sl.tolist() == lens
    ptr2, padded, _ = plan_inputs_padded(torch.from_numpy(table), torch.tensor(lens))
    assert padded.shape[0] == table.size
    assert np.array_equal(padded.numpy()[:want_idx.size], want_idx)
    assert not padded.numpy()[want_idx.size:].any()
    assert torch.equal(ptr, ptr2)


def test_length_longer_than_the_row_is_clipped_to_it():
    table = torch.arange(6, dtype=torch.int32).view(2, 3)
    ptr, idx, sl = plan_inputs(table, torch.tensor([64 * 5, 10]))
    assert ptr.tolist() == [0, 3, 4] and idx.tolist() == [0, 1, 2, 3]
    assert sl.tolist() == [320, 10]      # plan() refuses: 320 tokens on 3 pages


def test_refusals():
    table = torch.zeros(2, 3, dtype=torch.int32)
    with pytest.raises(ValueError, match="pages hold 64"):
        plan_inputs(table, torch.tensor([1, 2]), page_size=16)
    with pytest.raises(ValueError, match=r"seq_lens must be \[2\]"):
        plan_inputs(table, torch.tensor([1, 2, 3]))
    with pytest.raises(ValueError, match="block_table must be"):
        plan_inputs(table.view(-1), torch.tensor([1, 2]))


def test_last_page_lengths_and_slots():
    ptr = torch.tensor([0, 3, 3, 4], dtype=torch.int32)
    lens = seq_lens_of_last_page(ptr, torch.tensor([7, 1, 64]))
    assert lens.tolist() == [135, 0, 64]
    table = torch.tensor([[9, 4, 2], [5, 0, 0]], dtype=torch.int32)
    slots = slot_mapping_of(table, torch.tensor([130, 64 * 3]))
    assert slots.dtype == torch.int64
    assert slots.tolist() == [2 * 64 + 2, -1]
