"""The reference-facing launch helpers (`foscar_b200.reference_binding`) and the block-table
adapter, driven the way the reference's cache and wrapper drive theirs: pools and tensors made
by the caller, keyword launches, no PagedDecodeWrapper in between. Output against the CPU
oracle under the decode tests' tolerance (max-abs 2e-2, mean-abs 2e-3, LSE 5e-2)."""
import numpy as np
import pytest
import torch

from helpers import PAGE, cpu_twin, make_kv, make_q, oracle_outputs, paged_batch, assert_pools_equal

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 5e-2


def _written_cache(bits, d, hkv, seq, seed):
    """Pools written through launch_quant_append; returns everything the fold launch takes."""
    from foscar_b200 import QuantKVLayout
    from foscar_b200 import reference_binding as rb
    indptr, indices, slots, npages = paged_batch(seq, seed=seed)
    k, v = make_kv(len(slots), hkv, d, seed=seed)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages + 1)          # the engine's pool tensors
    cache.k_codes.zero_(); cache.v_codes.zero_(); cache.scales.zero_()
    writer = rb.compile_quant_append(layout)
    rb.launch_quant_append(writer, inputs=(k, v), slot_mapping=torch.from_numpy(slots).cuda(),
                           k_codes=cache.k_codes, v_codes=cache.v_codes, scales=cache.scales,
                           v_page_max=cache.v_page_max, v_max_hist=cache.v_max_hist)
    torch.cuda.synchronize()
    assert int(writer.status.item()) == 0
    pools = cpu_twin(cache, k, v, slots)
    assert_pools_equal(cache, pools)
    return layout, cache, pools, indptr, indices


@pytest.mark.parametrize("bits,d", [(2, 128), (4, 128), (4, 64), (2, 256)])
@pytest.mark.parametrize("kv_splits,fused", [(1, False), (4, True), (4, False)])
def test_launch_fold_against_oracle(bits, d, kv_splits, fused):
    from foscar_b200 import reference_binding as rb
    hq, hkv, seq = 16, 2, [65, 1000, 4097, 1]
    layout, cache, pools, indptr, indices = _written_cache(bits, d, hkv, seq, seed=bits + d)
    b = len(seq)
    q = make_q(b, hq, d, seed=5).view(b, 1, hq, d)
    out = torch.full((b, 1, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((b, 1, hq), float("nan"), device="cuda")
    fold = rb.compile_fold(layout, num_qo_heads=hq, has_lse=True, batch_size=b,
                           fused_merge=fused)
    parts = {}
    if kv_splits > 1:
        parts = dict(o_partial=torch.empty(kv_splits, b, 1, hq, d, device="cuda"),
                     l_partial=torch.empty(kv_splits, b, 1, hq, device="cuda"),
                     m_partial=torch.empty(kv_splits, b, 1, hq, device="cuda"))
    sm_scale = d ** -0.5
    for _ in range(2):       # twice: the fused merge must leave its counters at zero
        out.fill_(float("nan"))
        rb.launch_fold(fold, kv_splits=kv_splits, seqlens=torch.tensor(seq, dtype=torch.int32).cuda(),
                       table_offsets=torch.from_numpy(indptr).cuda(),
                       page_table=torch.from_numpy(indices).cuda(), q_bshd=q, o_bshd=out,
                       scale_s=sm_scale, mKq=cache.k_codes, mVq=cache.v_codes,
                       mScale=cache.scales, v_max_hist=cache.v_max_hist, lse=lse, **parts)
        torch.cuda.synchronize()
        assert int(fold.status.item()) == 0
        want, lse_want = oracle_outputs(pools, q.view(b, hq, d).cpu(), indptr, indices, seq,
                                        sm_scale)
        err = (out.view(b, hq, d).float().cpu() - want).abs()
        assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS
        assert (lse.view(b, hq).cpu() - lse_want).abs().max().item() <= LSE_ABS
    if fold.unit_counters is not None:
        assert not fold.unit_counters.any().item()


def test_launch_fold_refuses_what_it_was_not_compiled_for():
    from foscar_b200 import reference_binding as rb
    layout, cache, pools, indptr, indices = _written_cache(4, 128, 2, [64], seed=1)
    fold = rb.compile_fold(layout, num_qo_heads=8)
    q = make_q(1, 8, 128).view(1, 1, 8, 128)
    out = torch.empty(1, 1, 8, 128, dtype=torch.bfloat16, device="cuda")
    kw = dict(kv_splits=1, seqlens=torch.tensor([64], dtype=torch.int32).cuda(),
              table_offsets=torch.from_numpy(indptr).cuda(),
              page_table=torch.from_numpy(indices).cuda(), q_bshd=q, o_bshd=out,
              mKq=cache.k_codes, mVq=cache.v_codes, mScale=cache.scales,
              v_max_hist=cache.v_max_hist)
    with pytest.raises(TypeError, match="has_lse"):
        rb.launch_fold(fold, lse=torch.empty(1, 1, 8, device="cuda"), **kw)
    with pytest.raises(TypeError, match="has_q_descale"):
        rb.launch_fold(fold, q_descale=torch.ones(1, 8, device="cuda"), **kw)


def test_launch_dequant_matches_cache_readback():
    from foscar_b200 import reference_binding as rb
    seq = [130, 64, 1]
    layout, cache, pools, indptr, indices = _written_cache(2, 128, 2, seq, seed=9)
    total = sum(seq)
    k_out = torch.empty(total, 2, 128, dtype=torch.bfloat16, device="cuda")
    v_out = torch.empty_like(k_out)
    out_indptr = torch.tensor(np.concatenate([[0], np.cumsum(seq)]), dtype=torch.int32).cuda()
    rb.launch_dequant(rb.compile_dequant(layout), k_codes=cache.k_codes, v_codes=cache.v_codes,
                      scales=cache.scales, k_out=k_out, v_out=v_out,
                      page_indptr=torch.from_numpy(indptr).cuda(),
                      page_indices=torch.from_numpy(indices).cuda(),
                      seq_lens=torch.tensor(seq, dtype=torch.int32).cuda(), out_indptr=out_indptr)
    from oracle import ref_dequantize
    want = ref_dequantize(pools, indptr, indices, seq, rounded=True)
    assert torch.equal(k_out.cpu(), torch.cat([w[0] for w in want]))
    assert torch.equal(v_out.cpu(), torch.cat([w[1] for w in want]))


@pytest.mark.parametrize("padded", [False, True])
def test_block_table_adapter_feeds_plan(padded):
    """An engine's padded block table through the adapter gives the same output as the ragged
    page list it stands for; the padded form's tail entries are never read."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    from foscar_b200.adapters import plan_inputs, plan_inputs_padded, slot_mapping_of
    bits, d, hq, hkv, seq = 4, 128, 16, 2, [1, 64, 65, 700, 2049]
    b = len(seq)
    indptr, indices, slots, npages = paged_batch(seq, seed=4)
    width = max(-(-n // PAGE) for n in seq) + 2
    table = np.full((b, width), npages + 7, dtype=np.int32)     # unused cells: a page id outside
    for r in range(b):
        n = indptr[r + 1] - indptr[r]
        table[r, :n] = indices[indptr[r]:indptr[r + 1]]
    table_t = torch.from_numpy(table).cuda()
    lens_t = torch.tensor(seq, dtype=torch.int64).cuda()
    k, v = make_kv(len(slots), hkv, d, seed=4)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages + 1)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    # the last token of each request, located through the table
    last = slot_mapping_of(table_t, lens_t - 1)
    want_last = torch.tensor([slots[sum(seq[:r + 1]) - 1] for r in range(b)])
    assert torch.equal(last.cpu(), want_last)
    ptr, idx, sl = (plan_inputs_padded if padded else plan_inputs)(table_t, lens_t)
    if padded:
        assert idx.shape[0] == b * width
    w = PagedDecodeWrapper(torch.empty(32 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(ptr, idx, sl.cpu(), hq, layout)
    q = make_q(b, hq, d, seed=6)
    out = w.run(q, cache)
    torch.cuda.synchronize()
    assert w.last_status() == 0
    pools = cpu_twin(cache, k, v, slots)
    want, _ = oracle_outputs(pools, q.cpu(), indptr, indices, seq, d ** -0.5)
    err = (out.float().cpu() - want).abs()
    assert err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS
