"""Decode output through the public API against the fp32 oracle (fp32 dequantize + fp32 softmax
on CPU).

Tolerance (bf16 output vs the oracle): max-abs <= 2e-2 and mean-abs <= 2e-3; LSE within 5e-2
absolute. A second check scores the output against the cache's own bf16 read-back the way the
reference's GPU test does (global relative L2 < 6e-3, tests/test_cache_gpu.py:22-27) on N(0,1)
inputs, where the read-back's bf16 rounding does not dominate."""
import math

import numpy as np
import pytest
import torch

from helpers import PAGE, cpu_twin, make_kv, make_q, oracle_outputs, paged_batch

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 5e-2


def _run_case(bits, d, hq, hkv, seq, *, kv_splits=None, host_lens=True, outliers=False,
              q_scale=1.0, lse=True, q_descale=False, out_dtype=torch.bfloat16, seed=0,
              reduction="auto", max_kv_len=None, scale_dtype=None, k_quant=None):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    batch = len(seq)
    indptr, indices, slots, npages = paged_batch(seq, seed=seed)
    k, v = make_kv(len(slots), hkv, d, seed=seed, outliers=outliers)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda",
                                  scale_dtype=scale_dtype, k_quant=k_quant)
    cache = layout.allocate(npages + 1)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(batch, hq, d, seed=seed + 1, scale=q_scale)
    sm_scale = d ** -0.5 / q_scale
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    lens = torch.tensor(seq, dtype=torch.int32)
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           lens if host_lens else lens.cuda(), hq, layout, sm_scale=sm_scale,
           kv_splits=kv_splits, o_data_type=out_dtype, reduction=reduction,
           max_kv_len=max_kv_len)
    out = torch.full((batch, hq, d), float("nan"), dtype=out_dtype, device="cuda")
    lse_t = torch.full((batch, hq), float("nan"), device="cuda") if lse else None
    qd = None
    if q_descale:
        qd = (torch.rand(batch, hq, generator=torch.Generator().manual_seed(7)) + 0.5).cuda()
    w.run(q, cache, out=out, lse=lse_t, q_descale=qd)
    torch.cuda.synchronize()
    assert w.last_status() == 0, w.last_status()
    pools = cpu_twin(cache, k, v, slots)
    want, lse_want = oracle_outputs(pools, q.cpu(), indptr, indices, seq, sm_scale,
                                    None if qd is None else qd.cpu())
    err = (out.float().cpu() - want).abs()
    assert torch.isfinite(out.float()).all()
    assert err.max().item() <= MAX_ABS, f"max-abs {err.max().item():.3e}"
    assert err.mean().item() <= MEAN_ABS, f"mean-abs {err.mean().item():.3e}"
    if lse:
        assert (lse_t.cpu() - lse_want).abs().max().item() <= LSE_ABS
    if not outliers:
        back, _ = oracle_outputs(pools, q.cpu(), indptr, indices, seq, sm_scale,
                                 None if qd is None else qd.cpu(), rounded=True)
        rel = ((out.float().cpu() - back).norm() / back.norm()).item()
        assert rel < 6e-3, f"rel-L2 vs read-back {rel:.3e}"
    return w, out, err


def test_config1_cpu_reference_case():
    """INT4, B=2, 32/8 heads, D=128, two full pages per request."""
    _run_case(4, 128, 32, 8, [128, 128])


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 2), (8, 8), (24, 2)])
def test_ragged_batch(bits, hq, hkv):
    _run_case(bits, 128, hq, hkv, [1, 63, 64, 65, 129, 1000, 4097], seed=bits)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("hq,hkv", [(64, 8), (8, 2), (4, 4)])
def test_head_dim_64(bits, hq, hkv):
    """head_dim 64 (operand rows half used): ragged batch, planned splits."""
    _run_case(bits, 64, hq, hkv, [1, 64, 130, 2000, 9000], seed=3 + bits)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("hq,hkv", [(16, 2), (8, 2), (24, 1)])
def test_head_dim_256(bits, hq, hkv):
    """head_dim 256 (two operand rows per token, two channel halves of the PV product): ragged
    batch, planned splits, GQA 8 / 4 / 24 (three head tiles)."""
    _run_case(bits, 256, hq, hkv, [1, 63, 64, 65, 129, 1000, 4097, 9000], seed=17 + bits)


@pytest.mark.parametrize("bits", [2, 4])
def test_head_dim_256_splits_scales_and_outliers(bits):
    _run_case(bits, 256, 16, 2, [5000, 257], kv_splits=3, host_lens=False)
    _run_case(bits, 256, 16, 2, [3000, 130], scale_dtype=torch.bfloat16, seed=19)
    _run_case(bits, 256, 16, 2, [20000, 700], outliers=True, q_scale=8.0, seed=23, q_descale=True)


@pytest.mark.parametrize("bits,d", [(2, 128), (4, 128), (2, 64), (4, 64)])
def test_bf16_scale_pools(bits, d):
    """Scale records stored as bf16 pairs (8 bytes a token): the decode reads the pool's own
    rounded values, as the oracle's dequantize does."""
    _run_case(bits, d, 32, 8, [1, 64, 130, 3000], seed=11, scale_dtype=torch.bfloat16)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("hq,hkv", [(32, 8), (16, 2)])
def test_k_groups_of_64_channels(bits, hq, hkv):
    """K quantized per token over 64-channel groups (two (s, z) pairs per token, bf16 rings):
    each group's partial score comes out of its own S column."""
    _run_case(bits, 128, hq, hkv, [1, 64, 130, 3000, 700], seed=13, k_quant=("token", 64),
              outliers=True)


@pytest.mark.parametrize("bits", [2, 4])
def test_head_dim_64_uniform_splits(bits):
    _run_case(bits, 64, 64, 8, [5000, 257], kv_splits=3, host_lens=False)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("kv_splits", [1, 4, 7, None])
def test_uniform_and_planned_splits(bits, kv_splits):
    w, _, _ = _run_case(bits, 128, 32, 8, [4096, 700], kv_splits=kv_splits, host_lens=False,
                        max_kv_len=4096 if kv_splits is None else None)
    assert w.kv_splits >= 1


def test_balanced_plan_splits_long_request():
    w, _, _ = _run_case(2, 128, 32, 8, [20000, 130], seed=3)
    assert w.kv_splits > 1 and w.reduction == "kernel"


def test_outlier_keys_fp8_query_scale():
    """K with per-channel log-normal magnitudes, q = e4m3(8 q) with sm_scale / 8."""
    _run_case(2, 128, 32, 8, [3000, 5000], outliers=True, q_scale=8.0, seed=5)


@pytest.mark.parametrize("bits,d,hq,hkv", [(2, 128, 32, 8), (4, 64, 16, 2), (4, 256, 16, 2)])
def test_rows_that_carry_their_request_change_nothing(bits, d, hq, hkv):
    """A planned list whose rows carry the request's length and table offset (what plan() makes)
    and one whose rows leave them to the device arrays (a C caller's list that was not passed
    through fq_worklist_attach_requests) give the same bits."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = [9000, 1, 333, 4097]
    indptr, indices, slots, npages = paged_batch(seq, seed=13)
    k, v = make_kv(len(slots), hkv, d, seed=13)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(len(seq), hq, d)
    outs, lses = [], []
    for carry in (True, False):
        w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
        w.carry_requests = carry
        w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
               torch.tensor(seq, dtype=torch.int32), hq, layout)
        header = w._worklist[:8].cpu()
        assert int(header[4]) == int(carry)
        out = torch.empty(len(seq), hq, d, dtype=torch.bfloat16, device="cuda")
        lse = torch.empty(len(seq), hq, device="cuda")
        w.run(q, cache, out=out, lse=lse)
        torch.cuda.synchronize()
        assert w.last_status() == 0
        outs.append(out)
        lses.append(lse)
    assert torch.equal(outs[0], outs[1]) and torch.equal(lses[0], lses[1])


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_output_dtypes_and_descale(out_dtype):
    _run_case(4, 128, 16, 4, [300, 900], out_dtype=out_dtype, q_descale=True)


def test_reduction_none_forces_one_piece():
    w, _, _ = _run_case(2, 128, 32, 8, [9000], reduction="none")
    assert w.kv_splits == 1 and w.reduction == "none"


def test_run_is_deterministic():
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = [5000, 333, 8000]
    indptr, indices, slots, npages = paged_batch(seq, seed=9)
    k, v = make_kv(len(slots), 8, 128, seed=9)
    layout = QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=8, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(3, 32, 128)
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), 32, layout)
    outs = []
    for _ in range(3):
        out = torch.empty(3, 32, 128, dtype=torch.bfloat16, device="cuda")
        w.run(q, cache, out=out)
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("kv_splits", [5, None])
def test_in_kernel_merge_equals_merge_launch(kv_splits):
    """Split units merged by their last piece inside the decode launch give the bytes the
    separate merge launch gives (same arithmetic, same slot order), launch after launch: the
    arrival counters reset themselves."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = [7000, 150, 12000, 64]
    indptr, indices, slots, npages = paged_batch(seq, seed=4)
    k, v = make_kv(len(slots), 8, 128, seed=4)
    layout = QuantKVLayout.create(bits=4, head_dim=128, num_kv_heads=8, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(len(seq), 32, 128)
    lens = torch.tensor(seq, dtype=torch.int32)
    results = []
    for fused in (False, True, True):
        w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
        w.fused_merge = fused
        w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
               lens.cuda() if kv_splits else lens, 32, layout, kv_splits=kv_splits)
        assert w.kv_splits > 1
        for _ in range(2):
            out = torch.full((len(seq), 32, 128), float("nan"), dtype=torch.bfloat16,
                             device="cuda")
            lse = torch.full((len(seq), 32), float("nan"), device="cuda")
            before = w.launches
            w.run(q, cache, out=out, lse=lse)
            assert w.launches - before == (1 if fused else 2)
            results.append((out, lse))
        torch.cuda.synchronize()
        assert w.last_status() == 0
    for out, lse in results[1:]:
        assert torch.equal(out, results[0][0]) and torch.equal(lse, results[0][1])


def test_empty_request_in_a_batch():
    """A request of length 0 next to live ones: its rows come out zero with lse = -inf, the
    others are unaffected (uniform and balanced plans)."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = [300, 0, 70]
    indptr, indices, slots, npages = paged_batch(seq, seed=2)
    k, v = make_kv(len(slots), 8, 128, seed=2)
    layout = QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=8, device="cuda")
    cache = layout.allocate(npages + 1)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(3, 32, 128)
    live = [0, 2]
    for lens_on_host, splits in ((True, None), (False, 2)):
        w = PagedDecodeWrapper(torch.empty(16 << 20, dtype=torch.uint8, device="cuda"))
        lens = torch.tensor(seq, dtype=torch.int32)
        w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
               lens if lens_on_host else lens.cuda(), 32, layout, kv_splits=splits)
        out = torch.full((3, 32, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((3, 32), float("nan"), device="cuda")
        w.run(q, cache, out=out, lse=lse)
        torch.cuda.synchronize()
        assert w.last_status() == 0
        assert torch.all(out[1] == 0) and torch.all(torch.isneginf(lse[1]))
        assert torch.isfinite(out[0].float()).all() and torch.isfinite(out[2].float()).all()
        assert torch.isfinite(lse[0]).all() and torch.isfinite(lse[2]).all()
        # the live rows equal a batch without the empty request
        w2 = PagedDecodeWrapper(torch.empty(16 << 20, dtype=torch.uint8, device="cuda"))
        keep = np.concatenate([indices[indptr[0]:indptr[1]], indices[indptr[2]:indptr[3]]])
        ip2 = np.array([0, indptr[1] - indptr[0], indptr[1] - indptr[0] + indptr[3] - indptr[2]],
                       dtype=np.int32)
        w2.plan(torch.from_numpy(ip2).cuda(), torch.from_numpy(keep.astype(np.int32)).cuda(),
                torch.tensor([300, 70], dtype=torch.int32), 32, layout, kv_splits=1)
        ref = w2.run(q[live].contiguous(), cache)
        torch.cuda.synchronize()
        assert (out[live].float() - ref.float()).abs().max().item() <= 1e-2


@pytest.mark.parametrize("bits,d", [(4, 64), (2, 128), (4, 256)])
def test_many_single_tile_items(bits, d):
    """Hundreds of one-tile work items per CTA: most worker groups have no tile in most items,
    while the producer runs items ahead. Repeated launches must neither time out (status bit
    0x10) nor differ."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    rng = np.random.default_rng(5)
    seq = [int(x) for x in rng.integers(1, 200, 320)]
    hq, hkv = 64, 8
    indptr, indices, slots, npages = paged_batch(seq, seed=5)
    k, v = make_kv(len(slots), hkv, d, seed=5)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(len(seq), hq, d)
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), hq, layout)
    first = None
    for _ in range(30):
        out = w.run(q, cache)
        if first is None:
            first = out.clone()
    torch.cuda.synchronize()
    assert w.last_status() == 0, w.last_status()
    assert torch.equal(out, first)
    pools = cpu_twin(cache, k, v, slots)
    some = [0, 17, 319]
    for b in some:
        want, _ = oracle_outputs(pools, q.cpu()[b:b + 1], indptr[b:b + 2] - indptr[b],
                                 indices[indptr[b]:indptr[b + 1]], [seq[b]], d ** -0.5)
        err = (out[b].float().cpu() - want[0]).abs()
        assert err.max().item() <= MAX_ABS, (b, err.max().item())


@pytest.mark.parametrize("stages", ["4", "5", "6", "7"])
def test_shallow_rings(stages, monkeypatch):
    """The shared-memory ring at its smallest depths (the library rounds an odd request down):
    same results, no timeout. INT4 at head_dim 64 runs at six stages in production."""
    monkeypatch.setenv("FOSCAR_B200_RING_STAGES", stages)
    _run_case(2, 128, 32, 8, [9000, 4097, 130], seed=31)
    _run_case(4, 64, 64, 8, [9000, 300], seed=32)


def test_pdl_flag_does_not_change_the_result():
    """enable_pdl only changes how the launch is ordered after the one before it."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    seq = [2000, 130]
    indptr, indices, slots, npages = paged_batch(seq, seed=21)
    k, v = make_kv(len(slots), 8, 128, seed=21)
    layout = QuantKVLayout.create(bits=4, head_dim=128, num_kv_heads=8, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(2, 32, 128)
    w = PagedDecodeWrapper(torch.empty(16 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), 32, layout)
    a = w.run(q, cache, enable_pdl=True)
    b = w.run(q, cache, enable_pdl=False)
    c = w.run(q, cache, enable_pdl=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(a, c) and w.last_status() == 0
    # a decode step: the writer rewrites the last tokens, the decode follows on the same stream;
    # under a programmatic launch its set-up overlaps the writer's tail, its reads do not
    tail = torch.from_numpy(slots[-3:]).cuda()
    k2, v2 = make_kv(3, 8, 128, seed=22)
    outs = []
    for pdl in (True, False, True):
        cache.append(k2, v2, tail)
        outs.append(w.run(q, cache, enable_pdl=pdl))
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert not torch.equal(outs[0], a) and w.last_status() == 0 and cache.last_status() == 0


def test_bad_page_id_sets_status_without_fault():
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    layout = QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=2, device="cuda")
    cache = layout.allocate(4)
    k, v = make_kv(256, 2, 128)
    cache.append(k, v, torch.arange(256, device="cuda"))
    w = PagedDecodeWrapper(torch.empty(1 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.tensor([0, 4], dtype=torch.int32), torch.tensor([0, 99, 2, -5], dtype=torch.int32),
           torch.tensor([256], dtype=torch.int32), 8, layout)
    out = torch.empty(1, 8, 128, dtype=torch.bfloat16, device="cuda")
    w.run(make_q(1, 8, 128), cache, out=out)
    torch.cuda.synchronize()
    assert w.last_status() & 0x2
