"""The benchmark configurations at their own sizes, through the public API, against the fp32
oracle (fp32 dequantize of the cache's bytes + fp32 softmax on CPU).

* long-context INT2: 100,352-token prefixes (1,568 pages), batch 1 and 4: every request checked.
* serving sweep shape: head_dim 64, 64 query / 8 KV heads, INT2 and INT4, batch 256, lengths
  log-uniform in [64, 131072], eager and CUDA-graph mode: the longest, the shortest and a few
  seeded requests are checked per run (the oracle over all 4.5 M tokens would take minutes).
* the reference's own acceptance cases (tests/test_cache_gpu.py:98-122 there): 16 query / 2 KV
  heads, head_dim 64, kv_splits 1 / 4 / planner's choice, decode of a cache written by one
  append, by append_quantized, and by an append plus a 3-token tail append; both of its metrics
  (relative L2 < 6e-3 against the read-back rows, LSE within 5e-2).

Tolerance against the fp32 oracle: max-abs <= 2e-2, mean-abs <= 2e-3, LSE <= 5e-2."""
import math

import numpy as np
import pytest
import torch

from helpers import (PAGE, cpu_twin, make_kv, make_q, oracle_outputs, paged_batch,
                     pools_of_requests)

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 5e-2


def _fill_cache(layout, seq, hkv, d, seed, outliers, chunk=1 << 18):
    """A cache holding requests of `seq` tokens on a shuffled pool, written by the library's own
    append in chunks (K with per-channel log-normal magnitudes when `outliers`)."""
    indptr, indices, slots, npages = paged_batch(seq, seed=seed)
    cache = layout.allocate(npages)
    g = torch.Generator(device="cuda").manual_seed(seed)
    mult = torch.exp(torch.randn(1, hkv, d, device="cuda", generator=g)) if outliers else None
    slots_dev = torch.from_numpy(slots).cuda()
    for a in range(0, len(slots), chunk):
        n = min(chunk, len(slots) - a)
        k = torch.randn(n, hkv, d, device="cuda", generator=g)
        if mult is not None:
            k = k * mult
        v = torch.randn(n, hkv, d, device="cuda", generator=g)
        cache.append(k.to(torch.bfloat16), v.to(torch.bfloat16), slots_dev[a:a + n])
    torch.cuda.synchronize()
    assert cache.last_status() == 0
    return cache, indptr, indices


def _check_requests(out, lse, cache, q, indptr, indices, seq, requests, sm_scale):
    pools, ip, ix = pools_of_requests(cache, indptr, indices, requests)
    lens = [int(seq[b]) for b in requests]
    want, lse_want = oracle_outputs(pools, q.cpu()[requests], ip, ix, lens, sm_scale)
    got = out.float().cpu()[requests]
    err = (got - want).abs()
    assert torch.isfinite(got).all()
    assert err.max().item() <= MAX_ABS, f"max-abs {err.max().item():.3e} (requests {requests})"
    assert err.mean().item() <= MEAN_ABS, f"mean-abs {err.mean().item():.3e}"
    if lse is not None:
        assert (lse.cpu()[requests] - lse_want).abs().max().item() <= LSE_ABS


@pytest.mark.parametrize("batch", [1, 4])
def test_long_context_int2_at_100k_tokens(batch):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    hq, hkv, d, n = 32, 8, 128, 100352
    seq = [n] * batch
    layout = QuantKVLayout.create(bits=2, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache, indptr, indices = _fill_cache(layout, seq, hkv, d, seed=40 + batch, outliers=True)
    q = make_q(batch, hq, d, seed=3, scale=8.0)
    sm_scale = d ** -0.5 / 8.0
    w = PagedDecodeWrapper(torch.empty(256 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), hq, layout, sm_scale=sm_scale)
    assert w.kv_splits > 1 and w.reduction == "kernel"
    out = torch.full((batch, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((batch, hq), float("nan"), device="cuda")
    w.run(q, cache, out=out, lse=lse)
    torch.cuda.synchronize()
    assert w.last_status() == 0
    for b in range(batch):
        _check_requests(out, lse, cache, q, indptr, indices, seq, [b], sm_scale)


def _serving_lengths(batch, lo, hi, seed):
    rng = np.random.default_rng(seed)
    seq = np.round(np.exp(rng.uniform(math.log(lo), math.log(hi), batch))).astype(np.int64)
    seq[0], seq[1] = hi, lo          # both ends of the range are always present
    return [int(x) for x in seq]


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("graph", [False, True])
def test_serving_sweep_shape_batch_256(bits, graph):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    from foscar_b200.wrapper import graph_workspace_bytes
    batch, hq, hkv, d = 256, 64, 8, 64
    seq = _serving_lengths(batch, 64, 131072, seed=50 + bits)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache, indptr, indices = _fill_cache(layout, seq, hkv, d, seed=60 + bits, outliers=False)
    q = make_q(batch, hq, d, seed=4, scale=8.0)
    sm_scale = d ** -0.5 / 8.0
    out = torch.full((batch, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((batch, hq), float("nan"), device="cuda")
    if not graph:
        w = PagedDecodeWrapper(torch.empty(256 << 20, dtype=torch.uint8, device="cuda"))
        w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
               torch.tensor(seq, dtype=torch.int32), hq, layout, sm_scale=sm_scale)
        w.run(q, cache, out=out, lse=lse)
    else:
        max_pages = max(-(-n // PAGE) for n in seq)
        table = torch.zeros(batch, max_pages, dtype=torch.int32)
        for b in range(batch):
            row = indices[indptr[b]:indptr[b + 1]]
            table[b, :len(row)] = torch.from_numpy(row)
        table = table.cuda()
        lens_dev = torch.tensor(seq, dtype=torch.int32, device="cuda")
        need = graph_workspace_bytes(batch, hq, layout, max_kv_len=131072, device="cuda")
        w = PagedDecodeWrapper(torch.empty(need, dtype=torch.uint8, device="cuda"),
                               use_cuda_graph=True)
        w.plan(page_table=table, seq_lens=lens_dev, num_qo_heads=hq, layout=layout,
               max_kv_len=131072, sm_scale=sm_scale, lse=True)
        w.update(seq)
        w.run(q, cache, out=out, lse=lse)          # warm-up outside the graph
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            w.run(q, cache, out=out, lse=lse)
        out.fill_(float("nan"))
        # a skewed step first (one long request, the others short), then the step under test
        skew = [131072] + [64] * (batch - 1)
        lens_dev.copy_(torch.tensor(skew, dtype=torch.int32))
        w.update(skew)
        g.replay()
        lens_dev.copy_(torch.tensor(seq, dtype=torch.int32))
        w.update(seq)
        g.replay()
    torch.cuda.synchronize()
    assert w.last_status() == 0
    assert torch.isfinite(out.float()).all()
    rng = np.random.default_rng(7)
    sample = [0, 1] + [int(x) for x in rng.choice(np.arange(2, batch), 4, replace=False)]
    _check_requests(out, lse, cache, q, indptr, indices, seq, sample, sm_scale)


def _rel_l2(a, b):
    return ((a - b).norm() / b.norm()).item()


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("kv_splits", [1, 4, None])
@pytest.mark.parametrize("mode", ["normal", "prequantized", "short_tail"])
def test_reference_acceptance_cases(bits, kv_splits, mode):
    """16 query / 2 KV heads, head_dim 64: decode against the cache's own read-back rows, by the
    reference's two metrics."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    from oracle import quantize_rows
    hq, hkv, d = 16, 2, 64
    seq = [777, 2050, 64]
    tail = 3 if mode == "short_tail" else 0
    indptr, indices, slots, npages = paged_batch(seq, seed=70)
    k, v = make_kv(len(slots), hkv, d, seed=71)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages)
    slots_dev = torch.from_numpy(slots).cuda()
    if mode == "prequantized":
        kc, ks, kz = quantize_rows(k.float().cpu(), bits)
        vc, vs, vz = quantize_rows(v.float().cpu(), bits)
        cache.append_quantized(kc.cuda(), ks[..., 0].contiguous().cuda(),
                               kz[..., 0].contiguous().cuda(), vc.cuda(),
                               vs[..., 0].contiguous().cuda(), vz[..., 0].contiguous().cuda(),
                               slots_dev)
    elif mode == "short_tail":
        # every request's last 3 tokens arrive in a second append (a decode step's write)
        ends = np.cumsum(seq)
        is_tail = np.zeros(len(slots), dtype=bool)
        for e in ends:
            is_tail[e - tail:e] = True
        head_idx = torch.from_numpy(np.nonzero(~is_tail)[0]).cuda()
        tail_idx = torch.from_numpy(np.nonzero(is_tail)[0]).cuda()
        cache.append(k[head_idx], v[head_idx], slots_dev[head_idx])
        cache.append(k[tail_idx], v[tail_idx], slots_dev[tail_idx])
    else:
        cache.append(k, v, slots_dev)
    q = make_q(len(seq), hq, d, seed=72)
    sm_scale = d ** -0.5
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    lens = torch.tensor(seq, dtype=torch.int32)
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           lens if kv_splits is None else lens.cuda(), hq, layout, sm_scale=sm_scale,
           kv_splits=kv_splits)
    out = torch.empty(len(seq), hq, d, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(len(seq), hq, device="cuda")
    w.run(q, cache, out=out, lse=lse)
    torch.cuda.synchronize()
    assert w.last_status() == 0 and cache.last_status() == 0
    # the reference's check: fp32 attention over the cache's own bf16 read-back rows
    total = sum(seq)
    k_back = torch.empty(total, hkv, d, dtype=torch.bfloat16, device="cuda")
    v_back = torch.empty_like(k_back)
    out_indptr = torch.tensor(np.concatenate([[0], np.cumsum(seq)[:-1]]), dtype=torch.int32,
                              device="cuda")
    cache.dequantize(k_back, v_back, torch.from_numpy(indptr).cuda(),
                     torch.from_numpy(indices).cuda(), lens.cuda(), out_indptr)
    torch.cuda.synchronize()
    qf = q.float()
    a = 0
    for b, n in enumerate(seq):
        kb = k_back[a:a + n].float().repeat_interleave(hq // hkv, dim=1)   # [n, HQ, D]
        vb = v_back[a:a + n].float().repeat_interleave(hq // hkv, dim=1)
        scores = torch.einsum("hd,nhd->hn", qf[b], kb) * sm_scale
        want_lse = torch.logsumexp(scores, dim=-1)
        want = torch.einsum("hn,nhd->hd", torch.softmax(scores, dim=-1), vb)
        assert _rel_l2(out[b].float(), want) < 6e-3
        assert (lse[b] - want_lse).abs().max().item() < 5e-2
        a += n


def test_a_wait_that_runs_out_returns_and_leaves_the_context_usable():
    """The give-up path of the bounded device waits: a kernel whose threads wait ~1 ms for a
    barrier phase nothing completes returns with the time-out status bit; a decode launched
    afterwards on the same context gives the bytes it gave before."""
    import ctypes
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, _lib
    lib = _lib.load()
    seq = [3000, 130]
    indptr, indices, slots, npages = paged_batch(seq, seed=80)
    k, v = make_kv(len(slots), 8, 128, seed=80)
    layout = QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=8, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(2, 32, 128)
    w = PagedDecodeWrapper(torch.empty(16 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), 32, layout)
    before = w.run(q, cache).clone()
    torch.cuda.synchronize()
    words = torch.zeros(2, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.fq_wait_selftest(2_000_000, words.data_ptr(), words.data_ptr() + 4,
                              ctypes.c_void_p(stream))
    assert rc == 0
    torch.cuda.synchronize()
    status, gave_up = (int(x) for x in words.cpu())
    assert status == _lib.STATUS_TIMEOUT and gave_up == 1
    assert lib.fq_wait_selftest(0, words.data_ptr(), None, None) == _lib.ERR_BAD_ARG
    after = w.run(q, cache)
    torch.cuda.synchronize()
    assert w.last_status() == 0
    assert torch.equal(before, after)


def test_exchange_kernel_alone_and_its_give_up_path():
    """The sequence split's exchange kernel on one GPU: a world of one merges its own rows; in a
    world of two whose other rank never posts, the bounded wait runs out, the time-out bit is
    set, the output is left as it was and the context stays usable."""
    import ctypes
    from foscar_b200 import _lib
    lib = _lib.load()
    b, hq, d = 2, 8, 128
    o = torch.randn(b, hq, d, device="cuda")
    lse = torch.randn(b, hq, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # world of one
    buf = torch.zeros(int(lib.fq_exchange_bytes(1, b, hq, d)), dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
    out = torch.zeros(b, hq, d, device="cuda")
    lse_out = torch.zeros(b, hq, device="cuda")
    for step in (1, 2, 3):
        assert lib.fq_exchange_merge(ptrs, 0, 1, o.data_ptr(), lse.data_ptr(), b, hq, d, step,
                                     out.data_ptr(), 2, lse_out.data_ptr(), 0, status.data_ptr(),
                                     stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.allclose(out, o, atol=1e-6) and torch.allclose(lse_out, lse, atol=1e-6)
    # world of two, the other rank silent: ~1 ms, then the give-up path
    n2 = int(lib.fq_exchange_bytes(2, b, hq, d))
    mine = torch.zeros(n2, dtype=torch.uint8, device="cuda")
    other = torch.zeros(n2, dtype=torch.uint8, device="cuda")
    ptrs2 = (ctypes.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    out.fill_(7.0)
    # (step 2: the even steps use the first half of the staging area)
    assert lib.fq_exchange_merge(ptrs2, 0, 2, o.data_ptr(), lse.data_ptr(), b, hq, d, 2,
                                 out.data_ptr(), 2, None, 2_000_000, status.data_ptr(),
                                 stream) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.STATUS_TIMEOUT
    assert torch.all(out == 7.0)
    # the silent rank's slot holds what this rank sent it
    sent = other.view(torch.float32)[:b * hq * (d + 1)].view(b * hq, d + 1)
    assert torch.equal(sent[:, :d], o.view(b * hq, d)) and torch.equal(sent[:, d], lse.view(-1))
    assert lib.fq_exchange_merge(ptrs2, 2, 2, o.data_ptr(), lse.data_ptr(), b, hq, d, 1,
                                 out.data_ptr(), 2, None, 0, None, stream) == _lib.ERR_BAD_ARG
