"""Shared builders for the GPU parity tests: seeded inputs, caches written through the public
API, and the CPU oracle's twin of the same cache."""
import math

import numpy as np
import torch

from oracle import CpuPools, ref_append, ref_attention, ref_dequantize

PAGE = 64


def make_kv(tokens, hkv, d, seed=0, outliers=False, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    k = torch.randn(tokens, hkv, d, generator=g)
    v = torch.randn(tokens, hkv, d, generator=g)
    if outliers:
        k = k * torch.exp(torch.randn(1, hkv, d, generator=g))
    return k.to(torch.bfloat16).to(device), v.to(torch.bfloat16).to(device)


def make_q(batch, hq, d, seed=1, scale=1.0, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(batch, hq, d, generator=g) * scale).clamp(-448, 448)
    return q.to(torch.float8_e4m3fn).to(device)


def paged_batch(seq_lens, seed=0, shuffle=True):
    """(indptr, indices, slots, num_pages) for requests of `seq_lens` tokens on a shuffled pool."""
    pages = [-(-int(n) // PAGE) for n in seq_lens]
    total = sum(pages)
    rng = np.random.default_rng(seed)
    order = rng.permutation(total) if shuffle else np.arange(total)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    indices = order.astype(np.int32)
    slots = []
    for b, n in enumerate(seq_lens):
        t = np.arange(int(n))
        slots.append(indices[indptr[b] + t // PAGE].astype(np.int64) * PAGE + t % PAGE)
    return indptr, indices, np.concatenate(slots) if slots else np.zeros(0, np.int64), total


def oracle_outputs(pools: CpuPools, q_fp8_cpu, indptr, indices, seq_lens, sm_scale,
                   q_descale=None, rounded=False):
    """fp32 softmax attention over the oracle's fp32 dequantized values (or, with `rounded`,
    over the bf16 read-back rows): (out [B,HQ,D], lse [B,HQ])."""
    kv = ref_dequantize(pools, indptr, indices, seq_lens, rounded=rounded)
    outs, lses = [], []
    for b in range(len(seq_lens)):
        o, l = ref_attention(q_fp8_cpu[b].float(), kv[b][0], kv[b][1], sm_scale,
                             None if q_descale is None else q_descale[b])
        outs.append(o)
        lses.append(l)
    return torch.stack(outs), torch.stack(lses)


def cpu_twin(cache, k, v, slots):
    """The oracle's pools after the same append."""
    lay = cache.layout
    kg = lay.k_quant[1] if lay.k_quant[1] < lay.head_dim else None
    pools = CpuPools(cache.num_pages, lay.num_kv_heads, lay.head_dim, lay.bits, k_group=kg,
                     scale_dtype=lay.scale_dtype)
    ref_append(pools, k.cpu(), v.cpu(), np.asarray(slots))
    return pools


def assert_pools_equal(cache, pools: CpuPools, pages=None):
    sel = slice(None) if pages is None else torch.as_tensor(sorted(pages))
    assert torch.equal(cache.k_codes.cpu()[sel], pools.k_codes[sel]), "k_codes differ"
    assert torch.equal(cache.v_codes.cpu()[sel], pools.v_codes[sel]), "v_codes differ"
    got = cache.scales.cpu()[sel].contiguous().view(torch.uint8)
    want = pools.scales[sel].contiguous().view(torch.uint8)
    assert torch.equal(got, want), "scale bytes differ"
    if cache.v_page_max is not None:
        vpm = cache.v_page_max.view(torch.int32).cpu().numpy().view(np.uint32)
        assert np.array_equal(vpm, pools.v_page_max), "v_page_max differs"
        hist = cache.v_max_hist.view(torch.int32).cpu().numpy().view(np.uint32)
        assert np.array_equal(hist, pools.v_max_hist), "v_max_hist differs"


def pools_of_requests(cache, indptr, indices, requests):
    """The oracle's pools filled with the cache's own bytes for the pages of `requests` only,
    renumbered from 0: (pools, indptr', indices'). For batches too large to write twice (once on
    the GPU, once by the CPU writer); the writer's bytes are compared elsewhere."""
    lay = cache.layout
    pages, new_indptr = [], [0]
    for b in requests:
        pages.extend(int(p) for p in indices[indptr[b]:indptr[b + 1]])
        new_indptr.append(len(pages))
    sel = torch.as_tensor(pages, dtype=torch.long, device=cache.k_codes.device)
    kg = lay.k_quant[1] if lay.k_quant[1] < lay.head_dim else None
    pools = CpuPools(len(pages), lay.num_kv_heads, lay.head_dim, lay.bits, k_group=kg,
                     scale_dtype=lay.scale_dtype)
    pools.k_codes = cache.k_codes[sel].cpu()
    pools.v_codes = cache.v_codes[sel].cpu()
    pools.scales = cache.scales[sel].cpu()
    return pools, np.asarray(new_indptr, dtype=np.int32), np.arange(len(pages), dtype=np.int32)
