"""CPU restatement of the channel-wise K page format (K quantized per channel over the 64
tokens of a page, V per token over the whole head). TEST INFRASTRUCTURE ONLY, like the rest of
`oracle/`: imported by `tests/`, `__graft_entry__.smoke()` and `bench.py`'s CPU legs, never by
the product.

PARITY UNPINNED. The reference defines where these bytes sit and how its decode reads them:
  - scale block sections [K ring | V ring | K channel | V channel], the channel section being
    [2, D] = row 0 s_d, row 1 z_d of the page's token group: src/foscar/quant_layout.py:9-21,
    57-85;
  - its decode reads s_d at k_ch + d and z_d at k_ch + D + d of the group's page:
    src/foscar/_sm100/int_fold_decode.py:5012-5036;
  - code rows are the token rows of every layout: src/foscar/_sm100/code_layout.py:24-43;
but it ships no writer, packer, fixture or numeric test for them (its append refuses channel-wise
layouts, src/foscar/kv_cache.py:643-644, 769-774). The quantizer arithmetic below is therefore
this library's choice: the token-wise writer's (src/foscar/_append_core.py:533-587: exact
min/max, z = clamp(min), s = max(max - z, 1e-8) / qmax, q = min(rint(max(x - z, 2^-60) / s),
qmax), the stored record rounded to the pool dtype while the codes use the f32 s) applied along
the token axis of a page. What these functions pin is that the CUDA writer, read-back and decode
agree with this statement of it.
"""
from __future__ import annotations

import numpy as np
import torch

from .ref_quant import (PAGE, _fma_f32, pack_rows, quantize_rows, ref_v_max_hist, saturate_given,
                        unpack_rows)


class CpuChannelPools:
    """k_codes, v_codes uint8 [NP, HKV, 64, RB]; scales [NP, HKV, 128 + 2 D] in the pool dtype:
    V ring (token t's (s_v, z_v) at 2 t) then K channel rows s_d, z_d; v_page_max, v_max_hist."""

    def __init__(self, num_pages, num_kv_heads, head_dim, bits, scale_dtype=torch.float32):
        self.num_pages, self.hkv, self.d, self.bits = num_pages, num_kv_heads, head_dim, bits
        self.scale_dtype = scale_dtype
        rb = head_dim * bits // 8
        self.k_codes = torch.zeros((num_pages, num_kv_heads, PAGE, rb), dtype=torch.uint8)
        self.v_codes = torch.zeros((num_pages, num_kv_heads, PAGE, rb), dtype=torch.uint8)
        self.v_ring, self.k_ch = 0, 2 * PAGE
        self.scales = torch.zeros((num_pages, num_kv_heads, 2 * PAGE + 2 * head_dim),
                                  dtype=scale_dtype)
        self.v_page_max = np.zeros((num_pages, num_kv_heads), dtype=np.uint32)
        self.v_max_hist = np.zeros(256, dtype=np.uint32)


def _write_page(pools: CpuChannelPools, p: int, n: int, kc, ks, kz, vc, vs, vz):
    """Store one page's first n tokens: K codes [n, HKV, D] with channel records ks, kz
    [HKV, D]; V codes [n, HKV, D] with token records vs, vz [n, HKV] (all records f32, rounded
    to the pool dtype here). The page's V ring is rebuilt from 0 and its maximum recomputed."""
    d, sd = pools.d, pools.scale_dtype
    pools.k_codes[p, :, :n] = pack_rows(kc, pools.bits).permute(1, 0, 2)
    pools.scales[p, :, pools.k_ch:pools.k_ch + d] = ks.to(sd)
    pools.scales[p, :, pools.k_ch + d:pools.k_ch + 2 * d] = kz.to(sd)
    pools.v_codes[p, :, :n] = pack_rows(vc, pools.bits).permute(1, 0, 2)
    ring = torch.zeros(pools.hkv, PAGE, 2, dtype=sd)
    ring[:, :n, 0] = vs.to(sd).t()
    ring[:, :n, 1] = vz.to(sd).t()
    pools.scales[p, :, :2 * PAGE] = ring.reshape(pools.hkv, 2 * PAGE)
    stored = vs.to(sd).float().contiguous().numpy().view(np.uint32)           # [n, HKV]
    pools.v_page_max[p] = stored.max(axis=0)


def _page_groups(pools: CpuChannelPools, page_ids, valid):
    page_ids = np.asarray(page_ids, dtype=np.int64)
    valid = np.full(len(page_ids), PAGE) if valid is None else np.asarray(valid, dtype=np.int64)
    for i, (p, n) in enumerate(zip(page_ids, valid)):
        n = min(int(n), PAGE)
        if n <= 0:
            continue
        if p < 0 or p >= pools.num_pages:
            raise IndexError("page outside the cache")
        yield i, int(p), n


def ref_append_page_groups(pools: CpuChannelPools, k, v, page_ids, valid=None):
    """Write whole page groups: k, v bf16 [P * 64, HKV, D], page i's tokens being rows
    [64 i, 64 i + valid[i]); page_ids [P]. K statistics run over the page's valid tokens only;
    rows past them are not written, their V records are cleared (every page starts at 0)."""
    for i, p, n in _page_groups(pools, page_ids, valid):
        rows = slice(PAGE * i, PAGE * i + n)
        # K: per (head, channel) over the n tokens
        x = k[rows].float().permute(1, 2, 0).contiguous()            # [HKV, D, n]
        codes, s, z = quantize_rows(x, pools.bits)                   # [HKV, D, n], [HKV, D, 1]
        # V: per token over the head
        vc, vs, vz = quantize_rows(v[rows], pools.bits)              # [n, HKV, D], [n, HKV, 1]
        _write_page(pools, p, n, codes.permute(2, 0, 1).contiguous(), s[..., 0], z[..., 0],
                    vc, vs[..., 0], vz[..., 0])
    pools.v_max_hist[:] = ref_v_max_hist(pools.v_page_max)


def ref_append_quantized_page_groups(pools: CpuChannelPools, k_codes, k_scale, k_zero, v_codes,
                                     v_scale, v_zero, page_ids, valid=None):
    """The layout-only form: k_codes, v_codes uint8 [P * 64, HKV, D] one value per byte; k_scale,
    k_zero f32 [P, HKV, D]; v_scale, v_zero f32 [P * 64, HKV]. Codes masked to the stored width
    and records saturated as the token-wise layout-only write does
    (src/foscar/kv_cache.py:689-767, src/foscar/_append_core.py:709-717)."""
    mask = (1 << pools.bits) - 1
    for i, p, n in _page_groups(pools, page_ids, valid):
        rows = slice(PAGE * i, PAGE * i + n)
        ks, kz = saturate_given(k_scale[i].float(), k_zero[i].float(), pools.bits)
        vs, vz = saturate_given(v_scale[rows].float(), v_zero[rows].float(), pools.bits)
        _write_page(pools, p, n, k_codes[rows] & mask, ks, kz, v_codes[rows] & mask, vs, vz)
    pools.v_max_hist[:] = ref_v_max_hist(pools.v_page_max)


def ref_dequantize_channel(pools: CpuChannelPools, page_indptr, page_indices, seq_lens,
                           rounded=True):
    """Per request (k_hat, v_hat) [len, HKV, D]: K through its page's channel records, V through
    its token record; bf16-rounded (the read-back) or the f32 fma result."""
    out = []
    d = pools.d
    sc = pools.scales.float()
    for b, n in enumerate(np.asarray(seq_lens)):
        n = int(n)
        pages = np.asarray(page_indices[int(page_indptr[b]):int(page_indptr[b + 1])])
        t = np.arange(n)
        pg, pos = pages[t // PAGE], t % PAGE
        kq = unpack_rows(pools.k_codes[pg, :, pos], pools.bits, d)      # [n, HKV, D]
        vq = unpack_rows(pools.v_codes[pg, :, pos], pools.bits, d)
        ks = sc[pg, :, pools.k_ch:pools.k_ch + d]                        # [n, HKV, D]
        kz = sc[pg, :, pools.k_ch + d:pools.k_ch + 2 * d]
        ring = sc[torch.as_tensor(pg), :, :2 * PAGE].reshape(n, pools.hkv, PAGE, 2)
        vs = ring[torch.arange(n), :, torch.as_tensor(pos)]             # [n, HKV, 2]
        k_hat = _fma_f32(ks, kq, kz)
        v_hat = _fma_f32(vs[..., 0:1], vq, vs[..., 1:2])
        if rounded:
            k_hat, v_hat = k_hat.to(torch.bfloat16), v_hat.to(torch.bfloat16)
        out.append((k_hat, v_hat))
    return out
