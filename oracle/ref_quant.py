"""CPU oracle (torch on CPU, numpy) for the quantized-KV decode path. Test infrastructure:
never imported by the product.

Every function restates reference behaviour and cites the file:line (paths inside the
reference project) it follows. The reference's device kernels are CuTe-DSL programs with no CPU
form, so these are restatements of their arithmetic, not the reference's code.
"""
from __future__ import annotations

import math
import struct

import numpy as np
import torch

PAGE = 64
S_CLAMP = 1.0e-8                 # src/foscar/_append_core.py:199
INPUT_ENVELOPE = 2.0 ** 64       # src/foscar/_append_core.py:203
DIVIDEND_FLOOR = 2.0 ** -60      # src/foscar/_append_core.py:207


# ------------------------------------------------------------------------------------------
# Code placement (src/foscar/_sm100/code_layout.py:24-43; docs/K_STORE_PERM.md:31-65)
# ------------------------------------------------------------------------------------------

def code_channel(bits: int, word: int, field: int) -> int:
    """Channel held by field `field` of word `word`: W*word + field//2 + (W/2)*(field%2)."""
    per_word = 32 // bits
    return per_word * word + field // 2 + (per_word // 2) * (field % 2)


def _bit_offsets(bits: int, head_dim: int) -> np.ndarray:
    """Bit offset inside a token row of every channel (docs/K_STORE_PERM.md:47-54)."""
    per_word = 32 // bits
    c = np.arange(head_dim)
    within = c % per_word
    field = 2 * (within % (per_word // 2)) + within // (per_word // 2)
    return (c // per_word) * 32 + bits * field


def pack_rows(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """uint8 codes [..., D] (one per byte) -> packed rows uint8 [..., D*bits/8], little-endian
    32-bit words in the production store order."""
    d = codes.shape[-1]
    flat = codes.reshape(-1, d).numpy().astype(np.uint32) & ((1 << bits) - 1)
    off = _bit_offsets(bits, d)
    words = np.zeros((flat.shape[0], d * bits // 32), dtype=np.uint32)
    for c in range(d):
        words[:, off[c] // 32] |= flat[:, c] << np.uint32(off[c] % 32)
    out = words.view(np.uint8).reshape(*codes.shape[:-1], d * bits // 8)
    return torch.from_numpy(out.copy())


def unpack_rows(rows: torch.Tensor, bits: int, head_dim: int) -> torch.Tensor:
    """Packed rows uint8 [..., D*bits/8] -> codes uint8 [..., D] in channel order."""
    flat = np.ascontiguousarray(rows.reshape(-1, rows.shape[-1]).numpy()).view(np.uint32)
    off = _bit_offsets(bits, head_dim)
    mask = np.uint32((1 << bits) - 1)
    out = np.empty((flat.shape[0], head_dim), dtype=np.uint8)
    for c in range(head_dim):
        out[:, c] = (flat[:, off[c] // 32] >> np.uint32(off[c] % 32)) & mask
    return torch.from_numpy(out.reshape(*rows.shape[:-1], head_dim))


# ------------------------------------------------------------------------------------------
# Quantizer (src/foscar/_append_core.py:533-587)
# ------------------------------------------------------------------------------------------

def _f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def scale_range(qmax: int):
    """(lowest, highest) stored scale (src/foscar/_append_core.py:235-241)."""
    return _f32(_f32(S_CLAMP) / qmax), _f32(2.0 * INPUT_ENVELOPE / qmax)


def clip_rows(x: torch.Tensor, index: int) -> torch.Tensor:
    """Per-row clip to +-(the element at `index` of the row's sorted |x|)
    (src/foscar/kv_cache.py:104-118; src/foscar/_append_core.py:500-531)."""
    if index < 0:
        return x
    t = x.abs().sort(dim=-1).values[..., index:index + 1]
    return torch.minimum(torch.maximum(x, -t), t)


def quantize_rows(x: torch.Tensor, bits: int, groups: int = 1, clip_index: int = -1):
    """bf16/f32 rows [..., D] -> (codes uint8 [..., D], s f32 [..., groups], z f32 [..., groups]).

    All f32, each step one correctly rounded operation: z = clamp(min), s = max(clamp(max) - z,
    1e-8) / qmax, q = min(rint_even(max(x - z, 2^-60) / s), qmax). The clip threshold comes from
    the whole row even when K is grouped."""
    qmax = float((1 << bits) - 1)
    f = clip_rows(x.float(), clip_index)
    d = f.shape[-1]
    g = f.reshape(*f.shape[:-1], groups, d // groups)
    bound = torch.tensor(INPUT_ENVELOPE, dtype=torch.float32)
    mn = g.amin(dim=-1)
    mx = g.amax(dim=-1)
    z = torch.minimum(torch.maximum(mn, -bound), bound)
    top = torch.minimum(torch.maximum(mx, -bound), bound)
    s = torch.maximum(top - z, torch.tensor(S_CLAMP, dtype=torch.float32)) / qmax
    gc = torch.minimum(torch.maximum(g, -bound), bound)
    dividend = torch.maximum(gc - z.unsqueeze(-1), torch.tensor(DIVIDEND_FLOOR))
    # fmax semantics: a NaN dividend falls to the floor
    dividend = torch.where(torch.isnan(dividend), torch.tensor(DIVIDEND_FLOOR), dividend)
    q = torch.round(dividend / s.unsqueeze(-1)).clamp_max(qmax)
    codes = q.to(torch.uint8).reshape(*f.shape)
    return codes, s, z


def saturate_given(s: torch.Tensor, z: torch.Tensor, bits: int):
    """Saturation of engine-given records (src/foscar/_append_core.py:709-717): fmax then fmin,
    NaN to the lower bound."""
    lo, hi = scale_range((1 << bits) - 1)
    s = torch.where(torch.isnan(s), torch.tensor(lo), s).clamp(lo, hi)
    z = torch.where(torch.isnan(z), torch.tensor(-INPUT_ENVELOPE), z).clamp(-INPUT_ENVELOPE,
                                                                          INPUT_ENVELOPE)
    return s.float(), z.float()


# ------------------------------------------------------------------------------------------
# Page maxima (src/foscar/_sm100/fold_runtime.py:135-245)
# ------------------------------------------------------------------------------------------

def ref_vmax_bucket(bits):
    """Exponent bin of an f32 bit pattern; works on ints and numpy arrays."""
    if isinstance(bits, np.ndarray):
        b = np.minimum(bits.astype(np.int64) & 0x7FFFFFFF, 0x7F800000)
        return (b + 0x1FFFFF) >> 23
    return (min(int(bits) & 0x7FFFFFFF, 0x7F800000) + 0x1FFFFF) >> 23


def ref_v_max_hist(v_page_max: np.ndarray) -> np.ndarray:
    """Count table of a set of page maxima: cells with a nonzero magnitude, by bin."""
    bits = v_page_max.astype(np.int64).reshape(-1) & 0x7FFFFFFF
    hist = np.zeros(256, dtype=np.uint32)
    np.add.at(hist, ref_vmax_bucket(bits.astype(np.uint32))[bits != 0], 1)
    return hist


def ref_pscale_lp(hist: np.ndarray) -> int:
    """lp = 135 - max(top nonzero bin, 27) (src/foscar/_sm100/int_fold_decode.py:2528-2578)."""
    nz = np.nonzero(hist)[0]
    top = int(nz[-1]) if len(nz) else 0
    return 135 - max(top, 27)


# ------------------------------------------------------------------------------------------
# Pools and the writer (src/foscar/kv_cache.py:405-455; src/foscar/_append_core.py:18-22,73-109)
# ------------------------------------------------------------------------------------------

def _sections(k_groups: int, head_dim: int):
    """Scale-block sections of a token-wise layout (src/foscar/quant_layout.py:57-85)."""
    if k_groups == 1:
        return dict(legacy=True, block_tot=4 * PAGE, v_ring=0)
    kr = 2 * k_groups * PAGE
    return dict(legacy=False, block_tot=kr + 2 * PAGE, v_ring=kr)


class CpuPools:
    """CPU twin of a token-wise cache: k_codes, v_codes uint8 [NP,HKV,64,RB]; scales
    [NP,HKV,64,4] (whole-head K) or [NP,HKV,block_tot]; v_page_max uint32 [NP,HKV];
    v_max_hist uint32 [256]."""

    def __init__(self, num_pages, num_kv_heads, head_dim, bits, k_group=None,
                 scale_dtype=torch.float32, fill=0):
        self.num_pages, self.hkv, self.d, self.bits = num_pages, num_kv_heads, head_dim, bits
        self.k_groups = 1 if k_group is None else head_dim // k_group
        self.scale_dtype = scale_dtype
        self.sec = _sections(self.k_groups, head_dim)
        rb = head_dim * bits // 8
        self.k_codes = torch.full((num_pages, num_kv_heads, PAGE, rb), fill, dtype=torch.uint8)
        self.v_codes = torch.full((num_pages, num_kv_heads, PAGE, rb), fill, dtype=torch.uint8)
        shape = ((num_pages, num_kv_heads, PAGE, 4) if self.sec["legacy"]
                 else (num_pages, num_kv_heads, self.sec["block_tot"]))
        self.scales = torch.zeros(shape, dtype=scale_dtype)
        if fill:
            self.scales.view(torch.uint8).fill_(fill)
        self.v_page_max = np.zeros((num_pages, num_kv_heads), dtype=np.uint32)
        self.v_max_hist = np.zeros(256, dtype=np.uint32)

    # scale records as [NP,HKV,64,...] views ------------------------------------------------
    def _k_records(self):
        if self.sec["legacy"]:
            return self.scales[..., 0:2]
        return self.scales[..., :self.sec["v_ring"]].reshape(
            self.num_pages, self.hkv, PAGE, 2 * self.k_groups)

    def _v_records(self):
        if self.sec["legacy"]:
            return self.scales[..., 2:4]
        vr = self.sec["v_ring"]
        return self.scales[..., vr:vr + 2 * PAGE].reshape(self.num_pages, self.hkv, PAGE, 2)


def _write_tokens(pools: CpuPools, slots, k_codes, k_s, k_z, v_codes, v_s, v_z):
    """Lay quantized tokens out: code rows, scale records rounded to the pool dtype, tail clear
    of every page a token of this launch starts at position 0, page maxima and the count table.

    Final-state semantics of one launch without duplicate valid slots
    (src/foscar/_append_core.py:73-109): a page holding a position-0 token keeps (0,0) records at
    every position no token of the launch writes and its maximum is the largest stored s_v of the
    launch's tokens in it; any other page's maximum is max(old, that)."""
    slots = np.asarray(slots, dtype=np.int64)
    valid = slots >= 0
    if (slots[valid] >= pools.num_pages * PAGE).any():
        raise IndexError("slot outside the cache")
    idx = np.nonzero(valid)[0]
    if len(idx) == 0:
        return
    page, pos = slots[idx] // PAGE, slots[idx] % PAGE
    kq = pack_rows(k_codes[idx], pools.bits)
    vq = pack_rows(v_codes[idx], pools.bits)
    sd = pools.scale_dtype
    ks, kz = k_s[idx].to(sd), k_z[idx].to(sd)          # [n, HKV, groups]
    vs, vz = v_s[idx].to(sd), v_z[idx].to(sd)          # [n, HKV, 1]
    # tail clear first, then the launch's own records overwrite their positions
    starts = np.unique(page[pos == 0])
    krec, vrec = pools._k_records(), pools._v_records()
    for p in starts:
        krec[p] = 0
        vrec[p] = 0
    pools.k_codes[page, :, pos] = kq
    pools.v_codes[page, :, pos] = vq
    krec[page, :, pos] = torch.stack([ks, kz], dim=-1).reshape(len(idx), pools.hkv, -1)
    vrec[page, :, pos] = torch.stack([vs, vz], dim=-1).reshape(len(idx), pools.hkv, 2)
    # page maxima: bit pattern of the largest STORED s_v (widened to f32)
    sv_bits = vs[..., 0].float().contiguous().numpy().view(np.uint32)      # [n, HKV]
    for p in starts:
        pools.v_page_max[p] = 0
    np.maximum.at(pools.v_page_max, page, sv_bits)
    pools.v_max_hist[:] = ref_v_max_hist(pools.v_page_max)


def ref_append(pools: CpuPools, k: torch.Tensor, v: torch.Tensor, slots, k_clip_index=-1,
               v_clip_index=-1):
    """`QuantKVCache.append` (src/foscar/kv_cache.py:618-687): k, v bf16 [T, HKV, D]."""
    kc, ks, kz = quantize_rows(k, pools.bits, pools.k_groups, k_clip_index)
    vc, vs, vz = quantize_rows(v, pools.bits, 1, v_clip_index)
    _write_tokens(pools, slots, kc, ks, kz, vc, vs, vz)


def ref_append_quantized(pools: CpuPools, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero,
                         slots):
    """`QuantKVCache.append_quantized` (src/foscar/kv_cache.py:689-767): codes masked to the
    stored width, records saturated."""
    t, h = k_codes.shape[:2]
    ks, kz = saturate_given(k_scale.reshape(t, h, -1), k_zero.reshape(t, h, -1), pools.bits)
    vs, vz = saturate_given(v_scale.reshape(t, h, 1), v_zero.reshape(t, h, 1), pools.bits)
    mask = (1 << pools.bits) - 1
    _write_tokens(pools, slots, k_codes & mask, ks, kz, v_codes & mask, vs, vz)


# ------------------------------------------------------------------------------------------
# Read-back (src/foscar/_dequant_core.py:19-25) and the attention reference
# (tests/test_cache_gpu.py:84-95)
# ------------------------------------------------------------------------------------------

def _fma_f32(s, q, z):
    """fma.rn.f32(s, q, z): the product s*q is exact in f64 (24+4 bits) and the f64 sum of it
    and z rounds to f32 once more without double-rounding error for these magnitudes."""
    return (s.double() * q.double() + z.double()).float()


def ref_dequantize(pools: CpuPools, page_indptr, page_indices, seq_lens, rounded=True):
    """Per request, (k_hat, v_hat) [len, HKV, D] = bf16_rne(fma(s, q, z)), the cache's read-back.
    `rounded=False` keeps the f32 fma result: the "fp32 dequantize" the decode's tolerance is
    stated against (the decode never rounds a K or V value to bf16)."""
    out = []
    krec, vrec = pools._k_records().float(), pools._v_records().float()
    for b, n in enumerate(np.asarray(seq_lens)):
        n = int(n)
        pages = np.asarray(page_indices[int(page_indptr[b]):int(page_indptr[b + 1])])
        t = np.arange(n)
        pg, pos = pages[t // PAGE], t % PAGE
        kq = unpack_rows(pools.k_codes[pg, :, pos], pools.bits, pools.d)     # [n,HKV,D]
        vq = unpack_rows(pools.v_codes[pg, :, pos], pools.bits, pools.d)
        kr = krec[pg, :, pos].reshape(n, pools.hkv, pools.k_groups, 2)
        ks = kr[..., 0].repeat_interleave(pools.d // pools.k_groups, dim=-1)
        kz = kr[..., 1].repeat_interleave(pools.d // pools.k_groups, dim=-1)
        vr = vrec[pg, :, pos]
        k_hat = _fma_f32(ks, kq, kz)
        v_hat = _fma_f32(vr[..., 0:1], vq, vr[..., 1:2])
        if rounded:
            k_hat, v_hat = k_hat.to(torch.bfloat16), v_hat.to(torch.bfloat16)
        out.append((k_hat, v_hat))
    return out


def ref_attention(q: torch.Tensor, k_hat: torch.Tensor, v_hat: torch.Tensor, sm_scale: float,
                  q_descale=None):
    """fp32 softmax(q K^T * sm_scale) V for one request: q [HQ, D] (the FP8-rounded query as
    float), k_hat/v_hat [T, HKV, D]. Returns (out f32 [HQ, D], natural-log lse f32 [HQ])."""
    hq, d = q.shape
    hkv = k_hat.shape[1]
    g = hq // hkv
    qf = q.float()
    if q_descale is not None:
        qf = qf * q_descale.float().reshape(hq, 1)
    qb = qf.reshape(hkv, g, d)
    kb = k_hat.permute(1, 0, 2).float()
    vb = v_hat.permute(1, 0, 2).float()
    scores = torch.einsum("hgd,htd->hgt", qb, kb) * sm_scale
    lse = torch.logsumexp(scores, dim=-1).reshape(hq)
    out = torch.einsum("hgt,htd->hgd", torch.softmax(scores, -1), vb).reshape(hq, d)
    return out, lse


def ref_merge(o_partial, l_partial, m_partial, o_scale=1.0):
    """Split-KV merge (src/foscar/_sm100/gqa_decode.py:666-761): partials [S, ..., D], m in the
    log2 domain; rows whose M is -inf give zeros."""
    M = m_partial.max(dim=0).values
    w = torch.exp2(m_partial - M.unsqueeze(0))
    w = torch.where(torch.isfinite(M).unsqueeze(0), w, torch.zeros_like(w))
    den = (w * l_partial).sum(0)
    out = (w.unsqueeze(-1) * o_partial).sum(0) / den.unsqueeze(-1) * o_scale
    out = torch.where((den > 0).unsqueeze(-1), out, torch.zeros_like(out))
    lse = (M + torch.log2(den)) * math.log(2.0)
    return out, lse


# ------------------------------------------------------------------------------------------
# Model of the fold arithmetic (src/foscar/_sm100/int_fold_decode.py:5-22, 378-434): used to
# check that the E4M3 hi/lo P representation meets the stated tolerance before any GPU run.
# ------------------------------------------------------------------------------------------

def _e4m3(x: torch.Tensor) -> torch.Tensor:
    """Round to E4M3 (saturating to +-448) and widen back to f32."""
    return x.clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()


def emulate_fold_decode(q: torch.Tensor, k_codes, k_s, k_z, v_codes, v_s, v_z, sm_scale: float,
                        lp: int, tile: int = 128):
    """One (request, KV head): q [g, D] f32 (FP8 values), codes [T, D] uint8, records [T] f32.

    score = s_k (q . c_k) + z_k sum(q); running max per `tile` tokens; w = P s_v 2^lp stored as
    E4M3 hi + lo/16; O = sum w c_v; the V offset enters once through sum(w/s_v/2^lp * z_v).
    Returns (out f32 [g, D], natural-log lse [g])."""
    g, d = q.shape
    t_all = k_codes.shape[0]
    log2e = math.log2(math.e)
    qsum = q.sum(dim=-1)                                           # [g]
    m = torch.full((g,), -math.inf)
    l = torch.zeros(g)
    c = torch.zeros(g)
    o = torch.zeros(g, d)
    for t0 in range(0, t_all, tile):
        sl = slice(t0, min(t0 + tile, t_all))
        raw = k_codes[sl].float() @ q.t()                          # [n, g]
        x = (k_s[sl, None] * raw + k_z[sl, None] * qsum[None, :]) * (sm_scale * log2e)
        m_new = torch.maximum(m, x.max(dim=0).values)
        corr = torch.exp2(m - m_new)
        e = torch.exp2(x - m_new[None, :])
        w = e * (v_s[sl, None] * 2.0 ** lp)
        hi = _e4m3(w)
        lo = _e4m3((w - hi) * 16.0)
        wq = hi + lo / 16.0
        pq = torch.where(wq > 0, wq / (v_s[sl, None] * 2.0 ** lp), e)
        l = l * corr + e.sum(0)
        c = c * corr + (pq * v_z[sl, None]).sum(0)
        o = o * corr[:, None] + wq.t() @ v_codes[sl].float()
        m = m_new
    out = (o * 2.0 ** (-lp) + c[:, None]) / l[:, None]
    lse = (m + torch.log2(l)) * math.log(2.0)
    return out, lse
