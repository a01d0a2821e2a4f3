"""The CPU oracle against the reference's known-answer vectors and against vectors generated
from the reference's own host functions (tests/golden/reference_host.json)."""
import math
import struct

import numpy as np
import torch

from oracle import (CpuPools, code_channel, emulate_fold_decode, pack_rows, quantize_rows,
                    ref_append, ref_append_quantized, ref_attention, ref_dequantize, ref_merge,
                    ref_pscale_lp, ref_v_max_hist, ref_vmax_bucket, scale_range, unpack_rows)
from oracle.ref_quant import clip_rows


def test_packing_known_answers():
    # docs/K_STORE_PERM.md:63-64
    r = pack_rows(torch.tensor([[i % 4 for i in range(16)]], dtype=torch.uint8), 2)
    assert r.numpy().view(np.uint32)[0, 0] == 0xFA50FA50
    r = pack_rows(torch.tensor([list(range(8))], dtype=torch.uint8), 4)
    assert r.numpy().view(np.uint32)[0, 0] == 0x73625140


def test_channel_order_per_word():
    # docs/K_STORE_PERM.md:42-43
    assert [code_channel(2, 0, f) for f in range(16)] == [0, 8, 1, 9, 2, 10, 3, 11, 4, 12, 5, 13,
                                                           6, 14, 7, 15]
    assert [code_channel(4, 0, f) for f in range(8)] == [0, 4, 1, 5, 2, 6, 3, 7]


def test_code_field_matches_reference(golden):
    for bits in (2, 4):
        table = golden["code_field"][str(bits)]
        for w, row in enumerate(table):
            assert [code_channel(bits, w, f) for f in range(32 // bits)] == row


def test_pack_unpack_round_trip():
    g = torch.Generator().manual_seed(0)
    for bits, d in ((2, 64), (2, 128), (2, 256), (4, 64), (4, 128), (4, 256)):
        x = torch.randint(0, 1 << bits, (7, 3, d), dtype=torch.uint8, generator=g)
        packed = pack_rows(x, bits)
        assert packed.shape == (7, 3, d * bits // 8)
        assert torch.equal(unpack_rows(packed, bits, d), x)


def test_vmax_bucket_matches_reference(golden):
    for bits, want in golden["vmax_bucket"]:
        assert ref_vmax_bucket(bits) == want
    for bucket, lp in golden["pscale_lp_of_bucket"]:
        assert 135 - bucket == lp


def test_vmax_bucket_is_floor_log2_448_over_x():
    # tests/test_sm100_scale_dtype_host.py:165-191: every binade, boundary mantissas
    for e in range(1, 255):
        for mant in (0, 1, 0x5FFFFF, 0x600000, 0x600001, 0x7FFFFF):
            bits = (e << 23) | mant
            x = struct.unpack("<f", struct.pack("<I", bits))[0]
            assert 135 - ref_vmax_bucket(bits) == math.floor(math.log2(448.0 / x)), hex(bits)
    assert ref_pscale_lp(np.zeros(256, dtype=np.uint32)) == 108


def test_page_maxima_and_histogram_match_reference(golden):
    g = golden["v_page_max_for_pool"]
    sv = np.array(g["sv_bits"], dtype=np.int32).view(np.float32)         # [NP,HKV,64]
    m = sv.max(axis=-1)
    m = np.where(m > 0, m, 0).astype(np.float32)
    assert np.array_equal(m.view(np.int32), np.array(g["v_page_max"], dtype=np.int32))
    hist = ref_v_max_hist(m.view(np.uint32))
    assert np.array_equal(hist.astype(np.int64), np.array(g["v_max_hist"], dtype=np.int64))


def test_scale_range_matches_reference(golden):
    for qmax, (lo, hi) in golden["scale_range"].items():
        got = scale_range(int(qmax))
        assert [struct.unpack("<I", struct.pack("<f", x))[0] for x in got] == [lo, hi]


def test_quantizer_matches_the_reference_test_formula():
    """tests/test_cache_gpu.py:48-53 states the quantizer in torch; same codes and records."""
    g = torch.Generator().manual_seed(1)
    for bits in (2, 4):
        x = torch.randn(50, 4, 128, generator=g).bfloat16()
        f = x.float()
        mn, mx = f.amin(-1), f.amax(-1)
        s = (mx - mn).clamp_min(1e-8) / ((1 << bits) - 1)
        q = ((f - mn.unsqueeze(-1)) / s.unsqueeze(-1)).round().clamp(0, (1 << bits) - 1)
        codes, s2, z2 = quantize_rows(x, bits)
        assert torch.equal(codes, q.to(torch.uint8))
        assert torch.equal(s2.squeeze(-1), s) and torch.equal(z2.squeeze(-1), mn)


def test_quantizer_edges():
    for bits in (2, 4):
        qmax = (1 << bits) - 1
        x = torch.zeros(2, 128).bfloat16()
        x[1] = 3.0
        codes, s, z = quantize_rows(x, bits)
        assert codes.max() == 0 and torch.all(s == torch.tensor(1e-8) / qmax)
        x = torch.tensor([[-1e38, 1e38] + [0.0] * 62]).bfloat16()       # outside the envelope
        codes, s, z = quantize_rows(x, bits)
        assert float(z) == -(2.0 ** 64) and torch.isfinite(s).all()
        assert int(codes[0, 0]) == 0 and int(codes[0, 1]) == qmax
        g2 = quantize_rows(torch.randn(3, 128).bfloat16(), bits, groups=2)
        assert g2[1].shape == (3, 2)


def test_clip_matches_sorted_order_statistic():
    x = torch.randn(5, 128, generator=torch.Generator().manual_seed(2)).bfloat16().float()
    for idx in (0, 64, 126, 127):
        t = x.abs().sort(-1).values[:, idx]
        c = clip_rows(x, idx)
        assert torch.all(c.abs().amax(-1) <= t + 0)
    assert torch.equal(clip_rows(x, 127), x) and torch.equal(clip_rows(x, -1), x)


def test_append_tail_clear_and_page_maxima():
    hkv, d = 2, 64
    pools = CpuPools(3, hkv, d, 2)
    pools.scales.fill_(7.0)
    g = torch.Generator().manual_seed(3)
    k = torch.randn(70, hkv, d, generator=g).bfloat16()
    v = torch.randn(70, hkv, d, generator=g).bfloat16()
    ref_append(pools, k, v, np.arange(70))                  # page 0 full, page 1 positions 0..5
    assert torch.all(pools.scales[1, :, 6:] == 0)           # tail cleared
    assert torch.all(pools.scales[2] == 7.0)                # untouched page
    assert torch.all(pools.scales[0, :, :, 0] > 0)
    sv = pools.scales[..., 2]
    want = sv[:2].amax(-1).contiguous().numpy().view(np.uint32)
    assert np.array_equal(pools.v_page_max[:2], want) and np.all(pools.v_page_max[2] == 0)
    assert pools.v_max_hist.sum() == 4
    # a later token continues page 1 mid-page: no clear, maximum only rises
    big = (torch.randn(1, hkv, d, generator=g) * 50).bfloat16()
    before = pools.v_page_max.copy()
    ref_append(pools, big, big, np.array([64 + 6]))
    assert np.all(pools.v_page_max[1] > before[1]) and pools.v_max_hist.sum() == 4
    assert torch.all(pools.scales[1, :, 7:] == 0) and torch.all(pools.scales[1, :, 6, 0] > 0)
    # reuse of page 1 from position 0 resets it
    small = (torch.randn(2, hkv, d, generator=g) * 0.01).bfloat16()
    ref_append(pools, small, small, np.array([64, 65]))
    assert np.all(pools.v_page_max[1] < before[1])
    assert torch.all(pools.scales[1, :, 2:] == 0)
    # skipped slots write nothing
    snap = pools.k_codes.clone()
    ref_append(pools, small, small, np.array([-1, -5]))
    assert torch.equal(snap, pools.k_codes)


def test_append_quantized_saturates_and_masks():
    hkv, d, bits = 1, 64, 2
    pools = CpuPools(1, hkv, d, bits)
    codes = torch.full((2, hkv, d), 0xFE, dtype=torch.uint8)
    s = torch.tensor([[float("nan")], [1e30]])
    z = torch.tensor([[float("nan")], [-1e30]])
    ref_append_quantized(pools, codes, s, z, codes, s, z, np.array([0, 1]))
    lo, hi = scale_range(3)
    assert float(pools.scales[0, 0, 0, 0]) == lo and float(pools.scales[0, 0, 1, 0]) == hi
    assert float(pools.scales[0, 0, 0, 1]) == -(2.0 ** 64)
    assert torch.all(unpack_rows(pools.k_codes[0, 0, :2], bits, d) == 2)


def test_dequantize_is_fma_then_bf16():
    hkv, d, bits = 2, 128, 4
    pools = CpuPools(2, hkv, d, bits)
    g = torch.Generator().manual_seed(4)
    k = torch.randn(100, hkv, d, generator=g).bfloat16()
    v = torch.randn(100, hkv, d, generator=g).bfloat16()
    ref_append(pools, k, v, np.arange(100))
    (k_hat, v_hat), = ref_dequantize(pools, [0, 2], [0, 1], [100])
    codes, s, z = quantize_rows(k, bits)
    want = torch.from_numpy(np.float32(
        s.double().numpy() * codes.double().numpy() + z.double().numpy())).bfloat16()
    assert torch.equal(k_hat, want)
    assert (k_hat.float() - k.float()).abs().max() <= s.max() * 0.5 + 0.02


def test_merge_recombines_split_attention():
    g = torch.Generator().manual_seed(5)
    hq, d, t = 4, 32, 300
    q = torch.randn(hq, d, generator=g)
    k = torch.randn(t, 1, d, generator=g)
    v = torch.randn(t, 1, d, generator=g)
    full, lse = ref_attention(q, k, v, 0.2)
    parts = []
    for a, b in ((0, 100), (100, 260), (260, 300)):
        s = torch.einsum("hd,td->ht", q, k[a:b, 0]) * 0.2 * math.log2(math.e)
        m = s.max(-1).values
        p = torch.exp2(s - m[:, None])
        parts.append((p @ v[a:b, 0], p.sum(-1), m))
    o = torch.stack([p[0] for p in parts])
    l = torch.stack([p[1] for p in parts])
    m = torch.stack([p[2] for p in parts])
    out, lse2 = ref_merge(o, l, m)
    assert torch.allclose(out, full, atol=1e-5) and torch.allclose(lse2, lse, atol=1e-5)


def test_fold_model_meets_the_stated_tolerance():
    """The fold arithmetic (raw codes through the contraction, E4M3 hi/lo P) stays within
    max-abs 2e-2 / mean-abs 2e-3 of the fp32 oracle, outlier keys included."""
    g = torch.Generator().manual_seed(6)
    hkv, d, t, grp = 1, 128, 1500, 4
    for bits in (2, 4):
        k = (torch.randn(t, hkv, d, generator=g) * torch.exp(torch.randn(1, hkv, d, generator=g))
             ).bfloat16()
        v = torch.randn(t, hkv, d, generator=g).bfloat16()
        pools = CpuPools(-(-t // 64), hkv, d, bits)
        ref_append(pools, k, v, np.arange(t))
        q = (torch.randn(grp, d, generator=g) * 8).clamp(-448, 448).to(torch.float8_e4m3fn).float()
        sm = d ** -0.5 / 8
        (kf, vf), = ref_dequantize(pools, [0, pools.num_pages], np.arange(pools.num_pages), [t],
                                   rounded=False)
        want, lse = ref_attention(q, kf, vf, sm)
        kc = unpack_rows(pools.k_codes[:, 0].reshape(-1, d * bits // 8)[:t], bits, d)
        vc = unpack_rows(pools.v_codes[:, 0].reshape(-1, d * bits // 8)[:t], bits, d)
        sc = pools.scales[:, 0].reshape(-1, 4)[:t]
        got, lse2 = emulate_fold_decode(q, kc, sc[:, 0], sc[:, 1], vc, sc[:, 2], sc[:, 3], sm,
                                        ref_pscale_lp(pools.v_max_hist))
        err = (got - want).abs()
        assert err.max() <= 2e-2 and err.mean() <= 2e-3
        assert (lse2 - lse).abs().max() <= 5e-2
