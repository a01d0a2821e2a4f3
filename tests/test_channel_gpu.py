"""K quantized per channel over the 64 tokens of a page (V per token): writer, read-back and
decode against the CPU restatement in `oracle/ref_channel.py`.

PARITY UNPINNED: the reference ships no writer, packer or fixture for this layout (its append
refuses it, src/foscar/kv_cache.py:643-644), only the byte positions its decode reads
(src/foscar/quant_layout.py:57-85, src/foscar/_sm100/int_fold_decode.py:5012-5036). These tests
pin the CUDA path to this repository's own statement of the format: bytes bit-exact, decode
within max-abs 2e-2 / mean-abs 2e-3 of fp32 attention over the fp32 dequantized values."""
import numpy as np
import pytest
import torch

from helpers import PAGE, make_q
from oracle import (CpuChannelPools, quantize_rows, ref_append_page_groups,
                    ref_append_quantized_page_groups, ref_attention, ref_dequantize_channel)

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 5e-2


def _page_batch(seq, seed):
    """Requests of `seq` tokens on a shuffled pool: (indptr, indices, valid per page entry)."""
    pages = [-(-int(n) // PAGE) for n in seq]
    total = sum(pages)
    order = np.random.default_rng(seed).permutation(total).astype(np.int32)
    indptr = np.concatenate([[0], np.cumsum(pages)]).astype(np.int32)
    valid = []
    for n, p in zip(seq, pages):
        valid += [PAGE] * (p - 1) + [int(n) - PAGE * (p - 1)]
    return indptr, order, np.asarray(valid, dtype=np.int32), total


def _page_rows(seq, hkv, d, seed, outliers):
    """k, v bf16 [P * 64, HKV, D] with page i's tokens at rows [64 i, 64 i + valid[i])."""
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-int(n) // PAGE) for n in seq)
    k = torch.randn(pages * PAGE, hkv, d, generator=g)
    v = torch.randn(pages * PAGE, hkv, d, generator=g)
    if outliers:
        k = k * torch.exp(torch.randn(1, hkv, d, generator=g))
    return k.to(torch.bfloat16), v.to(torch.bfloat16)


def _build(bits, d, hkv, seq, seed, scale_dtype=None, outliers=True):
    from foscar_b200 import QuantKVLayout
    indptr, indices, valid, total = _page_batch(seq, seed)
    k, v = _page_rows(seq, hkv, d, seed, outliers)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda",
                                  k_quant=("channel", 64), scale_dtype=scale_dtype)
    cache = layout.allocate(total + 1)
    cache.append_page_groups(k.cuda(), v.cuda(), torch.from_numpy(indices).cuda(),
                             torch.from_numpy(valid).cuda())
    torch.cuda.synchronize()
    assert cache.last_status() == 0
    pools = CpuChannelPools(total + 1, hkv, d, bits, scale_dtype=layout.scale_dtype)
    ref_append_page_groups(pools, k, v, indices, valid)
    return layout, cache, pools, indptr, indices, valid


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("scale_dtype", [None, torch.bfloat16])
def test_page_group_writer_bytes(bits, d, scale_dtype):
    seq = [1, 64, 65, 200, 1000]
    layout, cache, pools, indptr, indices, valid = _build(bits, d, 2, seq, 11, scale_dtype)
    kc, vc = cache.k_codes.cpu(), cache.v_codes.cpu()
    for e, (p, n) in enumerate(zip(indices, valid)):
        assert torch.equal(kc[p, :, :n], pools.k_codes[p, :, :n]), f"K codes of page entry {e}"
        assert torch.equal(vc[p, :, :n], pools.v_codes[p, :, :n]), f"V codes of page entry {e}"
    sel = torch.as_tensor(np.sort(indices).astype(np.int64))
    got = cache.scales.cpu()[sel].contiguous().view(torch.uint8)
    want = pools.scales[sel].contiguous().view(torch.uint8)
    assert torch.equal(got, want), "scale blocks differ"
    vpm = cache.v_page_max.view(torch.int32).cpu().numpy().view(np.uint32)
    assert np.array_equal(vpm[np.sort(indices)], pools.v_page_max[np.sort(indices)])
    hist = cache.v_max_hist.view(torch.int32).cpu().numpy().view(np.uint32)
    assert np.array_equal(hist, pools.v_max_hist)


def _engine_quantized(k, v, bits, valid):
    """What an engine that quantizes by itself would hand over for the page rows k, v: codes one
    per byte, K records per (page, head, channel) over each page's valid tokens, V records per
    token. Codes carry junk in their high bits and rows past a page's valid tokens are random:
    the write has to mask the first and skip the second."""
    pages, (hkv, d) = len(valid), k.shape[1:]
    g = torch.Generator().manual_seed(5)
    kc = torch.randint(0, 256, (pages * PAGE, hkv, d), generator=g, dtype=torch.uint8)
    vc = torch.randint(0, 256, (pages * PAGE, hkv, d), generator=g, dtype=torch.uint8)
    ks, kz = torch.randn(pages, hkv, d, generator=g), torch.randn(pages, hkv, d, generator=g)
    vs, vz = torch.rand(pages * PAGE, hkv, generator=g), torch.randn(pages * PAGE, hkv, generator=g)
    junk = 256 - (1 << bits)
    for i, n in enumerate(valid):
        rows = slice(PAGE * i, PAGE * i + int(n))
        c, s, z = quantize_rows(k[rows].float().permute(1, 2, 0).contiguous(), bits)
        kc[rows] = c.permute(2, 0, 1).to(torch.uint8) | (kc[rows] & junk)
        ks[i], kz[i] = s[..., 0], z[..., 0]
        c, s, z = quantize_rows(v[rows], bits)
        vc[rows] = c.to(torch.uint8) | (vc[rows] & junk)
        vs[rows], vz[rows] = s[..., 0], z[..., 0]
    return kc, ks, kz, vc, vs, vz


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("scale_dtype", [None, torch.bfloat16])
def test_layout_only_page_group_write(bits, d, scale_dtype):
    """Pages an engine quantized itself: the bytes equal the CPU statement of the layout-only
    write, and, the engine having used the writer's own arithmetic, the bytes the quantizing
    page-group writer leaves for the same rows."""
    from foscar_b200 import QuantKVLayout
    seq, hkv = [1, 64, 65, 200, 1000], 2
    indptr, indices, valid, total = _page_batch(seq, 21)
    k, v = _page_rows(seq, hkv, d, 21, outliers=True)
    given = _engine_quantized(k, v, bits, valid)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda",
                                  k_quant=("channel", 64), scale_dtype=scale_dtype)
    ids, val = torch.from_numpy(indices).cuda(), torch.from_numpy(valid).cuda()
    cache = layout.allocate(total + 1)
    cache.append_quantized_page_groups(*(x.cuda() for x in given), ids, val)
    twin = layout.allocate(total + 1)
    twin.append_page_groups(k.cuda(), v.cuda(), ids, val)
    torch.cuda.synchronize()
    assert cache.last_status() == 0 and twin.last_status() == 0
    pools = CpuChannelPools(total + 1, hkv, d, bits, scale_dtype=layout.scale_dtype)
    ref_append_quantized_page_groups(pools, *given, indices, valid)
    sel = torch.as_tensor(np.sort(indices).astype(np.int64))
    kc, vc, tk, tv = (x.cpu() for x in (cache.k_codes, cache.v_codes, twin.k_codes, twin.v_codes))
    for e, (p, n) in enumerate(zip(indices, valid)):
        assert torch.equal(kc[p, :, :n], pools.k_codes[p, :, :n]), f"K codes of page entry {e}"
        assert torch.equal(vc[p, :, :n], pools.v_codes[p, :, :n]), f"V codes of page entry {e}"
        assert torch.equal(kc[p, :, :n], tk[p, :, :n]) and torch.equal(vc[p, :, :n], tv[p, :, :n])
    got = cache.scales.cpu()[sel].contiguous().view(torch.uint8)
    assert torch.equal(got, pools.scales[sel].contiguous().view(torch.uint8)), "scale blocks"
    assert torch.equal(got, twin.scales.cpu()[sel].contiguous().view(torch.uint8))
    vpm = cache.v_page_max.view(torch.int32).cpu().numpy().view(np.uint32)
    assert np.array_equal(vpm[np.sort(indices)], pools.v_page_max[np.sort(indices)])
    hist = cache.v_max_hist.view(torch.int32).cpu().numpy().view(np.uint32)
    assert np.array_equal(hist, pools.v_max_hist)


def test_layout_only_page_group_write_saturates_records():
    """Records outside the quantizing writer's ranges (and NaN) are saturated, as the token-wise
    layout-only write does; a page written again replaces its maximum."""
    from foscar_b200 import QuantKVLayout
    bits, d, hkv = 4, 256, 2
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda",
                                  k_quant=("channel", 64))
    cache = layout.allocate(3)
    pools = CpuChannelPools(3, hkv, d, bits, scale_dtype=layout.scale_dtype)
    g = torch.Generator().manual_seed(9)
    ids = np.array([2, 0], dtype=np.int32)
    for step in range(2):
        kc = torch.randint(0, 16, (2 * PAGE, hkv, d), generator=g, dtype=torch.uint8)
        vc = torch.randint(0, 16, (2 * PAGE, hkv, d), generator=g, dtype=torch.uint8)
        ks = torch.randn(2, hkv, d, generator=g)
        kz = torch.randn(2, hkv, d, generator=g)
        vs = torch.rand(2 * PAGE, hkv, generator=g) * (0.1 if step else 1.0)
        vz = torch.randn(2 * PAGE, hkv, generator=g)
        ks[0, 0, :4] = torch.tensor([0.0, -1.0, float("nan"), float("inf")])
        kz[1, 1, :3] = torch.tensor([float("inf"), -float("inf"), float("nan")])
        vs[3, 0], vs[4, 1], vz[5, 0] = 0.0, float("inf"), float("nan")
        given = (kc, ks, kz, vc, vs, vz)
        cache.append_quantized_page_groups(*(x.cuda() for x in given),
                                           torch.from_numpy(ids).cuda())
        ref_append_quantized_page_groups(pools, *given, ids)
        torch.cuda.synchronize()
        assert cache.last_status() == 0
        sel = torch.tensor([0, 2])
        assert torch.equal(cache.scales.cpu()[sel].contiguous().view(torch.uint8),
                           pools.scales[sel].contiguous().view(torch.uint8))
        assert torch.equal(cache.k_codes.cpu()[sel], pools.k_codes[sel])
        vpm = cache.v_page_max.view(torch.int32).cpu().numpy().view(np.uint32)
        assert np.array_equal(vpm[[0, 2]], pools.v_page_max[[0, 2]])
        hist = cache.v_max_hist.view(torch.int32).cpu().numpy().view(np.uint32)
        assert np.array_equal(hist, pools.v_max_hist)


@pytest.mark.parametrize("bits,d", [(4, 256), (2, 128)])
def test_read_back_rows(bits, d):
    seq = [130, 64, 7]
    layout, cache, pools, indptr, indices, valid = _build(bits, d, 2, seq, 12)
    total = sum(seq)
    k_out = torch.zeros(total, 2, d, dtype=torch.bfloat16, device="cuda")
    v_out = torch.zeros_like(k_out)
    out_indptr = torch.tensor(np.concatenate([[0], np.cumsum(seq)[:-1]]), dtype=torch.int32,
                              device="cuda")
    cache.dequantize(k_out, v_out, torch.from_numpy(indptr).cuda(),
                     torch.from_numpy(indices).cuda(),
                     torch.tensor(seq, dtype=torch.int32, device="cuda"), out_indptr)
    torch.cuda.synchronize()
    assert cache.last_status() == 0
    want = ref_dequantize_channel(pools, indptr, indices, seq, rounded=True)
    a = 0
    for b, n in enumerate(seq):
        assert torch.equal(k_out[a:a + n].cpu(), want[b][0]), f"K rows of request {b}"
        assert torch.equal(v_out[a:a + n].cpu(), want[b][1]), f"V rows of request {b}"
        a += n


def _decode_case(bits, hq, hkv, seq, seed, kv_splits=None, q_scale=8.0, scale_dtype=None):
    from foscar_b200 import PagedDecodeWrapper
    d = 256
    layout, cache, pools, indptr, indices, valid = _build(bits, d, hkv, seq, seed, scale_dtype)
    q = make_q(len(seq), hq, d, seed=seed + 1, scale=q_scale)
    sm_scale = d ** -0.5 / q_scale
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    lens = torch.tensor(seq, dtype=torch.int32)
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           lens if kv_splits is None else lens.cuda(), hq, layout, sm_scale=sm_scale,
           kv_splits=kv_splits)
    out = torch.full((len(seq), hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((len(seq), hq), float("nan"), device="cuda")
    w.run(q, cache, out=out, lse=lse)
    torch.cuda.synchronize()
    assert w.last_status() == 0
    kv = ref_dequantize_channel(pools, indptr, indices, seq, rounded=False)
    wants, lses = zip(*(ref_attention(q[b].float().cpu(), kv[b][0], kv[b][1], sm_scale)
                        for b in range(len(seq))))
    err = (out.float().cpu() - torch.stack(wants)).abs()      # over the batch, as the
    assert torch.isfinite(out.float()).all()                  # token-wise decode tests do
    assert err.max().item() <= MAX_ABS, f"max-abs {err.max().item():.3e}"
    assert err.mean().item() <= MEAN_ABS, f"mean-abs {err.mean().item():.3e}"
    assert (lse.cpu() - torch.stack(lses)).abs().max().item() <= LSE_ABS


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("hq,hkv", [(16, 2), (8, 2)])
def test_decode_channel_wise_k_head_dim_256(bits, hq, hkv):
    """The head_dim 256 / GQA 8 / K-channel-64 configuration: ragged batch with outlier keys."""
    _decode_case(bits, hq, hkv, [1, 63, 64, 65, 129, 1000, 4097, 9000], seed=31 + bits)


def test_decode_channel_wise_k_splits_and_bf16_records():
    _decode_case(4, 16, 2, [5000, 257], seed=41, kv_splits=3)
    _decode_case(4, 16, 2, [3000, 130], seed=42, scale_dtype=torch.bfloat16)
    _decode_case(4, 16, 2, [20000, 700], seed=43, q_scale=1.0)
