"""Cache writer and read-back on the device against the CPU oracle: packed codes, scale bytes,
page maxima and the count table must be bit-exact; read-back rows must be bit-exact."""
import numpy as np
import pytest
import torch

from helpers import PAGE, assert_pools_equal, cpu_twin, make_kv, paged_batch
from oracle import CpuPools, ref_append, ref_append_quantized, ref_dequantize, quantize_rows

pytestmark = pytest.mark.gpu


def _layout(bits, d, hkv, **kw):
    from foscar_b200 import QuantKVLayout
    return QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda", **kw)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("d", [64, 128, 256])
def test_append_bytes_match_oracle(bits, d):
    hkv, seq = 4, [300, 64, 1, 129]
    indptr, indices, slots, npages = paged_batch(seq, seed=d + bits)
    k, v = make_kv(len(slots), hkv, d, seed=bits, outliers=True)
    cache = _layout(bits, d, hkv).allocate(npages)
    cache.k_codes.fill_(0xA5); cache.v_codes.fill_(0xA5)
    cache.scales.view(torch.uint8).fill_(0x7F)
    pools = CpuPools(npages, hkv, d, bits, fill=0)
    pools.k_codes.fill_(0xA5); pools.v_codes.fill_(0xA5)
    pools.scales.view(torch.uint8).fill_(0x7F)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    ref_append(pools, k.cpu(), v.cpu(), slots)
    torch.cuda.synchronize()
    assert cache.last_status() == 0
    assert_pools_equal(cache, pools)


def test_config1_int4_identity_pages_bit_exact():
    """INT4, B=2, 8 KV heads, D=128, two full pages per request, slots = arange(256), seed 0."""
    hkv, d = 8, 128
    k, v = make_kv(256, hkv, d, seed=0)
    cache = _layout(4, d, hkv).allocate(4)
    slots = np.arange(256, dtype=np.int64)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    pools = cpu_twin(cache, k, v, slots)
    assert_pools_equal(cache, pools)


@pytest.mark.parametrize("bits", [2, 4])
def test_decode_step_appends_and_page_reuse(bits):
    """Prefill, then single-token steps that continue pages and start new ones, then a page
    reused from position 0: tail clear, page maxima and count table follow the oracle."""
    hkv, d, npages = 2, 128, 6
    cache = _layout(bits, d, hkv).allocate(npages)
    cache.k_codes.zero_(); cache.v_codes.zero_()
    cache.scales.view(torch.uint8).fill_(0xFF)
    pools = CpuPools(npages, hkv, d, bits)
    pools.scales.view(torch.uint8).fill_(0xFF)
    g = torch.Generator().manual_seed(5)

    def step(slots, scale=1.0):
        slots = np.asarray(slots, dtype=np.int64)
        k = (torch.randn(len(slots), hkv, d, generator=g) * scale).bfloat16()
        v = (torch.randn(len(slots), hkv, d, generator=g) * scale).bfloat16()
        cache.append(k.cuda(), v.cuda(), torch.from_numpy(slots).cuda())
        ref_append(pools, k, v, slots)

    step(np.concatenate([np.arange(0, 100), np.arange(3 * 64, 3 * 64 + 10)]))
    touched = {0, 1, 3}
    assert_pools_equal(cache, pools, pages=touched)
    step([100, 3 * 64 + 10], scale=4.0)            # continue both requests (raises maxima)
    step([101, -1, 3 * 64 + 11])                   # a skipped slot
    step(np.arange(2 * 64, 2 * 64 + 5), scale=0.1) # a new page for a new request
    touched.add(2)
    assert_pools_equal(cache, pools, pages=touched)
    step(np.arange(0, 7), scale=0.01)              # page 0 reused from position 0
    assert_pools_equal(cache, pools, pages=touched)
    assert cache.last_status() == 0


def test_bad_slot_sets_status_and_writes_nothing():
    hkv, d = 2, 128
    cache = _layout(2, d, hkv).allocate(2)
    cache.k_codes.zero_()
    k, v = make_kv(3, hkv, d)
    cache.append(k, v, torch.tensor([0, 2 * 64, 5], dtype=torch.int64, device="cuda"))
    torch.cuda.synchronize()
    assert cache.last_status() & 0x1


@pytest.mark.parametrize("bits", [2, 4])
def test_bf16_pool_and_grouped_k(bits):
    hkv, d = 2, 128
    seq = [70, 200]
    indptr, indices, slots, npages = paged_batch(seq, seed=3)
    k, v = make_kv(len(slots), hkv, d, seed=9)
    for kw in (dict(scale_dtype=torch.bfloat16), dict(k_quant=("token", 64))):
        cache = _layout(bits, d, hkv, **kw).allocate(npages)
        cache.k_codes.zero_(); cache.v_codes.zero_(); cache.scales.zero_()
        cache.append(k, v, torch.from_numpy(slots).cuda())
        pools = cpu_twin(cache, k, v, slots)
        assert_pools_equal(cache, pools)


@pytest.mark.parametrize("bits", [2, 4])
def test_append_quantized_matches_oracle(bits):
    hkv, d = 4, 128
    seq = [130, 64]
    indptr, indices, slots, npages = paged_batch(seq, seed=11)
    k, v = make_kv(len(slots), hkv, d, seed=2)
    kc, ks, kz = quantize_rows(k.cpu(), bits)
    vc, vs, vz = quantize_rows(v.cpu(), bits)
    ks, kz, vs, vz = (x.squeeze(-1).contiguous() for x in (ks, kz, vs, vz))
    ks[0, 0] = float("nan"); vz[1, 1] = 1e30
    kc = kc | 0xF0                                  # high bits are ignored
    cache = _layout(bits, d, hkv).allocate(npages)
    cache.k_codes.zero_(); cache.v_codes.zero_(); cache.scales.zero_()
    cache.append_quantized(kc.cuda(), ks.cuda(), kz.cuda(), vc.cuda(), vs.cuda(), vz.cuda(),
                           torch.from_numpy(slots).cuda())
    pools = CpuPools(npages, hkv, d, bits)
    ref_append_quantized(pools, kc, ks, kz, vc, vs, vz, slots)
    assert_pools_equal(cache, pools)


@pytest.mark.parametrize("clip", [(0.9, None), (None, 0.5), (0.97, 0.97)])
def test_clipped_append(clip):
    from foscar_b200.kv_cache import clip_index
    hkv, d, bits = 2, 128, 2
    seq = [90]
    indptr, indices, slots, npages = paged_batch(seq, seed=1)
    k, v = make_kv(len(slots), hkv, d, seed=4, outliers=True)
    cache = _layout(bits, d, hkv).allocate(npages)
    cache.k_codes.zero_(); cache.v_codes.zero_(); cache.scales.zero_()
    cache.append(k, v, torch.from_numpy(slots).cuda(), k_clip=clip[0], v_clip=clip[1])
    pools = CpuPools(npages, hkv, d, bits)
    ref_append(pools, k.cpu(), v.cpu(), slots, clip_index(clip[0], d), clip_index(clip[1], d))
    assert_pools_equal(cache, pools)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("d", [64, 128, 256])
def test_dequantize_bit_exact(bits, d):
    hkv = 2
    seq = [130, 1, 64, 200]
    indptr, indices, slots, npages = paged_batch(seq, seed=d)
    k, v = make_kv(len(slots), hkv, d, seed=d + bits)
    cache = _layout(bits, d, hkv).allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    pools = cpu_twin(cache, k, v, slots)
    total = sum(seq)
    k_out = torch.full((total + 3, hkv, d), 7.0, dtype=torch.bfloat16, device="cuda")
    v_out = torch.full_like(k_out, 7.0)
    out_indptr = np.concatenate([[0], np.cumsum(seq)[:-1]]).astype(np.int64) + 3
    cache.dequantize(k_out, v_out, torch.from_numpy(indptr).cuda(),
                     torch.from_numpy(indices).cuda(),
                     torch.tensor(seq, dtype=torch.int32, device="cuda"),
                     torch.from_numpy(out_indptr).cuda())
    torch.cuda.synchronize()
    assert cache.last_status() == 0
    want = ref_dequantize(pools, indptr, indices, seq)
    assert torch.equal(k_out[:3].cpu(), torch.full((3, hkv, d), 7.0, dtype=torch.bfloat16))
    for b, n in enumerate(seq):
        o = int(out_indptr[b])
        assert torch.equal(k_out[o:o + n].cpu(), want[b][0])
        assert torch.equal(v_out[o:o + n].cpu(), want[b][1])


def test_recount_rebuilds_table():
    hkv, d = 2, 128
    cache = _layout(2, d, hkv).allocate(8)
    k, v = make_kv(8 * 64, hkv, d, seed=0)
    cache.append(k, v, torch.arange(8 * 64, device="cuda"))
    before = cache.v_max_hist.view(torch.int32).clone()
    cache.v_page_max.view(torch.int32)[0, 0] |= -2**31          # a sign bit sneaks in
    cache.v_max_hist.view(torch.int32).zero_()
    cache.recount_v_max()
    torch.cuda.synchronize()
    assert torch.equal(cache.v_max_hist.view(torch.int32), before)
    assert int(cache.v_page_max.view(torch.int32)[0, 0]) > 0
