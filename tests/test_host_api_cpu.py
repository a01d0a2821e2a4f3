"""Host layer without a GPU: layout geometry against vectors from the reference's own layout
code, every refusal class, region-major bind, and plan()/run() wiring against a recording fake of
the C ABI (the way the reference tests its wrapper with fake backends)."""
import ctypes

import numpy as np
import pytest
import torch

import foscar_b200
from foscar_b200 import PagedDecodeWrapper, QuantKVCache, QuantKVLayout, _lib, device as dev
from foscar_b200 import kv_cache as kvc
from foscar_b200 import pool_format as pf
from foscar_b200 import wrapper as wr


def _layout(**kw):
    base = dict(bits=2, head_dim=128, num_kv_heads=8)
    base.update(kw)
    return QuantKVLayout._create("sm100", **base)


@pytest.fixture
def fake_b200(monkeypatch):
    """Pretend every device is a B200 so CPU tensors pass the architecture checks."""
    monkeypatch.setattr(dev, "require_arch", lambda device=None: "sm100")
    monkeypatch.setattr(dev, "sm_count", lambda device=None: 148)
    monkeypatch.setattr(dev, "on_device", lambda device: __import__("contextlib").nullcontext())
    monkeypatch.setattr(dev, "current_stream_ptr", lambda device=None: 0)


def test_public_names():
    for name in ("PagedDecodeWrapper", "QuantKVCache", "QuantKVLayout", "get_capabilities",
                 "is_supported", "graph_workspace_bytes", "__version__"):
        assert hasattr(foscar_b200, name)
    import foscar
    assert foscar.PagedDecodeWrapper is PagedDecodeWrapper


def test_capabilities_without_gpu_has_every_key():
    caps = foscar_b200.get_capabilities()
    assert set(caps) == {"arch", "paged", "dtypes", "head_dims", "page_sizes", "reductions",
                         "speculative", "atomic_reduction", "skip_softmax", "kv_layouts",
                         "quantized_bits", "quantized_validated", "quantized_page_sizes"}
    if not torch.cuda.is_available():
        assert caps["arch"] == "unsupported" and not foscar_b200.is_supported()


def test_capabilities_on_b200(monkeypatch):
    monkeypatch.setattr(dev, "is_supported", lambda device=None: True)
    caps = dev.get_capabilities()
    assert caps["arch"] == "sm100" and caps["dtypes"] == ["float8_e4m3fn"]
    assert caps["head_dims"] == "64,128,256" and caps["page_sizes"] == [64]
    assert caps["reductions"] == ["none", "kernel"] and caps["quantized_bits"] == [2, 4]
    assert caps["kv_layouts"] == ["QuantKVLayout"] and caps["paged"] is True
    assert not (caps["speculative"] or caps["atomic_reduction"] or caps["skip_softmax"])


def test_layout_geometry_matches_reference(golden):
    for rec in golden["layouts"]:
        sd = None if rec["scale_dtype"] is None else torch.bfloat16
        lay = QuantKVLayout._create(
            "sm100", bits=rec["bits"], head_dim=rec["head_dim"], num_kv_heads=rec["num_kv_heads"],
            k_quant=None if rec["k_quant"] is None else tuple(rec["k_quant"]),
            v_quant=None if rec["v_quant"] is None else tuple(rec["v_quant"]), scale_dtype=sd)
        want = rec["resolved"]
        assert list(lay.k_quant) == want["k_quant"] and list(lay.v_quant) == want["v_quant"]
        assert str(lay.scale_dtype).split(".")[-1] == want["scale_dtype"]
        assert lay.reader == want["reader"] and lay.code_pool_order == want["code_pool_order"]
        assert lay.k_pool_permuted == want["k_pool_permuted"]
        assert lay.v_pool_permuted == want["v_pool_permuted"]
        assert lay.has_v_page_max == want["has_v_page_max"]
        assert lay.bytes_per_page() == rec["bytes_per_page"]
        shapes = lay.pool_shapes(5)
        for name, shape in rec["pool_shapes"].items():
            assert (None if shapes[name] is None else list(shapes[name])) == shape, name


def test_scale_sections_match_reference(golden):
    for d, kq, vq, want in golden["quant_block_offsets"]:
        assert pf.scale_block_sections(tuple(kq), tuple(vq), d) == want


def test_headline_page_sizes():
    assert _layout(bits=4).bytes_per_page() == 73760           # config 1
    assert _layout(bits=2).bytes_per_page() == 40992           # configs 2 and 3
    assert _layout(bits=4, head_dim=256, num_kv_heads=2, k_quant=("channel", 64)
                   ).bytes_per_page() == 37896                  # config 4
    assert _layout(bits=2, head_dim=64).bytes_per_page() == 24608
    assert _layout(bits=4, head_dim=64).bytes_per_page() == 40992


def test_layout_is_a_frozen_value():
    a, b = _layout(), _layout()
    assert a == b and hash(a) == hash(b) and a != _layout(bits=4)
    with pytest.raises(Exception):
        a.bits = 4
    with pytest.raises(ValueError, match="built by QuantKVLayout.create"):
        QuantKVLayout(arch="sm100", bits=2, head_dim=128, num_kv_heads=8, k_quant=("token", 128),
                      v_quant=("token", 128), scale_dtype=torch.float32, reader="IntDecodeSm100",
                      code_pool_order="chunk16", k_pool_permuted=True, v_pool_permuted=True)


@pytest.mark.parametrize("kw,match", [
    (dict(bits=3), "bits must be one of"), (dict(bits=True), "bits must be one of"),
    (dict(head_dim=96), "is not accepted on sm100"), (dict(head_dim=0), "positive int"),
    (dict(num_kv_heads=0), "num_kv_heads must be a positive int"),
    (dict(scale_dtype=torch.float16), "scale_dtype must be one of"),
    (dict(k_quant=("token", 32)), "outside the decode's envelope"),
    (dict(v_quant=("token", 64)), "outside the decode's envelope"),
    (dict(k_quant=("channel", 32)), "outside the decode's envelope"),
    (dict(k_quant=("token", 64), scale_dtype=torch.float32), "bfloat16 scale"),
    (dict(k_quant=7), "must be an \\(axis, group\\) pair"),
])
def test_layout_refusals(kw, match):
    with pytest.raises(ValueError, match=match):
        _layout(**kw)


def test_create_refuses_a_device_without_a_kernel(monkeypatch):
    monkeypatch.setattr(dev, "cuda_index", lambda device=None: 0)
    monkeypatch.setattr(dev, "_cc", lambda index: (9, 0))
    with pytest.raises(RuntimeError, match="no kernel for compute capability 9.0"):
        QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=8)
    monkeypatch.setattr(dev, "_cc", lambda index: (10, 0))
    assert QuantKVLayout.create(bits=2, head_dim=128, num_kv_heads=8).arch == "sm100"


def test_clip_index_matches_reference(golden):
    for ratio, d, want in golden["clip_index"]:
        assert kvc.clip_index(ratio, d) == want
    for bad in (0, 1.5, -0.1, True, "0.5"):
        with pytest.raises(ValueError, match="clip ratio"):
            kvc.clip_index(bad, 128)


def test_bind_is_region_major_and_zeroes_only_the_maxima(fake_b200):
    lay = _layout(bits=4)
    n = 3
    buf = torch.full((n * lay.bytes_per_page() + 32,), 0xAB, dtype=torch.uint8)
    cache = lay.bind(buf, n)
    kb, sb = n * 8 * 64 * 64, n * 8 * 64 * 4 * 4
    assert cache.k_codes.data_ptr() == buf.data_ptr()
    assert cache.v_codes.data_ptr() == buf.data_ptr() + kb
    assert cache.scales.data_ptr() == buf.data_ptr() + 2 * kb
    assert cache.v_page_max.data_ptr() == buf.data_ptr() + 2 * kb + sb
    assert cache.k_codes.shape == (n, 8, 64, 64) and cache.scales.dtype == torch.float32
    assert int(cache.v_page_max.view(torch.int32).abs().sum()) == 0
    assert int(buf[0]) == 0xAB and int(buf[2 * kb]) == 0xAB
    assert cache.v_max_hist.shape == (256,) and cache.v_max_hist.dtype == torch.uint32
    assert cache.num_pages == n and cache.layout is lay
    for ptr in (cache.k_codes, cache.v_codes, cache.scales, cache.v_page_max):
        assert ptr.data_ptr() % 16 == 0
    assert _layout(v_quant=("channel", 64), k_quant=("channel", 64)).bind(
        torch.zeros(2 * 40000, dtype=torch.uint8), 1).v_page_max is None


def test_bind_refusals(fake_b200):
    lay = _layout()
    with pytest.raises(TypeError, match="torch.Tensor"):
        lay.bind([0] * 10, 1)
    with pytest.raises(ValueError, match="uint8"):
        lay.bind(torch.zeros(50000, dtype=torch.int8), 1)
    with pytest.raises(ValueError, match="needs 40992 bytes"):
        lay.bind(torch.zeros(100, dtype=torch.uint8), 1)
    with pytest.raises(ValueError, match="C-contiguous"):
        lay.bind(torch.zeros(2, 50000, dtype=torch.uint8)[:, ::2], 1)
    with pytest.raises(ValueError, match="16-byte aligned"):
        lay.bind(torch.zeros(50000, dtype=torch.uint8)[1:], 1)
    with pytest.raises(ValueError, match="positive int"):
        lay.bind(torch.zeros(50000, dtype=torch.uint8), 0)
    with pytest.raises(TypeError, match="allocate"):
        QuantKVCache()


def _cache(fake, **kw):
    lay = _layout(**kw)
    return lay, lay.bind(torch.zeros(4 * lay.bytes_per_page(), dtype=torch.uint8), 4)


def test_append_argument_refusals(fake_b200):
    lay, cache = _cache(fake_b200)
    k = torch.zeros(5, 8, 128, dtype=torch.bfloat16)
    slots = torch.arange(5)
    with pytest.raises(ValueError, match="k must be a bfloat16"):
        cache.append(k.float(), k, slots)
    with pytest.raises(ValueError, match="v must be a bfloat16"):
        cache.append(k, k[:, :4], slots)
    with pytest.raises(ValueError, match="contiguous \\[num_kv_heads, head_dim\\] row"):
        cache.append(torch.zeros(5, 8, 256, dtype=torch.bfloat16)[:, :, ::2], k, slots)
    with pytest.raises(ValueError, match="16-byte aligned"):
        cache.append(torch.zeros(5 * 8 * 128 + 8, dtype=torch.bfloat16)[1:1 + 5 * 1024].view(5, 8, 128),
                     k, slots)
    with pytest.raises(ValueError, match="k has 5 tokens and v has 4"):
        cache.append(k, k[:4], slots)
    with pytest.raises(ValueError, match="slot_mapping must be a contiguous int64"):
        cache.append(k, k, slots.int())
    with pytest.raises(ValueError, match="clip ratio"):
        cache.append(k, k, slots, k_clip=2.0)
    lay2, cache2 = _cache(fake_b200, k_quant=("channel", 64))
    with pytest.raises(NotImplementedError, match="token-wise layouts only"):
        cache2.append(k, k, slots)
    # K per channel over a page is written by whole pages and read back; a channel-wise V is not
    with pytest.raises(NotImplementedError, match="append_page_groups"):
        cache2.append(k, k, slots)
    with pytest.raises(ValueError, match="page_indices must be a contiguous int32"):
        cache2.append_page_groups(k, k, slots)
    with pytest.raises(ValueError, match="64 rows per page"):
        cache2.append_page_groups(k, k, torch.zeros(1, dtype=torch.int32))
    with pytest.raises(NotImplementedError, match="append_page_groups\\(\\) writes k_quant"):
        cache.append_page_groups(k, k, torch.zeros(1, dtype=torch.int32))
    c = torch.zeros(64, 8, 128, dtype=torch.uint8)
    rec, per_token, page = torch.zeros(1, 8, 128), torch.zeros(64, 8), torch.zeros(1, dtype=torch.int32)
    with pytest.raises(NotImplementedError, match="append_quantized_page_groups\\(\\) writes k_quant"):
        cache.append_quantized_page_groups(c, rec, rec, c, per_token, per_token, page)
    with pytest.raises(ValueError, match="k_scale must be a torch.float32 \\[1, 8, 128\\]"):
        cache2.append_quantized_page_groups(c, per_token, rec, c, per_token, per_token, page)
    with pytest.raises(ValueError, match="v_codes must be a torch.uint8 \\[64, 8, 128\\]"):
        cache2.append_quantized_page_groups(c, rec, rec, c[:32], per_token, per_token, page)
    with pytest.raises(ValueError, match="valid_tokens must be a contiguous int32"):
        cache2.append_quantized_page_groups(c, rec, rec, c, per_token, per_token, page,
                                            torch.zeros(2, dtype=torch.int32))
    lay3, cache3 = _cache(fake_b200, k_quant=("channel", 64), v_quant=("channel", 64))
    with pytest.raises(NotImplementedError, match="token-wise layouts only"):
        cache3.dequantize(k, k, slots.int(), slots.int(), slots.int(), slots.int())


def test_append_quantized_and_dequantize_refusals(fake_b200):
    lay, cache = _cache(fake_b200)
    c = torch.zeros(3, 8, 128, dtype=torch.uint8)
    s = torch.zeros(3, 8)
    slots = torch.arange(3)
    with pytest.raises(ValueError, match="k_scale must be a torch.float32"):
        cache.append_quantized(c, s.double(), s, c, s, s, slots)
    with pytest.raises(ValueError, match="v_codes must be a torch.uint8"):
        cache.append_quantized(c, s, s, c[:, :, :64], s, s, slots)
    out = torch.zeros(10, 8, 128, dtype=torch.bfloat16)
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32)
    with pytest.raises(ValueError, match="k_out must be a bfloat16"):
        cache.dequantize(out.float(), out, i32(0, 1), i32(0), i32(5), i32(0))
    with pytest.raises(ValueError, match="seq_lens must be a contiguous one-dimensional"):
        cache.dequantize(out, out, i32(0, 1), i32(0), torch.tensor([5]), i32(0))
    with pytest.raises(ValueError, match="page_indptr must have 2 entries"):
        cache.dequantize(out, out, i32(0, 1, 2), i32(0), i32(5), i32(0))


class _Recorder:
    """Stands in for the loaded library: records launches, runs the real host-only planners."""
    def __init__(self):
        self.real = _lib.load()
        self.calls = []

    def __getattr__(self, name):
        if name in ("fq_plan_splits", "fq_plan_worklist", "fq_worklist_words",
                    "fq_worklist_attach_requests", "fq_ctas_per_sm", "fq_tile_tokens",
                    "fq_piece_overhead",
                    "fq_workspace_bytes", "fq_error_string", "fq_version"):
            return getattr(self.real, name)

        def record(*args):
            self.calls.append((name, args))
            return 0
        return record


@pytest.fixture
def recorder(fake_b200, monkeypatch):
    rec = _Recorder()
    monkeypatch.setattr(_lib, "load", lambda: rec)
    return rec


def _plan_args(batch=2, pages=4):
    indptr = torch.arange(batch + 1, dtype=torch.int32) * pages
    indices = torch.arange(batch * pages, dtype=torch.int32)
    return indptr, indices


def test_plan_and_run_wiring(recorder):
    lay, cache = _cache(None)
    w = PagedDecodeWrapper(torch.zeros(8 << 20, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="Call plan\\(\\) before run\\(\\)"):
        w.run(torch.zeros(2, 32, 128).to(torch.float8_e4m3fn), cache)
    indptr, indices = _plan_args()
    w.plan(indptr, indices, torch.tensor([256, 200], dtype=torch.int32), 32, lay)
    assert w.bits == 2 and w.kv_splits >= 1 and w.reduction in ("none", "kernel")
    q = torch.zeros(2, 32, 128).to(torch.float8_e4m3fn)
    out = torch.zeros(2, 32, 128, dtype=torch.bfloat16)
    assert w.run(q, cache, out=out) is out
    names = [c[0] for c in recorder.calls]
    assert names[0] == "fq_decode" and set(names) <= {"fq_decode", "fq_merge"}
    args = ctypes.cast(recorder.calls[0][1][1], ctypes.POINTER(_lib.DecodeArgs)).contents
    assert args.batch == 2 and args.num_qo_heads == 32 and args.out_dtype == 0
    assert args.q == q.data_ptr() and args.out == out.data_ptr() and args.worklist
    assert abs(args.sm_scale - 128 ** -0.5) < 1e-7 and args.o_scale == 1.0
    assert w.run(q.view(2, 1, 32, 128), cache).shape == (2, 1, 32, 128)
    # uniform, device-resolved plan when the lengths must not be read
    w.plan(indptr, indices, torch.tensor([256, 200], dtype=torch.int32), 32, lay, kv_splits=4)
    assert w.kv_splits == 4 and w.reduction == "kernel"
    recorder.calls.clear()
    w.run(q, cache, out=out)
    # split units are merged inside the decode launch by default ...
    assert [c[0] for c in recorder.calls] == ["fq_decode"]
    args = ctypes.cast(recorder.calls[0][1][1], ctypes.POINTER(_lib.DecodeArgs)).contents
    assert args.unit_counters and not args.split_counts and args.kv_splits == 4
    # ... and by a second launch when that is switched off
    w.fused_merge = False
    w.plan(indptr, indices, torch.tensor([256, 200], dtype=torch.int32), 32, lay, kv_splits=4)
    recorder.calls.clear()
    w.run(q, cache, out=out)
    assert [c[0] for c in recorder.calls] == ["fq_decode", "fq_merge"]
    args = ctypes.cast(recorder.calls[0][1][1], ctypes.POINTER(_lib.DecodeArgs)).contents
    assert not args.unit_counters
    w.fused_merge = True
    w.plan(indptr, indices, torch.tensor([256, 200], dtype=torch.int32), 32, lay, kv_splits=1)
    assert w.kv_splits == 1 and w.reduction == "none"


def test_plan_refusals_are_transactional(recorder):
    lay, cache = _cache(None)
    w = PagedDecodeWrapper(torch.zeros(1 << 20, dtype=torch.uint8))
    indptr, indices = _plan_args()
    seq = torch.tensor([256, 200], dtype=torch.int32)
    w.plan(indptr, indices, seq, 32, lay)
    for bad, exc, match in [
        (dict(num_qo_heads=30), ValueError, "multiple of the layout's num_kv_heads"),
        (dict(q_len_per_req=0), ValueError, "q_len_per_req must be an int"),
        (dict(q_len_per_req=65), ValueError, "q_len_per_req must be an int"),
        (dict(q_data_type=torch.bfloat16), ValueError, "decode reads a"),
        (dict(o_data_type=torch.int8), ValueError, "decode writes a"),
        (dict(reduction="atomic"), NotImplementedError, "atomic"),
        (dict(reduction="bogus"), ValueError, "must be \"none\" or \"kernel\""),
        (dict(kv_splits=4, reduction="none"), ValueError, "requires kv_splits == 1"),
        (dict(bits=2), TypeError, "retired call form"),
        (dict(kernel_kwargs={}), TypeError, "kernel_kwargs is retired"),
    ]:
        kw = dict(num_qo_heads=32)
        kw.update(bad)
        hq = kw.pop("num_qo_heads")
        with pytest.raises(exc, match=match):
            w.plan(indptr, indices, seq, hq, lay, **kw)
        with pytest.raises(RuntimeError, match="Call plan"):
            w.run(torch.zeros(2, 32, 128).to(torch.float8_e4m3fn), cache)
        w.plan(indptr, indices, seq, 32, lay)
    with pytest.raises(TypeError, match="layout must be a QuantKVLayout"):
        w.plan(indptr, indices, seq, 32, 8)
    with pytest.raises(TypeError, match="extra positional"):
        w.plan(indptr, indices, seq, 32, lay, 128)
    with pytest.raises(ValueError, match="at least one request"):
        w.plan(indptr, indices, seq[:0], 32, lay)
    with pytest.raises(ValueError, match="seq_lens must be int32 or int64"):
        w.plan(indptr, indices, seq.float(), 32, lay)
    small = PagedDecodeWrapper(torch.zeros(64, dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="byte workspace"):
        small.plan(indptr, indices, seq, 32, lay, kv_splits=2)


def test_several_query_tokens_plan_as_columns(recorder):
    """q_len_per_req = L: the unit's columns, partial buffers and counters grow L-fold, the
    argument block carries q_len, and tensors take the [B, L, HQ, D] form."""
    lay, cache = _cache(None)
    w = PagedDecodeWrapper(torch.zeros(4 << 20, dtype=torch.uint8))
    indptr, indices = _plan_args()
    seq = torch.tensor([256, 200], dtype=torch.int32)
    w.plan(indptr, indices, seq, 32, lay, kv_splits=2, q_len_per_req=3)
    hkv = lay.num_kv_heads
    assert w._o_partial.shape == (2, 2, 1, 96, 128)
    assert w._unit_counters.numel() == 2 * hkv * ((32 // hkv * 3 + 7) // 8)
    q = torch.zeros(2, 3, 32, 128).to(torch.float8_e4m3fn)
    out = torch.zeros(2, 3, 32, 128, dtype=torch.bfloat16)
    lse = torch.zeros(2, 3, 32)
    recorder.calls.clear()
    w.run(q, cache, out=out, lse=lse, q_descale=torch.ones(2, 3, 32))
    args = ctypes.cast(recorder.calls[0][1][1], ctypes.POINTER(_lib.DecodeArgs)).contents
    assert args.q_len == 3 and args.num_qo_heads == 32
    assert (args.q_descale_stride_b, args.q_descale_stride_h) == (32, 1)
    with pytest.raises(ValueError, match=r"\[2, 3, 32, 128\]"):
        w.run(torch.zeros(2, 32, 128).to(torch.float8_e4m3fn), cache)
    with pytest.raises(ValueError, match="lse must be"):
        w.run(q, cache, out=out, lse=torch.zeros(2, 32))
    with pytest.raises(ValueError, match="seq_lens counts the 3 query tokens"):
        w.plan(indptr, indices, torch.tensor([256, 2], dtype=torch.int32), 32, lay,
               q_len_per_req=3)
    w.fused_merge = False
    with pytest.raises(NotImplementedError, match="in-kernel merge"):
        w.plan(indptr, indices, seq, 32, lay, q_len_per_req=2)
    w.fused_merge = True
    w.plan(indptr, indices, seq, 32, lay)
    assert w._q_len == 1 and w._cols == 32


def test_run_refusals(recorder):
    lay, cache = _cache(None)
    w = PagedDecodeWrapper(torch.zeros(1 << 20, dtype=torch.uint8))
    indptr, indices = _plan_args()
    w.plan(indptr, indices, torch.tensor([256, 200], dtype=torch.int32), 32, lay)
    q = torch.zeros(2, 32, 128).to(torch.float8_e4m3fn)
    with pytest.raises(TypeError, match="kv_cache must be a QuantKVCache"):
        w.run(q, torch.zeros(3))
    with pytest.raises(TypeError, match="retired call form"):
        w.run(q, cache, scale_pool=None)
    with pytest.raises(ValueError, match="mismatches the planned"):
        w.run(q.view(torch.uint8), cache)
    with pytest.raises(ValueError, match="the plan is for \\[2, 32, 128\\]"):
        w.run(torch.zeros(1, 16, 256).to(torch.float8_e4m3fn), cache)
    with pytest.raises(ValueError, match="lse must be"):
        w.run(q, cache, lse=torch.zeros(2, 32, dtype=torch.float64))
    with pytest.raises(ValueError, match="q_descale must be an fp32"):
        w.run(q, cache, q_descale=torch.zeros(2, 16))
    with pytest.raises(ValueError, match="out.dtype"):
        w.run(q, cache, out=torch.zeros(2, 32, 128))
    other_lay, other = _cache(None, bits=4)
    with pytest.raises(ValueError, match="another layout"):
        w.run(q, other)
    with pytest.raises(RuntimeError, match="graph mode's per-step call"):
        w.update([1, 2])


def test_graph_mode_refusals_before_any_device_work(fake_b200):
    lay = _layout()
    w = PagedDecodeWrapper(torch.zeros(1 << 20, dtype=torch.uint8), use_cuda_graph=True)
    assert type(w) is wr._GraphDecodeWrapper
    with pytest.raises(RuntimeError, match="plan\\(\\) it first"):
        w.update([1])
    # one long request alone wants the most pieces; a full bucket of long requests few
    assert 18 <= wr._graph_split_cap(1, 8, 1, 148, 784, 14) <= 64
    assert wr._graph_split_cap(1, 1, 1, 148, 784, 14) == 64
    assert 2 <= wr._graph_split_cap(64, 8, 1, 148, 784, 14) <= 16
    # the most skewed step of a bucket (one long request, the others one tile) still fits
    assert wr._graph_split_cap(19, 8, 1, 148, 782, 14) >= 15
    lens = wr._graph_host_lengths([5, 6], 2, 10)
    assert lens.dtype == np.int32
    with pytest.raises(ValueError, match="every length must be in"):
        wr._graph_host_lengths([5, 11], 2, 10)
    with pytest.raises(ValueError, match="integer lengths"):
        wr._graph_host_lengths([5.0, 1.0], 2, 10)


def test_plan_refuses_shapes_the_decode_kernel_lacks(recorder):
    """K groups other than 64 channels at head_dim 128 (and any sub-head K group at head_dim 256)
    are written and read back by this build but not decoded: plan() says so instead of failing
    at run()."""
    w = PagedDecodeWrapper(torch.zeros(1 << 20, dtype=torch.uint8))
    indptr, indices = _plan_args()
    seq = torch.tensor([256, 200], dtype=torch.int32)
    with pytest.raises(NotImplementedError, match="whole-head K groups at head_dim 256"):
        w.plan(indptr, indices, seq, 16, _layout(head_dim=256, num_kv_heads=2,
                                                 k_quant=("token", 128)))
    _, cache = _cache(None)
    with pytest.raises(RuntimeError, match="Call plan"):
        w.run(torch.zeros(2, 32, 128).to(torch.float8_e4m3fn), cache)
    w.plan(indptr, indices, seq, 16, _layout(head_dim=256, num_kv_heads=2))
    assert w.bits == 4 or w.bits == 2
    ok = _layout(head_dim=128, k_quant=("token", 64))
    w.plan(indptr, indices, seq, 32, ok)
    assert w.bits == ok.bits
