"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and
its host-only planners keep their invariants (every tile covered exactly once, balanced CTAs).
No compute entry point is called here."""
import os
import re

import numpy as np
import pytest

from foscar_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "foscar_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fq_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_loads_and_exports_the_header():
    path = _build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    names = _declared_functions()
    assert "fq_decode" in names and "fq_append" in names and len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == names
    assert lib.fq_version().decode().startswith("foscar_b200")
    assert lib.fq_error_string(-2).decode() == "unsupported configuration"


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("FOSCAR_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def _plan(lens, hkv, ht, ctas, cap=64, bits=4, d=128):
    lib = _lib.load()
    lens = np.asarray(lens, dtype=np.int32)
    words = int(lib.fq_worklist_words(len(lens), hkv, ht, ctas))
    work = np.zeros(words, dtype=np.int32)
    counts = np.zeros(len(lens) * hkv * ht, dtype=np.int32)
    n = lib.fq_plan_worklist(lens.ctypes.data, len(lens), hkv, ht, ctas, cap, work.ctypes.data,
                             words, counts.ctypes.data, bits, d)
    return n, work, counts


def _pieces_by_unit(n, work):
    rows = work[work[3]:work[3] + 8 * n].reshape(n, 8)
    seen = {}
    for b, kvh, t, t0, t1, slot, _, _ in rows:
        seen.setdefault((b, kvh, t), []).append((t0, t1, slot))
    return rows, seen


@pytest.mark.parametrize("lens,hkv,ht,ctas", [
    ([128, 128], 8, 1, 148), ([1, 63, 64, 65, 5000, 131072], 8, 1, 148), ([100352], 8, 1, 148),
    (list(range(1, 300, 7)), 2, 2, 148), ([0, 5, 0], 1, 1, 4), ([70000] * 3, 1, 1, 7),
])
@pytest.mark.parametrize("bits", [2, 4])
def test_worklist_covers_every_tile_once(lens, hkv, ht, ctas, bits):
    tt = _lib.tile_tokens(bits, 128)
    n, work, counts = _plan(lens, hkv, ht, ctas, bits=bits)
    assert n > 0 and work[0] == n and work[1] == len(lens) * hkv * ht and work[2] == ctas
    starts = work[8:8 + ctas + 1]
    assert starts[0] == 0 and starts[-1] == n and np.all(np.diff(starts) >= 0)
    rows = work[work[3]:work[3] + 8 * n].reshape(n, 8)
    tiles = {b: -(-l // tt) if l > 0 else 0 for b, l in enumerate(lens)}
    seen = {}
    for b, kvh, t, t0, t1, slot, _, _ in rows:
        assert 0 <= b < len(lens) and 0 <= kvh < hkv and 0 <= t < ht and 0 <= t0 <= t1
        seen.setdefault((b, kvh, t), []).append((t0, t1, slot))
    assert len(seen) == len(lens) * hkv * ht
    for (b, kvh, t), pieces in seen.items():
        pieces.sort()
        assert pieces[0][0] == 0 and pieces[-1][1] == tiles[b]
        for (a0, a1, _), (b0, _, _) in zip(pieces, pieces[1:]):
            assert a1 == b0 and a1 > a0
        k = counts[(b * hkv + kvh) * ht + t]
        assert k == len(pieces)
        assert [p[2] for p in pieces] == ([-1] if k == 1 else list(range(k)))
    load = np.array([(rows[starts[c]:starts[c + 1], 4] - rows[starts[c]:starts[c + 1], 3]).sum()
                     for c in range(ctas)])
    total = load.sum()
    if total > 50 * ctas:
        assert load.max() <= total / ctas * 1.15 + 8


@pytest.mark.parametrize("lens,hkv,ht,cap", [
    ([131072], 1, 1, 4), ([100000] + [1] * 18, 8, 1, 2), ([131072] + [128] * 63, 8, 1, 2),
    ([100352], 1, 1, 64), ([100352], 1, 1, 1), ([5000, 70000, 3], 2, 2, 3),
    ([131072] * 3 + [64] * 300, 1, 1, 5),
])
def test_worklist_never_exceeds_the_split_cap(lens, hkv, ht, cap):
    """No unit is cut into more pieces than the cap, whatever the skew: the planner raises the
    share per CTA instead of refusing (a graph-mode update() must never fail on valid lengths)."""
    n, work, counts = _plan(lens, hkv, ht, 148, cap=cap)
    assert n > 0
    assert counts.max() <= cap
    rows, seen = _pieces_by_unit(n, work)
    tt = _lib.tile_tokens(4, 128)
    for (b, kvh, t), pieces in seen.items():
        pieces.sort()
        assert len(pieces) <= cap
        assert pieces[0][0] == 0 and pieces[-1][1] == -(-lens[b] // tt)
        for (a0, a1, _), (b0, _, _) in zip(pieces, pieces[1:]):
            assert a1 == b0


def test_rows_take_their_requests_length_and_table_offset():
    """fq_worklist_attach_requests fills every row's two spare words from host arrays and marks
    the header; a list that is not passed through it keeps them 0."""
    lib = _lib.load()
    lens = [5000, 1, 70000]
    n, work, counts = _plan(lens, 2, 1, 148)
    rows = work[work[3]:work[3] + 8 * n].reshape(n, 8)
    assert work[4] == 0 and not rows[:, 6:].any()
    lens32 = np.asarray(lens, dtype=np.int32)
    offsets = np.asarray([0, 79, 80], dtype=np.int32)
    assert lib.fq_worklist_attach_requests(work.ctypes.data, len(work), lens32.ctypes.data,
                                           offsets.ctypes.data, 3) == 0
    assert work[4] == 1
    assert np.array_equal(rows[:, 6], lens32[rows[:, 0]])
    assert np.array_equal(rows[:, 7], offsets[rows[:, 0]])
    # a batch smaller than the rows' requests, a buffer shorter than the list, missing arrays
    assert lib.fq_worklist_attach_requests(work.ctypes.data, len(work), lens32.ctypes.data,
                                           offsets.ctypes.data, 2) == _lib.ERR_BAD_ARG
    assert lib.fq_worklist_attach_requests(work.ctypes.data, int(work[3]) + 8, lens32.ctypes.data,
                                           offsets.ctypes.data, 3) == _lib.ERR_BAD_ARG
    assert lib.fq_worklist_attach_requests(work.ctypes.data, len(work), None,
                                           offsets.ctypes.data, 3) == _lib.ERR_BAD_ARG


def test_worklist_refuses_a_short_buffer():
    lib = _lib.load()
    lens = np.array([100], dtype=np.int32)
    small = np.zeros(16, dtype=np.int32)
    counts = np.zeros(8, dtype=np.int32)
    assert lib.fq_plan_worklist(lens.ctypes.data, 1, 8, 1, 148, 64, small.ctypes.data, 16,
                                counts.ctypes.data, 2, 128) == _lib.ERR_TOO_LARGE


@pytest.mark.parametrize("batch,hkv,length", [(1, 8, 100352), (4, 8, 100352), (16, 8, 100352),
                                              (1, 1, 524288), (8, 2, 32768), (64, 8, 16384)])
def test_uniform_planner_agrees_with_the_balanced_one(batch, hkv, length):
    """On a uniform batch the closed-form planner (no host lengths) and the balanced piece list
    cut a unit into similar numbers of pieces: both count a piece's overhead in the same tile
    units."""
    lib = _lib.load()
    s = lib.fq_plan_splits(batch, hkv, 1, length, 2, 128, 148)
    n, work, counts = _plan([length] * batch, hkv, 1, 148, bits=2)
    most = int(counts.max())
    assert s >= 1 and n > 0
    assert most / 3 <= s <= max(most * 2.5, 2), (s, most)


def test_uniform_planner_behaviour():
    lib = _lib.load()
    assert lib.fq_plan_splits(64, 8, 1, 16384, 2, 128, 148) == 1      # enough units: no split
    s1 = lib.fq_plan_splits(1, 8, 1, 100352, 2, 128, 148)
    assert 8 <= s1 <= 64                                               # one long request: split
    assert lib.fq_plan_splits(1, 8, 1, 256, 2, 128, 148) == 1          # too short to split
    assert lib.fq_plan_splits(0, 8, 1, 256, 2, 128, 148) == _lib.ERR_BAD_ARG
    assert lib.fq_workspace_bytes(4, 2, 32, 128) == 4 * 4 * 2 * 32 * 130


def test_worklist_tiles_hold_256_tokens_at_head_dim_64():
    """At head_dim 64 a tile is 256 tokens (two per tensor-memory lane): the planner's tile
    ranges cover ceil(len / 256) tiles of every unit."""
    lib = _lib.load()
    lens = np.array([1, 256, 257, 5000, 100000], dtype=np.int32)
    hkv, ht, ctas = 8, 1, 148
    words = int(lib.fq_worklist_words(len(lens), hkv, ht, ctas))
    work = np.zeros(words, dtype=np.int32)
    counts = np.zeros(len(lens) * hkv * ht, dtype=np.int32)
    n = lib.fq_plan_worklist(lens.ctypes.data, len(lens), hkv, ht, ctas, 64, work.ctypes.data,
                             words, counts.ctypes.data, 2, 64)
    assert n > 0
    rows = work[work[3]:work[3] + 8 * n].reshape(n, 8)
    covered = {}
    for b, kvh, t, t0, t1, slot, _, _ in rows:
        covered[(b, kvh)] = covered.get((b, kvh), 0) + (t1 - t0)
    for b, l in enumerate(lens):
        for kvh in range(hkv):
            assert covered[(b, kvh)] == -(-int(l) // 256)
    assert _lib.tile_tokens(2, 64) == 256 and _lib.tile_tokens(4, 64) == 256
    assert _lib.tile_tokens(4, 128) == 128
    assert _lib.tile_tokens(2, 128) in (128, 256)     # two tokens per lane in the INT2 build
    assert _lib.piece_overhead(2, 128) > 0


def _fake_pools(**over):
    """Pool descriptor with made-up, 16-byte aligned addresses: enough for the argument checks,
    which run before any launch (nothing is dereferenced on the host)."""
    p = _lib.Pools(bits=2, head_dim=128, num_kv_heads=8, k_groups=1, scale_bf16=0, num_pages=4,
                   k_channel_group=0, k_codes=0x10000, v_codes=0x20000, scales=0x30000,
                   v_page_max=0x40000, v_max_hist=0x50000)
    for name, value in over.items():
        setattr(p, name, value)
    return p


def test_entry_points_refuse_misaligned_or_senseless_arguments_before_any_launch():
    import ctypes
    lib = _lib.load()
    ok, bad = 0x100000, 0x100002            # made-up device addresses
    p = _fake_pools()
    # writer: 16-byte rows and strides
    assert lib.fq_append(ctypes.byref(p), bad, ok, 1024, 1024, ok, 4, -1, -1, None, None) \
        == _lib.ERR_BAD_ARG
    assert lib.fq_append(ctypes.byref(p), ok, ok, 1020, 1024, ok, 4, -1, -1, None, None) \
        == _lib.ERR_BAD_ARG
    assert lib.fq_append(ctypes.byref(p), ok, ok, 1024, 1024, ok, 4, 128, -1, None, None) \
        == _lib.ERR_BAD_ARG                                  # clip index outside the row
    assert lib.fq_append_quantized(ctypes.byref(p), bad, ok, ok, ok, ok, ok, ok, 4, None, None) \
        == _lib.ERR_BAD_ARG
    # the layout-only page-group write: channel-wise K pools only, code rows 4-byte aligned
    pch = _fake_pools(head_dim=256, k_channel_group=64)
    assert lib.fq_append_quantized_page_groups(ctypes.byref(p), ok, ok, ok, ok, ok, ok, ok, None,
                                               1, None, None) == _lib.ERR_UNSUPPORTED
    assert lib.fq_append_quantized_page_groups(ctypes.byref(pch), ok, ok, ok, bad, ok, ok, ok,
                                               None, 1, None, None) == _lib.ERR_BAD_ARG
    assert lib.fq_append_quantized_page_groups(ctypes.byref(pch), ok, None, ok, ok, ok, ok, ok,
                                               None, 1, None, None) == _lib.ERR_BAD_ARG
    assert lib.fq_append_quantized_page_groups(ctypes.byref(pch), ok, ok, ok, ok, ok, ok, ok,
                                               None, 0, None, None) == 0
    assert lib.fq_append_quantized_page_groups(ctypes.byref(pch), ok, ok, ok, ok, ok, ok, ok,
                                               None, 1 << 26, None, None) == _lib.ERR_TOO_LARGE
    pz = _fake_pools(num_kv_heads=0)
    assert lib.fq_append(ctypes.byref(pz), ok, ok, 1024, 1024, ok, 4, -1, -1, None, None) \
        == _lib.ERR_BAD_ARG
    p96 = _fake_pools(head_dim=96)
    assert lib.fq_append(ctypes.byref(p96), ok, ok, 1024, 1024, ok, 4, -1, -1, None, None) \
        == _lib.ERR_UNSUPPORTED
    # read-back: 16-byte destinations, row strides in multiples of eight elements
    assert lib.fq_dequantize(ctypes.byref(p), bad, ok, 1024, 1024, 64, ok, ok, 1, ok, ok, 0, 1,
                             None, None) == _lib.ERR_BAD_ARG
    assert lib.fq_dequantize(ctypes.byref(p), ok, ok, 1028, 1024, 64, ok, ok, 1, ok, ok, 0, 1,
                             None, None) == _lib.ERR_BAD_ARG
    # decode
    def args(**over):
        a = _lib.DecodeArgs()
        a.batch, a.num_qo_heads, a.kv_splits, a.max_splits = 2, 32, 1, 1
        a.seq_lens = a.page_table = a.table_offsets = ok
        a.q, a.out, a.status = ok, ok, ok
        for name, value in over.items():
            setattr(a, name, value)
        return a
    def decode(pools, a):
        return lib.fq_decode(ctypes.byref(pools), ctypes.byref(a), None)
    assert decode(p, args(q=bad)) == _lib.ERR_BAD_ARG
    assert decode(p, args(worklist=bad, num_work=4)) == _lib.ERR_BAD_ARG
    assert decode(pz, args()) == _lib.ERR_BAD_ARG
    assert decode(p, args(num_qo_heads=30)) == _lib.ERR_BAD_ARG
    assert decode(p96, args()) == _lib.ERR_UNSUPPORTED
    assert decode(p, args(kv_splits=2, max_splits=1, o_partial=ok, l_partial=ok, m_partial=ok)) \
        == _lib.ERR_BAD_ARG
    # several query tokens: at most 64, and split units only with the in-kernel merge
    assert decode(p, args(q_len=65)) == _lib.ERR_BAD_ARG
    assert decode(p, args(q_len=2, kv_splits=2, max_splits=2, o_partial=ok, l_partial=ok,
                          m_partial=ok)) == _lib.ERR_UNSUPPORTED
    assert lib.fq_decode_split_static(ctypes.byref(p), ctypes.byref(args(q_len=2)), None) \
        == _lib.ERR_UNSUPPORTED
    grouped = _fake_pools(k_groups=2, scale_bf16=1)
    assert decode(grouped, args(q_len=2)) == _lib.ERR_UNSUPPORTED
