"""The split decode that allocates nothing (`fq_decode_split_static`), through the C ABI.

Some hosts of the library cannot hand it a workspace: an inference engine that owns the CUDA
allocator and forbids cudaMalloc from plugins, or a call site where allocating is illegal (inside
a stream capture, a latency-critical loop). For them the split partials live in a buffer that is
part of the library image. The entry point must give exactly what the regular path gives (decode
into a caller workspace, then merge), on two calls in a row, because the buffer keeps the previous
call's contents. Collected last on purpose: a failure here stops nothing else."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import make_kv, make_q, paged_batch

pytestmark = pytest.mark.gpu


def _args(lib_mod, w, q, out, lse, kv_splits):
    a = lib_mod.DecodeArgs()
    a.batch, a.num_qo_heads = w._batch_size, w._num_qo_heads
    a.out_dtype = 0
    a.kv_splits = kv_splits
    a.sm_scale, a.o_scale = w._sm_scale, 1.0
    a.seq_lens = w._seqlens.data_ptr()
    a.page_table = w._page_table.data_ptr()
    a.table_offsets = w._table_offsets.data_ptr()
    a.table_len = w._page_table.numel()
    a.q, a.out, a.lse = q.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.status = w._status_ptr()
    return a


@pytest.mark.parametrize("bits", [2, 4])
def test_static_scratch_split_matches_workspace_split(bits):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, _lib
    lib = _lib.load()
    hq, hkv, d, splits = 32, 8, 128, 4
    stream = torch.cuda.current_stream().cuda_stream
    for round_, seq in enumerate(([5000, 700, 1], [64, 9000, 3000])):
        indptr, indices, slots, npages = paged_batch(seq, seed=round_)
        k, v = make_kv(len(slots), hkv, d, seed=10 + round_)
        layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
        cache = layout.allocate(npages)
        cache.append(k, v, torch.from_numpy(slots).cuda())
        q = make_q(len(seq), hq, d, seed=20 + round_)
        w = PagedDecodeWrapper(torch.empty(32 << 20, dtype=torch.uint8, device="cuda"))
        w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
               torch.tensor(seq, dtype=torch.int32, device="cuda"), hq, layout, kv_splits=splits)
        want = torch.empty(len(seq), hq, d, dtype=torch.bfloat16, device="cuda")
        want_lse = torch.empty(len(seq), hq, device="cuda")
        w.run(q, cache, out=want, lse=want_lse)
        got = torch.full_like(want, float("nan"))
        got_lse = torch.full_like(want_lse, float("nan"))
        a = _args(_lib, w, q, got, got_lse, splits)
        rc = lib.fq_decode_split_static(ctypes.byref(cache._c_pools), ctypes.byref(a), stream)
        assert rc == 0, lib.fq_error_string(rc)
        torch.cuda.synchronize()
        assert w.last_status() == 0
        assert torch.equal(got, want), (got.float() - want.float()).abs().max()
        assert torch.equal(got_lse, want_lse)


def test_static_scratch_rejects_what_does_not_fit():
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, _lib
    lib = _lib.load()
    hq, hkv, d = 32, 8, 128
    batch = 64                      # 64 splits x 64 x 32 x 130 x 4 B = 68 MB > 8 MiB
    seq = [64] * batch
    indptr, indices, slots, npages = paged_batch(seq)
    layout = QuantKVLayout.create(bits=2, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages)
    w = PagedDecodeWrapper(torch.empty(1 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32, device="cuda"), hq, layout, kv_splits=1)
    q = make_q(batch, hq, d)
    out = torch.zeros(batch, hq, d, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(batch, hq, device="cuda")
    a = _args(_lib, w, q, out, lse, 64)
    rc = lib.fq_decode_split_static(ctypes.byref(cache._c_pools), ctypes.byref(a),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_SCRATCH_TOO_SMALL
    assert b"scratch" in lib.fq_error_string(rc)
    torch.cuda.synchronize()
    assert int(out.float().abs().sum()) == 0          # nothing was launched
