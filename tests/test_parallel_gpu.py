"""Multi-GPU decode on real GPUs (needs >= 2; skipped otherwise): one process per GPU over NCCL.

* sequence split: rank r caches and decodes only its page-aligned token range of one long
  context; one all_gather of (o, lse) and a local merge kernel give every rank the full result,
  checked against the fp32 oracle over the whole context (tolerance of the decode tests).
* KV-head tensor parallel: rank r caches and decodes its KV heads only; no communication on the
  data path; its output equals the oracle's slice for its query heads.
NVLS is switched off; the peers are reached through NCCL, and through plain stores and loads on
peer-mapped pointers in the library's exchange kernel (no multicast, no bulk copies)."""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from helpers import PAGE, cpu_twin, make_kv, make_q, oracle_outputs, paged_batch

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, parallel
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        bits, d, hq, hkv, seq = 2, 128, 32, 8, 20000
        k, v = make_kv(seq, hkv, d, seed=5, device=dev)          # same context on every rank
        q = make_q(1, hq, d, seed=6, device=dev)
        sm = d ** -0.5
        # ---- sequence split
        a, b = parallel.split_sequence(seq, rank, world)
        n = b - a
        layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device=dev)
        indptr, indices, slots, npages = paged_batch([n], seed=rank)
        cache = layout.allocate(npages)
        cache.append(k[a:b], v[a:b], torch.from_numpy(slots).to(dev))
        w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device=dev))
        w.plan(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev),
               torch.tensor([n], dtype=torch.int32), hq, layout, sm_scale=sm,
               o_data_type=torch.float32)
        out = parallel.sequence_split_decode(w, q, cache)
        torch.cuda.synchronize(dev)
        assert w.last_status() == 0
        # the same step through the one-launch exchange (peer stores + flags), three times over
        # (both parities of its staging area): the rows equal the all_gather form's
        ex = parallel.SequenceSplitExchange(1, hq, d, device=dev)
        fused_ok = True
        for _ in range(3):
            out2 = parallel.sequence_split_decode(w, q, cache, exchange=ex)
            torch.cuda.synchronize(dev)
            fused_ok = fused_ok and ex.last_status() == 0 and \
                (out2.float() - out.float()).abs().max().item() <= 1e-2
        # oracle over the whole context, cached the same way (token-wise records do not depend
        # on which page a token sits in)
        f_indptr, f_indices, f_slots, f_pages = paged_batch([seq], seed=9)
        full = layout.allocate(f_pages)
        full.append(k, v, torch.from_numpy(f_slots).to(dev))
        pools = cpu_twin(full, k, v, f_slots)
        want, _ = oracle_outputs(pools, q.cpu(), f_indptr, f_indices, [seq], sm, None)
        err = (out.float().cpu() - want).abs()
        seq_ok = err.max().item() <= MAX_ABS and err.mean().item() <= MEAN_ABS
        # ---- KV-head tensor parallel
        qh, kvh = parallel.shard_kv_heads(hq, hkv, rank, world)
        lay_tp = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=len(kvh), device=dev)
        cache_tp = lay_tp.allocate(f_pages)
        ks = k[:, kvh.start:kvh.stop].contiguous()
        vs = v[:, kvh.start:kvh.stop].contiguous()
        cache_tp.append(ks, vs, torch.from_numpy(f_slots).to(dev))
        w2 = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device=dev))
        w2.plan(torch.from_numpy(f_indptr).to(dev), torch.from_numpy(f_indices).to(dev),
                torch.tensor([seq], dtype=torch.int32), len(qh), lay_tp, sm_scale=sm)
        q_tp = q[:, qh.start:qh.stop].contiguous()
        out_tp = w2.run(q_tp, cache_tp)
        torch.cuda.synchronize(dev)
        err2 = (out_tp.float().cpu() - want[:, qh.start:qh.stop]).abs()
        tp_ok = err2.max().item() <= MAX_ABS and err2.mean().item() <= MEAN_ABS
        ret[rank] = (bool(seq_ok and fused_ok), bool(tp_ok), float(err.max()), float(err2.max()))
    finally:
        dist.destroy_process_group()


def test_sequence_split_and_tensor_parallel_over_nccl():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = 29500 + os.getpid() % 2000
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank, args=(world, port, ret), nprocs=world, join=True)
    got = dict(ret)
    assert sorted(got) == list(range(world)), got
    assert all(v[0] and v[1] for v in got.values()), got
