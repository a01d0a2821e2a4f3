"""run() inside a CUDA graph: eager-mode capture replays bit-identically, and graph mode
(plan once, update(lengths) per step, replay) follows each step's lengths."""
import numpy as np
import pytest
import torch

from helpers import cpu_twin, make_kv, make_q, oracle_outputs, paged_batch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [2, 4])
def test_eager_run_replays_identically(bits):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    hq, hkv, d, seq = 16, 2, 128, [8192, 8192]
    indptr, indices, slots, npages = paged_batch(seq, shuffle=False)
    k, v = make_kv(len(slots), hkv, d)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    q = make_q(2, hq, d)
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32, device="cuda"), hq, layout)
    out = torch.empty(2, hq, d, dtype=torch.bfloat16, device="cuda")
    w.run(q, cache, out=out)
    torch.cuda.synchronize()
    eager = out.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            w.run(q, cache, out=out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w.run(q, cache, out=out)
    torch.cuda.synchronize()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    assert w.last_status() == 0


@pytest.mark.parametrize("bits,hq,hkv,d", [(2, 32, 8, 128), (4, 64, 8, 64), (2, 64, 8, 64)])
def test_graph_mode_follows_updates(bits, hq, hkv, d):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, graph_workspace_bytes
    batch, max_len = 3, 6000
    max_pages = -(-max_len // 64)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(batch * max_pages)
    table = torch.arange(batch * max_pages, dtype=torch.int32, device="cuda").view(batch, max_pages)
    seq_dev = torch.ones(batch, dtype=torch.int32, device="cuda")
    # fill every request to max_len once; steps then decode at shorter lengths
    full = [max_len] * batch
    slots = np.concatenate([np.arange(max_len) + b * max_pages * 64 for b in range(batch)])
    k, v = make_kv(len(slots), hkv, d, seed=2)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    pools = cpu_twin(cache, k, v, slots)
    ws = torch.empty(graph_workspace_bytes(batch, hq, layout, max_kv_len=max_len),
                     dtype=torch.uint8, device="cuda")
    w = PagedDecodeWrapper(ws, use_cuda_graph=True)
    w.plan(page_table=table, seq_lens=seq_dev, num_qo_heads=hq, layout=layout, max_kv_len=max_len)
    q = make_q(batch, hq, d)
    out = torch.empty(batch, hq, d, dtype=torch.bfloat16, device="cuda")
    w.run(q, cache, out=out)            # warm-up at the plan's length-1 list
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w.run(q, cache, out=out)
    indptr = np.arange(batch + 1, dtype=np.int32) * max_pages
    indices = np.arange(batch * max_pages, dtype=np.int32)
    for lengths in ([1, 1, 1], [6000, 64, 3000], [129, 5999, 17], [6000, 6000, 6000]):
        seq_dev.copy_(torch.tensor(lengths, dtype=torch.int32))
        w.update(lengths)
        graph.replay()
        torch.cuda.synchronize()
        want, _ = oracle_outputs(pools, q.cpu(), indptr, indices, lengths, d ** -0.5)
        err = (out.float().cpu() - want).abs()
        # the bf16 output's own rounding (2^-9 relative) is allowed on top of the mean tolerance:
        # at length 1 the output is a single V row of magnitude ~1
        mean_tol = 2e-3 + want.abs().mean().item() * 2.0 ** -9
        assert err.max().item() <= 2e-2 and err.mean().item() <= mean_tol, (lengths, err.max())
    assert w.last_status() == 0
