"""Several query tokens per request (q_len_per_req = L > 1, speculative / multi-token decode):
query token l of a request attends to positions < seq_len - (L - 1 - l). The reference refuses
this form (src/foscar/wrapper.py:756-761), so the check is the oracle's fp32 attention run once
per query token over the prefix that token sees. Tolerance as for one token: max-abs 2e-2,
mean-abs 2e-3, LSE 5e-2."""
import numpy as np
import pytest
import torch

from helpers import PAGE, cpu_twin, make_kv, paged_batch
from oracle import ref_attention, ref_dequantize

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_ABS = 2e-2, 2e-3, 5e-2


def _case(bits, d, hq, hkv, L, seq, *, kv_splits=None, k_channel=False, graph=False,
          descale=False, seed=0):
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout
    b = len(seq)
    indptr, indices, slots, npages = paged_batch(seq, seed=seed)
    k, v = make_kv(len(slots), hkv, d, seed=seed)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(npages + 1)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    g = torch.Generator().manual_seed(seed + 11)
    q = torch.randn(b, L, hq, d, generator=g).clamp(-448, 448).to(torch.float8_e4m3fn).cuda()
    qd = (torch.rand(b, L, hq, generator=g) + 0.5).cuda() if descale else None
    sm_scale = d ** -0.5
    w = PagedDecodeWrapper(torch.empty(64 << 20, dtype=torch.uint8, device="cuda"))
    w.plan(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(),
           torch.tensor(seq, dtype=torch.int32), hq, layout, q_len_per_req=L,
           kv_splits=kv_splits)
    out = torch.full((b, L, hq, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((b, L, hq), float("nan"), device="cuda")
    for _ in range(2):      # twice: split units must leave their counters at zero
        out.fill_(float("nan"))
        w.run(q, cache, out=out, lse=lse, q_descale=qd)
        torch.cuda.synchronize()
        assert w.last_status() == 0
    pools = cpu_twin(cache, k, v, slots)
    kv = ref_dequantize(pools, indptr, indices, seq, rounded=False)
    worst = mean = lse_worst = 0.0
    for r, n in enumerate(seq):
        for l in range(L):
            sees = n - (L - 1 - l)
            want, lse_want = ref_attention(q[r, l].cpu().float(), kv[r][0][:sees],
                                           kv[r][1][:sees], sm_scale,
                                           None if qd is None else qd[r, l].cpu())
            err = (out[r, l].float().cpu() - want).abs()
            assert torch.isfinite(out[r, l].float()).all(), (r, l)
            worst, mean = max(worst, err.max().item()), mean + err.mean().item()
            lse_worst = max(lse_worst, (lse[r, l].cpu() - lse_want).abs().max().item())
    assert worst <= MAX_ABS, f"max-abs {worst:.3e}"
    assert mean / (len(seq) * L) <= MEAN_ABS
    assert lse_worst <= LSE_ABS, f"lse {lse_worst:.3e}"
    return w


# lengths around the tile edges: 129 and 257 leave one token in the last 128/256-token tile,
# which every column but the last query token's then sees nothing of
SEQ = [4, 64, 128, 129, 130, 257, 1000, 4097]


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("d,hq,hkv,L", [(128, 32, 8, 2),    # 4 heads x 2 tokens: one head tile
                                        (128, 16, 2, 3),    # 8 heads x 3 tokens: a tile a token
                                        (128, 12, 4, 4),    # 3 heads x 4 tokens: tiles mix tokens
                                        (64, 8, 8, 4),      # 1 head x 4 tokens
                                        (256, 16, 2, 2)])   # head_dim 256
def test_tokens_against_oracle(bits, d, hq, hkv, L):
    _case(bits, d, hq, hkv, L, SEQ, seed=bits + d + L)


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("kv_splits", [1, 4, 33])
def test_uniform_splits_and_descale(d, kv_splits):
    """Uniform pieces (the last piece of the 4097- and 129-token requests is the last tile
    alone), with q_descale per (request, token, head)."""
    w = _case(4, d, 16, 2, 2, [129, 257, 4097, 700], kv_splits=kv_splits, descale=True, seed=5)
    assert w.kv_splits == kv_splits


def test_minimum_length_and_single_request():
    """seq_len == q_len: token 0 sees one position."""
    _case(2, 128, 32, 8, 4, [4], seed=2)
    _case(4, 128, 32, 8, 2, [2, 3], seed=3)


def test_graph_mode_with_two_query_tokens():
    """Graph mode: plan once with q_len_per_req=2, capture, then update lengths and replay."""
    from foscar_b200 import PagedDecodeWrapper, QuantKVLayout, graph_workspace_bytes
    bits, hq, hkv, d, L = 2, 32, 8, 128, 2
    batch, max_len = 3, 3000
    max_pages = -(-max_len // 64)
    layout = QuantKVLayout.create(bits=bits, head_dim=d, num_kv_heads=hkv, device="cuda")
    cache = layout.allocate(batch * max_pages)
    table = torch.arange(batch * max_pages, dtype=torch.int32, device="cuda").view(batch, max_pages)
    seq_dev = torch.full((batch,), L, dtype=torch.int32, device="cuda")
    slots = np.concatenate([np.arange(max_len) + b * max_pages * 64 for b in range(batch)])
    k, v = make_kv(len(slots), hkv, d, seed=4)
    cache.append(k, v, torch.from_numpy(slots).cuda())
    pools = cpu_twin(cache, k, v, slots)
    # workspace for the columns of two query tokens: sized as for twice the heads
    ws = torch.empty(graph_workspace_bytes(batch, hq * L, layout, max_kv_len=max_len),
                     dtype=torch.uint8, device="cuda")
    w = PagedDecodeWrapper(ws, use_cuda_graph=True)
    w.plan(page_table=table, seq_lens=seq_dev, num_qo_heads=hq, layout=layout, max_kv_len=max_len,
           q_len_per_req=L)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(batch, L, hq, d, generator=g).to(torch.float8_e4m3fn).cuda()
    out = torch.empty(batch, L, hq, d, dtype=torch.bfloat16, device="cuda")
    w.run(q, cache, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        w.run(q, cache, out=out)
    indptr = np.arange(batch + 1, dtype=np.int32) * max_pages
    indices = np.arange(batch * max_pages, dtype=np.int32)
    for lengths in ([2, 129, 3000], [2999, 257, 64]):
        seq_dev.copy_(torch.tensor(lengths, dtype=torch.int32))
        w.update(lengths)
        graph.replay()
        torch.cuda.synchronize()
        assert w.last_status() == 0
        kv = ref_dequantize(pools, indptr, indices, lengths, rounded=False)
        for r, n in enumerate(lengths):
            for l in range(L):
                sees = n - (L - 1 - l)
                want, _ = ref_attention(q[r, l].cpu().float(), kv[r][0][:sees], kv[r][1][:sees],
                                        d ** -0.5)
                err = (out[r, l].float().cpu() - want).abs()
                tol = 2e-3 + want.abs().mean().item() * 2.0 ** -9
                assert err.max().item() <= MAX_ABS and err.mean().item() <= tol, (lengths, r, l)
