"""The merge of attention states from sequence shards (`fq_merge_states`, the kernel under
`parallel.merge_states` and `gather_and_merge`) on one GPU, against the closed form in float64:
out = sum_r exp(lse_r - LSE) o_r with LSE = log sum_r exp(lse_r); a shard with lse = -inf (an
empty token range) contributes nothing and a row whose every shard is empty gives zeros and
lse = -inf. Tolerance: 2e-6 relative on f32 outputs, one bf16 ulp on bf16 outputs."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _want(o, lse):
    o, lse = o.double().cpu(), lse.double().cpu()
    top = torch.logsumexp(lse, dim=0)                                    # [B, HQ]
    w = torch.exp(lse - torch.where(torch.isinf(top), torch.zeros_like(top), top))
    w = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(w), w)
    return (w[..., None] * o).sum(0), top


def _shards(n, b, hq, d, seed, empty=True):
    g = torch.Generator().manual_seed(seed)
    o = torch.randn(n, b, hq, d, generator=g)
    lse = torch.randn(n, b, hq, generator=g) * 4.0
    if empty:
        lse[0, 0, :] = -float("inf")            # one shard empty for a request
        lse[:, b - 1, 0] = -float("inf")        # a row no shard saw
    return o.cuda(), lse.cuda()


@pytest.mark.parametrize("n,b,hq,d", [(2, 3, 8, 64), (8, 4, 32, 128), (3, 2, 16, 256), (1, 1, 4, 128)])
def test_merge_states_matches_the_closed_form(n, b, hq, d):
    from foscar_b200 import parallel
    o, lse = _shards(n, b, hq, d, seed=n * 100 + d, empty=n > 1)
    out = torch.full((b, hq, d), float("nan"), dtype=torch.float32, device="cuda")
    got_lse = torch.full((b, hq), float("nan"), device="cuda")
    parallel.merge_states(o, lse, out=out, lse=got_lse)
    torch.cuda.synchronize()
    want, want_lse = _want(o, lse)
    assert torch.allclose(out.double().cpu(), want, rtol=2e-6, atol=2e-6)
    finite = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(got_lse.cpu()), finite)
    assert torch.allclose(got_lse.double().cpu()[finite], want_lse[finite], rtol=2e-6, atol=2e-6)
    if n > 1:
        assert (out[b - 1, 0] == 0).all() and got_lse[b - 1, 0].item() == -float("inf")
    half = parallel.merge_states(o, lse)                                  # bf16 by default
    torch.cuda.synchronize()
    assert half.dtype == torch.bfloat16
    assert torch.equal(half.cpu(), out.cpu().to(torch.bfloat16))


def test_merge_states_reads_packed_rows_in_place():
    """The form the all_gather exchange uses: rows of D + 1 floats (o then lse), merged through
    strides without unpacking."""
    from foscar_b200 import _lib, device as dev
    n, b, hq, d = 4, 5, 32, 128
    o, lse = _shards(n, b, hq, d, seed=7)
    packed = torch.cat([o, lse[..., None]], dim=-1).contiguous()          # [N, B, HQ, D + 1]
    out = torch.empty(b, hq, d, dtype=torch.float32, device="cuda")
    got_lse = torch.empty(b, hq, device="cuda")
    base = packed.data_ptr()
    _lib.check(_lib.load().fq_merge_states(base, base + 4 * d, n, b, hq, d, out.data_ptr(), 2,
                                           got_lse.data_ptr(), d + 1, d + 1,
                                           dev.current_stream_ptr(out.device)), "merge_states")
    torch.cuda.synchronize()
    want, _ = _want(o, lse)
    assert torch.allclose(out.double().cpu(), want, rtol=2e-6, atol=2e-6)
    plain = torch.empty_like(out)
    from foscar_b200 import parallel
    parallel.merge_states(o, lse, out=plain)
    torch.cuda.synchronize()
    assert torch.equal(plain, out)


def test_merge_states_of_a_large_batch():
    """A batch larger than L2: 8 shards x 2048 x 32 rows of 128 channels (268 MB of f32 states)."""
    from foscar_b200 import parallel
    n, b, hq, d = 8, 2048, 32, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    o = torch.randn(n, b, hq, d, device="cuda", generator=g)
    lse = torch.randn(n, b, hq, device="cuda", generator=g) * 4.0
    out = torch.empty(b, hq, d, dtype=torch.float32, device="cuda")
    parallel.merge_states(o, lse, out=out)
    torch.cuda.synchronize()
    rows = torch.tensor([0, 1, 777, 2047])
    want, _ = _want(o[:, rows], lse[:, rows])
    assert torch.allclose(out[rows].double().cpu(), want, rtol=2e-6, atol=2e-6)
