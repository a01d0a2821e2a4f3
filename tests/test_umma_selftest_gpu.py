"""The tensor-core building blocks of the decode kernel on known operands, through the C ABI:
S = C_K . Q^T with the K operand in tensor memory (mode 0) and in shared memory (mode 1), and
O^T = C_V^T . P with MN-major operands. Operand bytes are raw codes (E4M3 value code * 2^-9,
subnormal for codes < 8), so exactness here is what lets the kernel skip dequantization."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _e4m3_values():
    return torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("qmax", [3, 15])
def test_umma_tile_matches_integer_arithmetic(mode, qmax):
    from foscar_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(mode * 7 + qmax)
    table = _e4m3_values()
    k = rng.integers(0, qmax + 1, (128, 128), dtype=np.uint8)
    v = rng.integers(0, qmax + 1, (128, 128), dtype=np.uint8)
    q = torch.randn(16, 128, generator=torch.Generator().manual_seed(3)).to(
        torch.float8_e4m3fn).view(torch.uint8).numpy()
    p = (torch.rand(128, 16, generator=torch.Generator().manual_seed(4)) * 400).to(
        torch.float8_e4m3fn).view(torch.uint8).numpy()
    dev = "cuda"
    kd, qd, vd, pd = (torch.from_numpy(x.copy()).to(dev) for x in (k, q, v, p))
    s_out = torch.zeros(128, 16, device=dev)
    o_out = torch.zeros(128, 16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    code = lib.fq_umma_selftest(mode, kd.data_ptr(), qd.data_ptr(), vd.data_ptr(), pd.data_ptr(),
                                s_out.data_ptr(), o_out.data_ptr(), status.data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
    assert code == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    kf, vf, qf, pf = table[k], table[v], table[q], table[p]
    s_want = kf.astype(np.float64) @ qf.astype(np.float64).T          # [tok, head]
    o_want = vf.astype(np.float64).T @ pf.astype(np.float64)          # [ch, col]
    s_got, o_got = s_out.cpu().numpy(), o_out.cpu().numpy()
    assert np.abs(s_got - s_want).max() <= 1e-5 * np.abs(s_want).max() + 1e-7
    assert np.abs(o_got - o_want).max() <= 1e-5 * np.abs(o_want).max() + 1e-6
