"""The tensor-core operand conventions on the device: TMA swizzled tiles, thread-written swizzled tiles, K-major and
MN-major descriptors, tensor-memory load layout.  Small-integer e4m3 operands make every fp32 sum exact, so the check
is bit-exact."""
import pytest
import torch

from delta_matching_b200 import _lib

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


def _tile(seed):
    g = torch.Generator("cpu").manual_seed(seed)
    return torch.randint(-4, 5, (128, 128), generator=g).float()


@pytest.mark.parametrize("a_mn,b_mn,n_cols,via_st", [(0, 0, 128, 0), (0, 0, 64, 0), (0, 1, 128, 0), (1, 1, 128, 0), (1, 0, 128, 0),
                                                      (0, 0, 128, 1), (0, 1, 128, 1), (1, 1, 128, 1)])
def test_mma_operand_conventions(a_mn, b_mn, n_cols, via_st):
    a, b = _tile(1 + a_mn), _tile(7 + b_mn)
    A = a.t() if a_mn else a                    # logical [M, K]
    Bm = b.t() if b_mn else b                   # logical [N, K]
    ref = A @ Bm[:n_cols].t()
    c, echo = _lib.probe_mma(a.to(E4M3).cuda(), b.to(E4M3).cuda(), a_mn, b_mn, n_cols, via_st)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(c.cpu(), ref), f"max abs diff {(c.cpu() - ref).abs().max().item()}"
    if via_st:
        assert torch.equal(echo.cpu(), a.to(E4M3).view(torch.uint8))
