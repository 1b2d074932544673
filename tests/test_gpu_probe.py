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


@pytest.mark.parametrize("mode,b_mn,n_cols", [(2, 0, 128), (2, 1, 128), (2, 0, 64), (3, 1, 128), (4, 1, 128), (4, 0, 128)])
def test_a_operand_in_tensor_memory(mode, b_mn, n_cols):
    """A written into tensor memory by tcgen05.st (four e4m3 per 32-bit column, lane = row): contiguous K steps, K steps 32
    columns apart, and (mode 4) an accumulator written over the operand by the very next MMA, which must not disturb the
    product that reads it."""
    a, b = _tile(21), _tile(27 + b_mn)
    Bm = b.t() if b_mn else b
    ref = a @ Bm[:n_cols].t()
    c, _ = _lib.probe_mma(a.to(E4M3).cuda(), b.to(E4M3).cuda(), 0, b_mn, n_cols, mode)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(c[:128].cpu(), ref), f"max abs diff {(c[:128].cpu() - ref).abs().max().item()}"
    if mode == 4:
        assert torch.equal(c[128:].cpu(), ref)      # the second product has the same operands, read from shared memory


def test_a_wait_that_runs_out_is_reported_and_the_kernel_ends():
    """The bounded-wait path itself: a kernel whose barrier is never armed returns by itself, both of its waits come back
    unsatisfied (the second one early, through the CTA's abort flag), the status word says so once, and the context stays
    usable."""
    assert _lib.device_status() == 0
    flags = _lib.selftest_wait_timeout()
    assert _lib.device_status() == 1          # DM_DEV_TIMEOUT; reading clears the word
    assert flags.tolist() == [0, 0]
    assert _lib.device_status() == 0
    a, b = _tile(1), _tile(7)
    c, _ = _lib.probe_mma(a.to(E4M3).cuda(), b.to(E4M3).cuda(), 0, 0, 128, 0)
    assert torch.equal(c.cpu(), a @ b.t()) and _lib.device_status() == 0


def test_init_is_idempotent():
    _lib.init()
    _lib.init()
    assert _lib.device_status() == 0
