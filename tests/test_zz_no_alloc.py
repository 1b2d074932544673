"""The allocation-free K-mean entry point (dm_kmean_noalloc) against the ordinary one.

Some users of this library cannot allocate device memory when they call it: their process has given the whole of HBM to
its own arena, or sits in a loop that cannot afford cudaMalloc's device-wide synchronisation.  For them the K mean has a
variant whose partial sums live in a fixed 4 MiB array inside the library.  This file checks, through the C ABI, that the
variant gives the ordinary entry point's result bit for bit (the tolerance every quantizer test here uses) on two calls
in a row that reuse the shared array with different shapes, and that a shape beyond the array is refused.  It sorts last
so a run that stops at the first failure has already run every other test."""
import pytest
import torch

from delta_matching_b200 import _lib

pytestmark = pytest.mark.gpu


def test_noalloc_kmean_matches_the_ordinary_entry_point_twice_in_a_row():
    g = torch.Generator("cpu").manual_seed(31)
    shapes = [(2, 1024, 4, 128), (1, 512, 2, 256)]          # (B, N, Hk, D); the second call reuses the array with another shape
    inputs = [(torch.randn(B, N, Hk, D, generator=g) + 0.5).to(torch.bfloat16).cuda() for (B, N, Hk, D) in shapes]
    outs = [torch.full((B * Hk, D), float("nan"), device="cuda") for (B, N, Hk, D) in shapes]
    _lib.kmean_noalloc(inputs[0], outs[0])                   # first call on the device: module load and the array's address lookup
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    steady = False
    for _ in range(3):                                       # (the driver's count is device-wide: give an unrelated change a second look)
        free_before = torch.cuda.mem_get_info()[0]           # free bytes as the driver counts them: sees a raw cudaMalloc too
        for k, out in zip(inputs, outs):                     # back to back on one stream
            _lib.kmean_noalloc(k, out)
        torch.cuda.synchronize()
        steady = steady or torch.cuda.mem_get_info()[0] >= free_before
    assert torch.cuda.memory_allocated() == before           # the wrapper itself allocated nothing
    assert steady                                            # and neither did the library
    for k, out in zip(inputs, outs):
        assert torch.equal(out, _lib.kmean(k))
    # again, same shapes, after the array has held other data
    for k, out in zip(inputs, outs):
        out.fill_(float("nan"))
        _lib.kmean_noalloc(k, out)
        assert torch.equal(out, _lib.kmean(k))


def test_noalloc_kmean_refuses_shapes_beyond_its_array():
    limit = _lib.lib().dm_kmean_noalloc_max_bytes()
    assert limit == 4 * 2 ** 20
    B, N, Hk, D = 2, 65536, 8, 128                           # 8 MiB of partial sums
    assert _lib.lib().dm_kmean_scratch_bytes(B, Hk, N, D) > limit
    k = torch.empty(1, 1, 1, D, dtype=torch.bfloat16, device="cuda").expand(B, N, Hk, D)     # never read: refused first
    out = torch.empty(B * Hk, D, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        _lib.kmean_noalloc(k, out)
