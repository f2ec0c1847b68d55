"""The allocation-free sum-of-squares entry point (``eo_sumsq_f32_noalloc``) against the regular one.

Some embedders of the library cannot obtain device scratch at the point where they need the Frobenius norm: code
running inside an allocator callback, a loop that has promised a fixed memory footprint, a host that only gets
raw device pointers from another runtime.  For them the partial sums live in an array built into the library.
This test calls that entry point through the C ABI twice in a row, on inputs of different sizes so that the second
call finds the first call's leftovers in the shared array, and requires the same bits as ``eo_sumsq_f32``
(both run the same kernels in the same order; the tolerance used elsewhere for this quantity, rtol 1e-12, is
therefore met with equality).  The file name sorts after every other test file, so these cases are collected
and run last.
"""


import pytest
import torch

from emerging_optimizers_b200 import _native as nat


pytestmark = pytest.mark.gpu


def _randn(*shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).cuda()


def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row():
    big = _randn(1024, 4096, seed=1)          # 128 partial sums
    small = _randn(3, 100, 36, seed=2) * 1e-3  # 3 matrices, 1 partial sum each: reuses slots the first call filled
    out_big = torch.full((1,), float("nan"), dtype=torch.float64, device="cuda")
    out_small = torch.full((3,), float("nan"), dtype=torch.float64, device="cuda")
    want_big, want_small = nat.sumsq(big), nat.sumsq(small)
    torch.cuda.synchronize()

    before = torch.cuda.memory_allocated()
    nat.sumsq_noalloc(big, out_big)
    nat.sumsq_noalloc(small, out_small)
    assert torch.cuda.memory_allocated() == before  # nothing went through torch's allocator
    torch.cuda.synchronize()

    assert torch.equal(out_big, want_big)
    assert torch.equal(out_small, want_small)
    ref = (small.double() ** 2).sum(dim=(-2, -1))
    assert torch.allclose(out_small, ref, rtol=1e-12, atol=0)
    # transposed view: same storage walked in its physical order, same bits
    out_t = torch.empty(1, dtype=torch.float64, device="cuda")
    nat.sumsq_noalloc(big.T, out_t)
    assert torch.equal(out_t, want_big)
    assert nat.read_device_status() == 0


def test_noalloc_rejects_requests_beyond_its_capacity():
    lib = nat.lib()
    cap = lib.eo_sumsq_noalloc_max_partials()
    assert cap == 65536
    # batch * blocks_per_matrix > capacity: refused before any launch, with a message that names the way out
    x = torch.zeros(8, device="cuda")
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    rc = lib.eo_sumsq_f32_noalloc(x.data_ptr(), 65, 8192, 8192, 8192, 8192 * 8192, out.data_ptr(), None)
    assert rc == 4  # EO_ERR_WORKSPACE
    msg = lib.eo_last_error().decode()
    assert "built-in scratch" in msg and "eo_sumsq_f32" in msg
    with pytest.raises(nat.NativeLibraryError, match="EO_ERR_WORKSPACE"):
        big_batch = torch.zeros(cap + 1, 1, 1, device="cuda")
        nat.sumsq_noalloc(big_batch, torch.zeros(cap + 1, dtype=torch.float64, device="cuda"))
    torch.cuda.synchronize()
    assert nat.read_device_status() == 0
