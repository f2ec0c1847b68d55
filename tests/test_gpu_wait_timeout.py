"""Bounded waits: a kernel whose peer never shows up gives up, records a status code and returns.

No GPU is hung or faulted here: the owner-side reduce kernel of the tensor-parallel Gram exchange is run for a
two-rank group of which only rank 0 exists (rank 1's buffers are ordinary local allocations that nobody writes), so
the flag words of rank 1 never reach the awaited sequence number.  The kernel's wait runs out after its cycle budget
(about a second), it sets the device status word and exits; the host reads and clears the word, and the context
stays usable.
"""

import ctypes

import pytest
import torch

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200 import triton_kernels as tk


pytestmark = pytest.mark.gpu

STATUS_TIMEOUT_PEER = 0x40


def test_missing_peer_flag_ends_in_status_code_not_in_a_hang():
    lib = nat.lib()
    n, k, world = 256, 64, 2
    x = torch.randint(-1, 2, (n, k), device="cuda").to(torch.bfloat16)
    inbox_elems = lib.eo_tp_gram_inbox_bytes(n, world) // 2
    nflags = lib.eo_tp_gram_flag_count(n, world)
    inbox = [torch.zeros(inbox_elems, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(nflags, dtype=torch.int32, device="cuda") for _ in range(world)]
    gram = [torch.zeros(n, n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    assert nat.read_device_status() == 0

    def ptrs(ts):
        arr = (ctypes.c_void_p * world)()
        for i, t in enumerate(ts):
            arr[i] = t.data_ptr()
        return arr

    rc = lib.eo_tp_gram_allreduce(
        x.data_ptr(), 0, k, n, k, world, 0, ptrs(inbox), ptrs(flags), ptrs(gram), n, 1,
        torch.cuda.current_stream().cuda_stream,
    )  # fmt: skip
    assert rc == 0  # the launch itself succeeds; the failure is reported by the device
    torch.cuda.synchronize()
    # rank 0's own partials and flags arrived ...
    assert int((flags[0][: nflags // world] == 1).sum()) + int((flags[1][: nflags // world] == 1).sum()) > 0
    # ... rank 1's never did: the reduce kernel gave up and said so
    assert nat.read_device_status() == STATUS_TIMEOUT_PEER
    assert nat.read_device_status() == 0  # reading clears the word

    # the context is still healthy: an ordinary kernel of the library runs and is correct
    a = torch.randint(-2, 3, (256, 128), device="cuda").to(torch.bfloat16)
    assert torch.equal(tk.tsyrk_ex(a), (a.float() @ a.float().T).bfloat16())
    assert nat.read_device_status() == 0
