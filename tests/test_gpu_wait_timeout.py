"""Bounded waits: a kernel whose peer never shows up gives up, records a status code, poisons what it could not
compute and returns; the Python-level exchange then raises.

No GPU is hung or faulted here: the tensor-parallel Gram exchange is run for a two-rank group of which only rank 0
exists (rank 1's buffers are ordinary local allocations that nobody writes), so the flag words rank 1 would raise
never reach the awaited sequence number.  The reducer warps' wait runs out after its budget (set to 0.3 s here),
they set the device status word, fill the tiles they own with NaN and the kernel exits; the host sees the status at
its next call, and the context stays usable.
"""

import pytest
import torch

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200 import triton_kernels as tk
from emerging_optimizers_b200.distributed.tensor_parallel import GramExchange


pytestmark = pytest.mark.gpu

STATUS_TIMEOUT_PEER = 0x40


def test_missing_peer_ends_in_status_code_poisoned_tiles_and_a_python_exception():
    lib = nat.lib()
    n, k, world = 256, 64, 2
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.randint(-1, 2, (n, k), device="cuda").to(torch.bfloat16)
    part_elems = lib.eo_tp_gram_inbox_bytes(n, world) // 2
    nflags = lib.eo_tp_gram_flag_count(n, world)
    partials = [torch.zeros(part_elems, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(nflags, dtype=torch.int32, device="cuda") for _ in range(world)]
    gram = [torch.zeros(n, n, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    assert nat.read_device_status() == 0
    nat.set_option("peer_wait_ms", 300)
    try:
        ex = GramExchange.from_raw(n, world, 0, dev, [t.data_ptr() for t in partials], [t.data_ptr() for t in flags],
                                   [t.data_ptr() for t in gram], gram[0])  # fmt: skip
        a = ex.allreduce_gram(x)  # the launch itself succeeds; the failure is reported by the device
        torch.cuda.synchronize()
    finally:
        nat.set_option("peer_wait_ms", 10000)
    # rank 0 raised its own flags (for the tiles it owns in its own words, for rank 1's tiles in rank 1's words) ...
    slots = nflags // world
    assert int((flags[0][:slots] == 1).sum()) + int((flags[1][:slots] == 1).sum()) > 0
    # ... rank 1 never did: the tiles rank 0 owns are NaN on both "ranks", nothing else was written
    assert bool(torch.isnan(a.float()).any())
    assert bool(torch.isnan(gram[1].float()).any())
    # the exchange object has seen the status word: the next call (and an explicit check) raises, once
    with pytest.raises(nat.NativeLibraryError, match="did not deliver"):
        ex.allreduce_gram(x)
    assert nat.read_device_status() == 0  # raising cleared the word
    ex.raise_if_failed()

    # the context is still healthy: an ordinary kernel of the library runs and is correct
    m = torch.randint(-2, 3, (256, 128), device="cuda").to(torch.bfloat16)
    assert torch.equal(tk.tsyrk_ex(m), (m.float() @ m.float().T).bfloat16())
    assert nat.read_device_status() == 0


def test_raw_status_word_round_trip():
    """eo_read_device_status / eo_peek_device_status_async on a healthy device: zero, and stays zero."""
    pinned = torch.full((1,), 7, dtype=torch.int32).pin_memory()
    dev = torch.device("cuda", torch.cuda.current_device())
    nat.peek_device_status_async(pinned, dev)
    torch.cuda.synchronize()
    assert int(pinned[0]) == 0
    assert nat.read_device_status() == 0
