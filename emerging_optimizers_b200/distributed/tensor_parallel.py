"""Tensor-parallel Newton-Schulz support: the Gram all-reduce fused into the SYRK kernel, and the sharded
``S = b A + c A^2`` product whose epilogue is the all-gather.

In ``newton_schulz_tp(..., tp_mode="distributed")`` every rank holds a shard ``X_r`` along the contraction
dimension and each iteration needs ``A = sum_r X_r X_r^T`` on every rank.  The reference computes the partial
product and then calls ``all_reduce`` on the full m x m matrix (``muon_utils.py:370-372, 434-436`` there), and
computes ``S`` redundantly on every rank (``:374``).  Here

- one kernel per rank does SYRK and all-reduce (``eo_tp_gram_allreduce``): the epilogue leaves each bf16 partial
  tile in the rank's own symmetric buffer and raises a flag at the tile's owner; reducer warps of the same kernel
  sum the tiles they own with NVSwitch load-reduce instructions (fp32 accumulation, one rounding) and
  multicast-store the tile and its mirror image into every rank's Gram matrix.  Without multicast support the
  same warps read and write the peers one by one.
- for groups of four ranks or more each rank computes m / P rows of ``S`` and its epilogue multicast-stores them
  into every rank's buffer (``eo_gemm_multicast``): product and all-gather in one kernel.

One group barrier follows each of the two kernels.  Buffers live in symmetric memory (``PeerBuffer``) and are
cached per (process group, matrix size, device).

A wait for another rank that runs out (``eo_set_option("peer_wait_ms")``, default 10 s) fills the affected Gram
tiles with NaN on every rank and sets the device status word.  The status word is copied to pinned host memory
behind every exchange without synchronising; the next exchange (or :func:`check`) raises ``NativeLibraryError`` if
it is non-zero.  With ``STRICT = True`` every exchange synchronises and checks at once.
"""

from __future__ import annotations

import os
import weakref

import torch
import torch.distributed as dist

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer


__all__ = ["GramExchange", "fused_gram_available", "fused_gram", "sharded_gram_poly", "check", "clear", "STRICT"]

# Synchronise and check the device status after every exchange (costs the launch-ahead of the caller's stream).
STRICT = os.environ.get("EO_TP_STRICT", "0") == "1"

# The exchange delivers the lower triangle only and every rank mirrors its own copy (whole-row accesses in the
# reducers, half the NVLink bytes); False lets the reducers store the mirror image over NVLink themselves.
LOWER_ONLY = os.environ.get("EO_TP_LOWER_ONLY", "1") == "1"

# How the row blocks of S = b A + c A^2 reach the other ranks: "copy" (default): plain product into the local
# buffer, then one multicast copy kernel (512 contiguous bytes per warp); "epilogue": the product's epilogue
# stores through the multicast address itself (one kernel, but 16-byte multicast stores at a row stride).
POLY_GATHER = os.environ.get("EO_TP_POLY", "copy")

# process group -> {(m, device index): GramExchange}; entries die with their group
_EXCHANGES: "weakref.WeakKeyDictionary[dist.ProcessGroup, dict[tuple, GramExchange]]" = weakref.WeakKeyDictionary()


class GramExchange:
    """Partial tiles, flag words, Gram matrix and S matrix of one rank for m x m matrices over ``group`` (built
    collectively), or over raw pointers handed in by :meth:`from_raw`."""

    def __init__(self, m: int, group: "dist.ProcessGroup", device: torch.device):
        self.m, self.group, self.device = m, group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lib = _native.lib()
        self.ld = (m + 7) // 8 * 8
        self.partials = PeerBuffer(lib.eo_tp_gram_inbox_bytes(m, self.world) // 2, torch.bfloat16, device, group)
        self.flags = PeerBuffer(lib.eo_tp_gram_flag_count(m, self.world), torch.int32, device, group)
        self.gram = PeerBuffer(m * self.ld, torch.bfloat16, device, group)
        self.poly = PeerBuffer(m * self.ld, torch.bfloat16, device, group)  # S = b A + c A^2, gathered by multicast
        self.multicast = bool(self.partials.multicast_ptr and self.gram.multicast_ptr)
        self._setup_common(
            self.partials.ptrs, self.flags.ptrs, self.gram.ptrs,
            self.partials.multicast_ptr if self.multicast else 0, self.gram.multicast_ptr if self.multicast else 0,
            self.gram.local, self.gram.barrier,
        )  # fmt: skip
        self.flags.local.zero_()
        torch.cuda.synchronize(device)
        self.flags.barrier()  # nobody raises a flag before every rank has cleared its words

    def _setup_common(self, partial_ptrs, flag_ptrs, gram_ptrs, partials_mc, gram_mc, gram_local, barrier) -> None:
        self._partial_ptrs, self._flag_ptrs, self._gram_ptrs = list(partial_ptrs), list(flag_ptrs), list(gram_ptrs)
        self._partials_mc, self._gram_mc = int(partials_mc), int(gram_mc)
        self._gram_local, self._barrier = gram_local, barrier
        self.seq = 0
        self._host_status = torch.zeros(1, dtype=torch.int32).pin_memory()

    @classmethod
    def from_raw(cls, m: int, world: int, rank: int, device: torch.device, partial_ptrs, flag_ptrs, gram_ptrs,
                 gram_local: torch.Tensor, barrier=None) -> "GramExchange":  # fmt: skip
        """An exchange over buffers the caller has mapped itself (``world`` device pointers each; no multicast).
        ``barrier`` is called after every exchange (default: nothing, for a caller that synchronises itself)."""
        self = object.__new__(cls)
        self.m, self.group, self.device, self.world, self.rank = m, None, device, world, rank
        self.ld = (m + 7) // 8 * 8
        self.multicast = False
        self._setup_common(partial_ptrs, flag_ptrs, gram_ptrs, 0, 0, gram_local, barrier or (lambda: None))
        return self

    def raise_if_failed(self, synchronize: bool = False) -> None:
        """Raise if a kernel of this library on this device has reported a wait that ran out.  Without
        ``synchronize`` only what the last status copy has already delivered to the host is looked at."""
        if synchronize:
            code = _native.read_device_status(self.device)
        else:
            code = int(self._host_status[0])
            if code != 0:
                self._host_status[0] = 0
                _native.read_device_status(self.device)  # synchronises and clears the device word
        if code != 0:
            raise _native.NativeLibraryError(
                f"a kernel gave up waiting (device status {code:#x}"
                + (": a rank of the tensor-parallel group did not deliver its Gram tiles in time; the affected tiles "
                   "were filled with NaN" if code == 0x40 else "")
                + ")"
            )  # fmt: skip

    def allreduce_gram(self, x: torch.Tensor) -> torch.Tensor:
        """``sum over ranks of x @ x.mT`` for this rank's bf16 shard ``x`` (m x k_r, row- or column-major).

        Returns a view of this rank's Gram buffer (both triangles filled), valid until the next call.
        """
        self.raise_if_failed()
        self.seq += 1
        _native.set_option("tp_lower_only", 1 if LOWER_ONLY else 0)
        _native.tp_gram_allreduce(x, self.world, self.rank, self._partial_ptrs, self._flag_ptrs, self._gram_ptrs,
                                  self._partials_mc, self._gram_mc, self.ld, self.seq)  # fmt: skip
        # Orders every owner's stores before any rank reads its Gram matrix, and every owner's reads of the partial
        # tiles before the next exchange overwrites them.
        self._barrier()
        if LOWER_ONLY:
            _native.tp_gram_mirror(self._gram_local, self.m, self.ld)
        _native.peek_device_status_async(self._host_status, self.device)
        if STRICT:
            self.raise_if_failed(synchronize=True)
        return self._gram_local.view(self.m, self.ld)[:, : self.m]

    def sharded_poly(self, A: torch.Tensor, b: float, c: float) -> torch.Tensor | None:
        """``S = b A + c A A`` with this rank computing rows ``[rank m / P, (rank + 1) m / P)`` and its epilogue
        storing them into every rank's S buffer.  ``None`` if the shape or the box does not allow it."""
        m, world = self.m, self.world
        if self.group is None or not self.poly.multicast_ptr or m % (32 * world) != 0 or self.ld != m:
            return None
        rows = m // world
        r0 = self.rank * rows
        S = self.poly.local.view(m, m)
        if POLY_GATHER == "epilogue":
            _native.gemm_multicast(A[r0 : r0 + rows], A, A[r0 : r0 + rows], S[r0 : r0 + rows],
                                   self.poly.multicast_ptr + r0 * m * 2, alpha=c, beta=b)  # fmt: skip
        else:
            _native.gemm(A[r0 : r0 + rows], A, A[r0 : r0 + rows], S[r0 : r0 + rows], alpha=c, beta=b)
            _native.multicast_copy(S[r0 : r0 + rows], self.poly.multicast_ptr + r0 * m * 2)
        # every rank's rows have landed everywhere; also keeps the next iteration's stores behind this one's readers
        self.poly.barrier()
        return S


def fused_gram_available(x: torch.Tensor, group: "dist.ProcessGroup | None") -> bool:
    """Whether the fused exchange is used for this shard: 2-D bf16 CUDA, TMA-addressable sizes, 2..8 ranks.

    ``EO_TP_GRAM=nccl`` forces the plain path (SYRK kernel, then ``torch.distributed.all_reduce``).
    """
    if group is None or not x.is_cuda or x.dim() != 2 or x.dtype != torch.bfloat16:
        return False
    if os.environ.get("EO_TP_GRAM", "auto") == "nccl":
        return False
    world = dist.get_world_size(group)
    return 2 <= world <= 8 and x.size(0) % 8 == 0 and x.size(1) % 8 == 0


def _exchange(m: int, group: "dist.ProcessGroup", device: torch.device) -> GramExchange:
    per_group = _EXCHANGES.setdefault(group, {})
    key = (m, device.index)
    ex = per_group.get(key)
    if ex is None:
        ex = per_group[key] = GramExchange(m, group, device)
    return ex


def fused_gram(x: torch.Tensor, group: "dist.ProcessGroup") -> torch.Tensor:
    return _exchange(x.size(0), group, x.device).allreduce_gram(x)


def sharded_gram_poly(A: torch.Tensor, b: float, c: float, group: "dist.ProcessGroup") -> torch.Tensor | None:
    """``b A + c A A`` in row blocks, one per rank, gathered by multicast stores; ``None`` if not applicable."""
    if not A.is_cuda or A.dim() != 2 or A.dtype != torch.bfloat16 or not A.is_contiguous():
        return None
    return _exchange(A.size(0), group, A.device).sharded_poly(A, b, c)


def check(device: torch.device | None = None) -> None:
    """Synchronise ``device`` and raise ``NativeLibraryError`` if any kernel of the library gave up waiting."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    code = _native.read_device_status(dev)
    if code != 0:
        raise _native.NativeLibraryError(f"a kernel gave up waiting (device status {code:#x})")


def clear(group: "dist.ProcessGroup | None" = None) -> None:
    """Drop the cached exchanges (and with them their symmetric buffers) of ``group``, or of all groups."""
    if group is None:
        _EXCHANGES.clear()
    else:
        _EXCHANGES.pop(group, None)
