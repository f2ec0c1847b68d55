"""Tensor-parallel Newton-Schulz support: the Gram all-reduce fused into the SYRK epilogue.

In ``newton_schulz_tp(..., tp_mode="distributed")`` every rank holds a shard ``X_r`` along the contraction
dimension and each iteration needs ``A = sum_r X_r X_r^T`` on every rank.  The reference computes the partial
product and then calls ``all_reduce`` on the full m x m matrix (``muon_utils.py:370-372, 434-436`` there).  Here the
SYRK kernel's epilogue stores each finished partial tile directly into the memory of the tile's owner rank, the
owners sum their tiles and store the lower-triangle results into every rank's Gram matrix, one group barrier
closes the exchange and every rank mirrors its own copy: only lower-triangle data travels, in bf16, overlapped
with the SYRK main loop.

Buffers live in symmetric memory (``PeerBuffer``) and are cached per (process group, matrix size, device).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer


__all__ = ["GramExchange", "fused_gram_available", "fused_gram"]

_EXCHANGES: dict[tuple, "GramExchange"] = {}


class GramExchange:
    """Inbox, flag words and Gram matrix of one rank for m x m Gram matrices over ``group`` (built collectively)."""

    def __init__(self, m: int, group: "dist.ProcessGroup", device: torch.device):
        self.m, self.group, self.device = m, group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lib = _native.lib()
        self.ld = (m + 7) // 8 * 8
        self.inbox = PeerBuffer(lib.eo_tp_gram_inbox_bytes(m, self.world) // 2, torch.bfloat16, device, group)
        self.flags = PeerBuffer(lib.eo_tp_gram_flag_count(m, self.world), torch.int32, device, group)
        self.gram = PeerBuffer(m * self.ld, torch.bfloat16, device, group)
        self.flags.local.zero_()
        self.seq = 0
        torch.cuda.synchronize(device)
        self.flags.barrier()  # nobody publishes a flag before every rank has cleared its words

    def allreduce_gram(self, x: torch.Tensor) -> torch.Tensor:
        """``sum over ranks of x @ x.mT`` for this rank's bf16 shard ``x`` (m x k_r, row- or column-major).

        Returns a view of this rank's Gram buffer, valid until the next call.
        """
        self.seq += 1
        _native.tp_gram_allreduce(x, self.world, self.rank, self.inbox.ptrs, self.flags.ptrs, self.gram.ptrs,
                                  self.ld, self.seq)  # fmt: skip
        # Orders every owner's stores before any rank reads its Gram matrix, and this exchange before the next.
        self.gram.barrier()
        # The owners sent lower triangles only; complete the local copy.
        _native.tp_gram_mirror(self.gram.local, self.m, self.ld)
        return self.gram.local.view(self.m, self.ld)[:, : self.m]


# Largest group for which the fused exchange is chosen by default.  Measured on 8192 x 28672 (five steps, B200,
# NVSwitch): fused 15.7 / 10.6 / 8.4 ms on 2 / 4 / 8 ranks against 15.5 / 10.0 / 7.6 ms with NCCL's all-reduce: on
# par for a pair of GPUs, while on larger groups the owners' point-to-point broadcast of the reduced tiles loses to
# the in-switch reduction NCCL uses.
FUSED_MAX_WORLD = 2


def fused_gram_available(x: torch.Tensor, group: "dist.ProcessGroup | None") -> bool:
    """Whether the fused exchange is used for this shard: 2-D bf16 CUDA, TMA-addressable sizes, 2..8 ranks.

    ``EO_TP_GRAM=fused`` / ``EO_TP_GRAM=nccl`` force one or the other; by default (``auto``) groups of up to
    ``FUSED_MAX_WORLD`` ranks take the fused exchange and larger ones NCCL.
    """
    if group is None or not x.is_cuda or x.dim() != 2 or x.dtype != torch.bfloat16:
        return False
    mode = os.environ.get("EO_TP_GRAM", "auto")
    if mode == "nccl":
        return False
    world = dist.get_world_size(group)
    if not (2 <= world <= 8 and x.size(0) % 8 == 0 and x.size(1) % 8 == 0):
        return False
    return mode == "fused" or world <= FUSED_MAX_WORLD


def fused_gram(x: torch.Tensor, group: "dist.ProcessGroup") -> torch.Tensor:
    key = (id(group), x.size(0), x.device.index)
    ex = _EXCHANGES.get(key)
    if ex is None:
        ex = _EXCHANGES[key] = GramExchange(x.size(0), group, x.device)
    return ex.allreduce_gram(x)
