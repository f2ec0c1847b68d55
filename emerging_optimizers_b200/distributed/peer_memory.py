"""Peer-visible device buffers inside one NVSwitch box and collectives built on them.

``torch.distributed._symmetric_memory`` allocates a buffer on every rank of a group and maps all of them into
every rank's address space (CUDA virtual-memory handles exchanged over the process group), so a rank can write a
peer's buffer with an ordinary device-to-device copy or an ordinary store from a kernel.  Two uses here:

- :meth:`PeerBuffer.all_gather_slots`: an all-gather made of copy-engine transfers (one ``cudaMemcpyAsync`` per
  peer, on its own stream) followed by a group barrier.  It occupies no SM, so it does not take SMs away from the
  persistent tensor-core kernels it overlaps with, which a kernel-based collective does.
- the raw peer pointers (:attr:`PeerBuffer.ptrs`) and the NVSwitch multicast address
  (:attr:`PeerBuffer.multicast_ptr`, 0 if the box has no multicast support or ``EO_MULTICAST=0``) handed to kernels
  that load from / store to peers directly.

Only plain copies, plain loads/stores, ``multimem`` load-reduce / stores and the library's own barrier touch peer
memory; no TMA load with cluster multicast ever reads it.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist


__all__ = ["PeerBuffer", "MULTICAST_PUSH"]

# all_gather_slots pushes a slot with one multicast-store kernel instead of P - 1 copy-engine transfers.
MULTICAST_PUSH = os.environ.get("EO_MULTICAST_PUSH", "0") == "1"


class PeerBuffer:
    """A symmetric buffer of ``numel`` elements of ``dtype`` on every rank of ``group``.

    Must be constructed collectively (every rank, same arguments, same order).
    """

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group: "dist.ProcessGroup | None" = None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.numel, self.dtype, self.device = numel, dtype, device
        self.local = symm.empty(numel, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.local, self.group)
        # Addresses of element 0 on every rank, and through the multicast (NVLS) mapping if the box has one.  The
        # handle describes the allocation the tensor lives in; the tensor's offset inside it is the same on all
        # ranks and is taken from this rank's own pair of addresses.
        base = [int(p) for p in self.handle.buffer_ptrs]
        delta = self.local.data_ptr() - base[self.rank]
        self.ptrs = [p + delta for p in base]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc + delta if mc and os.environ.get("EO_MULTICAST", "1") != "0" else 0
        self._copy_streams = [torch.cuda.Stream(device=device) for _ in range(max(self.world - 1, 1))]

    def peer_view(self, peer: int, numel: int, offset: int = 0) -> torch.Tensor:
        """``numel`` elements of rank ``peer``'s buffer starting at element ``offset``, as a local tensor."""
        if peer == self.rank:
            return self.local[offset : offset + numel]
        return self.handle.get_buffer(peer, (numel,), self.dtype, offset)

    def barrier(self) -> None:
        """Group barrier enqueued on the current stream (every rank's stream passes it together)."""
        self.handle.barrier(channel=0)

    def all_gather_slots(self, base: int, slot_numel: int, barrier: bool = True) -> None:
        """All-gather in place: region ``base + r * slot_numel`` holds rank r's slot on every rank afterwards.

        The caller has filled its own slot of its own buffer.  Enqueued on the current stream: the slot is pushed
        to every peer by copy engines (parallel streams), then the group barrier orders the arrival of all pushes
        before anything enqueued after this call.  With ``barrier=False`` only the pushes are enqueued (a caller that
        gathers several disjoint regions needs one barrier behind the last of them, not one each).
        """
        cur = torch.cuda.current_stream(self.device)
        mine = base + self.rank * slot_numel
        src = self.local[mine : mine + slot_numel]
        if MULTICAST_PUSH and self.multicast_ptr and (slot_numel * src.element_size()) % 16 == 0:
            # One kernel reads the slot once and stores it through the NVSwitch multicast address: 1 / (P - 1) of
            # the local HBM reads and NVLink egress of P - 1 point-to-point copies (the switch replicates).
            from emerging_optimizers_b200 import _native

            _native.multicast_copy(src, self.multicast_ptr + mine * src.element_size())
            if barrier:
                self.barrier()
            return
        ready = torch.cuda.Event()
        ready.record(cur)
        for k in range(1, self.world):
            peer = (self.rank + k) % self.world
            s = self._copy_streams[k - 1]
            with torch.cuda.stream(s):
                s.wait_event(ready)
                self.peer_view(peer, slot_numel, mine).copy_(src, non_blocking=True)
            cur.wait_stream(s)
        if barrier:
            self.barrier()
