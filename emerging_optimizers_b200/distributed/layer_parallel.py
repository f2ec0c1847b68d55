"""Layer-parallel Muon: each rank orthogonalizes 1/P of the parameter matrices, then the ranks all-gather the
orthogonalized updates and every rank applies all of them.

The reference only describes this scheme in prose (``docs/primer/layerwise-distributed-optimizer.md:24-33, 39-87``
there) and points at an external implementation; the single-process ``Muon.step`` over *all* matrices is its
specification: after :meth:`LayerParallelMuon.step` every rank holds exactly the parameters that a single process
would hold.

Design for one NVSwitch box (one process per GPU, NCCL through ``torch.distributed``):

- Matrices are independent units.  They are assigned to ranks by longest-processing-time-first on the cost
  ``m (m + 1) n + m^2 (m + 1) + 2 m^2 n`` (tensor-core FLOPs of one iteration, m <= n).  Gradients are assumed to
  be identical on all ranks already (the data-parallel reduction happens upstream of the optimizer).
- The owner keeps the momentum buffer of a matrix (1/P of the optimizer state per rank), updates it, applies
  Nesterov and runs Newton-Schulz.  On the bf16 path the Newton-Schulz result is bf16-valued, so it is exchanged
  as bf16 without loss: 2 bytes per parameter cross NVLink instead of 4.
- The exchange is one all-gather per bucket of matrices, issued on a side stream as soon as the bucket's matrices
  are done, so it overlaps the Newton-Schulz work of the next bucket.  On GPUs it is made of copy-engine pushes
  into the peers' symmetric buffers plus a group barrier (no SM is taken from the persistent tensor-core
  kernels); host ranks (gloo, used by the tests) call ``all_gather_into_tensor``.
- Weight decay and ``p -= lr * scale * update`` are then applied by every rank to every matrix with the same fp32
  arithmetic, which makes the parameters bitwise identical across ranks and equal to the single-process result.
- ``exchange="parameters"`` is the alternative in which only the owner applies the update and the *updated
  parameters* travel (4 bytes per parameter instead of 2, but the update kernel touches 1/P of the parameters
  instead of all of them, and that kernel is the part of the step that does not shrink with P).  On GPUs the
  parameters are moved, once, into a symmetric buffer laid out like the exchange slots, so the owners' copy-engine
  pushes land directly in the peers' parameter storage and the receiving side does no work at all.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Sequence

import torch
import torch.distributed as dist
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import _native, mixin, utils
from emerging_optimizers_b200.orthogonalized_optimizers import _fused_step, muon_utils
from emerging_optimizers_b200.orthogonalized_optimizers.muon import _NS_FUNCTIONS, _SHRINK, get_muon_scale_factor


__all__ = ["ns_cost", "partition_by_cost", "LayerParallelMuon"]

# exchange="parameters": close every bucket's pushes with a group barrier of its own (only for comparison runs).
PER_BUCKET_BARRIER = False


def ns_cost(shape: Sequence[int]) -> float:
    """Tensor-core FLOPs of one Newton-Schulz iteration on a matrix of this shape (symmetric outputs once)."""
    m, n = sorted((int(shape[-2]), int(shape[-1])))
    batch = 1
    for s in shape[:-2]:
        batch *= int(s)
    return batch * (m * (m + 1.0) * n + m * m * (m + 1.0) + 2.0 * m * m * n)


def partition_by_cost(costs: Sequence[float], world: int) -> list[int]:
    """Owner rank of every item: largest cost first onto the least loaded rank (ties: lower index, lower rank).

    Deterministic, so every rank computes the same assignment without communication.
    """
    if world < 1:
        raise ValueError(f"world must be at least 1, got {world}")
    owners = [0] * len(costs)
    load = [0.0] * world
    for i in sorted(range(len(costs)), key=lambda j: (-costs[j], j)):
        r = min(range(world), key=lambda q: (load[q], q))
        owners[i] = r
        load[r] += costs[i]
    return owners


@dataclass
class _Bucket:
    """One exchange: for every rank the (parameter index, offset in the rank's slot) pairs it contributes."""

    per_rank: list[list[tuple[int, int]]] = field(default_factory=list)
    slot_numel: int = 0


def _plan_buckets(
    numels: Sequence[int], owners: Sequence[int], world: int, bucket_numel: int, shapes: Sequence[tuple] | None = None
) -> list[_Bucket]:
    """Cut every rank's owned list into groups; group j of all ranks forms bucket j.

    A group is closed once it holds ``bucket_numel`` elements.  With ``shapes`` a rank's list is first ordered by
    shape, largest matrices first, and a group is also closed where the shape changes: every group is then a stack
    of equally shaped matrices, i.e. one batched Newton-Schulz run, and the last buckets (whose exchange nothing
    is left to hide behind) hold the smallest matrices.  Without ``shapes`` the list stays in index order.  The slot
    size of a bucket is the largest group in it (rounded up to 8 elements), so the all-gather has equal-sized slots.
    """
    owned: list[list[int]] = [[] for _ in range(world)]
    for i, r in enumerate(owners):
        owned[r].append(i)
    if shapes is not None:
        for r in range(world):
            owned[r].sort(key=lambda i: (-numels[i], tuple(shapes[i]), i))
    groups: list[list[list[tuple[int, int]]]] = []
    for r in range(world):
        mine: list[list[tuple[int, int]]] = [[]]
        fill = 0
        for i in owned[r]:
            new_shape = shapes is not None and mine[-1] and tuple(shapes[mine[-1][-1][0]]) != tuple(shapes[i])
            if (fill >= bucket_numel or new_shape) and mine[-1]:
                mine.append([])
                fill = 0
            mine[-1].append((i, fill))
            fill += (numels[i] + 7) // 8 * 8
        groups.append(mine if mine[-1] or len(mine) > 1 else [[]])
    n_buckets = max(len(g) for g in groups)
    buckets = []
    for j in range(n_buckets):
        b = _Bucket(per_rank=[g[j] if j < len(g) else [] for g in groups])
        for r in range(world):
            for i, off in b.per_rank[r]:
                b.slot_numel = max(b.slot_numel, off + (numels[i] + 7) // 8 * 8)
        buckets.append(b)
    return buckets


class LayerParallelMuon(mixin.WeightDecayMixin, torch.optim.Optimizer):
    """Muon over 2-D parameters with the Newton-Schulz work divided among the ranks of ``group``.

    A ``torch.optim.Optimizer``: ``params`` may be an iterable of parameters or of parameter-group dicts, the
    per-group ``lr``, ``momentum`` and ``weight_decay`` are honoured (so learning-rate schedulers work),
    ``zero_grad`` and ``add_param_group``-free use behave as usual, and the per-parameter state key is
    ``"momentum_buffer"`` as in ``orthogonalized_optimizer.py:136-154`` of the reference; a rank holds state only
    for the matrices it owns.  The remaining hyper-parameters have the meaning they have for
    :class:`~emerging_optimizers_b200.orthogonalized_optimizers.Muon`.  ``step()`` must be called by all ranks of the
    group, with identical gradients on all of them.

    Args:
        params: the 2-D parameters (or parameter groups), in the same order on every rank.
        group: process group to divide the work over (``None``: the default group; a single process if
            torch.distributed is not initialised).
        bucket_numel: elements per rank and exchange; smaller buckets start communicating earlier, larger ones
            give the batched Newton-Schulz runs more matrices per launch.  A bucket holds matrices of one shape.
            The default (32 Mi elements) was the fastest of 16 / 32 / 64 / 256 Mi on the Llama-3-8B-shaped step on
            eight GPUs (73.6 / 65.1 / 67.6 / 81.5 ms).
        exchange_dtype: dtype of the gathered updates.  ``None`` picks bf16 on the "medium" path (lossless there)
            and fp32 otherwise.
        exchange: "updates": all-gather the orthogonalized updates, every rank applies all of them.
            "parameters": the owner alone applies its updates and the updated fp32 parameters are all-gathered.  On
            GPUs the first step then moves every ``p.data`` into a symmetric buffer owned by this object (a
            collective call; tensors that alias the old storage are not updated any more), and from then on peers
            write the new values straight into that storage.
            "mixed": per bucket one or the other.  Parameters cost 4 bytes per element of NVLink ingress and nothing
            else on the receivers; updates cost 2 bytes per element and an HBM-bound weight update on every rank.
            Both run behind the Newton-Schulz work of the following buckets.  On eight B200s a half-and-half
            mixture measured no better than the better of the two (the step runs at the power cap, where moved
            bytes cost time wherever they overlap); kept for systems with other ratios of link to HBM speed.
            "auto": "parameters" for groups of up to four ranks, "updates" beyond.  A rank receives
            4 (W - 1) / W bytes per element under "parameters" while its share of the Newton-Schulz work shrinks
            with 1 / W; on eight B200s the 24 GB of pushes per step take 33 - 54 ms alone (box dependent) against
            53 - 55 ms of compute and end up on the critical path (70 ms per step), while half the bytes hide and
            the additional weight updates cost less (65 ms).  At four ranks the pushes hide completely (96 %).
        updates_fraction: with ``exchange="mixed"``, the fraction of the elements (in whole buckets, spread evenly
            over the step) that travel as updates.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 3e-4,
        momentum: float = 0.95,
        weight_decay: float = 0.01,
        *,
        nesterov: bool = False,
        weight_decay_method: mixin.WeightDecayT = "decoupled",
        fp32_matmul_prec: utils.FP32MatmulPrecT = "medium",
        coefficient_type: muon_utils.NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        scale_mode: str = "spectral",
        extra_scale_factor: float = 1.0,
        use_syrk: bool = False,
        group: "dist.ProcessGroup | None" = None,
        bucket_numel: int = 32 * 1024 * 1024,
        exchange_dtype: torch.dtype | None = None,
        exchange: str = "updates",
        updates_fraction: float = 0.5,
    ) -> None:
        if num_ns_steps < 1:
            raise ValueError(f"num_ns_steps must be at least 1, got {num_ns_steps}")
        if exchange not in ("updates", "parameters", "mixed", "auto"):
            raise ValueError(f"exchange must be 'updates', 'parameters', 'mixed' or 'auto', got {exchange!r}")
        if not 0.0 <= updates_fraction <= 1.0:
            raise ValueError(f"updates_fraction must lie in [0, 1], got {updates_fraction}")
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay))
        self.exchange = exchange  # "auto" is resolved below, once the group size is known
        # Flat view of the parameter groups: index i everywhere below is the position in this list, which is also
        # the index torch's state_dict() packs the parameter under.
        self.params = [p for g in self.param_groups for p in g["params"]]
        self._group_of = [g for g in self.param_groups for _ in g["params"]]
        for p in self.params:
            if p.ndim != 2:
                raise ValueError("Only 2D parameters are supported.")
        self.nesterov, self.weight_decay_method = nesterov, weight_decay_method
        self.fp32_matmul_prec = fp32_matmul_prec
        self.coefficient_type, self.num_ns_steps = coefficient_type, num_ns_steps
        self.scale_mode, self.extra_scale_factor, self.use_syrk = scale_mode, extra_scale_factor, use_syrk
        self.group = group
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        if exchange == "auto":
            self.exchange = "parameters" if self.world <= 4 else "updates"
        self.exchange_dtype = exchange_dtype or (torch.bfloat16 if fp32_matmul_prec == "medium" else torch.float32)

        self.owners = partition_by_cost([ns_cost(p.shape) for p in self.params], self.world)
        self.buckets = _plan_buckets([p.numel() for p in self.params], self.owners, self.world, bucket_numel,
                                     [tuple(p.shape) for p in self.params])  # fmt: skip
        # exchange="mixed": which buckets travel as updates (error diffusion over the element counts, so that the two
        # kinds alternate through the step in the requested proportion).
        self._as_updates = [False] * len(self.buckets)
        if self.exchange == "mixed":
            owed = 0.0
            for j, b in enumerate(self.buckets):
                owed += updates_fraction * b.slot_numel
                if owed >= 0.5 * b.slot_numel:
                    self._as_updates[j] = True
                    owed -= b.slot_numel
        self._ns_streams: list = []  # two streams the buckets' Newton-Schulz work alternates between (GPU ranks)
        self._side: "torch.cuda.Stream | None" = None
        self._peer = None  # symmetric exchange buffer, created collectively at the first multi-GPU step
        self._param_peer = None  # exchange="parameters": the symmetric buffer the parameters live in
        self._exchanges = 0

    # -- pieces of the step ------------------------------------------------------------------------------
    def owned_indices(self) -> list[int]:
        return [i for i, r in enumerate(self.owners) if r == self.rank]

    def _hyper(self, i: int) -> tuple[float, float, float]:
        """(lr, momentum, weight_decay) of parameter ``i``, read from its parameter group at call time."""
        g = self._group_of[i]
        return g["lr"], g["momentum"], g["weight_decay"]

    def _shrink(self, i: int) -> float:
        lr, _, wd = self._hyper(i)
        return _SHRINK[self.weight_decay_method](lr, wd) if wd != 0.0 else 0.0

    def _momentum_buffer(self, i: int) -> torch.Tensor:
        st = self.state[self.params[i]]
        if "momentum_buffer" not in st:
            st["momentum_buffer"] = torch.zeros_like(self.params[i].data)
        return st["momentum_buffer"]

    def _by_group(self, idxs: Sequence[int]) -> list[list[int]]:
        """``idxs`` split into runs that share a parameter group (one fused call each), order preserved."""
        runs: dict[int, list[int]] = {}
        for i in idxs:
            runs.setdefault(id(self._group_of[i]), []).append(i)
        return list(runs.values())

    def _fork_compute_streams(self, dev: torch.device) -> list:
        """Two streams, made to wait for everything enqueued on the current stream so far.  The Newton-Schulz work
        of consecutive buckets alternates between them: each product is a persistent launch whose last wave leaves
        SMs idle, and with an independent chain of launches in flight those SMs pick up the other bucket's tiles."""
        if dev.type != "cuda":
            return []
        if not self._ns_streams:
            self._ns_streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
        fork = torch.cuda.Event()
        fork.record(torch.cuda.current_stream(dev))
        for s in self._ns_streams:
            s.wait_event(fork)
        return self._ns_streams

    def _join_compute_streams(self, dev: torch.device) -> None:
        cur = torch.cuda.current_stream(dev)
        for s in self._ns_streams:
            cur.wait_stream(s)

    def _orthogonalize_owned(self, i: int) -> torch.Tensor:
        """Momentum update, Nesterov and Newton-Schulz for parameter ``i`` (owned by this rank); unscaled."""
        p = self.params[i]
        _, momentum, wd = self._hyper(i)
        grad = p.grad
        if self.weight_decay_method == "l2" and wd != 0.0:
            grad = grad.add(p, alpha=wd)
        buf = self._momentum_buffer(i)
        buf.lerp_(grad, 1 - momentum)
        update = grad.lerp(buf, momentum) if self.nesterov else buf
        with utils.fp32_matmul_precision(self.fp32_matmul_prec):
            return muon_utils.newton_schulz(
                update, steps=self.num_ns_steps, coefficient_type=self.coefficient_type, use_syrk=self.use_syrk
            )

    def _use_fused_kernels(self) -> bool:
        """Static decision, identical on every rank: all parameters are contiguous fp32 CUDA matrices, the bf16
        path is selected and the driver functions are the package's own."""
        return (
            self.fp32_matmul_prec == "medium"
            and self.weight_decay_method in _SHRINK
            and self.coefficient_type in muon_utils._COEFFICIENT_SETS
            and all(_fused_step.eligible(p.data, p.grad) for p in self.params)
            and all(getattr(muon_utils, name) is fn for name, fn in _NS_FUNCTIONS.items())
        )

    def _orthogonalize_many(self, idxs: Sequence[int], fused: bool) -> dict[int, torch.Tensor]:
        """Unscaled orthogonalized updates of the owned parameters ``idxs``."""
        if not fused:
            return {i: self._orthogonalize_owned(i) for i in idxs}
        out: dict[int, torch.Tensor] = {}
        for run in self._by_group(idxs):
            _, momentum, wd = self._hyper(run[0])
            ups = _fused_step.orthogonalized_updates(
                [self.params[i].data for i in run],
                [self.params[i].grad for i in run],
                [self._momentum_buffer(i) for i in run],
                momentum=momentum,
                nesterov=self.nesterov,
                l2_weight_decay=wd if self.weight_decay_method == "l2" else 0.0,
                steps=self.num_ns_steps,
                coefficient_type=self.coefficient_type,
                use_syrk=self.use_syrk,
            )
            out.update(zip(run, ups))
        return out

    def _apply_many(self, idxs: Sequence[int], updates: Sequence[torch.Tensor], fused: bool) -> None:
        """Weight decay and ``p -= lr * (update * scale * extra)`` for the parameters ``idxs``, with the arithmetic
        of the single-process step; one fused launch sequence per parameter group."""
        if not fused:
            for i, u in zip(idxs, updates):
                p = self.params[i]
                lr, _, wd = self._hyper(i)
                scale = get_muon_scale_factor(p.size(-2), p.size(-1), mode=self.scale_mode)
                if self.weight_decay_method != "l2":
                    self._apply_weight_decay_inplace(p.data, p.grad, lr, wd)
                p.data.add_(u.view_as(p).to(torch.float32) * scale * self.extra_scale_factor, alpha=-lr)
            return
        by_idx = dict(zip(idxs, updates))
        for run in self._by_group(idxs):
            lr = self._hyper(run[0])[0]
            scales = [get_muon_scale_factor(*self.params[i].shape[-2:], mode=self.scale_mode) for i in run]
            _native.muon_apply_batch(
                [self.params[i].data for i in run], [by_idx[i] for i in run], scales, self._shrink(run[0]),
                self.extra_scale_factor, lr,
            )  # fmt: skip

    @torch.no_grad()
    def step(self, closure=None) -> None:  # type: ignore[no-untyped-def,override]
        """One optimizer step; on return every rank holds the same updated parameters.  ``closure`` is not
        supported and must be ``None`` (as for the single-process optimizers)."""
        if closure is not None:
            raise ValueError("closure is not supported")
        for i, p in enumerate(self.params):
            if p.grad is None:
                raise RuntimeError(f"parameter {i} has no gradient; layer-parallel Muon needs all gradients")
        fused = self._use_fused_kernels()
        dev = self.params[0].device
        if self.world == 1:
            streams = self._fork_compute_streams(dev) if fused else []
            for j, b in enumerate(self.buckets):
                idxs = [i for i, _ in b.per_rank[0]]
                with torch.cuda.stream(streams[j % 2]) if streams else contextlib.nullcontext():
                    orths = self._orthogonalize_many(idxs, fused)
                    self._apply_many(idxs, [orths[i] for i in idxs], fused)
            if streams:
                self._join_compute_streams(dev)
            return

        if self.exchange in ("parameters", "mixed"):
            self._step_exchanging_parameters(fused, dev)
            return
        if dev.type != "cuda":
            # Host ranks (tests on gloo): plain collective, no overlap.
            for b in self.buckets:
                self._host_bucket_as_updates(b, fused, dev)
            return

        # GPU ranks: the exchange of bucket j (copy-engine pushes into the peers' symmetric buffers, a group
        # barrier) and its weight update run on a side stream behind the Newton-Schulz work of bucket j + 1.
        # The copies use no SM and the update is HBM-bound while the iteration is tensor-bound.  The symmetric
        # buffer has two halves used alternately; a half is rewritten only after the barrier of the exchange in
        # between, which every rank enters after it has consumed that half.
        max_slot = max(b.slot_numel for b in self.buckets)
        if self._peer is None:
            from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer

            self._side = torch.cuda.Stream(device=dev)
            self._peer = PeerBuffer(2 * self.world * max_slot, self.exchange_dtype, dev, self.group)
            self._exchanges = 0
        peer, side = self._peer, self._side
        streams = self._fork_compute_streams(dev)
        for j, b in enumerate(self.buckets):
            mine = b.per_rank[self.rank]
            with torch.cuda.stream(streams[j % 2]):
                orths = self._orthogonalize_many([i for i, _ in mine], fused)
                ready = torch.cuda.Event()
                ready.record()
            base = (self._exchanges % 2) * self.world * max_slot
            self._exchanges += 1
            with torch.cuda.stream(side):
                side.wait_event(ready)
                own = base + self.rank * b.slot_numel
                for i, off in mine:
                    peer.local[own + off : own + off + orths[i].numel()].copy_(orths[i].reshape(-1))
                    orths[i].record_stream(side)
                peer.all_gather_slots(base, b.slot_numel)
                self._apply_bucket(b, peer.local[base : base + self.world * b.slot_numel], fused)
        self._join_compute_streams(dev)
        torch.cuda.current_stream().wait_stream(side)

    def _host_bucket_as_updates(self, b: _Bucket, fused: bool, dev: torch.device) -> None:
        slot = torch.empty(b.slot_numel, dtype=self.exchange_dtype, device=dev)
        mine = b.per_rank[self.rank]
        orths = self._orthogonalize_many([i for i, _ in mine], fused)
        for i, off in mine:
            slot[off : off + orths[i].numel()].copy_(orths[i].reshape(-1))
        gathered = torch.empty(self.world * b.slot_numel, dtype=self.exchange_dtype, device=dev)
        dist.all_gather_into_tensor(gathered, slot, group=self.group)
        self._apply_bucket(b, gathered, fused)

    # -- exchange="parameters" and "mixed" ------------------------------------------------------------------
    def _bucket_bases(self) -> list[int]:
        """Element offset of every bucket in the flat parameter buffer (bucket-major, then rank, then slot offset)."""
        bases, at = [], 0
        for b in self.buckets:
            bases.append(at)
            at += self.world * b.slot_numel
        return bases + [at]

    def _adopt_parameters(self, dev: torch.device) -> None:
        """Move every parameter into one symmetric fp32 buffer laid out like the exchange slots (collective)."""
        from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer

        bases = self._bucket_bases()
        self._param_peer = PeerBuffer(max(bases[-1], 8), torch.float32, dev, self.group)
        for b, base in zip(self.buckets, bases):
            for r in range(self.world):
                for i, off in b.per_rank[r]:
                    p = self.params[i]
                    if p.dtype != torch.float32 or not p.data.is_contiguous():
                        raise TypeError("exchange='parameters' needs contiguous float32 parameters")
                    at = base + r * b.slot_numel + off
                    home = self._param_peer.local[at : at + p.numel()].view_as(p.data)
                    home.copy_(p.data)
                    p.data = home
        # Nobody may push into a rank's buffer before that rank has moved its parameters in.
        torch.cuda.current_stream(dev).synchronize()
        self._param_peer.barrier()
        self._side = torch.cuda.Stream(device=dev)

    def _step_exchanging_parameters(self, fused: bool, dev: torch.device) -> None:
        if dev.type != "cuda":
            # Host ranks (tests on gloo): the owners' new values are gathered and copied over the other ranks' copies.
            for j, b in enumerate(self.buckets):
                if self._as_updates[j]:
                    self._host_bucket_as_updates(b, fused, dev)
                    continue
                mine = [i for i, _ in b.per_rank[self.rank]]
                orths = self._orthogonalize_many(mine, fused)
                self._apply_many(mine, [orths[i] for i in mine], fused)
                slot = torch.zeros(b.slot_numel, dtype=torch.float32, device=dev)
                for i, off in b.per_rank[self.rank]:
                    slot[off : off + self.params[i].numel()].copy_(self.params[i].data.reshape(-1))
                gathered = torch.empty(self.world * b.slot_numel, dtype=torch.float32, device=dev)
                dist.all_gather_into_tensor(gathered, slot, group=self.group)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    for i, off in b.per_rank[r]:
                        p = self.params[i]
                        p.data.copy_(gathered[r * b.slot_numel + off : r * b.slot_numel + off + p.numel()].view_as(p))
            return

        # GPU ranks: the parameters live in the symmetric buffer, a rank's matrices of one bucket contiguously in
        # its slot.  After the owner has updated them, pushing the slot to every peer (copy engines, side stream)
        # IS the parameter update of the peers; it overlaps the Newton-Schulz work of the next bucket.  During a
        # step a rank reads only matrices it owns, and peers write only matrices it does not own.
        if self._param_peer is None:
            self._adopt_parameters(dev)
        peer, side = self._param_peer, self._side
        max_slot = max([b.slot_numel for j, b in enumerate(self.buckets) if self._as_updates[j]], default=0)
        if max_slot and self._peer is None:
            # "mixed": the buckets that travel as updates use the two-halves buffer of exchange="updates" (a half is
            # rewritten only after the barrier of the exchange in between, see there).
            from emerging_optimizers_b200.distributed.peer_memory import PeerBuffer

            self._peer = PeerBuffer(2 * self.world * max_slot, self.exchange_dtype, dev, self.group)
        # Entry barrier: a peer may write my copy of its matrices only after everything I enqueued before this step
        # (the backward pass that read them) is done, and symmetrically.
        peer.barrier()
        streams = self._fork_compute_streams(dev)
        for j, (b, base) in enumerate(zip(self.buckets, self._bucket_bases())):
            mine = [i for i, _ in b.per_rank[self.rank]]
            with torch.cuda.stream(streams[j % 2]):
                orths = self._orthogonalize_many(mine, fused)
                if not self._as_updates[j]:
                    self._apply_many(mine, [orths[i] for i in mine], fused)
                ready = torch.cuda.Event()
                ready.record()
            with torch.cuda.stream(side):
                side.wait_event(ready)
                if self._as_updates[j]:
                    ubase = (self._exchanges % 2) * self.world * max_slot
                    self._exchanges += 1
                    own = ubase + self.rank * b.slot_numel
                    for i, off in b.per_rank[self.rank]:
                        self._peer.local[own + off : own + off + orths[i].numel()].copy_(orths[i].reshape(-1))
                        orths[i].record_stream(side)
                    self._peer.all_gather_slots(ubase, b.slot_numel)
                    self._apply_bucket(b, self._peer.local[ubase : ubase + self.world * b.slot_numel], fused)
                    continue
                # No barrier per bucket: the buckets' regions are disjoint and nobody reads a pushed matrix before
                # the step ends, so a rank's pushes never wait for the slowest rank's previous bucket.
                peer.all_gather_slots(base, b.slot_numel, barrier=PER_BUCKET_BARRIER)
        with torch.cuda.stream(side):
            peer.barrier()  # every rank's pushes have landed everywhere
        self._join_compute_streams(dev)
        torch.cuda.current_stream().wait_stream(side)

    def _apply_bucket(self, b: _Bucket, gathered: torch.Tensor, fused: bool) -> None:
        idxs, ups = [], []
        for r in range(self.world):
            base = r * b.slot_numel
            for i, off in b.per_rank[r]:
                idxs.append(i)
                ups.append(gathered[base + off : base + off + self.params[i].numel()])
        self._apply_many(idxs, ups, fused)

    # -- checkpointing -----------------------------------------------------------------------------------
    # ``state_dict()`` is torch's: ``{"state": {index: {"momentum_buffer": tensor}}, "param_groups": [...]}`` with
    # entries only for the matrices this rank owns (the union over ranks is the full checkpoint).

    def gathered_state_dict(self) -> dict:
        """The full checkpoint on every rank, in the layout of ``state_dict()``: each momentum buffer is broadcast
        by its owner.

        Collective (all ranks of the group, same call order).  Every stepped parameter index is present, so the
        result can be saved by one rank and later loaded on a group of any size: :meth:`load_state_dict` keeps the
        entries of the matrices the loading rank owns.  Matrices that have not been stepped yet have no entry.
        """
        sd = self.state_dict()
        sd["owners"] = list(self.owners)
        if self.world == 1:
            return sd
        # Which matrices have state is the same question on every rank only if the owners answer it.
        has = torch.zeros(len(self.params), dtype=torch.int32, device=self.params[0].device if self.params else "cpu")
        for i, p in enumerate(self.params):
            if "momentum_buffer" in self.state.get(p, {}):
                has[i] = 1
        dist.all_reduce(has, op=dist.ReduceOp.MAX, group=self.group)
        full: dict[int, dict[str, torch.Tensor]] = {}
        for i in has.nonzero().flatten().tolist():
            p, owner = self.params[i], self.owners[i]
            buf = self.state[p]["momentum_buffer"] if owner == self.rank else torch.empty_like(p.data)
            dist.broadcast(buf, src=dist.get_global_rank(self.group, owner) if self.group is not None else owner,
                           group=self.group)  # fmt: skip
            full[i] = {"momentum_buffer": buf}
        sd["state"] = full
        return sd

    def load_state_dict(self, state_dict: dict) -> None:  # type: ignore[override]
        """Load a checkpoint written by ``state_dict()`` or :meth:`gathered_state_dict`; of the per-parameter
        entries, only those of the matrices this rank owns are kept (as copies)."""
        mine = {
            int(i): {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in st.items()}
            for i, st in state_dict["state"].items()
            if self.owners[int(i)] == self.rank
        }
        super().load_state_dict({"state": mine, "param_groups": state_dict["param_groups"]})
