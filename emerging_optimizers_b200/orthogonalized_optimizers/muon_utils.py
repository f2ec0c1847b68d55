"""Newton-Schulz orthogonalization driver and its tensor-parallel helpers, on the sm_100a kernels.

Public names, signatures, coefficient presets, error messages and the precision switch follow
``emerging_optimizers/orthogonalized_optimizers/muon_utils.py`` of the reference, so this module is a drop-in
for it on CUDA tensors.  What differs is underneath: every product of the iteration

    A = X X^T,   B = b A + c A^2,   X <- a X + B X

is one launch of the tcgen05 kernels in ``libeo_b200.so`` (the affine terms ``b A`` and ``a X`` are folded into
the kernels' epilogues), the Frobenius normalisation and the bf16 down-cast are a single fused pass, and the last
product of the last step writes fp32 directly.  There is no CPU path: CPU tensors are rejected.
"""

from __future__ import annotations

import os

from itertools import chain, cycle, islice, repeat
from typing import Any, Iterator, Literal, Sequence

import torch
from absl import logging

from emerging_optimizers_b200 import _native, triton_kernels


__all__ = ["newton_schulz", "newton_schulz_tp", "NSCoeffT", "get_coefficient_iterator", "CoeffIterMode"]

CoeffIterMode = Literal["cycle", "repeat_last"]

NSCoeffT = Literal["simple", "quintic", "polar_express", "cans", "aol", "deepseekv4", "custom", "cubic5"]

# (a, b, c) schedules; values and sources as in the reference (muon_utils.py:30-90).
_COEFFICIENT_SETS = {
    "simple": [
        (3.4445, -4.7750, 2.0315),
    ],
    # Tuned quintic schedule (leloykun.github.io/ponder/muon-opt-coeffs; numbers from modded-nanogpt).
    "quintic": [
        (4.0848, -6.8946, 2.9270),
        (3.9505, -6.3029, 2.6377),
        (3.7418, -5.5913, 2.3037),
        (2.8769, -3.1427, 1.2046),
        (2.8366, -3.0525, 1.2012),
    ],
    # Polar Express (arXiv:2505.16932), with its 1.01^degree safety division folded in.
    "polar_express": [
        (8.2051, -22.9019, 16.4607),
        (4.0664, -2.8612, 0.5184),
        (3.9096, -2.8234, 0.5250),
        (3.2856, -2.4153, 0.4853),
        (2.2779, -1.6198, 0.3985),
        (1.8726, -1.2307, 0.3585),
        (1.8564, -1.2132, 0.3568),
        (1.8750, -1.2500, 0.3750),
    ],
    # CANS (arXiv:2506.10935), Remez + adaptive interval.
    "cans": [
        (8.4703, -25.1081, 18.6293),
        (4.1828, -3.1087, 0.5806),
        (3.9619, -2.9541, 0.5630),
        (3.2866, -2.4647, 0.5074),
        (2.2737, -1.6447, 0.4162),
    ],
    # AOL schedule (thib-s/flash-newton-schulz).
    "aol": [
        (4.0098, -7.0585, 2.4635),
        (3.4585, -5.5479, 2.5959),
        (2.7573, -3.2939, 1.4254),
        (2.7215, -3.0494, 1.3169),
    ],
    # DeepSeek-V4 report: eight "simple" steps then two (2, -1.5, 0.5) steps.
    "deepseekv4": [(3.4445, -4.7750, 2.0315)] * 8 + [(2.0, -1.5, 0.5)] * 2,
    # Relaxed cubic five-step schedule (arXiv:2606.00371); c == 0 drops the A^2 product.
    "cubic5": [
        (3.3656576, -3.3420992, 0.0),
        (2.5744352, -1.4957376, 0.0),
        (2.5368962, -1.4312570, 0.0),
        (2.4418906, -1.2764040, 0.0),
        (2.2230472, -0.9630650, 0.0),
    ],
}

# Schedules that keep yielding their last tuple once exhausted; the others start over.
_REPEAT_LAST_TYPES = ("polar_express", "cans", "deepseekv4")


def get_coefficient_iterator(
    steps: int,
    coefficient_sets: Sequence[tuple[float, float, float]],
    mode: CoeffIterMode = "cycle",
) -> Iterator[tuple[float, float, float]]:
    """Yield ``steps`` coefficient tuples from ``coefficient_sets``.

    Args:
        steps: how many tuples to yield.
        coefficient_sets: non-empty sequence of ``(a, b, c)``.
        mode: "cycle" starts over after the last tuple, "repeat_last" keeps yielding it.

    Raises:
        ValueError: empty ``coefficient_sets`` or unknown ``mode``.
    """
    logging.debug("Iterating through %s steps with %s mode.", steps, mode)
    if not coefficient_sets:
        raise ValueError("coefficient_sets must be non-empty.")
    if mode == "cycle":
        source: Iterator[tuple[float, float, float]] = cycle(coefficient_sets)
    elif mode == "repeat_last":
        source = chain(coefficient_sets, repeat(coefficient_sets[-1]))
    else:
        raise ValueError(f"Invalid mode: {mode}. Expected 'cycle' or 'repeat_last'.")
    return islice(source, steps)


# ---------------------------------------------------------------------------------------------------------
# Kernel-facing helpers
# ---------------------------------------------------------------------------------------------------------
def _round_up(v: int, to: int) -> int:
    return (v + to - 1) // to * to


def _empty_matrix(shape: Sequence[int], dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """Row-major (.., R, C) buffer whose row stride is padded to 16 bytes so that TMA can address it."""
    *lead, rows, cols = shape
    per = 16 // torch.empty((), dtype=dtype).element_size()
    ld = _round_up(cols, per)
    if ld == cols:
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    mat = _round_up(rows * ld, per)
    base = torch.empty((*lead, mat), dtype=dtype, device=device)
    return base[..., : rows * ld].unflatten(-1, (rows, ld))[..., :cols]


def _as_kernel_operand(x: torch.Tensor) -> torch.Tensor:
    """Return ``x`` itself if the kernels can address it, else a padded row-major copy."""
    if _native.is_matrix_layout(x):
        mn, ld, bs = _native._mat_layout(x)
        per = 16 // x.element_size()
        if x.data_ptr() % 16 == 0 and ld % per == 0 and (x.dim() == 2 or bs % per == 0):
            return x
    # Copy in the orientation that keeps the contiguous dim contiguous.
    if x.stride(-2) == 1 and x.size(-2) > 1:
        y = _empty_matrix(x.mT.shape, x.dtype, x.device)
        y.copy_(x.mT)
        return y.mT
    y = _empty_matrix(x.shape, x.dtype, x.device)
    y.copy_(x)
    return y


def _is_split(X: torch.Tensor) -> bool:
    """fp32 iterates run on split-bf16 operands (fp32-accurate products); bf16 iterates run as they are."""
    return X.dtype == torch.float32


def _prepare(X: torch.Tensor) -> torch.Tensor:
    """Make ``X`` addressable by the kernels (bf16: TMA alignment; fp32: row- or column-major)."""
    if _is_split(X):
        return X if _native.is_matrix_layout(X) else X.contiguous()
    return _as_kernel_operand(X)


def _gram(X: torch.Tensor, use_syrk: bool, x_op: "torch.Tensor | _native.Split3 | None" = None) -> torch.Tensor:
    """A = X @ X.mT as a row-major (.., m, m) tensor of X's dtype."""
    x_op = X if x_op is None else x_op
    m = X.size(-2)
    A = _empty_matrix((*X.shape[:-2], m, m), X.dtype, X.device)
    if use_syrk or _is_split(X):
        # The fp32-accurate product costs six tensor-core passes, so it always takes the triangular kernel.
        _native.syrk(x_op, None, A)
    else:
        _native.gemm(x_op, x_op.mT, None, A)
    return A


def _gram_poly(A: torch.Tensor, b: float, c: float, use_syrk: bool) -> torch.Tensor:
    """B = b * A + c * A @ A for symmetric A."""
    Bm = _empty_matrix(A.shape, A.dtype, A.device)
    if _is_split(A):
        _native.syrk(_native.Split3(A), A, Bm, alpha=c, beta=b)
    elif use_syrk:
        _native.syrk(A, A, Bm, alpha=c, beta=b)
    else:
        _native.gemm(A, A, A, Bm, alpha=c, beta=b)
    return Bm


def _apply(
    S: torch.Tensor,
    X: torch.Tensor,
    alpha: float,
    beta: float,
    out_fp32: bool = False,
    x_op: "torch.Tensor | _native.Split3 | None" = None,
) -> torch.Tensor:
    """alpha * S @ X + beta * X for symmetric S, keeping X's orientation (row- or column-major).

    With ``out_fp32`` and a bf16 ``X`` the result is rounded to bf16 and widened to fp32 in the kernel epilogue,
    which equals ``(...).to(torch.bfloat16).to(torch.float32)``.
    """
    split = _is_split(X)
    x_op = X if x_op is None else x_op
    s_op = _native.Split3(S) if split else S
    out_dtype = torch.float32 if (out_fp32 or split) else X.dtype
    round_bf16 = out_fp32 and not split
    dense_out = out_fp32 or split

    def new(shape: Sequence[int]) -> torch.Tensor:
        if dense_out:
            return torch.empty(tuple(shape), dtype=out_dtype, device=X.device)
        return _empty_matrix(shape, out_dtype, X.device)

    mn, _, _ = _native._mat_layout(X)
    if mn == 0:
        out = new(X.shape)
        _native.gemm(s_op, x_op, X, out, alpha=alpha, beta=beta, round_bf16=round_bf16)
        return out
    # Column-major X: work on its row-major transpose, X'^T = beta X^T + alpha X^T S (S symmetric).
    out_t = new(X.mT.shape)
    _native.gemm(x_op.mT, s_op.mT, X.mT, out_t, alpha=alpha, beta=beta, round_bf16=round_bf16)
    return out_t.mT


# Matrices of at least this many elements (and more than 128 rows on the short side) take the deferred Frobenius
# normalisation on the bf16 path: one pass writes bf16(x) and the sum of squares, and the division is applied in the
# epilogues of the first Gram and the first update product.  The first iterate is then bf16(x) / |x| instead of
# bf16(x / |x|): the same accuracy, different last bits.  On a large matrix that is invisible in the result
# (1024 x 4096, five "simple" steps: 5.3e-3 from the reference's bf16 result either way); on matrices of a few
# hundred elements single roundings show (up to 1e-1 on a 16 x 32 case), so those keep the reference's order of
# operations.  0 disables it.  Stacks of wide matrices of at most 128 rows (the per-head kernel) take it from 2^20
# elements per matrix: a 128 x 8192 head is as far from the fp32 result either way (1.1e-2 after five "simple" steps).
FOLD_NORMALIZATION_MIN_NUMEL = 1 << 22
FOLD_NORMALIZATION_MIN_NUMEL_SMALL = 1 << 20


def _defer_normalization(rows: int, cols: int, steps: int) -> bool:
    """Whether a (stack of) ``rows x cols`` matrices in this physical orientation takes the deferred normalisation."""
    if FOLD_NORMALIZATION_MIN_NUMEL <= 0 or steps < 1:
        return False
    if min(rows, cols) > 128:
        return rows * cols >= FOLD_NORMALIZATION_MIN_NUMEL
    small_kernel = rows <= 128 and cols >= 256 and steps <= 16  # what the library routes to the per-head kernel
    return small_kernel and rows * cols >= FOLD_NORMALIZATION_MIN_NUMEL_SMALL


# Smallest tensor-parallel group for which S = b A + c A^2 is computed in row blocks, one per rank, and all-gathered,
# instead of redundantly on every rank as the reference does.  A rank's block costs 2 m^3 / P FLOP as a general
# product against m^3 for the symmetric kernel on the whole matrix, so the split pays from four ranks on.
TP_SHARD_GRAM_POLY_MIN_WORLD = 4


def _gram_poly_sharded(
    A: torch.Tensor, b: float, c: float, tp_group: "torch.distributed.ProcessGroup"
) -> torch.Tensor | None:
    """S = b A + c A A with the rows of S divided among the ranks of ``tp_group`` and all-gathered in place.

    Returns ``None`` when the split does not apply (small group, batched or fp32 iterate, rows not divisible).
    Every element is the same dot product with the same rounding as in :func:`_gram_poly`, so the result is
    identical on every rank and to the unsharded computation.
    """
    world = torch.distributed.get_world_size(tp_group)
    m = A.size(-1)
    if world < TP_SHARD_GRAM_POLY_MIN_WORLD or A.dim() != 2 or _is_split(A) or not A.is_cuda:
        return None
    if m % (8 * world) != 0 or not A.is_contiguous():
        return None
    from emerging_optimizers_b200.distributed import tensor_parallel

    if os.environ.get("EO_TP_GRAM", "auto") != "nccl":
        # product + all-gather in one kernel: the epilogue stores this rank's rows into every rank's buffer
        S = tensor_parallel.sharded_gram_poly(A, b, c, tp_group)
        if S is not None:
            return S
    rows = m // world
    r0 = torch.distributed.get_rank(tp_group) * rows
    S = torch.empty((m, m), dtype=A.dtype, device=A.device)
    _native.gemm(A[r0 : r0 + rows], A, A[r0 : r0 + rows], S[r0 : r0 + rows], alpha=c, beta=b)
    torch.distributed.all_gather_into_tensor(S.view(-1), S[r0 : r0 + rows].reshape(-1), group=tp_group)
    return S


def _ns_step(
    X: torch.Tensor,
    a: float,
    b: float,
    c: float,
    tp_group: "torch.distributed.ProcessGroup | None",
    use_syrk: bool,
    out_fp32: bool = False,
) -> torch.Tensor:
    """One iteration on the native kernels; the Gram all-reduce goes through torch.distributed."""
    _native.require_cuda(X, "X")
    X = _prepare(X)
    x_op = _native.Split3(X) if _is_split(X) else X
    if tp_group is not None and use_syrk and X.is_cuda:
        from emerging_optimizers_b200.distributed import tensor_parallel

        if tensor_parallel.fused_gram_available(X, tp_group):
            # Gram all-reduce fused into the SYRK epilogue (peer stores over NVLink), see tensor_parallel.py.
            A = tensor_parallel.fused_gram(X, tp_group)
            if c != 0.0:
                S = _gram_poly_sharded(A, b, c, tp_group)
                if S is None:
                    S = _gram_poly(A, b, c, use_syrk)
                return _apply(S, X, 1.0, a, out_fp32, x_op)
            return _apply(A, X, b, a, out_fp32, x_op)
    A = _gram(X, use_syrk, x_op)
    if tp_group is not None:
        if not A.is_contiguous():
            Ac = A.contiguous()
            torch.distributed.all_reduce(Ac, op=torch.distributed.ReduceOp.SUM, group=tp_group)
            A.copy_(Ac)
        else:
            torch.distributed.all_reduce(A, op=torch.distributed.ReduceOp.SUM, group=tp_group)
    if c != 0.0:
        S = _gram_poly_sharded(A, b, c, tp_group) if tp_group is not None else None
        if S is None:
            S = _gram_poly(A, b, c, use_syrk)
        return _apply(S, X, 1.0, a, out_fp32, x_op)
    return _apply(A, X, b, a, out_fp32, x_op)


def distributed_normalize_p2(
    x: torch.Tensor, eps: float, group: "torch.distributed.ProcessGroup", normalize_in_double: bool = False
) -> torch.Tensor:
    """Divide a sharded tensor by its global Frobenius norm.

    Every rank reduces its shard's sum of squares on the device (float64 accumulation, so tiny entries do not
    underflow when squared), the scalars are all-reduced over ``group`` and each rank divides its shard by the
    norm.  Without ``normalize_in_double`` the norm is clamped from below by ``eps``.
    """
    return _normalize(x, eps, group, normalize_in_double, torch.float32)


def _normalize(
    x: torch.Tensor,
    eps: float,
    group: "torch.distributed.ProcessGroup | None",
    normalize_in_double: bool,
    out_dtype: torch.dtype,
) -> torch.Tensor:
    _native.require_cuda(x, "x")
    if not _native.is_matrix_layout(x):
        x = x.contiguous()
    ss = _native.sumsq(x)
    if group is not None:
        # One scalar per rank (muon_utils.py:141-142 of the reference); a 3-D input shares one norm across its
        # batch there, because the whole local tensor is reduced.
        ss = ss.sum().reshape(1).expand(ss.numel()).contiguous() if ss.numel() > 1 else ss
        torch.distributed.all_reduce(ss, op=torch.distributed.ReduceOp.SUM, group=group)
    return _native.normalize(x, ss, eps, not normalize_in_double, out_dtype)


def newton_schulz(
    x: torch.Tensor,
    steps: int,
    coefficient_type: NSCoeffT = "quintic",
    custom_coefficient_sets: list[tuple[float, float, float]] | None = None,
    eps: float = 1e-15,
    transpose: bool | None = None,
    tp_group: "torch.distributed.ProcessGroup | None" = None,
    use_syrk: bool = False,
    normalize_in_double: bool = False,
) -> torch.Tensor:
    """Approximate the orthogonal polar factor of ``x`` by Newton-Schulz iteration.

    ``x`` is divided by its Frobenius norm (so its spectral norm is at most one), oriented so that the Gram
    matrix is taken over the shorter side, and iterated ``steps`` times with ``X <- a X + (b A + c A^2) X``,
    ``A = X X^T``.  With the tuned schedules the result is ``U S' V^T`` with ``S'`` close to one rather than the
    exact ``U V^T``.

    The ambient ``torch.get_float32_matmul_precision()`` selects the arithmetic, as in the reference: "medium"
    runs the iteration on bf16 operands with fp32 accumulation (A, B and X are rounded to bf16 once per product);
    "high" / "highest" keep fp32 storage and use split-bf16 tensor-core products accurate to fp32 round-off.

    Args:
        x: fp32 CUDA tensor, ``(M, N)`` or batched ``(B, M, N)``.
        steps: number of iterations.
        coefficient_type: "simple", "quintic", "polar_express", "cans", "aol", "deepseekv4", "cubic5" or
            "custom".
        custom_coefficient_sets: the tuples for "custom".
        eps: lower clamp of the norm.
        transpose: iterate on ``x.mT``; by default decided from the shape (rows > cols).
        tp_group: process group over which ``x`` is sharded along its long (contraction) dimension.
        use_syrk: compute ``A`` and ``A^2`` with the lower-triangular SYRK kernel instead of the general GEMM
            kernel ("medium" precision only; needs both dims to be multiples of 8, else the GEMM kernel is used).
        normalize_in_double: take the norm in float64 and skip the ``eps`` clamp.

    Returns:
        A new fp32 tensor with the shape of ``x``.
    """
    if x.ndim < 2 or x.ndim > 3:
        raise TypeError(f"Input tensor x must be 2d or 3d (batched 2d), got {x.ndim}d")
    if x.dtype != torch.float32:
        raise TypeError(f"Input tensor x must be in float32, got {x.dtype}")

    if coefficient_type in _COEFFICIENT_SETS:
        coefficient_sets = _COEFFICIENT_SETS[coefficient_type]
    elif coefficient_type == "custom":
        if custom_coefficient_sets is None:
            raise ValueError("custom_coefficient_sets must be provided when coefficient_type is 'custom'.")
        coefficient_sets = custom_coefficient_sets
    else:
        raise ValueError(f"Invalid coefficient type: {coefficient_type}")
    if coefficient_type == "cubic5" and steps != len(coefficient_sets):
        raise ValueError(
            f"cubic5 is a fixed {len(coefficient_sets)}-step schedule; got steps={steps}. "
            "Use steps=5, or pass explicit custom coefficients."
        )
    iter_mode: CoeffIterMode = "repeat_last" if coefficient_type in _REPEAT_LAST_TYPES else "cycle"
    schedule = list(get_coefficient_iterator(steps, coefficient_sets, mode=iter_mode))

    _native.require_cuda(x, "x")

    if transpose is None:
        transpose = x.size(-2) > x.size(-1)
    if transpose:
        x = x.mT

    bf16_path = torch.get_float32_matmul_precision() == "medium"
    # The step functions are looked up on the module at call time so that a caller may replace them.
    ns_step_fn = newton_schulz_step if x.ndim == 2 else batched_newton_schulz_step
    if bf16_path:
        if use_syrk:
            if x.size(-1) % 8 != 0 or x.size(-2) % 8 != 0:
                logging.log_first_n(
                    logging.ERROR,
                    "[SYRK-SKIP] skipping SYRK for shape %s because GEMM M or N is not 16-byte "
                    "aligned, which is incompatible with TMA.",
                    8,
                    tuple(x.shape),
                )
            else:
                ns_step_fn = newton_schulz_step_tsyrk if x.ndim == 2 else batched_newton_schulz_step_tsyrk
        logging.log_first_n(logging.INFO, "Using BF16 I/O kernels for Newton-Schulz iteration.", 1)

    native_fn = _NATIVE_STEP_FNS.get(ns_step_fn)

    if bf16_path and native_fn is not None and tp_group is None and not normalize_in_double and schedule:
        # Deferred normalisation: no pass of its own (see FOLD_NORMALIZATION_MIN_NUMEL).
        x_phys = x.mT if transpose else x  # the input's own orientation
        natural = transpose == (x_phys.size(-2) > x_phys.size(-1))
        if (
            natural
            and _defer_normalization(x_phys.size(-2), x_phys.size(-1), len(schedule))
            and x_phys.stride(-1) == 1
            and x_phys.size(-1) % 8 == 0
            and _native.is_matrix_layout(x_phys)
        ):
            xb, scales = _native.cast_sumsq(x_phys, eps)
            return _native.newton_schulz_bf16(xb, schedule, native_fn, out_dtype=torch.float32, scales=scales)

    # Normalise and (on the bf16 path) narrow in one pass over x.
    X = _normalize(x, eps, tp_group, normalize_in_double, torch.bfloat16 if bf16_path else torch.float32)

    # Whole loop in one library call when nothing needs to happen between the products: no Gram all-reduce, step
    # functions not replaced, default orientation and (bf16 path, which reads the iterate by TMA) addressable rows.
    X_phys = X.mT if transpose else X  # the input's own orientation
    natural = transpose == (X_phys.size(-2) > X_phys.size(-1))  # the library call transposes exactly when rows > cols
    one_call = native_fn is not None and tp_group is None and schedule and natural and X_phys.stride(-1) == 1
    if one_call and bf16_path and X_phys.size(-1) % 8 == 0 and (X_phys.dim() == 2 or X_phys.stride(0) % 8 == 0):
        return _native.newton_schulz_bf16(X_phys, schedule, native_fn, out_dtype=torch.float32)
    if one_call and not bf16_path:
        return _native.newton_schulz_f32(X_phys, schedule)

    for i, (a, b, c) in enumerate(schedule):
        if native_fn is not None and bf16_path and i == len(schedule) - 1:
            # Last step: the kernel epilogue rounds to bf16 and widens to fp32, saving the separate cast pass.
            X = _ns_step(X, a, b, c, tp_group, use_syrk=native_fn, out_fp32=True)
        else:
            X = ns_step_fn(X, a, b, c, tp_group=tp_group)

    X = X.to(torch.float32)
    if transpose:
        X = X.mT
    return X


def newton_schulz_tp(
    x: torch.Tensor,
    steps: int,
    coefficient_type: NSCoeffT,
    tp_group: "torch.distributed.ProcessGroup",
    partition_dim: int | None = None,
    tp_mode: Literal["duplicated", "distributed"] = "duplicated",
    use_syrk: bool = False,
) -> torch.Tensor:
    """Newton-Schulz on a tensor that is sharded over ``tp_group`` along ``partition_dim``.

    - ``partition_dim is None``: ``x`` is not sharded; plain :func:`newton_schulz`.
    - ``tp_mode="duplicated"``: all-gather the shards, orthogonalize the full matrix on every rank, return this
      rank's chunk.
    - ``tp_mode="distributed"``: every rank keeps its shard; the iteration contracts over the sharded dimension
      (``transpose`` is set from ``partition_dim``), the partial Gram matrices are all-reduced each step and the
      update of the shard stays local.  Sharding along the short dimension still works but wastes compute.

    ``use_syrk`` is forwarded to :func:`newton_schulz` on every path.
    """
    if partition_dim is None:
        return newton_schulz(x, steps, coefficient_type, use_syrk=use_syrk)

    common: dict[str, Any] = {"steps": steps, "coefficient_type": coefficient_type, "use_syrk": use_syrk}

    if tp_mode == "duplicated":
        world = tp_group.size()
        gathered = [torch.empty_like(x) for _ in range(world)]
        torch.distributed.all_gather(gathered, x, tp_group)
        full = newton_schulz(torch.cat(gathered, dim=partition_dim), tp_group=None, **common)
        return full.chunk(world, dim=partition_dim)[tp_group.rank()]
    if tp_mode == "distributed":
        if partition_dim not in (0, 1):
            raise ValueError(f"Invalid partition_dim: {partition_dim}")
        return newton_schulz(x, **common, transpose=(partition_dim == 0), tp_group=tp_group)
    raise ValueError(f"Invalid tp_mode: {tp_mode}")


def newton_schulz_step(
    X: torch.Tensor, a: float, b: float, c: float, tp_group: "torch.distributed.ProcessGroup | None" = None
) -> torch.Tensor:
    """One iteration ``X <- a X + (b A + c A^2) X`` (``X <- a X + b A X`` when ``c == 0``) with the general
    tensor-core GEMM kernel for every product.

    If ``tp_group`` is given, ``X`` is this rank's shard along the contraction dimension and the Gram matrix is
    all-reduced over the group; the caller is responsible for sharding along that dimension.
    """
    return _ns_step(X, a, b, c, tp_group, use_syrk=False)


def batched_newton_schulz_step(
    X: torch.Tensor, a: float, b: float, c: float, tp_group: "torch.distributed.ProcessGroup | None" = None
) -> torch.Tensor:
    """:func:`newton_schulz_step` for ``X`` of shape ``(B, M, N)``; the batch is one launch per product."""
    return _ns_step(X, a, b, c, tp_group, use_syrk=False)


def newton_schulz_step_tsyrk(
    X: torch.Tensor, a: float, b: float, c: float, tp_group: "torch.distributed.ProcessGroup | None" = None
) -> torch.Tensor:
    """One iteration with the symmetric products (``X X^T`` and ``A A``) on the lower-triangular SYRK kernel.

    ``X`` must be bfloat16 with both dims multiples of 8.
    """
    assert triton_kernels.HAS_TRITON_340, "libeo_b200.so has not been built; the SYRK kernel is unavailable."
    return _ns_step(X, a, b, c, tp_group, use_syrk=True)


def batched_newton_schulz_step_tsyrk(
    X: torch.Tensor, a: float, b: float, c: float, tp_group: "torch.distributed.ProcessGroup | None" = None
) -> torch.Tensor:
    """:func:`newton_schulz_step_tsyrk` for ``X`` of shape ``(B, M, N)``."""
    assert triton_kernels.HAS_TRITON_340, "libeo_b200.so has not been built; the SYRK kernel is unavailable."
    return _ns_step(X, a, b, c, tp_group, use_syrk=True)


# Step functions as defined above -> whether they use the SYRK kernel.  `newton_schulz` fuses the final fp32 cast
# only when the function it looked up is still one of these (i.e. has not been replaced by the caller).
_NATIVE_STEP_FNS = {
    newton_schulz_step: False,
    batched_newton_schulz_step: False,
    newton_schulz_step_tsyrk: True,
    batched_newton_schulz_step_tsyrk: True,
}
