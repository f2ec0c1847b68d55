"""CPU oracle for the Newton-Schulz / Muon hot path.  TEST INFRASTRUCTURE ONLY.

A plain numpy restatement of the reference algorithm (NVIDIA-NeMo/Emerging-Optimizers), used only as the
checker in ``tests/``, in ``__graft_entry__.smoke()`` and as the timed CPU baseline in ``bench.py``.  Nothing in
the shipped package imports this module.

Parity is pinned: ``tests/test_oracle_golden.py`` checks every function here against vectors produced by running
the reference itself (``tests/golden/make_golden.py``, outputs committed under ``tests/golden/``).

Each function cites the reference file:line it follows (paths inside the reference repository).
"""

from __future__ import annotations

import itertools
from typing import Iterator, Sequence

import numpy as np


# emerging_optimizers/orthogonalized_optimizers/muon_utils.py:30-90
COEFFICIENT_SETS: dict[str, list[tuple[float, float, float]]] = {
    "simple": [(3.4445, -4.7750, 2.0315)],
    "quintic": [
        (4.0848, -6.8946, 2.9270),
        (3.9505, -6.3029, 2.6377),
        (3.7418, -5.5913, 2.3037),
        (2.8769, -3.1427, 1.2046),
        (2.8366, -3.0525, 1.2012),
    ],
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
    "cans": [
        (8.4703, -25.1081, 18.6293),
        (4.1828, -3.1087, 0.5806),
        (3.9619, -2.9541, 0.5630),
        (3.2866, -2.4647, 0.5074),
        (2.2737, -1.6447, 0.4162),
    ],
    "aol": [
        (4.0098, -7.0585, 2.4635),
        (3.4585, -5.5479, 2.5959),
        (2.7573, -3.2939, 1.4254),
        (2.7215, -3.0494, 1.3169),
    ],
    "deepseekv4": [(3.4445, -4.7750, 2.0315)] * 8 + [(2.0, -1.5, 0.5)] * 2,
    "cubic5": [
        (3.3656576, -3.3420992, 0.0),
        (2.5744352, -1.4957376, 0.0),
        (2.5368962, -1.4312570, 0.0),
        (2.4418906, -1.2764040, 0.0),
        (2.2230472, -0.9630650, 0.0),
    ],
}

# muon_utils.py:239 -- schedules that hold their last tuple instead of cycling
REPEAT_LAST_TYPES = ("polar_express", "cans", "deepseekv4")


def coefficient_iterator(
    steps: int, coefficient_sets: Sequence[tuple[float, float, float]], mode: str = "cycle"
) -> Iterator[tuple[float, float, float]]:
    """muon_utils.py:93-129 (get_coefficient_iterator)."""
    if not coefficient_sets:
        raise ValueError("coefficient_sets must be non-empty.")
    if mode == "cycle":
        base = itertools.cycle(coefficient_sets)
    elif mode == "repeat_last":
        base = itertools.chain(coefficient_sets, itertools.repeat(coefficient_sets[-1]))
    else:
        raise ValueError(f"Invalid mode: {mode}. Expected 'cycle' or 'repeat_last'.")
    return itertools.islice(base, steps)


def coefficient_schedule(
    steps: int, coefficient_type: str, custom: Sequence[tuple[float, float, float]] | None = None
) -> list[tuple[float, float, float]]:
    """muon_utils.py:224-241: preset lookup, cubic5 length guard, cycle / repeat_last choice."""
    if coefficient_type in COEFFICIENT_SETS:
        sets = COEFFICIENT_SETS[coefficient_type]
    elif coefficient_type == "custom":
        if custom is None:
            raise ValueError("custom_coefficient_sets must be provided when coefficient_type is 'custom'.")
        sets = list(custom)
    else:
        raise ValueError(f"Invalid coefficient type: {coefficient_type}")
    if coefficient_type == "cubic5" and steps != len(sets):
        raise ValueError(f"cubic5 is a fixed {len(sets)}-step schedule; got steps={steps}.")
    mode = "repeat_last" if coefficient_type in REPEAT_LAST_TYPES else "cycle"
    return list(coefficient_iterator(steps, sets, mode))


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bfloat16 (ties to even) and return it widened to fp32 again.

    Models ``X.to(torch.bfloat16)`` (muon_utils.py:262) and the bf16 output cast of every bf16 kernel.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    nan = np.isnan(x)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = (bits + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = rounded.view(np.float32).copy()
    out[nan] = np.nan
    return out


def _mT(x: np.ndarray) -> np.ndarray:
    return np.swapaxes(x, -1, -2)


def frobenius_normalize(x: np.ndarray, eps: float = 1e-15, in_double: bool = False) -> np.ndarray:
    """muon_utils.py:215-222: per-matrix x / max(||x||_F, eps); the float64 variant skips the clamp."""
    x = np.asarray(x, dtype=np.float32)
    if in_double:
        norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=(-2, -1), keepdims=True)).astype(np.float32)
        return (x / norm).astype(np.float32)
    norm = np.sqrt((x.astype(np.float64) ** 2).sum(axis=(-2, -1), keepdims=True)).astype(np.float32)
    return (x / np.maximum(norm, np.float32(eps))).astype(np.float32)


def syrk_ex(
    a: np.ndarray, c: np.ndarray | None = None, alpha: float = 1.0, beta: float = 0.0, bf16: bool = True
) -> np.ndarray:
    """``alpha * a @ a.mT + beta * c`` with fp32 accumulation and fp32 epilogue, bf16 output when ``bf16``.

    emerging_optimizers/triton_kernels/syrk.py:195-215 and batched_syrk.py:209-227 (accumulate in fp32, scale by
    alpha, add beta * c in fp32, cast to bf16).
    """
    a = np.asarray(a, dtype=np.float32)
    d = np.float32(alpha) * np.matmul(a, _mT(a))
    if c is not None and beta != 0.0:
        d = d + np.float32(beta) * np.asarray(c, dtype=np.float32)
    d = d.astype(np.float32)
    return bf16_round(d) if bf16 else d


def newton_schulz_step(x: np.ndarray, a: float, b: float, c: float, bf16: bool, gram_reduce=None) -> np.ndarray:
    """muon_utils.py:348-378 (and :381-411 batched): A = XX^T; B = bA + cA^2; X' = aX + BX; cubic when c == 0.

    ``gram_reduce`` stands for the tensor-parallel all-reduce of the Gram matrix (:371-372).
    With ``bf16`` every product is rounded to bf16 on output, as the bf16 GEMMs of the "medium" path do.
    """
    rnd = bf16_round if bf16 else (lambda v: v.astype(np.float32))
    f = np.float32
    A = rnd(np.matmul(x, _mT(x)))
    if gram_reduce is not None:
        A = gram_reduce(A)
    if c != 0.0:
        B = rnd(f(b) * A + f(c) * np.matmul(A, A))
        return rnd(f(a) * x + np.matmul(B, x))
    return rnd(f(a) * x + f(b) * np.matmul(A, x))


def newton_schulz(
    x: np.ndarray,
    steps: int,
    coefficient_type: str = "quintic",
    custom_coefficient_sets: Sequence[tuple[float, float, float]] | None = None,
    eps: float = 1e-15,
    transpose: bool | None = None,
    precision: str = "highest",
    normalize_in_double: bool = False,
) -> np.ndarray:
    """muon_utils.py:149-274.  ``precision`` is the ambient fp32 matmul precision the reference reads at :245:
    "medium" runs the iteration on bf16-rounded operands, anything else stays in fp32."""
    x = np.asarray(x)
    if x.ndim < 2 or x.ndim > 3:
        raise TypeError(f"Input tensor x must be 2d or 3d (batched 2d), got {x.ndim}d")
    if x.dtype != np.float32:
        raise TypeError(f"Input tensor x must be in float32, got {x.dtype}")
    if transpose is None:
        transpose = x.shape[-2] > x.shape[-1]
    if transpose:
        x = _mT(x)
    X = frobenius_normalize(x, eps, normalize_in_double)
    schedule = coefficient_schedule(steps, coefficient_type, custom_coefficient_sets)
    bf16 = precision == "medium"
    if bf16:
        X = bf16_round(X)
    for a, b, c in schedule:
        X = newton_schulz_step(X, a, b, c, bf16)
    X = X.astype(np.float32)
    if transpose:
        X = _mT(X)
    return X


def newton_schulz_deferred_norm(
    x: np.ndarray,
    steps: int,
    coefficient_type: str = "quintic",
    custom_coefficient_sets: Sequence[tuple[float, float, float]] | None = None,
    eps: float = 1e-15,
    transpose: bool | None = None,
) -> np.ndarray:
    """The bf16 path of :func:`newton_schulz` with the Frobenius normalisation deferred, as the device kernels run
    it on large matrices: the iterate starts as the un-normalised ``bf16(x)``, and ``s = 1 / max(|x|, eps)`` enters
    the first iteration's two products instead (``A = bf16(s^2 X X^T)``, ``X' = bf16(s (a X + S X))``).  Not a
    restatement of the reference (which normalises first, muon_utils.py:242): it states what the variant computes,
    so that its distance to the reference's results can be measured without a GPU."""
    x = np.asarray(x)
    if x.dtype != np.float32 or x.ndim < 2 or x.ndim > 3:
        raise TypeError("x must be a float32 matrix or stack of matrices")
    if transpose is None:
        transpose = x.shape[-2] > x.shape[-1]
    if transpose:
        x = _mT(x)
    f = np.float32
    sumsq = (x.astype(np.float64) ** 2).sum(axis=(-2, -1), keepdims=True)
    s = (f(1.0) / np.maximum(np.sqrt(sumsq).astype(np.float32), f(eps))).astype(np.float32)
    X0 = bf16_round(x)
    X = None
    for i, (a, b, c) in enumerate(coefficient_schedule(steps, coefficient_type, custom_coefficient_sets)):
        if i > 0:
            X = newton_schulz_step(X, a, b, c, True)
            continue
        A = bf16_round((s * s) * np.matmul(X0, _mT(X0)))
        if c != 0.0:
            S = bf16_round(f(b) * A + f(c) * np.matmul(A, A))
            X = bf16_round(s * (f(a) * X0 + np.matmul(S, X0)))
        else:
            X = bf16_round(s * (f(a) * X0 + f(b) * np.matmul(A, X0)))
    if X is None:  # no iteration at all: the normalised input
        X = bf16_round(s * X0)
    X = X.astype(np.float32)
    if transpose:
        X = _mT(X)
    return X


def newton_schulz_tp_distributed(
    shards: Sequence[np.ndarray],
    steps: int,
    coefficient_type: str,
    partition_dim: int,
    precision: str = "highest",
    eps: float = 1e-15,
) -> list[np.ndarray]:
    """Single-process model of ``newton_schulz_tp(..., tp_mode="distributed")`` (muon_utils.py:334-341):
    every rank normalises by the global Frobenius norm (:132-146), all-reduces its partial Gram each step
    (:370-372) and updates its own shard."""
    if partition_dim not in (0, 1):
        raise ValueError(f"Invalid partition_dim: {partition_dim}")
    transpose = partition_dim == 0
    xs = [np.asarray(s, dtype=np.float32) for s in shards]
    if transpose:
        xs = [_mT(s) for s in xs]
    total = sum(float((s.astype(np.float32) * s.astype(np.float32)).sum()) for s in xs)
    norm = max(np.float32(np.sqrt(np.float32(total))), np.float32(eps))
    Xs = [(s / norm).astype(np.float32) for s in xs]
    bf16 = precision == "medium"
    rnd = bf16_round if bf16 else (lambda v: v.astype(np.float32))
    if bf16:
        Xs = [bf16_round(X) for X in Xs]
    f = np.float32
    for a, b, c in coefficient_schedule(steps, coefficient_type):
        # The reference rounds each partial Gram to X's dtype before summing (A inherits X's dtype).
        A = rnd(sum(rnd(np.matmul(X, _mT(X))) for X in Xs))
        if c != 0.0:
            B = rnd(f(b) * A + f(c) * np.matmul(A, A))
            Xs = [rnd(f(a) * X + np.matmul(B, X)) for X in Xs]
        else:
            Xs = [rnd(f(a) * X + f(b) * np.matmul(A, X)) for X in Xs]
    if transpose:
        Xs = [_mT(X) for X in Xs]
    return [np.ascontiguousarray(X, dtype=np.float32) for X in Xs]


def muon_scale_factor(size_out: int, size_in: int, mode: str = "spectral") -> float:
    """emerging_optimizers/orthogonalized_optimizers/muon.py:190-216."""
    if mode == "shape_scaling":
        return max(1, size_out / size_in) ** 0.5
    if mode == "spectral":
        return max(size_out, size_in) ** 0.5
    if mode == "unit_rms_norm":
        return (size_out / size_in) ** 0.5
    raise ValueError(f"Invalid mode for Muon update scale factor: {mode}")


def _lerp(start: np.ndarray, end: np.ndarray, weight: float) -> np.ndarray:
    """torch.lerp in fp32: start + w (end - start) for w < 0.5, else end - (end - start)(1 - w)."""
    w = np.float32(weight)
    diff = end - start
    if abs(weight) < 0.5:
        return (start + w * diff).astype(np.float32)
    return (end - diff * (np.float32(1.0) - w)).astype(np.float32)


def apply_weight_decay(p: np.ndarray, grad: np.ndarray, lr: float, weight_decay: float, method: str) -> None:
    """emerging_optimizers/mixin.py:35-56, in place on ``p`` or ``grad``."""
    if weight_decay == 0.0:
        return
    if method == "decoupled":
        p += np.float32(-weight_decay * lr) * p
    elif method == "independent":
        p += np.float32(-weight_decay) * p
    elif method == "l2":
        grad += np.float32(weight_decay) * p
    elif method == "palm":
        p += np.float32(-(weight_decay * lr * lr)) * p
    else:
        raise ValueError(f"Invalid weight decay method: {method}")


def muon_step(
    params: list[np.ndarray],
    grads: list[np.ndarray],
    momenta: list[np.ndarray],
    lr: float = 3e-4,
    momentum: float = 0.95,
    weight_decay: float = 0.01,
    nesterov: bool = False,
    weight_decay_method: str = "decoupled",
    precision: str = "medium",
    coefficient_type: str = "quintic",
    num_ns_steps: int = 5,
    scale_mode: str = "spectral",
    extra_scale_factor: float = 1.0,
) -> None:
    """One ``Muon.step()`` over fp32 2-D parameters, in place on ``params`` and ``momenta``.

    emerging_optimizers/orthogonalized_optimizers/orthogonalized_optimizer.py:164-212 (weight decay, momentum
    ``lerp_``, Nesterov ``lerp``, orthogonalize, ``p.add_(update, alpha=-lr)``) with Muon's closure
    (muon.py:117-132: Newton-Schulz, then ``* scale * extra``).
    """
    for p, g, m in zip(params, grads, momenta):
        g = g.astype(np.float32).copy()
        apply_weight_decay(p, g, lr, weight_decay, weight_decay_method)
        m[...] = _lerp(m, g, 1 - momentum)
        u = _lerp(g, m, momentum) if nesterov else m
        o = newton_schulz(u, num_ns_steps, coefficient_type, precision=precision)
        scale = muon_scale_factor(u.shape[-2], u.shape[-1], scale_mode)
        o = (o * np.float32(scale) * np.float32(extra_scale_factor)).astype(np.float32)
        p += np.float32(-lr) * o


def ns_flops(m: int, n: int, steps: int, cubic: bool = False) -> tuple[float, float]:
    """(dense-equivalent, symmetric-credited) FLOPs of ``steps`` iterations on an m x n matrix, m <= n after the
    wide transpose: Gram 2m^2n + A^2 2m^3 + BX 2m^2n; symmetric outputs counted once in the second figure."""
    if m > n:
        m, n = n, m
    if cubic:
        return steps * 4.0 * m * m * n, steps * (m * (m + 1.0) * n + 2.0 * m * m * n)
    dense = 4.0 * m * m * n + 2.0 * m**3
    sym = m * (m + 1.0) * n + m * m * (m + 1.0) + 2.0 * m * m * n
    return steps * dense, steps * sym
