"""AdaptiveMuon: Muon with a second-moment normalisation between orthogonalization and update scaling.

Same constructor, state keys (``momentum_buffer``, ``moment2_buffer``), per-group ``beta2`` / ``eps``, variants and
arithmetic as ``emerging_optimizers/orthogonalized_optimizers/adaptive_muon.py:38-331`` of the reference.
"""

from typing import Callable, Literal

import torch
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import mixin as opt_mixin
from emerging_optimizers_b200 import registry, utils
from emerging_optimizers_b200.orthogonalized_optimizers import _consumers, muon
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import OrthogonalizedOptimizer
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["AdaptiveMuon", "Moment2MethodT"]

Moment2MethodT = Literal["adamuon", "normuon", "namo"]


def _reduced_dim(shape: torch.Size) -> int:
    """NorMuon averages the squared update along the longer side (ties: along the last dimension)."""
    return -1 if shape[-2] >= shape[-1] else -2


@registry.register_optimizer("adaptive_muon")
class AdaptiveMuon(OrthogonalizedOptimizer):
    """Muon whose raw Newton-Schulz output is normalised by an EMA of second moments before Muon's scale factor.

    Variants (``moment2_method``):

    - "adamuon" (arXiv:2507.11005): elementwise, ``o / (sqrt(v) + eps)`` with ``v <- lerp(v, o^2, 1 - beta2)``.
    - "normuon" (arXiv:2510.05491): one second moment per row (or per column, whichever side is shorter),
      ``o * rsqrt(max(v, eps))``, then rescaled to the Frobenius norm the raw output had.
    - "namo" (arXiv:2602.17080): one scalar, ``o * |u|_F / (sqrt(v) + eps)`` with ``v`` the EMA of the squared
      Frobenius norm of the raw gradient and ``u`` the (Nesterov) momentum that was orthogonalized.

    Args:
        params: iterable of parameters or of dicts defining parameter groups.
        lr: learning rate.
        momentum: EMA coefficient of the momentum buffer.
        weight_decay: weight-decay strength.
        nesterov: use the Nesterov look-ahead of the momentum.
        weight_decay_method: see :data:`emerging_optimizers_b200.mixin.WeightDecayT`; "l2" is refused with "namo".
        fp32_matmul_prec: fp32 matmul precision while orthogonalizing.
        coefficient_type: Newton-Schulz schedule name.
        num_ns_steps: number of Newton-Schulz iterations (at least 1).
        scale_mode: Muon update scale, see
            :func:`~emerging_optimizers_b200.orthogonalized_optimizers.muon.get_muon_scale_factor`.
        extra_scale_factor: extra multiplier of the update.
        moment2_method: "adamuon", "normuon" or "namo".
        beta2: EMA coefficient of the second moment (per-group default).
        eps: stabiliser of the normalisation (per-group default).
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float,
        momentum: float,
        weight_decay: float,
        *,
        nesterov: bool = False,
        weight_decay_method: opt_mixin.WeightDecayT = "decoupled",
        fp32_matmul_prec: FP32MatmulPrecT = "medium",
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        scale_mode: muon.MuonScaleT = "spectral",
        extra_scale_factor: float = 1.0,
        moment2_method: Moment2MethodT = "adamuon",
        beta2: float = 0.95,
        eps: float = 1e-8,
    ):
        if moment2_method == "namo" and weight_decay_method == "l2":
            raise ValueError('moment2_method="namo" is incompatible with weight_decay_method="l2"')
        _consumers.check_steps(num_ns_steps)

        self.scale_mode = scale_mode
        self.extra_scale_factor = extra_scale_factor

        def unscaled_polar_factor(grad: torch.Tensor) -> torch.Tensor:
            # Muon's scale factor comes after the second-moment normalisation, not here.
            return _consumers.msign(grad, num_ns_steps, coefficient_type)

        super().__init__(
            params,
            lr,
            momentum,
            weight_decay,
            nesterov=nesterov,
            weight_decay_method=weight_decay_method,
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=unscaled_polar_factor,
        )
        self.moment2_method = moment2_method
        for group in self.param_groups:
            group.setdefault("beta2", beta2)
            group.setdefault("eps", eps)

    def _apply_muon_scale(self, update: torch.Tensor, size_out: int, size_in: int) -> torch.Tensor:
        return update * muon.get_muon_scale_factor(size_out, size_in, mode=self.scale_mode) * self.extra_scale_factor

    def _match_frobenius_norm(self, update: torch.Tensor, reference: torch.Tensor, eps: float) -> torch.Tensor:
        """``update`` rescaled to the Frobenius norm of ``reference``."""
        have = torch.linalg.vector_norm(update)
        want = torch.linalg.vector_norm(reference)
        return update * (want / have.clamp_min(eps))

    def _moment2_like(self, p: torch.Tensor) -> torch.Tensor:
        """A zero second-moment buffer of the shape the configured variant needs for parameter ``p``."""
        data = p.data
        if self.moment2_method == "adamuon":
            return torch.zeros_like(data)
        if self.moment2_method == "normuon":
            if data.ndim != 2:
                raise ValueError(
                    f"{self.__class__.__name__} only supports 2D parameters, got shape {tuple(data.shape)}"
                )
            shape = list(data.shape)
            shape[_reduced_dim(data.shape)] = 1
            return torch.zeros(shape, dtype=data.dtype, device=data.device)
        if self.moment2_method == "namo":
            return torch.zeros(1, dtype=data.dtype, device=data.device)
        raise TypeError(f"Invalid second moment method: {self.moment2_method}")

    @torch.no_grad()
    def _init_group(self, group: dict, skip_non_grad_params: bool = True) -> None:
        """Create ``momentum_buffer`` and ``moment2_buffer`` of every parameter that has no state yet."""
        for p in group["params"]:
            if skip_non_grad_params and p.grad is None:
                continue
            state = self.state[p]
            if len(state) == 0:
                state["momentum_buffer"] = torch.zeros_like(p.data)
                state["moment2_buffer"] = self._moment2_like(p)

    def _apply_moment2_normalization(
        self,
        orth_grad: torch.Tensor,
        moment2: torch.Tensor,
        beta2: float,
        eps: float,
        *,
        raw_grad: torch.Tensor | None = None,
        pre_orth_grad: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """EMA-update ``moment2`` in place and return the normalised update (before Muon's scale factor).

        Args:
            orth_grad: raw Newton-Schulz output.
            moment2: the parameter's second-moment buffer.
            beta2: EMA coefficient.
            eps: stabiliser.
            raw_grad: "namo" only: the gradient before the momentum update.
            pre_orth_grad: "namo" only: the tensor that was orthogonalized.
        """
        method = self.moment2_method
        if method == "adamuon":
            moment2.lerp_(orth_grad.square(), 1 - beta2)
            return orth_grad / (moment2.sqrt() + eps)
        if method == "normuon":
            per_line = orth_grad.square().mean(dim=_reduced_dim(orth_grad.shape), keepdim=True)
            moment2.lerp_(per_line, 1 - beta2)
            normalised = orth_grad * moment2.clamp_min(eps).rsqrt_()
            return self._match_frobenius_norm(normalised, orth_grad, eps)
        if method == "namo":
            if raw_grad is None or pre_orth_grad is None:
                raise RuntimeError("NAMO requires raw_grad and pre_orth_grad")
            moment2.lerp_(torch.linalg.vector_norm(raw_grad).square(), 1 - beta2)
            return orth_grad * (torch.linalg.vector_norm(pre_orth_grad) / (moment2.sqrt() + eps))
        raise TypeError(f"Invalid second moment method: {method}")

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        """One optimization step.  ``closure`` is not supported and must be ``None``."""
        if closure is not None:
            raise ValueError("closure is not supported")
        namo = self.moment2_method == "namo"

        for group in self.param_groups:
            self._init_group(group)
            lr = group["lr"]
            group_kwargs = {k: v for k, v in group.items() if k != "params"}

            for p in group["params"]:
                if p.dim() != 2:
                    raise ValueError(f"{self.__class__.__name__} only supports 2D parameters")
                grad = p.grad
                if grad is None:
                    continue
                state = self.state[p]

                self._apply_weight_decay_inplace(p, grad, lr, group["weight_decay"])
                direction = self._momentum_update(grad, state["momentum_buffer"], group["momentum"])

                with utils.fp32_matmul_precision(self.fp32_matmul_prec):
                    raw = self.orthogonalize(p, direction, **group_kwargs)

                update = self._apply_moment2_normalization(
                    raw,
                    state["moment2_buffer"],
                    group["beta2"],
                    group["eps"],
                    raw_grad=grad if namo else None,
                    pre_orth_grad=direction if namo else None,
                )
                update = self._apply_muon_scale(update, update.size(-2), update.size(-1))

                self.pre_weight_update_fn_inplace(p, update)
                p.add_(update, alpha=-lr)
                self.post_weight_update_fn_inplace(p)

        return None
