"""Base class of the orthogonalized optimizers: SGD-with-momentum whose update is orthogonalized before it is
applied.

Constructor arguments, state layout (``state[p]["momentum_buffer"]``), the order of operations inside
:meth:`OrthogonalizedOptimizer.step`, the override points and the error messages follow
``emerging_optimizers/orthogonalized_optimizers/orthogonalized_optimizer.py:46-269`` of the reference, so that
subclasses and checkpoints written for it keep working.
"""

from __future__ import annotations

from typing import Any, Callable, Generic, cast

import torch
import torch.optim as optim
from absl import logging
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import mixin as opt_mixin
from emerging_optimizers_b200 import utils
from emerging_optimizers_b200.utils import FP32MatmulPrecT
from emerging_optimizers_b200.weight_update_hooks import NoOpWeightUpdateHook, WeightUpdateHook
from emerging_optimizers_b200.weight_update_hooks.base import HookStateT


__all__ = ["OrthogonalizedOptimizer"]

_args_doc = """params: iterable of parameters or of dicts defining parameter groups.
        lr: learning rate of the inner SGD.
        momentum: EMA coefficient of the momentum buffer.
        weight_decay: weight-decay strength (see ``weight_decay_method``).
        nesterov: use the Nesterov look-ahead of the momentum.
        weight_decay_method: one of :data:`emerging_optimizers_b200.mixin.WeightDecayT`.
        fp32_matmul_prec: fp32 matmul precision in force while the update is orthogonalized
            ("medium" selects the bf16 tensor-core kernels).
        weight_update_hook: optional hook around the final in-place weight update.
"""


class OrthogonalizedOptimizer(opt_mixin.WeightDecayMixin, optim.Optimizer, Generic[HookStateT]):
    """Momentum SGD whose per-parameter update passes through ``scaled_orthogonalize_fn``.

    Per parameter and step: weight decay, ``m <- lerp(m, g, 1 - momentum)``, optional Nesterov
    ``u = lerp(g, m, momentum)`` (else ``u = m``), ``o = orthogonalize(p, u)`` under the configured fp32 matmul
    precision, then ``p <- p - lr * o`` bracketed by the pre/post update functions and the weight-update hook.

    Fused parameters (for example a stacked QKV weight, or per-head blocks) can be orthogonalized piecewise by
    overriding :meth:`orthogonalize` in a subclass: split ``grad``, call ``self.scaled_orthogonalize_fn`` on each
    piece (or once on a 3-D stack of equally sized pieces) and concatenate the results.

    Args:
        {_args_doc}
        scaled_orthogonalize_fn: maps the momentum tensor to the scaled orthogonalized update; identity if None.
        **kwargs: extra per-group defaults handed to ``torch.optim.Optimizer`` unchecked.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float,
        momentum: float,
        weight_decay: float,
        *,
        nesterov: bool,
        weight_decay_method: opt_mixin.WeightDecayT,
        fp32_matmul_prec: FP32MatmulPrecT,
        scaled_orthogonalize_fn: Callable | None = None,
        weight_update_hook: WeightUpdateHook[HookStateT] | None = None,
        **kwargs: Any,
    ):
        if scaled_orthogonalize_fn is None:
            logging.warning("scaled_orthogonalize_fn not provided. Using noop")
            scaled_orthogonalize_fn = torch.nn.Identity()

        self.fp32_matmul_prec = fp32_matmul_prec
        self.nesterov = nesterov
        self.weight_decay_method = weight_decay_method
        if weight_update_hook is None:
            weight_update_hook = cast(WeightUpdateHook[HookStateT], NoOpWeightUpdateHook())
        self._weight_update_hook: WeightUpdateHook[HookStateT] = weight_update_hook

        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay, **kwargs)
        super().__init__(params, defaults)
        self.scaled_orthogonalize_fn = scaled_orthogonalize_fn

    @torch.no_grad()
    def _init_group(self, group: dict, skip_non_grad_params: bool = True) -> None:
        """Create the zero momentum buffer of every parameter of ``group`` that does not have one yet."""
        for p in group["params"]:
            if skip_non_grad_params and p.grad is None:
                continue
            state = self.state[p]
            if len(state) == 0:
                state["momentum_buffer"] = torch.zeros_like(p.data)

    def _momentum_update(self, grad: torch.Tensor, buf: torch.Tensor, momentum: float) -> torch.Tensor:
        """EMA the buffer towards ``grad`` in place and return the tensor to orthogonalize."""
        buf.lerp_(grad, 1 - momentum)
        if self.nesterov:
            return grad.lerp(buf, momentum)
        return buf

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:
        """Run one optimization step.  ``closure`` is not supported and must be ``None``."""
        if closure is not None:
            raise ValueError("closure is not supported")

        for group in self.param_groups:
            self._init_group(group)
            for p in group["params"]:
                if p.grad is not None:
                    self._step_param(group, p)

        return None

    def _step_param(self, group: dict, p: torch.Tensor) -> None:
        """The update of one parameter: weight decay, momentum, orthogonalize, hooks, ``p -= lr * update``."""
        lr = group["lr"]
        grad = p.grad
        self._apply_weight_decay_inplace(p, grad, lr, group["weight_decay"])
        update = self._momentum_update(grad, self.state[p]["momentum_buffer"], group["momentum"])

        with utils.fp32_matmul_precision(self.fp32_matmul_prec):
            group_kwargs = {k: v for k, v in group.items() if k != "params"}
            orth = self.orthogonalize(p, update, **group_kwargs)

        self.pre_weight_update_fn_inplace(p, orth)
        hook_state = self._weight_update_hook.pre_weight_update_inplace(p, orth)
        p.add_(orth, alpha=-lr)
        self.post_weight_update_fn_inplace(p)
        self._weight_update_hook.post_weight_update_inplace(p, hook_state)

    def orthogonalize(self, p: torch.Tensor, grad: torch.Tensor, **kwargs: Any) -> torch.Tensor:
        """Map the momentum tensor of ``p`` to its orthogonalized update.

        The default accepts 2-D tensors only and calls ``self.scaled_orthogonalize_fn``.  Subclasses override this
        to reshape N-D parameters (e.g. convolution weights to ``[out, in * kh * kw]``) or to split fused ones;
        ``p`` is passed because such decisions usually depend on attributes of the parameter, and ``kwargs`` holds
        the non-"params" entries of its parameter group.
        """
        if grad.ndim != 2:
            raise ValueError("Only 2D parameters are supported.")
        return self.scaled_orthogonalize_fn(grad)

    def pre_weight_update_fn_inplace(self, p: torch.Tensor, update: torch.Tensor) -> None:
        """Experimental override point: called before ``p -= lr * update``."""

    def post_weight_update_fn_inplace(self, p: torch.Tensor) -> None:
        """Experimental override point: called after ``p`` has been updated."""


OrthogonalizedOptimizer.__doc__ = OrthogonalizedOptimizer.__doc__.format(_args_doc=_args_doc)  # type: ignore[union-attr]
