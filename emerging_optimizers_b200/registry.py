"""Name -> optimizer-class registry (boundary only: keeps ``"muon"`` resolvable by name).

Same functions as ``emerging_optimizers/registry.py:27-93`` of the reference.
"""

from functools import partial
from inspect import signature
from typing import Any, Callable

from torch import optim


_OPTIMIZERS: dict[str, type] = {}


def register_optimizer(name: str) -> Callable[[type], type]:
    """Class decorator: make ``cls`` available as ``get_optimizer_cls(name)`` (case-insensitive)."""
    key = name.lower()

    def decorator(cls: type) -> type:
        if key in _OPTIMIZERS:
            raise ValueError(f"Optimizer {name} already registered.")
        _OPTIMIZERS[key] = cls
        return cls

    return decorator


def get_optimizer_name_list() -> list[str]:
    return list(_OPTIMIZERS)


def get_optimizer_cls(name: str) -> type:
    """Look a class up by name; the module defining it must have been imported first."""
    try:
        return _OPTIMIZERS[name.lower()]
    except KeyError:
        raise ValueError(f"Optimizer {name} not found in the registry.") from None


def validate_optimizer_args(opt_cls: type, kwargs: dict[str, Any]) -> None:
    """Raise ``TypeError`` when ``kwargs`` holds a name the constructor of ``opt_cls`` does not take."""
    accepted = set(signature(opt_cls).parameters)
    unknown_args = set(kwargs) - accepted - {"params"}
    if unknown_args:
        raise TypeError(
            f"Optimizer '{opt_cls.__name__}' does not accept arguments: {unknown_args}.\n"
            f"Valid options are: {list(accepted)}"
        )


def get_configured_optimizer_cls(name: str, **kwargs: Any) -> Callable[..., optim.Optimizer]:
    """``partial(cls, **kwargs)`` after checking the keyword names against the constructor."""
    opt_cls = get_optimizer_cls(name)
    validate_optimizer_args(opt_cls, kwargs)
    return partial(opt_cls, **kwargs)
