"""ATREX public operator surface for the sm_100a (B200) FlashAttention build.

Importing this package is free: no torch import, no library load, no compile.
Each public name is a small proxy that imports its implementation module on the
first call and then replaces itself with the real function, as
``_lazy_import_and_call`` does in the reference (python/atrex/__init__.py:13-39).
This build exports the FlashAttention entry points
(python/atrex/__init__.py:66-73 in the reference) and compact sparse attention (:74-77).
"""

from __future__ import annotations

from collections.abc import Callable as _Callable
from importlib import import_module as _import_module
from typing import Any as _Any

__all__: tuple[str, ...] = ()


def _lazy_import_and_call(
    func_name: str,
    module_name: str,
    *,
    public_name: str | None = None,
) -> _Callable[..., _Any]:
    """Build a proxy for ``module_name.func_name`` exported as ``public_name``.

    The proxy resolves the implementation when called.  Only after the lookup
    succeeded does it rebind the exported name to the real callable, so a failed
    import leaves the proxy in place and the next call tries again.
    """
    exported = func_name if public_name is None else public_name

    def _proxy(*args: _Any, **kwargs: _Any) -> _Any:
        implementation = getattr(_import_module(module_name), func_name)
        if not callable(implementation):
            raise TypeError(f"{module_name}.{func_name} is not callable")
        globals()[exported] = implementation
        return implementation(*args, **kwargs)

    _proxy.__name__ = _proxy.__qualname__ = exported
    _proxy.__module__ = __name__
    return _proxy


can_use_flash_attn_varlen_func = _lazy_import_and_call(
    "can_use_flash_attn_varlen_func", "atrex.api.flash_attn"
)
flash_attn_varlen_func = _lazy_import_and_call(
    "flash_attn_varlen_func", "atrex.api.flash_attn"
)

qsa_compact = _lazy_import_and_call("qsa_compact", "atrex.api.qsa")

__all__ = ("can_use_flash_attn_varlen_func", "flash_attn_varlen_func", "qsa_compact")
