"""Kernel-source package.

A wheel copies the repository's ``src/`` tree to ``atrex/src`` (the reference's
packaging does the same, setup.py:27-37).  In a source checkout the tree sits
three levels up, so it is appended to this package's search path and
``atrex.src.nvidia.flash_attn.sm100`` resolves in both layouts.
"""

from pathlib import Path as _Path

_checkout_src = _Path(__file__).resolve().parents[3] / "src"
if _checkout_src.is_dir():
    __path__.append(str(_checkout_src))
