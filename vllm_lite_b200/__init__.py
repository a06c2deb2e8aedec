"""Importable name of the engine whose sources live in the folder `vllm-lite_b200/`.

A Python package name cannot hold a hyphen, so this package redirects its
search path to the sibling folder; `vllm_lite_b200.config` is the file
`vllm-lite_b200/config/__init__.py`, and so on.
"""
from pathlib import Path as _Path

_src = _Path(__file__).resolve().parent.parent / "vllm-lite_b200"
if not _src.is_dir():
    raise ImportError(f"engine sources not found at {_src}")
__path__.insert(0, str(_src))

__version__ = "0.1.0"

from .api import *  # noqa: E402,F401,F403
from .api import __all__  # noqa: E402,F401
