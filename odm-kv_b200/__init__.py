"""odmkv_b200 -- B200 (sm_100a) implementation of ODM-KV's compress-then-decode path.

The directory name carries a hyphen, so import it with
``importlib.import_module("odm-kv_b200")``; the package then also answers to the plain name
``odmkv_b200`` (``import odmkv_b200`` / ``from odmkv_b200 import make_press``).
"""
from __future__ import annotations

import importlib
import sys

from . import _lib, codebook, ops  # noqa: F401
from ._lib import OdmkvError  # noqa: F401

_SUBMODULES = ["_lib", "codebook", "ops", "build", "tq_backend", "allocator", "scorer", "tq_adaptive_backend",
               "attention_patch", "packed_cache", "adaptive_backend_press", "press_factory", "dist"]

for _name in _SUBMODULES:
    try:
        _mod = importlib.import_module(f"{__name__}.{_name}")
    except ModuleNotFoundError as exc:  # a submodule that does not exist yet in a partial checkout
        if exc.name != f"{__name__}.{_name}":
            raise
        continue
    sys.modules.setdefault(f"odmkv_b200.{_name}", _mod)
sys.modules.setdefault("odmkv_b200", sys.modules[__name__])

for _exported in ("allocator", "scorer", "adaptive_backend_press", "press_factory", "tq_adaptive_backend", "packed_cache"):
    _m = sys.modules.get(f"odmkv_b200.{_exported}")
    if _m is not None:
        for _k in getattr(_m, "__all__", []):
            globals()[_k] = getattr(_m, _k)
