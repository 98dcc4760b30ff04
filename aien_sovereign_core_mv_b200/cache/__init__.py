"""The cache manager's Python face.

The manager itself is C++ (``csrc/host/cache_manager.{h,cpp}``: pages, block tables per layer
group, reference counts, copy-on-write fork, truncate, state slots) and is compiled at first
use; the names here load it on demand, so importing the package compiles nothing.
"""
from __future__ import annotations

_NAMES = ("CacheManager", "GroupSpec", "GroupKind", "CacheExhausted", "EXHAUSTED_PREFIX")


def __getattr__(name):
    if name in _NAMES:
        from ..csrc import build
        return getattr(build.load_host(), name)
    raise AttributeError(name)


__all__ = list(_NAMES)
