"""Loader of the native CUDA extension (``fast_b200._C``).

On a machine with a GPU a missing or stale extension is an error, never a silent fallback: the
kernels are the product. Without a GPU (build box, CPU tests) ``ext()`` still imports the
extension if it was built, and ``available()`` tells whether kernels can actually launch.
"""
from __future__ import annotations

import importlib

import torch

_EXT = None


def ext():
    global _EXT
    if _EXT is None:
        try:
            _EXT = importlib.import_module("fast_b200._C")
        except ImportError as e:
            from . import _build

            try:
                _build.build_cuda()
                _EXT = importlib.import_module("fast_b200._C")
            except Exception as e2:  # pragma: no cover - build environment problem
                raise RuntimeError(f"fast_b200._C is not built and could not be built here: {e2}") from e
    return _EXT


def available() -> bool:
    return torch.cuda.is_available()


SITE_NAMES = {1: "entry-ready", 2: "balance-arrival", 3: "rail-arrival", 4: "output-arrival", 5: "counts-arrival",
              6: "combine-ready", 7: "buffer-reuse", 8: "mbarrier", 9: "test-probe", 10: "receive-capacity", 11: "expert-id"}


class CollectiveTimeout(RuntimeError):
    """A device-side wait ran out of time; carries where and what it was waiting for."""

    def __init__(self, code, site, detail, seen, want):
        self.code, self.site, self.detail, self.seen, self.want = code, site, detail, seen, want
        if site == 10:
            super().__init__(f"MoE step refused: a rank needs {seen} receive rows but capacity_rows is {want}")
        elif site == 11:
            super().__init__(f"MoE step refused: routing entry {detail} names expert {seen if seen < 2**31 else seen - 2**32}, outside 0..{want - 1}")
        else:
            super().__init__(f"device wait gave up at {SITE_NAMES.get(site, site)} (detail {detail}): saw {seen}, wanted {want}")
