"""Run-time switches, all read from the environment once at import.

The reference has no run-time configuration (compile-time #defines in
nvidia/src/include/fast_alltoall/alltoall_define.h:21-80 and hard-coded experiment parameters);
these are the knobs of this implementation:

  FASTB_GEMM=pair|one     grouped GEMM kernel: CTA pairs (cta_group::2, default) or one CTA per tile
  FASTB_BAND=<rows>       rows of a GEMM raster band (0 = kernel default 4096)
  FASTB_NVTX=1            NVTX ranges around the phases of the expert-parallel engine
  FASTB_TIMEOUT_S=<sec>   default limit of device-side waits for new communicators (default 5)
  FASTB_LOG=1             one line per scheduled collective (stages, ops, modeled time) on rank 0
  FASTB_CHECK_SYMM=1      every symmetric allocation is compared across ranks (one host collective each)
  FASTB_A2A_BULK=1        all-to-all(v) kernel moves 16-byte aligned pieces with bulk copies through shared memory
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class Config:
    gemm: str = os.environ.get("FASTB_GEMM", "pair")
    band_rows: int = int(os.environ.get("FASTB_BAND", "0"))
    nvtx: bool = os.environ.get("FASTB_NVTX", "0") == "1"
    timeout_s: float = float(os.environ.get("FASTB_TIMEOUT_S", "5"))
    log: bool = os.environ.get("FASTB_LOG", "0") == "1"
    check_symm: bool = os.environ.get("FASTB_CHECK_SYMM", "0") == "1"
    a2a_bulk: bool = os.environ.get("FASTB_A2A_BULK", "0") == "1"


CONFIG = Config()


class nvtx_range:
    """``with nvtx_range("dispatch"):`` — a no-op unless FASTB_NVTX=1."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if CONFIG.nvtx:
            import torch

            torch.cuda.nvtx.range_push("fastb:" + self.name)

    def __exit__(self, *exc):
        if CONFIG.nvtx:
            import torch

            torch.cuda.nvtx.range_pop()
        return False
