"""Grouped bf16 GEMMs of the expert MLP on the tcgen05 kernel (forward, dgrad, wgrad).

Rows of all groups live in one matrix; ``group_off`` (int32[G+1], device) gives each group's row
range and every offset is a multiple of 128, so tiles never straddle two groups and the rows
between a group's real end and its padded end are zero.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime
from ..utils.config import CONFIG

FORWARD, DGRAD, WGRAD = 0, 1, 2
STORE, SWIGLU, SWIGLU_BWD = 0, 1, 2
_BM, _BN, _BK = 128, 256, 64
# CTA-pair kernel (256 x 256 tiles, cta_group::2); set False to fall back to the one-CTA kernel.
USE_PAIR = CONFIG.gemm != "one"
# Rows of a raster band (see csrc/kernels/gemm_common.cuh); 0 = kernel default.
BAND_ROWS = CONFIG.band_rows
# CTA-pair kernel: True = epilogue threads write global memory row by row; False = staged tiles + TMA stores.
DIRECT_EPILOGUE = False


def row_align() -> int:
    """Rows every group must be padded to for the kernel in use."""
    return 256 if USE_PAIR else 128


_status = None
_maps: dict = {}


def _st():
    global _status
    if _status is None:
        _status = runtime.ext().StatusBlock()
    return _status


def check() -> None:
    """Raise if a GEMM launched through this module gave up on an mbarrier wait."""
    code, site, detail, seen, want = _st().read()
    if code:
        raise runtime.CollectiveTimeout(code, site, detail, seen, want)


def _tmap(t: torch.Tensor, box_rows: int):
    assert t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
    m = _maps.get(key)
    if m is None:
        if len(_maps) > 4096:
            _maps.clear()
        m = runtime.ext().TensorMap2D(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), 64, box_rows)
        _maps[key] = m
    return m


def _out_maps(c: torch.Tensor, c2: Optional[torch.Tensor]):
    """Tensor maps of the outputs for the CTA-pair kernel's TMA stores (boxes of 64 columns x 128 rows)."""
    if not USE_PAIR:
        return None, None
    return _tmap(c, _BM), (_tmap(c2, _BM) if c2 is not None else None)


def _ctas() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def pad_group_offsets(counts: torch.Tensor) -> torch.Tensor:
    """int32[G+1] offsets with every group rounded up to row_align() rows (host/torch helper for tests)."""
    ra = row_align()
    padded = (counts.to(torch.int64) + ra - 1) // ra * ra
    off = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    off[1:] = torch.cumsum(padded, 0)
    return off.to(torch.int32)


def _tmap_bytes(t: torch.Tensor, box_rows: int):
    assert t.dtype == torch.uint8 and t.dim() == 2 and t.stride(1) == 1
    key = (t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows, "u8")
    m = _maps.get(key)
    if m is None:
        m = runtime.ext().TensorMap2D.bytes(t.data_ptr(), t.shape[0], t.shape[1], t.stride(0), box_rows)
        _maps[key] = m
    return m


def grouped_gemm_fwd(a: torch.Tensor, w: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor, swiglu: bool = False,
                     gate_up_out: Optional[torch.Tensor] = None, timeout_s: float = 5.0, gate=None, a_scales: Optional[torch.Tensor] = None,
                     group_rows: Optional[torch.Tensor] = None, gate_tile_rows: int = 0, ctas: Optional[int] = None) -> torch.Tensor:
    """out[rows of g] = a[rows of g] @ w[g].T  (a [R, K], w [G, N, K], out [R, N]).

    With ``swiglu`` the N columns of every 256-wide tile are [128 gate | 128 up] of the same 128
    features and ``out`` is [R, N/2] = silu(gate) * up; ``gate_up_out`` ([R, N]) optionally keeps
    the raw tile for the backward pass. ``gate=(counter_ptr, target)`` makes the TMA producer
    wait, group by group, until ``counter[g] >= target[g]`` (rows pushed by peers have landed);
    with ``gate_tile_rows`` > 0 the counters are per tile of that many rows of ``a`` instead of per
    group, so a tile is loaded as soon as its own rows are in.

    ``a`` may be uint8 e4m3 rows with ``a_scales`` (float [R, K/128], one scale per 128 elements):
    the CTA-pair kernel then converts them to bf16 tiles in shared memory on the way to the tensor
    core (no dequantised copy of ``a`` exists in global memory). ``group_rows`` (int32[G], real rows
    per group) makes that path treat the rows between a group's real and padded end as zeros.
    """
    G, N, K = w.shape
    assert a.shape[1] == K and K % _BK == 0 and N % _BN == 0 and a.shape[0] % _BM == 0
    assert out.shape[0] == a.shape[0] and out.shape[1] == (N // 2 if swiglu else N)
    C = runtime.ext()
    map_b = _tmap(w.view(G * N, K), 128 if USE_PAIR else _BN)
    if a.dtype == torch.uint8:
        assert USE_PAIR and a_scales is not None and K % 128 == 0 and a.is_contiguous(), "e4m3 operand: CTA-pair kernel, scales given, K a multiple of 128"
        map_a = _tmap_bytes(a, _BM)
    else:
        assert a_scales is None
        map_a = _tmap(a, _BM)
    C.grouped_gemm(FORWARD, SWIGLU if swiglu else STORE, map_a, map_b, group_off, N // _BN, 0, K, N,
                   0, out, gate_up_out, _st().ptr(), int(timeout_s * 1e9), min(ctas or _ctas(), _ctas()), *(gate or (0, None)), USE_PAIR, BAND_ROWS,
                   *_out_maps(out, gate_up_out), DIRECT_EPILOGUE and a_scales is None, a_scales, group_rows, gate_tile_rows)
    return out


def grouped_gemm_dgrad(dy: torch.Tensor, w: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor, timeout_s: float = 5.0, gate=None,
                       swiglu_bwd_of: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[rows of g] = dy[rows of g] @ w[g]  (dy [R, N], w [G, N, K], out [R, K]).

    With ``swiglu_bwd_of`` (the saved gate|up tiles [R, 2K]) the product is taken as d(act) and the
    epilogue writes d(gate|up) [R, 2K] into ``out`` instead (CTA-pair kernel only): the SwiGLU
    backward costs no extra pass over memory.
    """
    G, N, K = w.shape
    assert dy.shape[1] == N and N % _BK == 0 and K % _BN == 0 and dy.shape[0] % _BM == 0
    C = runtime.ext()
    if swiglu_bwd_of is not None:
        assert USE_PAIR and out.shape[1] == 2 * K and swiglu_bwd_of.shape == out.shape
        C.grouped_gemm(DGRAD, SWIGLU_BWD, _tmap(dy, _BM), _tmap(w.view(G * N, K), _BK), group_off, K // _BN, 0, N, N, 0, out, swiglu_bwd_of,
                       _st().ptr(), int(timeout_s * 1e9), _ctas(), *(gate or (0, None)), USE_PAIR, BAND_ROWS, *_out_maps(out, swiglu_bwd_of), DIRECT_EPILOGUE)
        return out
    C.grouped_gemm(DGRAD, STORE, _tmap(dy, _BM), _tmap(w.view(G * N, K), _BK), group_off, K // _BN, 0, N, N, 0, out, None, _st().ptr(),
                   int(timeout_s * 1e9), _ctas(), *(gate or (0, None)), USE_PAIR, BAND_ROWS, *_out_maps(out, None), DIRECT_EPILOGUE)
    return out


def grouped_gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor, timeout_s: float = 5.0) -> torch.Tensor:
    """out[g] = dy[rows of g].T @ x[rows of g]  (dy [R, N], x [R, K], out [G, N, K]). Rows between a
    group's real end and its padded end must be zero in at least one operand and finite in both."""
    G, N, K = out.shape
    bm = 256 if USE_PAIR else _BM
    assert dy.shape[1] == N and x.shape[1] == K and N % bm == 0 and K % _BN == 0
    C = runtime.ext()
    C.grouped_gemm(WGRAD, STORE, _tmap(dy, _BK), _tmap(x, _BK), group_off, K // _BN, N // bm, 0, 0, N, out.view(G * N, K), None, _st().ptr(),
                   int(timeout_s * 1e9), _ctas(), 0, None, USE_PAIR, BAND_ROWS, *_out_maps(out.view(G * N, K), None), DIRECT_EPILOGUE)
    return out
