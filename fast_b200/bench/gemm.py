"""Grouped GEMM throughput: the tcgen05 kernel against torch.matmul (cuBLAS) per expert.

    python -m fast_b200.bench.gemm [--rows 65536] [--hidden 4096] [--inter 14336] [--experts 8]

CUDA-event timing after warm-up; operands (>= 1 GB) exceed the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import gemm


def _time(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--kernel", default="pair", choices=["pair", "one"])
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--direct-epilogue", action="store_true", help="CTA-pair kernel: row-per-thread global accesses in the epilogue instead of TMA stores")
    ap.add_argument("--band-rows", type=int, default=0, help="rows of a raster band (0 = kernel default)")
    ap.add_argument("--only", default="", help="comma-separated case names to run (default: all)")
    ap.add_argument("--sustain-s", type=float, default=0.0, help="also time back-to-back launches for this many seconds (power-capped regime)")
    a = ap.parse_args()
    gemm.USE_PAIR = a.kernel == "pair"
    gemm.DIRECT_EPILOGUE = a.direct_epilogue
    if a.band_rows:
        gemm.BAND_ROWS = a.band_rows
    G, H, I = a.experts, a.hidden, a.inter
    per = a.rows // G // 256 * 256
    R = per * G
    dev = "cuda"
    off = torch.arange(G + 1, device=dev, dtype=torch.int32) * per
    x = torch.randn(R, H, device=dev, dtype=torch.bfloat16)
    w13 = torch.randn(G, 2 * I, H, device=dev, dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(G, H, I, device=dev, dtype=torch.bfloat16) * 0.02
    act = torch.empty(R, I, device=dev, dtype=torch.bfloat16)
    gu = torch.empty(R, 2 * I, device=dev, dtype=torch.bfloat16)
    y = torch.empty(R, H, device=dev, dtype=torch.bfloat16)
    dact = torch.empty(R, I, device=dev, dtype=torch.bfloat16)
    dw2 = torch.empty_like(w2)
    dw13 = torch.empty_like(w13)
    dx = torch.empty(R, H, device=dev, dtype=torch.bfloat16)
    dgu = torch.empty(R, 2 * I, device=dev, dtype=torch.bfloat16)
    xq = xs = None
    if gemm.USE_PAIR and H % 128 == 0:
        grp = x.float().view(R, H // 128, 128)
        xs = (grp.abs().amax(-1).clamp_min(1e-12) / 448.0).contiguous()
        xs = ((xs.view(torch.int32) + 0xFFFF) & ~0xFFFF).view(torch.float32)  # bf16-representable scales, as the dispatch kernel sends them
        xq = (grp / xs.unsqueeze(-1)).to(torch.float8_e4m3fn).view(R, H).view(torch.uint8).contiguous()
        del grp
    rows_real = torch.full((G,), per, device=dev, dtype=torch.int32)
    cases = {
        **({"fwd_w13_swiglu_from_e4m3": (lambda: gemm.grouped_gemm_fwd(xq, w13, off, act, swiglu=True, a_scales=xs, group_rows=rows_real), 2 * R * H * 2 * I)} if xq is not None else {}),
        "fwd_w13_swiglu_act_only": (lambda: gemm.grouped_gemm_fwd(x, w13, off, act, swiglu=True), 2 * R * H * 2 * I),
        "fwd_w13_swiglu": (lambda: gemm.grouped_gemm_fwd(x, w13, off, act, swiglu=True, gate_up_out=gu), 2 * R * H * 2 * I),
        "fwd_w13_plain": (lambda: gemm.grouped_gemm_fwd(x, w13, off, gu), 2 * R * H * 2 * I),
        "fwd_w2": (lambda: gemm.grouped_gemm_fwd(act, w2, off, y), 2 * R * H * I),
        "dgrad_w2": (lambda: gemm.grouped_gemm_dgrad(y, w2, off, dact), 2 * R * H * I),
        **({"dgrad_w2_swiglu_bwd": (lambda: gemm.grouped_gemm_dgrad(y, w2, off, dgu, swiglu_bwd_of=gu), 2 * R * H * I)} if gemm.USE_PAIR else {}),
        "wgrad_w2": (lambda: gemm.grouped_gemm_wgrad(y, act, off, dw2), 2 * R * H * I),
        "dgrad_w13": (lambda: gemm.grouped_gemm_dgrad(gu, w13, off, dx), 2 * R * H * 2 * I),
        "wgrad_w13": (lambda: gemm.grouped_gemm_wgrad(gu, x, off, dw13), 2 * R * H * 2 * I),
    }
    if a.only:
        cases = {k: v for k, v in cases.items() if k in a.only.split(",")}
    out = {}
    for name, (fn, flops) in cases.items():
        if a.sustain_s > 0:
            break
        ms = _time(fn, a.iters)
        out[name] = {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1)}
    gemm.check()
    if a.sustain_s > 0:
        def sustained(fn, flops):
            ms1 = _time(fn, 3, 1)
            n = max(3, int(a.sustain_s * 1e3 / ms1))
            ms = _time(fn, n, 0)
            return {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1), "launches": n}
        for name, (fn, flops) in cases.items():
            out["sustained_" + name] = sustained(fn, flops)
        if not a.no_cublas:
            sl = lambda t, g: t[g * per:(g + 1) * per]
            cub = {
                "fwd_w13": (lambda: [torch.matmul(sl(x, g), w13[g].t(), out=sl(gu, g)) for g in range(G)], 2 * R * H * 2 * I),
                "fwd_w2": (lambda: [torch.matmul(sl(act, g), w2[g].t(), out=sl(y, g)) for g in range(G)], 2 * R * H * I),
                "dgrad_w2": (lambda: [torch.matmul(sl(y, g), w2[g], out=sl(dact, g)) for g in range(G)], 2 * R * H * I),
                "wgrad_w2": (lambda: [torch.matmul(sl(y, g).t(), sl(act, g), out=dw2[g]) for g in range(G)], 2 * R * H * I),
                "dgrad_w13": (lambda: [torch.matmul(sl(gu, g), w13[g], out=sl(dx, g)) for g in range(G)], 2 * R * H * 2 * I),
                "wgrad_w13": (lambda: [torch.matmul(sl(gu, g).t(), sl(x, g), out=dw13[g]) for g in range(G)], 2 * R * H * 2 * I),
            }
            for name, (fn, flops) in cub.items():
                out["sustained_cublas_" + name] = sustained(fn, flops)
            print(json.dumps({"kernel": a.kernel, "rows": R, "hidden": H, "inter": I, "experts": G, **out}))
            return
    if a.no_cublas:
        print(json.dumps({"kernel": a.kernel, "rows": R, "hidden": H, "inter": I, "experts": G, **out}))
        return
    # cuBLAS reference for the same math, expert by expert
    def cublas_fwd():
        for g in range(G):
            torch.matmul(x[g * per:(g + 1) * per], w13[g].t(), out=gu[g * per:(g + 1) * per])
    ms = _time(cublas_fwd, a.iters)
    out["cublas_fwd_w13"] = {"ms": round(ms, 3), "tflops": round(2 * R * H * 2 * I / ms / 1e9, 1)}
    def cublas_wgrad():
        for g in range(G):
            torch.matmul(gu[g * per:(g + 1) * per].t(), x[g * per:(g + 1) * per], out=dw13[g])
    ms = _time(cublas_wgrad, a.iters)
    out["cublas_wgrad_w13"] = {"ms": round(ms, 3), "tflops": round(2 * R * H * 2 * I / ms / 1e9, 1)}
    print(json.dumps({"kernel": a.kernel, "rows": R, "hidden": H, "inter": I, "experts": G, **out}))


if __name__ == "__main__":
    main()
