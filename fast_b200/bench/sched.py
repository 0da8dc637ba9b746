"""Host scheduler timing on CPU: decomposition and whole-plan time per topology, next to the
reference's own simulator when it has been built (baseline/build_ref_sim.sh).

    python -m fast_b200.bench.sched [--servers 8 16 32 64] [--gpus 8] [--seed 3] [--out rows.jsonl]

One JSON row per topology: stages, ops, pad + decompose time, whole-plan time, validation time,
and the reference simulator's stage count and pad + decompose time on the same matrix.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import time

import numpy as np

from .. import sched
from ..sched import Topology
from ..utils.results import ResultLog

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def reference_row(m: np.ndarray, S: int, G: int):
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_sim")
    if not os.path.exists(exe):
        return None
    text = f"{S} {G} 0.7 22 0.1 2.3 1e-3\n" + " ".join(str(int(x)) for x in m.reshape(-1))
    out = subprocess.run([exe], input=text, capture_output=True, text=True, check=True).stdout
    return json.loads(out.strip().splitlines()[-1])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--servers", type=int, nargs="+", default=[8, 16, 32, 64])
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--seed", type=int, default=3)
    ap.add_argument("--max-entry", type=int, default=10000)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    log = ResultLog(a.out or None, "sched")
    for S in a.servers:
        G = a.gpus
        m = sched.workload_uniform(S * G, a.max_entry, a.seed, False)
        t = time.perf_counter()
        p = sched.build_plan(m, Topology(S, G))
        plan_ms = (time.perf_counter() - t) * 1e3
        t = time.perf_counter()
        err = p.validate()
        validate_ms = (time.perf_counter() - t) * 1e3
        sm = np.ascontiguousarray(p.server_matrix)
        reps = 20 if S <= 16 else 3
        dec_us = min(sched.decompose_time_us(sm, reps=reps) for _ in range(3))
        row = {"servers": S, "gpus": G, "stages": int(p.num_stages), "ops": int(p.num_ops), "valid": err == "",
               "decompose_us": round(dec_us, 1), "plan_ms": round(plan_ms, 2), "validate_ms": round(validate_ms, 2)}
        ref = reference_row(m, S, G)
        if ref is not None:
            row.update({"ref_stages": ref["stages"], "ref_decompose_us": round(ref["decompose_us"], 1), "ref_exact": ref["exact"]})
        print(json.dumps(row), flush=True)
        log.add(row)


if __name__ == "__main__":
    main()
