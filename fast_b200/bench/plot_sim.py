"""Plots of the simulator's JSON lines (needs matplotlib, which is optional):

    build/fastb-sim grid > grid.jsonl && python -m fast_b200.bench.plot_sim grid.jsonl out_dir

One figure per command found in the file: `grid` -> speed-up and scheduler-time heat maps over
servers x GPUs, `skew` / `size` / `fabric` / `topology` -> line charts. Counterpart of the reference's
simulation/plot/*.py.
"""
from __future__ import annotations

import json
import os
import sys
from collections import defaultdict


def load(path):
    rows = defaultdict(list)
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("{"):
                j = json.loads(line)
                rows[j.get("cmd", "?")].append(j)
    return rows


def series(rows, cmd):
    """(x label, {series name: [(x, y), ...]}) for the line-chart commands."""
    r = rows[cmd]
    if cmd == "skew":
        return "Zipf skew", {"speed-up": [(j["skew"], j["speedup"]) for j in r]}
    if cmd == "size":
        return "MB per unit", {k: [(j["mb_per_unit"], j[k]) for j in r] for k in ("no_scale", "alpha_beta_scale", "always_scale")}
    if cmd == "fabric":
        return "intra-server Tb/s", {"speed-up": [(j["intra_tbps"], j["speedup"]) for j in r], "exposed intra share": [(j["intra_tbps"], j["exposed_intra_share"]) for j in r]}
    if cmd == "topology":
        out = defaultdict(list)
        for j in r:
            out[j["fabric"]].append((j["servers"], j["speedup"]))
        return "servers", dict(out)
    raise KeyError(cmd)


def main(argv):
    if len(argv) < 3:
        print(__doc__)
        return 2
    rows = load(argv[1])
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        print("matplotlib is not installed; parsed commands:", {k: len(v) for k, v in rows.items()})
        return 1
    os.makedirs(argv[2], exist_ok=True)
    if rows.get("grid"):
        S = sorted({j["servers"] for j in rows["grid"]})
        G = sorted({j["gpus"] for j in rows["grid"]})
        for key in ("speedup", "scheduler_ms"):
            z = [[next((j[key] for j in rows["grid"] if j["servers"] == s and j["gpus"] == g), float("nan")) for g in G] for s in S]
            fig, ax = plt.subplots()
            im = ax.imshow(z, aspect="auto")
            ax.set_xticks(range(len(G)), G)
            ax.set_yticks(range(len(S)), S)
            ax.set_xlabel("GPUs per server")
            ax.set_ylabel("servers")
            fig.colorbar(im, label=key)
            fig.savefig(os.path.join(argv[2], f"grid_{key}.png"), dpi=150)
    for cmd in ("skew", "size", "fabric", "topology"):
        if not rows.get(cmd):
            continue
        xlabel, ser = series(rows, cmd)
        fig, ax = plt.subplots()
        for name, pts in ser.items():
            ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=name)
        if cmd in ("size",):
            ax.set_xscale("log")
        ax.set_xlabel(xlabel)
        ax.legend()
        fig.savefig(os.path.join(argv[2], f"{cmd}.png"), dpi=150)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
