"""Flagship benchmark: Mixtral-8x7B-shaped MoE block training step, expert-parallel over N B200s.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Per rank: 8 sequences x 4096 random token ids (vocab 32000) -> embedding -> RMSNorm -> top-2 of 8
SwiGLU experts (hidden 4096, FFN 14336; 8/N experts per rank) with fused dispatch/combine ->
residual -> mean-square loss; backward through the transposed all-to-all; AdamW step on every
parameter. bf16 compute, fp32 accumulation / master weights. Weak scaling: per-GPU tokens fixed.

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events, max over ranks) with the
step's inputs already on the device; `e2e.value` times the same step through the public API with
the token ids copied from pinned host memory and the loss read back every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEQS, SEQ_LEN, VOCAB, HIDDEN, FFN, EXPERTS, TOP_K = 8, 4096, 32000, 4096, 14336, 8, 2


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.t_begin, self.t_end = 0.0, float("inf")

    def window_begin(self):
        self.t_begin = time.monotonic()

    def window_end(self):
        self.t_end = time.monotonic()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, pw = [], [], set(), []
        inside = [r for t, r in self.rows if self.t_begin <= t <= self.t_end + 0.15]
        for r in inside or [r for _, r in self.rows[-3:]]:  # nvidia-smi can start slowly: fall back to the latest samples
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); pw.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


REF_NO_HEADLINE = ("the reference (MangoBoost/FAST) has no MoE layer, GEMM or training step, so the headline metric cannot be run on it; its root has no "
                   "setup.py/pyproject (the offline pip install fails) and its NVIDIA library, built for sm_100a from the unmodified sources by "
                   "baseline/build_ref_nvshmem.sh, exports only all-to-all self-tests on a self-generated workload")


def reference_arm(args):
    """Runs the UNMODIFIED reference library (baseline/_ref/nv_build/libflash.so) through its own stock
    path, ``flash_comm_t.test_flash_alltoall()`` (nvidia/alltoall_nvshmem.cpp:563-601): one process per
    GPU, every GPU a server of its own, the reference's own workload generator, warm-up and timing.
    The training headline has no counterpart there, so the line keeps ``unavailable`` for it and
    carries the reference's all-to-all(v) result in ``alltoallv_reference_workload``; the same key of
    the other arm is this runtime on the identical matrix. With one GPU the reference's scheduler is a
    no-op and its tester would dereference a null scheduler (:551, :576), so nothing is run."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    n = args.gpus
    out = {"impl": "reference", "unavailable": REF_NO_HEADLINE, "n_gpus": n}
    lib = os.path.join(ROOT, "baseline", "_ref", "nv_build", "libflash.so")
    if n < 2:
        out["alltoallv_reference_workload"] = None
        out["unavailable"] += "; on one GPU its scheduler does nothing and test_flash_alltoall would dereference a null scheduler"
    elif not os.path.exists(lib):
        out["alltoallv_reference_workload"] = None
        out["unavailable"] += "; baseline/_ref/nv_build/libflash.so is not built on this machine"
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import run_ref_flash as ref

        port = int(os.environ.get("MASTER_PORT", "29500")) + 17      # the launcher's own store keeps MASTER_PORT
        if world == n:                                                 # one process per GPU already: this process runs its rank
            results = [ref.spawn_rank(rank, n, "flash", port, args.ref_timeout)]
        else:                                                          # plain launch: start every rank from here
            from concurrent.futures import ThreadPoolExecutor

            with ThreadPoolExecutor(max_workers=n) as ex:
                results = list(ex.map(lambda r: ref.spawn_rank(r, n, "flash", port, args.ref_timeout), range(n)))
        rc = max(code for code, _ in results)
        text = "".join(o for _, o in results)
        if rank == 0:
            res = ref.parse(text)
            if rc == 0 and "algbw_GBps" in res:
                res.update(workload="uniform_distribution(2**23) x 8-byte units (nvidia/alltoall_nvshmem.cpp:565-569)", warmup=50, iters=50,
                           servers=n, gpus_per_server=1, timing="the reference's own CUDA events (perf_flash)")
                out["alltoallv_reference_workload"] = res
            else:
                out["alltoallv_reference_workload"] = None
                out["unavailable"] += f"; its test_flash_alltoall run ended with code {rc}" + (" (stopped at the timeout)" if rc == 124 else "")
                out["reference_output_tail"] = text[-1500:]
    if rank == 0:  # one line per job, also when launched with one process per GPU
        print(json.dumps(out), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-timeout", type=float, default=420.0, help="--impl reference: seconds before the reference's processes are stopped")
    ap.add_argument("--seqs", type=int, default=SEQS)
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--hidden", type=int, default=HIDDEN, help="model width (default: the benchmark's 4096; smaller only for profiling runs)")
    ap.add_argument("--ffn", type=int, default=FFN, help="expert FFN width (default: the benchmark's 14336)")
    ap.add_argument("--capacity-factor", type=float, default=0.0, help="receive rows per rank as a multiple of tokens*top_k (0 = worst case)")
    ap.add_argument("--early-step", action="store_true", help="apply W2's AdamW update inside the backward pass on a side stream (measured neutral under the 1000 W cap)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the torch + NCCL arm of the same step (vs_baseline becomes null)")
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-metrics measured after the training benchmark (skewed all-to-all(v) vs NCCL when N > 1; MoE forward dispatch+combine)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from fast_b200 import runtime
    from fast_b200.models import MixtralBlockModel
    from fast_b200.parallel import Communicator
    from fast_b200.utils import FusedAdamW

    C = runtime.ext()
    tokens = args.seqs * args.seq_len
    El = EXPERTS // world
    worst = world * tokens * min(TOP_K, El) + 256 * El  # every expert's rows are padded to 256
    cap = worst if args.capacity_factor <= 0 else min(worst, int(args.capacity_factor * tokens * TOP_K) + 256 * El)
    heap = 4 * cap * args.hidden * 2 + (256 << 20) + (0 if world == 1 or args.no_extras else (1100 << 20))
    comm = Communicator(heap_bytes=heap, device=local, timeout_s=20.0)
    model = MixtralBlockModel(comm, vocab=VOCAB, hidden=args.hidden, inter=args.ffn, num_experts=EXPERTS, top_k=TOP_K, max_tokens=tokens, capacity_rows=cap)
    opt_experts = FusedAdamW(model.expert_parameters(), lr=1e-4, weight_decay=0.01)
    opt_repl = FusedAdamW(model.replicated_parameters(), lr=1e-4, weight_decay=0.0)
    if args.early_step:
        model.moe.attach_optimizer(opt_experts)  # W2's AdamW update overlaps the W13 backward GEMMs

    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = 4
    host_ids = [torch.randint(0, VOCAB, (args.seqs, args.seq_len), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_ids = [h.cuda() for h in host_ids]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def train_step(ids):
        opt_experts.zero_grad()
        opt_repl.zero_grad()
        loss = model(ids)
        loss.backward()
        works = []
        if world > 1:  # replicated parameters: average gradients over the data-parallel ranks
            # NCCL's stream picks the gradients up once the backward pass is done; the experts' AdamW
            # (the rank's own shard, nothing to reduce) streams through HBM meanwhile.
            works = [dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, async_op=True) for p in model.replicated_parameters()]
        opt_experts.step()
        for w in works:
            w.wait()
        opt_repl.step()
        return loss

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()  # started before the warm-up so that it is already streaming when the timed region begins
    for i in range(warmup):
        train_step(dev_ids[i % n_batches])
    comm.check()

    # ---- device-timed: K steps, CUDA events, max over ranks ------------------------------------
    fence()
    sampler.window_begin()
    launches0 = C.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        train_step(dev_ids[i % n_batches])
    e1.record()
    fence()
    sampler.window_end()
    launches = C.launch_count() - launches0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    # ---- end to end: pinned host ids -> H2D every step, loss -> D2H every step -----------------
    fence()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        ids = host_ids[i % n_batches].cuda(non_blocking=True)
        loss = train_step(ids)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        last = float(loss_host[0])
    fence()
    e2e_s = time.perf_counter() - t0
    comm.check()

    # ---- collective sub-metric (N > 1): skewed all-to-all(v), this runtime vs NCCL on the same ranks ----
    a2av = None
    if world > 1 and not args.no_extras:
        from fast_b200.bench.a2a import skewed_point

        a2av = skewed_point(comm, 256 << 20, 1.0, matrices=3, iters=5, warmup=3)
        a2av["speedup_vs_nccl"] = round(a2av["nccl_alltoallv"]["ms"] / min(a2av["ours_fanout"]["ms"], a2av["ours_staged"]["ms"]), 3)

    # ---- the reference's own tester workload (its rand() matrix, 8-byte units) on this runtime: the other arm's key of the same name ----
    ref_wl = None
    if world > 1 and not args.no_extras:
        from fast_b200.compat import FlashComm
        from fast_b200.sched import PlanKind

        fc = FlashComm(rank, world, world, comm=comm, generator="glibc", quiet=True)
        staged = fc.test_flash_alltoall(warmup=20, iters=50)
        fanout = fc._run(PlanKind.FANOUT, 8, 20, 50, "fanout")
        best = min(staged, fanout, key=lambda r: r["time_ms"])
        ref_wl = {"algbw_GBps": round(best["algbw_GBps"], 2), "time_ms": round(best["time_ms"], 4), "per_gpu_MB": round(best["per_gpu_MB"], 3),
                  "verified": staged["verified"] and fanout["verified"], "staged_ms": round(staged["time_ms"], 4), "fanout_ms": round(fanout["time_ms"], 4),
                  "workload": "uniform_distribution(2**23) x 8-byte units, the reference tester's matrix (nvidia/alltoall_nvshmem.cpp:565-569)",
                  "warmup": 20, "iters": 50, "timing": "CUDA events around 50 collectives, max over ranks"}

    # ---- library arm of the same training step: torch ops (cuBLAS) + NCCL all-to-all + torch AdamW, same data, same process ----
    del model, opt_experts, opt_repl
    torch.cuda.empty_cache()
    baseline = None
    if not args.no_baseline:
        from fast_b200.bench import torch_block

        baseline = torch_block.measure(dev_ids, steps=min(args.steps, 5), warmup=3, hidden=args.hidden, inter=args.ffn, num_experts=EXPERTS, top_k=TOP_K, vocab=VOCAB)

    # ---- MoE forward sub-metric: dispatch + combine latency on DeepSeek-V3-like shapes, fp8 dispatch ----
    moe_fwd = None
    if not args.no_extras:
        from fast_b200.bench import moe_fwd as mf

        comm2 = Communicator(heap_bytes=mf.heap_bytes_needed(world, 4096, 7168, 8, 32, True), device=local, timeout_s=20.0)
        moe_fwd = mf.measure(comm2, fp8=True, iters=10, warmup=3, skip_nccl=True)

    t = torch.tensor([ms, e2e_s * 1e3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    total_tokens = tokens * world * args.steps
    value = total_tokens / (ms * 1e-3)
    if rank == 0:
        out = {
            "metric": "moe_block_train_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / baseline["tokens_per_s"], 3) if baseline else None,
            "dtype": "bf16", "data": "synthetic (seeded random token ids, random-init weights)",
            "config": {"model": f"Mixtral-8x7B-shaped MoE block (hidden {args.hidden}, FFN {args.ffn} SwiGLU, 8 experts, top-2)", "global_batch": args.seqs * world,
                       "seq_len": args.seq_len, "parallelism": f"ep{world}", "tokens_per_gpu": tokens,
                       "baseline_config": "BASELINE.json configs[4] (Mixtral-8x7B-shaped MoE block training step, tokens/s at 1/2/4/8 B200); the headline "
                                          "collective metrics of configs[2] and configs[3] are the sub-metrics alltoallv_skewed and moe_forward_fp8_dispatch", "capacity_rows": cap,
                       "l2": "per-step working set (weights 2.8 GB/GPU at N=1, activations > 10 GB) far exceeds the 126 MB L2; no flush needed",
                       "optimizer": "AdamW, fp32 master weights, in the timed step", "timing": "CUDA events around K steps, max over ranks"},
            "clocks": clocks,
            "e2e": {"value": round(total_tokens / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms / args.steps, 3),
                    "h2d_bytes_per_step": host_ids[0].numel() * host_ids[0].element_size(), "d2h_bytes_per_step": 4, "last_loss": last},
            "baseline": baseline,
            "alltoallv_skewed": a2av,
            "alltoallv_reference_workload": ref_wl,
            "moe_forward_fp8_dispatch": moe_fwd,
            "gpu_launches": int(launches),
            "gpu_launches_per_step": launches / max(args.steps, 1),
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
