"""Named model configurations and a per-GPU memory / FLOP plan for them.

The reference ships no model (it is the transport under expert parallelism); the two shapes its
successor is measured on are kept here so that benchmarks, tests and users name them once:
a Mixtral-8x7B-shaped MoE block (training) and a DeepSeek-V3-like routed-expert layer (forward,
fp8 dispatch). ``memory_plan`` mirrors the allocations of ``ExpertParallel`` and ``MoELayer`` /
``FusedAdamW`` so that shards can be sized for a 180 GB GPU before anything is allocated.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict

HBM_BYTES = 180 * 10**9   # B200: 180 GB HBM3e per GPU


@dataclass(frozen=True)
class MoEConfig:
    name: str
    hidden: int
    inter: int                 # FFN width of one expert (SwiGLU: gate and up are each this wide)
    num_experts: int
    top_k: int
    tokens_per_rank: int
    fp8_dispatch: bool = False
    training: bool = True
    vocab: int = 0             # > 0: the block has a token embedding (and its gradient)

    def with_(self, **kw) -> "MoEConfig":
        return replace(self, **kw)

    def experts_per_rank(self, world: int) -> int:
        if self.num_experts % world:
            raise ValueError(f"{self.num_experts} experts do not divide over {world} ranks")
        return self.num_experts // world

    def capacity_rows(self, world: int, capacity_factor: float = 0.0) -> int:
        """Receive rows per rank: the worst case (every token of every rank picks only local experts),
        or ``capacity_factor x tokens x top_k`` when that is smaller; padded as the engine pads it."""
        el = self.experts_per_rank(world)
        worst = world * self.tokens_per_rank * min(self.top_k, el) + 256 * el
        cap = worst if capacity_factor <= 0 else min(worst, int(capacity_factor * self.tokens_per_rank * self.top_k) + 256 * el)
        return (cap + 255) // 256 * 256


MIXTRAL_8X7B_BLOCK = MoEConfig("mixtral-8x7b-block", hidden=4096, inter=14336, num_experts=8, top_k=2, tokens_per_rank=8 * 4096,
                               training=True, vocab=32000)
DEEPSEEK_V3_MOE_LAYER = MoEConfig("deepseek-v3-moe-layer", hidden=7168, inter=2048, num_experts=256, top_k=8, tokens_per_rank=4096,
                                  fp8_dispatch=True, training=False)
CONFIGS: Dict[str, MoEConfig] = {c.name: c for c in (MIXTRAL_8X7B_BLOCK, DEEPSEEK_V3_MOE_LAYER)}


def memory_plan(cfg: MoEConfig, world: int, capacity_factor: float = 0.0) -> Dict[str, int]:
    """Bytes per GPU by category, their total and whether it fits one B200.

    ``symmetric_heap``: receive / return rows that peers write or read (x, y and, in training,
    dy and dx; fp8 rows carry one fp32 scale per 128 values). ``workspace``: local expert
    activations (act; in training also gate|up, d(act), d(gate|up)). ``weights``: bf16 expert
    weights of this rank plus the replicated router (and embedding). ``grads`` and ``optimizer``:
    bf16 gradients and AdamW's fp32 master copy and two moments. ``tokens``: the layer's input,
    output and routing tensors for ``tokens_per_rank`` tokens."""
    H, I, K, T = cfg.hidden, cfg.inter, cfg.top_k, cfg.tokens_per_rank
    el, cap = cfg.experts_per_rank(world), cfg.capacity_rows(world, capacity_factor)
    row = cap * H
    x_recv_symm = row + cap * (H // 128) * 4 if cfg.fp8_dispatch else 2 * row
    symmetric = x_recv_symm + 2 * row + (2 * 2 * row if cfg.training else 0)
    workspace = 2 * cap * I + (2 * row if cfg.fp8_dispatch else 0)
    if cfg.training:
        workspace += 2 * cap * (2 * I + I + 2 * I)
    params = el * 3 * H * I + H * cfg.num_experts + cfg.vocab * H
    weights = 2 * params
    grads = 2 * params if cfg.training else 0
    optimizer = 12 * params if cfg.training else 0
    tokens = T * H * 2 * (4 if cfg.training else 2) + T * cfg.num_experts * 4 + T * K * 12
    total = symmetric + workspace + weights + grads + optimizer + tokens
    return {"capacity_rows": cap, "symmetric_heap": symmetric, "workspace": workspace, "weights": weights, "grads": grads,
            "optimizer": optimizer, "tokens": tokens, "total": total, "fits_b200": total <= int(0.92 * HBM_BYTES)}


def max_tokens_per_rank(cfg: MoEConfig, world: int, capacity_factor: float = 0.0, quantum: int = 1024) -> int:
    """Largest ``tokens_per_rank`` (multiple of ``quantum``) whose plan still fits one GPU."""
    lo, hi = 0, 1
    while memory_plan(cfg.with_(tokens_per_rank=hi * quantum), world, capacity_factor)["fits_b200"] and hi < (1 << 20):
        lo, hi = hi, hi * 2
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if memory_plan(cfg.with_(tokens_per_rank=mid * quantum), world, capacity_factor)["fits_b200"]:
            lo = mid
        else:
            hi = mid
    return lo * quantum


def flops_per_step(cfg: MoEConfig, world: int) -> Dict[str, float]:
    """Tensor-core FLOPs per rank and step, for balanced routing (each rank receives
    ``tokens_per_rank x top_k`` rows): three GEMMs forward (gate, up, down), and in training the
    same again twice for data and weight gradients."""
    rows = cfg.tokens_per_rank * cfg.top_k
    fwd = 2.0 * rows * cfg.hidden * cfg.inter * 3
    total = fwd * (3 if cfg.training else 1)
    router = 2.0 * cfg.tokens_per_rank * cfg.hidden * cfg.num_experts * (3 if cfg.training else 1)
    return {"expert_gemm_fwd": fwd, "expert_gemm_total": total, "router": router, "total": total + router}


def step_roofline(cfg: MoEConfig, world: int, bf16_tflops: float, hbm_gbs: float, nvlink_gbs: float = 770.0) -> Dict[str, float]:
    """Lower bound of one step on one GPU, in ms, from the measured peaks: tensor-core time of the
    expert GEMMs, memory time of the passes that must stream HBM once (optimizer state, saved
    activations that do not fit on chip) and NVLink time of the all-to-alls (balanced routing).
    The phases overlap little in this design (GEMMs, then optimizer), so the bound is their sum."""
    f = flops_per_step(cfg, world)
    el = cfg.experts_per_rank(world)
    rows = cfg.tokens_per_rank * cfg.top_k
    params = el * 3 * cfg.hidden * cfg.inter
    gemm_ms = f["expert_gemm_total"] / (bf16_tflops * 1e12) * 1e3
    # AdamW: bf16 grad + bf16 weight (read, write) + fp32 master, m, v (read, write) = 2 + 4 + 24 bytes per parameter
    adamw_ms = (params * 28 / (hbm_gbs * 1e9) * 1e3) if cfg.training else 0.0
    # rows that leave the GPU: dispatch + combine (and their transposes in training), (world - 1) / world of them
    row_bytes = cfg.hidden * (1 if cfg.fp8_dispatch else 2)
    off_gpu = rows * (world - 1) / max(world, 1)
    a2a_bytes = off_gpu * (row_bytes + cfg.hidden * 2) * (2 if cfg.training else 1)
    a2a_ms = a2a_bytes / (nvlink_gbs * 1e9) * 1e3
    return {"gemm_ms": gemm_ms, "adamw_ms": adamw_ms, "a2a_ms": a2a_ms, "total_ms": gemm_ms + adamw_ms + a2a_ms}
