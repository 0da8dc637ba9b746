from .moe import MoELayer, MixtralBlockModel, reference_moe  # noqa: F401
from .configs import CONFIGS, DEEPSEEK_V3_MOE_LAYER, MIXTRAL_8X7B_BLOCK, MoEConfig, flops_per_step, max_tokens_per_rank, memory_plan, step_roofline  # noqa: F401
