from .moe import MoELayer, MixtralBlockModel, reference_moe  # noqa: F401
