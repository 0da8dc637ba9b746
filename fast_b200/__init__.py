"""fast_b200: a Blackwell-native all-to-all(v) scheduler and runtime with a fused MoE path.

Layers (bottom up): ``fast_b200.sched`` host scheduler (C++), ``fast_b200.runtime`` symmetric
memory + signals (C++/CUDA), ``fast_b200.ops`` sm_100a kernels, ``fast_b200.parallel``
communicator / expert parallelism, ``fast_b200.models`` MoE blocks, ``fast_b200.utils``.
"""
from . import sched  # noqa: F401

__version__ = "0.1.0"
