from .config import CONFIG, nvtx_range  # noqa: F401
from .optim import FusedAdamW  # noqa: F401
