from .optim import FusedAdamW  # noqa: F401
