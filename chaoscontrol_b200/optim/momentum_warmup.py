"""Module path kept for users of ``chaoscontrol.optim.momentum_warmup``."""
from .schedule import apply_momentum_warmup

__all__ = ["apply_momentum_warmup"]
