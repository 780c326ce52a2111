"""Module path kept for users of ``chaoscontrol.optim.weight_ema``."""
from .schedule import WeightEMA, eval_with_ema

__all__ = ["WeightEMA", "eval_with_ema"]
