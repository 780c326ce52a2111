"""Module path kept for users of ``chaoscontrol.optim.step_wrapper``."""
from .schedule import wrap_optimizer_step

__all__ = ["wrap_optimizer_step"]
