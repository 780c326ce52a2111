"""Module path kept for users of ``chaoscontrol.eval_stream.delta_mod``."""
from .state import DeltaModulator

__all__ = ["DeltaModulator"]
