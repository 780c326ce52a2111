"""Module path kept for users of ``chaoscontrol.eval_stream.ttt_runner``."""
from .state import ADAPT_SET_PATTERNS, select_adapt_params

__all__ = ["ADAPT_SET_PATTERNS", "select_adapt_params"]
