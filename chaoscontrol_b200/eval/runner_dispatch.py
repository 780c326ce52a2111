"""Module path kept for users of ``chaoscontrol.eval.runner_dispatch``."""
from .registry import dispatch_eval_for_config

__all__ = ["dispatch_eval_for_config"]
