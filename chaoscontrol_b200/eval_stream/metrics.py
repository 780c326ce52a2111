"""Module path kept for users of ``chaoscontrol.eval_stream.metrics``."""
from .io import MetricsCollector

__all__ = ["MetricsCollector"]
