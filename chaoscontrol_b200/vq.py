"""Import location kept for callers of the reference layout (src/chaoscontrol/vq.py)."""
from .models.routing import vector_quantize

__all__ = ["vector_quantize"]
