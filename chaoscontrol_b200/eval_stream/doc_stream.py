"""Module path kept for users of ``chaoscontrol.eval_stream.doc_stream``."""
from .io import DocStreamer

__all__ = ["DocStreamer"]
