"""Module path kept for users of ``chaoscontrol.eval_stream.val_cache``."""
from .io import CachedDoc, ValCache, load_val_cache, write_synthetic_val_cache, write_val_cache

__all__ = ["CachedDoc", "ValCache", "load_val_cache", "write_synthetic_val_cache", "write_val_cache"]
