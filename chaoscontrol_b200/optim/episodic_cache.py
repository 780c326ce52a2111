"""Import location kept for callers of the reference layout
(src/chaoscontrol/optim/episodic_cache.py); the classes live in ``episodic.cache``."""
from ..episodic.cache import CacheEntry, EpisodicCache

__all__ = ["CacheEntry", "EpisodicCache"]
