"""Import location kept for callers of the reference layout
(src/chaoscontrol/wake_cache_txn.py); the classes live in ``wake_cache``."""
from .wake_cache import CacheTxn, CausalEventClock, TransactionalWakeCache

__all__ = ["CacheTxn", "CausalEventClock", "TransactionalWakeCache"]
