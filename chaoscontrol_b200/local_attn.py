"""Module path kept for users of ``chaoscontrol.local_attn``; the classes live in
:mod:`chaoscontrol_b200.models.attention`."""
from .models.attention import LocalAttention, RollingKVCache

__all__ = ["LocalAttention", "RollingKVCache"]
