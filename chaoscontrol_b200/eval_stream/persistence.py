"""Module path kept for users of ``chaoscontrol.eval_stream.persistence``."""
from .state import PERSISTENCE_MODES, StateManager, attach_trainable_h0, detach_trainable_h0

__all__ = ["PERSISTENCE_MODES", "StateManager", "attach_trainable_h0", "detach_trainable_h0"]
