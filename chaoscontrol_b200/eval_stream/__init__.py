from .budget import BudgetTracker, EvalDeadline, compute_usable_ttt_budget
from .io import (CachedDoc, DocStreamer, MetricsCollector, ValCache, load_val_cache,
                 write_synthetic_val_cache, write_val_cache)
from .legality import LeakDetectedError, LegalityController
from .state import (ADAPT_SET_PATTERNS, DeltaModulator, StateManager, attach_trainable_h0,
                    detach_trainable_h0, select_adapt_params)
from .temporal_heads import (PreviousChunkPriorityGate, TemporalHeadChunkResult, TemporalHeadConfig,
                             make_same_horizon_virtual_depth_config,
                             online_exp_weighted_logprob_mixture, score_temporal_heads_chunk,
                             uniform_logprob_mixture, update_online_exp_weighted_log_weights,
                             weighted_logprob_mixture)
from .types import ChunkRecord, DocRecord, RunConfig

__all__ = ["BudgetTracker", "EvalDeadline", "compute_usable_ttt_budget", "CachedDoc", "DocStreamer",
           "MetricsCollector", "ValCache", "load_val_cache", "write_synthetic_val_cache",
           "write_val_cache", "LeakDetectedError", "LegalityController", "ADAPT_SET_PATTERNS",
           "DeltaModulator", "StateManager", "attach_trainable_h0", "detach_trainable_h0",
           "select_adapt_params", "ChunkRecord", "DocRecord", "RunConfig", "PreviousChunkPriorityGate",
           "TemporalHeadChunkResult", "TemporalHeadConfig", "make_same_horizon_virtual_depth_config",
           "online_exp_weighted_logprob_mixture", "score_temporal_heads_chunk", "uniform_logprob_mixture",
           "update_online_exp_weighted_log_weights", "weighted_logprob_mixture"]
