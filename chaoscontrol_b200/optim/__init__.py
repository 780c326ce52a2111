from .lamb import LAMB
from .muon import Muon, newton_schulz_orthogonalize
from .param_groups import (SPECTRAL_SUFFIXES, build_optimizer_params, classify_param,
                           ssm_three_group_params)
from .schedule import (WeightEMA, apply_momentum_warmup, eval_with_ema, wrap_optimizer_step)
from .semantic import SemanticOptimizer
from .scopt import ScarcityAwareOptimizer
from .criticality import CriticalityDistillation

__all__ = ["LAMB", "Muon", "newton_schulz_orthogonalize", "SPECTRAL_SUFFIXES", "build_optimizer_params",
           "classify_param", "ssm_three_group_params", "WeightEMA", "apply_momentum_warmup",
           "eval_with_ema", "wrap_optimizer_step", "SemanticOptimizer", "ScarcityAwareOptimizer",
           "CriticalityDistillation"]
