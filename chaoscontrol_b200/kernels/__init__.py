"""Kernel-level public ops under the names the reference exposes from
``chaoscontrol.kernels`` (ssm_scan, the LM-head / loss family, the fp8 linear)."""
from ..ops.scan import ssm_scan
from .lm_head_loss import (fused_linear_cross_entropy, fused_linear_cross_entropy_weighted,
                           fused_linear_cross_entropy_with_ce,
                           fused_lm_head_forward_with_ce_entropy, fused_rms_linear_cross_entropy,
                           fused_rms_linear_cross_entropy_with_ce, fused_rms_norm)

__all__ = ["ssm_scan", "fused_rms_norm", "fused_linear_cross_entropy",
           "fused_linear_cross_entropy_with_ce", "fused_linear_cross_entropy_weighted",
           "fused_rms_linear_cross_entropy", "fused_rms_linear_cross_entropy_with_ce",
           "fused_lm_head_forward_with_ce_entropy"]
