"""Module path kept for users of ``chaoscontrol.eval.ttt_eval`` (registry in :mod:`.registry`)."""
from .registry import (CALC_TYPE_METADATA, CALC_TYPE_REGISTRY, CalcTypeContext, CalcTypeResult, calc_type_metadata,
                       evaluate_with_calc_types, list_registered_calc_types, register_calc_type)

__all__ = ["CALC_TYPE_METADATA", "CALC_TYPE_REGISTRY", "CalcTypeContext", "CalcTypeResult", "calc_type_metadata",
           "evaluate_with_calc_types", "list_registered_calc_types", "register_calc_type"]
