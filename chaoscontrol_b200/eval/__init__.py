from .registry import (CALC_TYPE_METADATA, CALC_TYPE_REGISTRY, CalcTypeContext, CalcTypeResult,
                       calc_type_metadata, dispatch_eval_for_config, evaluate_with_calc_types,
                       list_registered_calc_types, register_calc_type)
from . import calc_types  # noqa: F401  registers the built-in passes

__all__ = ["CALC_TYPE_METADATA", "CALC_TYPE_REGISTRY", "CalcTypeContext", "CalcTypeResult",
           "calc_type_metadata", "dispatch_eval_for_config", "evaluate_with_calc_types",
           "list_registered_calc_types", "register_calc_type"]
