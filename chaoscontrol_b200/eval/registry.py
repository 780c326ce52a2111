"""Calc-type registry: each evaluation *calc type* is one pass over the
validation cache with its own per-document loop and state discipline
(cf. src/chaoscontrol/eval/ttt_eval.py:73-193, runner_dispatch.py:32-127)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch
import torch.nn as nn


@dataclass
class CalcTypeContext:
    model: nn.Module
    val_cache: Any
    device: torch.device
    base_bytes_lut: Optional[torch.Tensor]
    has_leading_space_lut: Optional[torch.Tensor]
    is_boundary_token_lut: Optional[torch.Tensor]
    config: dict[str, Any]


@dataclass
class CalcTypeResult:
    bpb: float
    loss: float
    docs_scored: int
    tokens_scored: int
    raw_bytes: int
    hyperparams: dict[str, Any]
    extra: dict[str, Any] = field(default_factory=dict)


CalcTypeFn = Callable[[CalcTypeContext], CalcTypeResult]
CALC_TYPE_REGISTRY: dict[str, CalcTypeFn] = {}
CALC_TYPE_METADATA: dict[str, dict[str, Any]] = {}


def register_calc_type(name: str, *, requires_source_order: bool = False, requires_grad: bool = False,
                       description: str = "") -> Callable[[CalcTypeFn], CalcTypeFn]:
    """``requires_source_order``: the pass is not invariant to document order
    (state or weights carry across documents).  ``requires_grad``: the pass runs
    its own autograd scope."""
    def deco(fn: CalcTypeFn) -> CalcTypeFn:
        if name in CALC_TYPE_REGISTRY:
            raise ValueError(f"calc_type {name!r} already registered")
        CALC_TYPE_REGISTRY[name] = fn
        CALC_TYPE_METADATA[name] = {"requires_source_order": bool(requires_source_order),
                                    "requires_grad": bool(requires_grad), "description": str(description)}
        return fn
    return deco


def calc_type_metadata(name: str) -> dict[str, Any]:
    if name not in CALC_TYPE_METADATA:
        raise ValueError(f"unknown calc_type: {name!r}")
    return dict(CALC_TYPE_METADATA[name])


def list_registered_calc_types() -> list[str]:
    return sorted(CALC_TYPE_REGISTRY)


def evaluate_with_calc_types(*, model: nn.Module, val_cache, calc_types: list[str],
                             calc_type_configs: Optional[dict[str, dict[str, Any]]] = None,
                             device: torch.device, base_bytes_lut=None, has_leading_space_lut=None,
                             is_boundary_token_lut=None, source_order_preserved: bool = True
                             ) -> dict[str, dict[str, Any]]:
    from . import calc_types as _builtin  # noqa: F401  (registers the built-in passes)
    cfgs = calc_type_configs or {}
    unknown = [n for n in calc_types if n not in CALC_TYPE_REGISTRY]
    if unknown:
        raise ValueError(f"unknown calc_type(s): {unknown!r}; registered={sorted(CALC_TYPE_REGISTRY)}")
    if not source_order_preserved:
        bad = [n for n in calc_types if CALC_TYPE_METADATA[n]["requires_source_order"]]
        if bad:
            raise ValueError(f"calc_type(s) {bad!r} require source-ordered docs but "
                             "source_order_preserved=False")
    out: dict[str, dict[str, Any]] = {}
    for name in calc_types:
        res = CALC_TYPE_REGISTRY[name](CalcTypeContext(
            model=model, val_cache=val_cache, device=device, base_bytes_lut=base_bytes_lut,
            has_leading_space_lut=has_leading_space_lut, is_boundary_token_lut=is_boundary_token_lut,
            config=dict(cfgs.get(name, {}))))
        out[name] = {"bpb": float(res.bpb), "loss": float(res.loss), "docs_scored": int(res.docs_scored),
                     "tokens_scored": int(res.tokens_scored), "raw_bytes": int(res.raw_bytes),
                     "hyperparams": dict(res.hyperparams), **dict(res.extra)}
    return out


def dispatch_eval_for_config(config: dict[str, Any], *, model: nn.Module, val_cache, val_tokens=None,
                             eval_starts=None, batch_size: int = 0, seq_len: int = 0,
                             device: torch.device, base_bytes_lut=None, has_leading_space_lut=None,
                             is_boundary_token_lut=None, legacy_evaluate_fn=None) -> dict[str, Any]:
    """Calc-type evaluation when ``config["calc_types"]`` is set, else the legacy
    windowed evaluator.  Non-finite results raise."""
    calc_types = list(config.get("calc_types") or [])
    if not calc_types:
        if legacy_evaluate_fn is None:
            raise ValueError("config has no calc_types and no legacy_evaluate_fn was given")
        return legacy_evaluate_fn(model, tokens=val_tokens, eval_starts=eval_starts, batch_size=batch_size,
                                  seq_len=seq_len, device=device, base_bytes_lut=base_bytes_lut,
                                  has_leading_space_lut=has_leading_space_lut,
                                  is_boundary_token_lut=is_boundary_token_lut)
    if val_cache is None:
        raise ValueError("config sets calc_types but val_cache is None; pass --val-cache-dir to the runner")
    results = evaluate_with_calc_types(
        model=model, val_cache=val_cache, calc_types=calc_types,
        calc_type_configs=dict(config.get("calc_type_configs") or {}), device=device,
        base_bytes_lut=base_bytes_lut, has_leading_space_lut=has_leading_space_lut,
        is_boundary_token_lut=is_boundary_token_lut, source_order_preserved=True)
    head = config.get("headline_calc_type")
    if head is not None:
        head = str(head)
        if head not in results:
            raise ValueError(f"headline_calc_type must be one of calc_types; got {head!r} for {list(results)}")
    else:
        head = "score_only_reset" if "score_only_reset" in results else next(iter(results))
    bad = [n for n, e in results.items() if not (math.isfinite(e["bpb"]) and math.isfinite(e["loss"]))]
    if bad:
        raise RuntimeError(f"non-finite bpb/loss for calc_type(s) {bad!r}")
    return {"calc_types": results, "headline_calc_type": head, "bpb": results[head]["bpb"],
            "loss": results[head]["loss"], "docs_scored": results[head]["docs_scored"],
            "tokens_scored": results[head]["tokens_scored"]}
