"""Typed run configuration.

``ChaosControlConfig`` carries every key of the reference's YAML / checkpoint
config (src/chaoscontrol/config.py:9-226) so its config dicts round-trip:
the field table (name, type, default) lives in ``config_schema.json`` and the
dataclass is generated from it.  ``from_dict`` accepts the reference's key
names, ignores nothing silently (unknown keys raise unless ``strict=False``)
and ``model_kwargs`` projects a config onto ``CareStudentLM``'s constructor.
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any, Optional

_SCHEMA = json.loads((Path(__file__).with_name("config_schema.json")).read_text())
_TYPES = {"str": str, "int": int, "float": float, "bool": bool}

VALID_BUFFER_MODES = ("legacy", "append_only")
VALID_RETRIEVAL_MODES = ("softmax_all", "bucket_mean", "bucket_recent", "bucket_topk")
VALID_POSTERIOR_MODES = ("none", "global_delta", "bucket_delta", "residual_cache")


def _field(entry: dict):
    typ = _TYPES.get(entry["type"], Any)
    if entry.get("required"):
        return (entry["name"], typ)
    default = entry["default"]
    if isinstance(default, (list, dict)):
        return (entry["name"], typ, dataclasses.field(default_factory=lambda d=default: type(d)(d)))
    return (entry["name"], typ, dataclasses.field(default=default))


def _post_init(self) -> None:
    for attr, valid in (("buffer_mode", VALID_BUFFER_MODES), ("retrieval_mode", VALID_RETRIEVAL_MODES),
                        ("posterior_mode", VALID_POSTERIOR_MODES)):
        v = getattr(self, attr, None)
        if v is not None and v not in valid:
            raise ValueError(f"{attr} must be one of {valid}, got {v!r}")


def _from_dict(cls, d: dict, strict: bool = True):
    known = {f.name for f in dataclasses.fields(cls)}
    extra = set(d) - known
    if extra and strict:
        raise ValueError(f"unknown config keys: {sorted(extra)}")
    return cls(**{k: v for k, v in d.items() if k in known})


def _from_yaml(cls, path, **overrides):
    import yaml
    data = yaml.safe_load(Path(path).read_text()) or {}
    data.update(overrides)
    return cls.from_dict(data)


_MODEL_KEYS = {
    "vocab_size": "vocab_size", "model_dim": "dim", "num_layers": "num_layers", "ff_mult": "ff_mult",
    "a_mode": "a_mode", "a_full_rank": "a_full_rank", "a_full_gamma": "a_full_gamma",
    "rich_b_mode": "rich_b_mode", "rich_b_bottleneck": "rich_b_bottleneck",
    "rich_b_num_subnets": "rich_b_num_subnets", "rich_b_settling_steps": "rich_b_settling_steps",
    "outer_model_dim": "outer_model_dim", "outer_model_type": "outer_model_type",
    "outer_max_slots": "outer_max_slots", "outer_compress_ratio": "outer_compress_ratio",
    "consolidation_mode": "consolidation_mode", "consolidation_ema_decay": "consolidation_ema_decay",
    "consolidation_trigger": "consolidation_trigger", "consolidation_window": "consolidation_window",
    "wernicke_enabled": "wernicke_enabled", "wernicke_k_max": "wernicke_k_max",
    "wernicke_window": "wernicke_window", "wernicke_router": "wernicke_router",
    "wernicke_balance_weight": "wernicke_balance_weight", "wernicke_expert_dim": "wernicke_expert_dim",
    "wernicke_layers": "wernicke_layers", "wernicke_k_max_fine": "wernicke_k_max_fine",
    "buffer_mode": "buffer_mode", "retrieval_mode": "retrieval_mode", "retrieval_k": "retrieval_k",
    "bucket_prototypes": "bucket_prototypes", "prototype_dim": "prototype_dim",
    "prototype_update_rate": "prototype_update_rate", "semantic_tier_bases": "semantic_tier_bases",
    "semantic_tier_update_rate": "semantic_tier_update_rate", "typed_storage": "typed_storage",
    "typed_consolidation": "typed_consolidation", "compression_consequence": "compression_consequence",
    "cue_projection": "cue_projection", "dynamic_crit_per_layer": "dynamic_crit_per_layer",
    "compression_selection": "compression_selection", "posterior_mode": "posterior_mode",
    "posterior_lr": "posterior_lr", "residual_cache_k": "residual_cache_k",
    "local_attn_window": "local_attn_window", "local_attn_heads": "local_attn_heads",
    "local_attn_dim": "local_attn_dim", "local_attn_topk": "local_attn_topk",
    "local_attn_topk_random": "local_attn_topk_random",
}


def _model_kwargs(self) -> dict:
    """Constructor kwargs of ``CareStudentLM`` implied by this config."""
    out = {}
    for cfg_key, ctor_key in _MODEL_KEYS.items():
        if hasattr(self, cfg_key):
            out[ctor_key] = getattr(self, cfg_key)
    return out


ChaosControlConfig = dataclasses.make_dataclass(
    "ChaosControlConfig", [_field(e) for e in _SCHEMA],
    namespace={"__post_init__": _post_init, "from_dict": classmethod(_from_dict),
               "from_yaml": classmethod(_from_yaml), "model_kwargs": _model_kwargs,
               "to_dict": lambda self: dataclasses.asdict(self)})
ChaosControlConfig.__module__ = __name__
ChaosControlConfig.__doc__ = "All knobs of the legacy YAML runner and of serialized artifacts."


def ssm_constructor_kwargs(config: dict) -> dict:
    """``CareStudentLM`` kwargs from a plain dict config of the modern runners
    (the checkpoint ``"config"`` schema; cf.
    experiments/21_sgns_tokenizer/runner_exp21.py:83-143)."""
    get = config.get
    kw = dict(vocab_size=int(config["vocab_size"]), dim=int(get("model_dim", get("dim", 256))),
              num_layers=int(get("num_layers", 4)), ff_mult=int(get("ff_mult", 2)),
              a_mode=str(get("a_mode", "diag")), a_full_rank=int(get("a_full_rank", 8)),
              a_full_gamma=float(get("a_full_gamma", 0.05)),
              ssm_delta_rank=int(get("ssm_delta_rank", 0)),
              local_attn_window=int(get("local_attn_window", 0)),
              local_attn_heads=int(get("local_attn_heads", 1)),
              local_attn_dim=int(get("local_attn_dim", 64)),
              local_attn_topk=int(get("local_attn_topk", 0)),
              local_attn_topk_random=bool(get("local_attn_topk_random", False)),
              activation_checkpoint=bool(get("activation_checkpoint", False)))
    for opt in ("block_type", "attention_num_heads", "attention_dropout", "outer_model_dim",
                "outer_model_type", "outer_max_slots", "buffer_mode", "retrieval_mode", "retrieval_k",
                "wernicke_enabled", "wernicke_k_max", "wernicke_window", "wernicke_router",
                "depth_recurrence_shared_layers", "depth_recurrence_count", "tie_embeddings", "log_a_init"):
        if opt in config:
            kw[opt] = config[opt]
    return kw
