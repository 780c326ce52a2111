"""Stable public entry points for a submission script
(surface of src/chaoscontrol/public/engine_entry.py:25-198):

``init_arm_topology``   which role a rank plays (train / packet-serving / maintenance)
``build_arm_config``    hyper-parameter object -> runner config dict
``run_arm_submission``  train + eval through ``runner_fast_path.run_condition``

The runner lives in this package, so nothing is resolved through environment
variables or ``sys.path`` edits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

__all__ = ["RoleInfo", "init_arm_topology", "build_arm_config", "run_arm_submission"]


@dataclass
class RoleInfo:
    rank: int
    world_size: int
    packet_rank: int
    maintenance_rank: int
    is_train_rank: bool
    is_packet_rank: bool
    is_maintenance_rank: bool
    split_memory_ranks: bool


def init_arm_topology(rank: int, world_size: int, *, split_memory_ranks: bool = False) -> RoleInfo:
    """Ranks ``0 .. N-2`` train and the last rank owns both memory roles; with
    ``split_memory_ranks`` the last two ranks take packet serving and maintenance
    separately.  A single rank is a train rank with no memory rank."""
    world = int(world_size)
    if world > 0:
        assert 0 <= rank < world, f"rank {rank} out of range for world_size {world}"
    split = bool(split_memory_ranks) and world >= 3
    packet, maint = world - (2 if split else 1), world - 1
    solo = world <= 1
    is_packet = (not solo) and rank == packet
    is_maint = (not solo) and rank == maint
    return RoleInfo(rank=rank, world_size=world, packet_rank=packet, maintenance_rank=maint,
                    is_train_rank=not (is_packet or is_maint), is_packet_rank=is_packet,
                    is_maintenance_rank=is_maint, split_memory_ranks=split)


# locked defaults of the submission arm: fast/slow consolidation and score-only evaluation through the
# online packet cache
_ARM_LOCK: dict[str, Any] = {
    "fast_slow_enabled": True, "fast_slow_interval": 64, "fast_slow_alpha": 0.25,
    "lm_head_backward_mode": "fused_streaming_cached", "lm_head_tile_size": 8192, "optimizer": "muon",
    "precision": "bf16", "dtype": "bf16", "grad_clip_norm": 1.0, "fused_grad_clip": True, "fused_muon": True,
    "stop_check_interval": 4, "stop_margin_seconds": 2.0, "prefetch_batches": True, "train_sampling_mode": "random",
    "calc_types": ["packet_online_cache"], "headline_calc_type": "packet_online_cache",
    "online_episodic_write_tokens_per_chunk": 64,
}
_FORWARD_KEYS = (
    "vocab_size", "model_dim", "num_layers", "ssm_delta_rank", "seq_len", "batch_size", "seed", "budget_seconds",
    "data_path", "val_cache_dir", "sp_model_path", "activation_checkpoint", "lm_head_tile_size", "base_lr",
    "weight_decay", "grad_clip_norm", "optimizer_log_a_beta_coupling", "optimizer_log_a_beta_ema",
    "optimizer_log_a_beta_min", "muon_momentum", "muon_momentum_warmup_start", "muon_momentum_warmup_steps",
    "weight_ema_decay", "weight_ema_fake_quant_bits", "online_episodic_write_tokens_per_chunk", "max_steps",
    "eval_only", "checkpoint_path", "calc_types", "headline_calc_type", "calc_type_configs", "distributed_muon",
    "warmup_steps", "restore_after_warmup", "stride", "eval_batches",
)
_REQUIRED = ("vocab_size", "model_dim", "num_layers", "seq_len", "batch_size")


def build_arm_config(hyperparams: Any) -> dict[str, Any]:
    """Locked arm defaults overlaid with every forwardable attribute present on
    ``hyperparams`` (an object or a mapping)."""
    cfg = dict(_ARM_LOCK)
    get = hyperparams.get if isinstance(hyperparams, dict) else lambda k, d=None: getattr(hyperparams, k, d)
    missing_marker = object()
    for k in _FORWARD_KEYS:
        v = get(k, missing_marker)
        if v is not missing_marker:
            cfg[k] = v
    missing = [k for k in _REQUIRED if k not in cfg]
    if missing:
        raise ValueError(f"build_arm_config: missing required keys {missing}. Set them on your Hyperparameters "
                         "object or pass them in config.")
    return cfg


def run_arm_submission(config: dict[str, Any], *, data_path: str, sp_model_path: Optional[str], budget_seconds: float,
                       output_json: Optional[str], val_cache_dir: Optional[str], output_ckpt: Optional[str] = None,
                       world_size_override: Optional[int] = None) -> dict[str, Any]:
    """``{"config", "params", "train", "eval", "artifact", "exp24"}`` from the production runner."""
    from ..runner_fast_path import run_condition
    return run_condition(dict(config), data_path=data_path, sp_model_path=sp_model_path,
                         budget_seconds=float(budget_seconds), output_json=output_json, output_ckpt=output_ckpt,
                         world_size_override=world_size_override, val_cache_dir=val_cache_dir)
