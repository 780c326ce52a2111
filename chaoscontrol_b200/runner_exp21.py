"""Lean train + eval runner with a model-type switch and a constructor-kwargs checkpoint
(behaviour of experiments/21_sgns_tokenizer/runner_exp21.py:83-608).

``model_type: transformer_nanogpt_lean`` builds the transformer baseline, anything else the
bare-SSM ``CareStudentLM``.  ``embed_init_path`` loads a pretrained embedding table (e.g. SGNS
vectors after moment matching).  ``--output-ckpt`` writes ``{"model": cpu state dict, "config":
constructor kwargs[, "episodic_cache", "online_eval_state"]}`` so that evaluation rebuilds the
model with ``Cls(**config)`` + ``load_state_dict(strict=True)``.  Training goes through the
library loop ``train_ssm_for_budget``; rank 0 evaluates bits-per-byte; a non-finite loss or bpb
refuses to write a result unless ``allow_nonfinite`` is set.
"""
from __future__ import annotations

import argparse
import json
import math
import random
import sys
from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch
import torch.distributed as dist

from .config import ssm_constructor_kwargs
from .data import build_lm_starts, choose_eval_starts, resolve_param_dtype
from .models.core import verify_diag_recurrence
from .models.model import CareStudentLM
from .optim import LAMB, Muon
from .runner_fast_path import _apply_embed_init, _init_distributed, _pick_device
from .sp_eval import build_sentencepiece_luts, evaluate_bpb_sp, load_sp_data
from .train_ssm import _reject_unsupported, train_ssm_for_budget

TRANSFORMER = "transformer_nanogpt_lean"

__all__ = ["ssm_constructor_kwargs", "transformer_constructor_kwargs", "constructor_kwargs", "build_model",
           "apply_embed_init", "build_optimizer", "shard_train_starts", "save_output_ckpt", "run_ddp", "main"]


def transformer_constructor_kwargs(config: dict[str, Any]) -> dict[str, Any]:
    """``NanoGPTLeanLM`` kwargs (``max_seq_len`` left at the class default on purpose: training did too)."""
    d = int(config["model_dim"])
    return dict(vocab_size=int(config["vocab_size"]), d_model=d, n_head=int(config.get("n_head", max(1, d // 64))),
                n_layer=int(config["num_layers"]), ffn_mult=int(config.get("ff_mult", 4)),
                activation_checkpoint=bool(config.get("activation_checkpoint", False)))


def _crct_checked(config: dict[str, Any]) -> dict[str, Any]:
    """SSM kwargs with the memory defaults that ``crct_enabled`` implies, and its consistency rules."""
    cfg = dict(config)
    if bool(cfg.get("crct_enabled", False)):
        cfg.setdefault("outer_model_dim", 64)
        cfg.setdefault("outer_model_type", "multislot")
        cfg.setdefault("outer_max_slots", 4096)
        cfg.setdefault("buffer_mode", "append_only")
        cfg.setdefault("retrieval_k", 16)
        if int(cfg["outer_model_dim"]) <= 0:
            raise ValueError("crct_enabled=True requires outer_model_dim > 0; otherwise memory_mode='force_on' "
                             "is identical to memory_mode='off'.")
        if cfg["buffer_mode"] != "append_only":
            raise ValueError("crct_enabled=True requires buffer_mode='append_only' so the fast runner can "
                             "populate memory from encode() hidden states.")
        if cfg["outer_model_type"] != "multislot":
            raise ValueError("crct_enabled=True requires outer_model_type='multislot' for append-only memory writes.")
    else:
        cfg["outer_model_dim"] = 0
    return ssm_constructor_kwargs(cfg)


def constructor_kwargs(config: dict[str, Any]) -> dict[str, Any]:
    if str(config.get("model_type", "")).strip() == TRANSFORMER:
        return transformer_constructor_kwargs(config)
    return _crct_checked(config)


def build_model(config: dict[str, Any], device: torch.device, param_dtype: torch.dtype) -> torch.nn.Module:
    if str(config.get("model_type", "")).strip() == TRANSFORMER:
        from .baselines_nanogpt_lean import NanoGPTLeanLM
        model: torch.nn.Module = NanoGPTLeanLM(**transformer_constructor_kwargs(config))
    else:
        model = CareStudentLM(**_crct_checked(config))
    model = model.to(device)
    return model.to(dtype=param_dtype) if device.type == "cuda" else model


apply_embed_init = _apply_embed_init


def build_optimizer(name: str, model: torch.nn.Module, *, base_lr: float, weight_decay: float) -> torch.optim.Optimizer:
    params = list(model.parameters())
    if name == "adamw":
        return torch.optim.AdamW(params, lr=base_lr, weight_decay=weight_decay)
    if name == "muon":
        opt = Muon(params, lr=base_lr, weight_decay=weight_decay, adamw_lr=base_lr, adamw_weight_decay=weight_decay)
        opt.bind_param_names(list(model.named_parameters()))
        return opt
    if name == "lamb":
        return LAMB(params, lr=base_lr, weight_decay=weight_decay)
    raise ValueError(f"Unknown optimizer: {name!r}. Expected one of {{'adamw', 'muon', 'lamb'}}.")


def shard_train_starts(train_starts: list[int], *, rank: int, world_size: int) -> list[int]:
    """Stride sharding: rank ``r`` keeps starts ``r, r + ws, ...``."""
    if world_size <= 1:
        return list(train_starts)
    mine = train_starts[rank::world_size]
    if not mine:
        raise RuntimeError(f"rank {rank} has no train_starts after stride-sharding ({len(train_starts)} total "
                           f"starts across world_size={world_size}).")
    return list(mine)


def _to_cpu(v: Any) -> Any:
    if torch.is_tensor(v):
        return v.detach().to("cpu")
    if isinstance(v, dict):
        return {k: _to_cpu(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return type(v)(_to_cpu(x) for x in v)
    return v


def save_output_ckpt(output_ckpt: str, model: torch.nn.Module, config: dict[str, Any], episodic_cache: Any = None,
                     online_eval_state: Optional[dict] = None) -> None:
    blob: dict[str, Any] = {"model": _to_cpu(dict(model.state_dict())), "config": constructor_kwargs(config)}
    if episodic_cache is not None:
        if not isinstance(episodic_cache, dict):
            to_dict = getattr(episodic_cache, "to_dict", None)
            if not callable(to_dict):
                raise TypeError("episodic_cache must be a dict or expose to_dict() when passed to save_output_ckpt")
            episodic_cache = to_dict()
        blob["episodic_cache"] = episodic_cache
    if isinstance(online_eval_state, dict) and online_eval_state:
        blob["online_eval_state"] = online_eval_state
    out = Path(output_ckpt)
    out.parent.mkdir(parents=True, exist_ok=True)
    tmp = out.with_suffix(out.suffix + ".tmp")
    torch.save(blob, tmp)
    tmp.rename(out)


def _finite_gate(result: dict[str, Any], config: dict[str, Any]) -> None:
    bad = []
    if not math.isfinite(result["train"]["final_loss"]):
        bad.append(f"train.final_loss={result['train']['final_loss']} is not finite")
    bad += [f"eval.{k}={result['eval'][k]} is not finite" for k in ("bpb", "loss")
            if k in result["eval"] and not math.isfinite(float(result["eval"][k]))]
    if not bad:
        return
    if not bool(config.get("allow_nonfinite", False)):
        raise RuntimeError("runner_exp21: refusing to write poisoned result JSON — " + "; ".join(bad))
    result["nonfinite"] = {"flag": True, "violations": bad}
    print(f"[rank 0] allow_nonfinite=true — preserving divergent run as datapoint: {'; '.join(bad)}", flush=True)


def run_ddp(config: dict[str, Any], *, data_path: str, sp_model_path: str, budget_seconds: float,
            output_json: Optional[str], world_size_override: Optional[int], output_ckpt: Optional[str] = None,
            max_steps: Optional[int] = None) -> dict[str, Any]:
    rank, world_size, local_rank = _init_distributed(world_size_override)
    ddp = world_size > 1
    device = _pick_device(local_rank, str(config.get("device", "auto")))
    dtype = resolve_param_dtype(str(config.get("dtype", "bf16")), device)
    seed = int(config.get("seed", 1337))
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    verify_diag_recurrence(device)
    vocab = int(config["vocab_size"])
    train_tokens, val_tokens, _ = load_sp_data(data_path, vocab)
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor()
    sp.Load(sp_model_path)
    luts = build_sentencepiece_luts(sp, vocab, device)
    seq_len, batch = int(config["seq_len"]), int(config["batch_size"])
    stride = int(config.get("stride", seq_len // 2))
    eval_starts = choose_eval_starts(build_lm_starts(int(val_tokens.numel()), seq_len, stride), batch_size=batch,
                                     eval_batches=int(config.get("eval_batches", 16)), seed=seed)
    train_starts = shard_train_starts(build_lm_starts(int(train_tokens.numel()), seq_len, stride), rank=rank,
                                      world_size=world_size)
    model = build_model(config, device, dtype)
    apply_embed_init(model, config, device)
    _reject_unsupported(model)
    precision = str(config.get("precision", "bf16"))
    if precision in ("fp8", "fp8_fused"):
        from .precision import maybe_promote_linears_to_fused_fp8
        n = maybe_promote_linears_to_fused_fp8(model, True, scaling=str(config.get("fp8_scaling", "tensor")))
        if rank == 0:
            print(f"[rank 0] promoted {n} nn.Linear modules to fp8", flush=True)
    params = sum(p.numel() for p in model.parameters())
    name = str(config.get("optimizer", "")).strip()
    if not name:
        raise ValueError("runner_exp21 requires config['optimizer'] to be set explicitly "
                         "(one of {'adamw', 'muon', 'lamb'}).")
    opt = build_optimizer(name, model, base_lr=float(config.get("base_lr", 2e-3)),
                          weight_decay=float(config.get("weight_decay", 1e-2)))
    tr = train_ssm_for_budget(model, train_tokens=train_tokens, train_starts=train_starts, seq_len=seq_len,
                              batch_size=batch, device=device, optimizer=opt, budget_seconds=budget_seconds,
                              chunk_size=int(config.get("chunk_size", 64)),
                              grad_clip_norm=float(config.get("grad_clip_norm", 1.0)), seed=seed, rank=rank,
                              world_size=world_size, precision=precision, max_steps=max_steps)
    if ddp:
        dist.barrier()
    ev = (evaluate_bpb_sp(model, tokens=val_tokens, eval_starts=eval_starts, batch_size=batch, seq_len=seq_len,
                          device=device, base_bytes_lut=luts[0], has_leading_space_lut=luts[1],
                          is_boundary_token_lut=luts[2]) if rank == 0 else {})
    if ddp:
        dist.barrier()
    last = tr["history"][-1] if tr["history"] else {}
    result = {"config": config, "params": params, "eval": ev, "train": {
        "steps": int(tr["steps"]), "elapsed_s": float(tr["elapsed_s"]),
        "steps_per_second": float(tr["steps"] / max(tr["elapsed_s"], 1e-9)),
        "final_loss": float(last.get("loss", float("nan"))), "peak_vram_mb": float(tr.get("peak_vram_mb", 0.0)),
        "ddp_rank": int(tr.get("rank", rank)), "ddp_world_size": int(tr.get("world_size", world_size))}}
    if rank == 0:
        _finite_gate(result, config)
        if output_json:
            out = Path(output_json)
            out.parent.mkdir(parents=True, exist_ok=True)
            tmp = out.with_suffix(".tmp")
            tmp.write_text(json.dumps(result, indent=2, default=str))
            tmp.rename(out)
        if output_ckpt:
            save_output_ckpt(output_ckpt, model, config)
        print(f"[rank {rank}/{world_size}] done: bpb={ev.get('bpb', float('nan')):.4f} steps={result['train']['steps']} "
              f"steps/s={result['train']['steps_per_second']:.2f}", flush=True)
    if ddp and dist.is_initialized():
        dist.destroy_process_group()
    return result


def main(argv: Optional[list[str]] = None) -> int:
    import yaml
    ap = argparse.ArgumentParser(description="lean train + eval runner")
    ap.add_argument("--config", required=True)
    ap.add_argument("--data-path", required=True)
    ap.add_argument("--sp-model-path", required=True)
    ap.add_argument("--budget", type=float, default=600.0)
    ap.add_argument("--output-json", default=None)
    ap.add_argument("--output-ckpt", default=None)
    ap.add_argument("--world-size", type=int, default=None)
    a = ap.parse_args(argv)
    config = yaml.safe_load(Path(a.config).read_text())
    run_ddp(config, data_path=a.data_path, sp_model_path=a.sp_model_path, budget_seconds=a.budget,
            output_json=a.output_json, world_size_override=a.world_size, output_ckpt=a.output_ckpt)
    return 0


if __name__ == "__main__":
    sys.exit(main())
