"""YAML-driven single-experiment runner for the research configurations
(``python -m chaoscontrol_b200.runner --config cfg.yaml --data-path DIR``):
config -> model (SSM / transformer / NanoGPT-lean / Mamba-2) [+ learned tokenizer]
-> all-features trainer -> bpb evaluation [-> warming curve] [-> checkpoint]
(surface of src/chaoscontrol/runner.py:21-354)."""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any, Optional

import torch

from .config import ChaosControlConfig, ssm_constructor_kwargs
from .data import build_lm_starts, choose_eval_starts, prepare_fineweb_splits, resolve_device, resolve_param_dtype
from .evaluation import evaluate_chaoscontrol_bpb, evaluate_warming_curve
from .models.model import CareStudentLM
from .training import train_chaoscontrol_for_budget

__all__ = ["load_config", "build_model", "save_checkpoint", "load_checkpoint", "run_experiment"]


def _cfg_dict(cfg) -> dict[str, Any]:
    return {k: v for k, v in vars(cfg).items() if not k.startswith("_")}


def load_config(path: str, *, data_path: str, budget_seconds: Optional[float] = None) -> ChaosControlConfig:
    import yaml
    raw = yaml.safe_load(Path(path).read_text())
    raw["data_path"] = data_path
    if budget_seconds is not None:
        raw["budget_seconds"] = budget_seconds
    return ChaosControlConfig(**raw)


def build_model(cfg: ChaosControlConfig, device: torch.device, param_dtype: torch.dtype):
    mt = cfg.model_type
    if mt == "transformer":
        from .baselines import SimpleTransformerLM
        model = SimpleTransformerLM(vocab_size=cfg.vocab_size, dim=cfg.model_dim, num_layers=cfg.num_layers,
                                    num_heads=max(1, cfg.model_dim // 32))
    elif mt == "transformer_nanogpt_lean":
        from .baselines_nanogpt_lean import NanoGPTLeanLM
        model = NanoGPTLeanLM(vocab_size=cfg.vocab_size, d_model=cfg.model_dim, n_head=max(1, cfg.model_dim // 64),
                              n_layer=cfg.num_layers, ffn_mult=cfg.ff_mult)
    elif mt == "mamba2":
        from .baselines import Mamba2LM
        model = Mamba2LM(vocab_size=cfg.vocab_size, dim=cfg.model_dim, num_layers=cfg.num_layers)
    else:
        model = CareStudentLM(**ssm_constructor_kwargs(_cfg_dict(cfg)))
    model = model.to(device)
    if device.type == "cuda":
        model = model.to(dtype=param_dtype)
    if getattr(cfg, "embed_init_path", None):
        table = torch.load(cfg.embed_init_path, map_location=device)
        assert table.shape == model.embed.weight.shape, (f"embed_init_path shape mismatch: got {tuple(table.shape)}, "
                                                         f"expected {tuple(model.embed.weight.shape)}")
        with torch.no_grad():
            model.embed.weight.copy_(table.to(model.embed.weight))
    return model


def _build_tokenizer(cfg, device, param_dtype):
    if cfg.tokenizer_type != "fixed_stride":
        return None
    from .tokenizer import FixedStrideTokenizer
    tok = FixedStrideTokenizer(byte_dim=cfg.tokenizer_byte_dim, token_dim=cfg.tokenizer_token_dim,
                               codebook_size=cfg.tokenizer_codebook_size, stride=cfg.tokenizer_stride,
                               beta=cfg.tokenizer_beta).to(device)
    if device.type == "cuda":
        tok = tok.to(dtype=param_dtype)
    cfg.vocab_size = cfg.tokenizer_codebook_size         # the model then predicts codebook ids
    return tok


def save_checkpoint(checkpoint_dir: Path, name: str, model: Any, tokenizer: Any | None, structured_proj: Any | None,
                    cfg: ChaosControlConfig) -> Path:
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    path = checkpoint_dir / f"{name}.pt"
    payload: dict[str, Any] = {"model_state_dict": model.state_dict(), "config": _cfg_dict(cfg)}
    if tokenizer is not None:
        payload["tokenizer_state_dict"] = tokenizer.state_dict()
    if structured_proj is not None:
        payload["structured_proj"] = structured_proj
    torch.save(payload, path)
    print(f"Checkpoint saved: {path} ({path.stat().st_size / 1024:.0f} KB)")
    return path


def load_checkpoint(ckpt_path: Path, device: torch.device, param_dtype: torch.dtype) -> dict[str, Any]:
    payload = torch.load(ckpt_path, map_location=device, weights_only=False)
    cfg = ChaosControlConfig(**payload["config"])
    tokenizer = _build_tokenizer(cfg, device, param_dtype)
    model = build_model(cfg, device, param_dtype)
    model.load_state_dict(payload["model_state_dict"])
    if tokenizer is not None and "tokenizer_state_dict" in payload:
        tokenizer.load_state_dict(payload["tokenizer_state_dict"])
    return {"model": model, "tokenizer": tokenizer, "structured_proj": payload.get("structured_proj"), "config": cfg}


_TRAIN_KEYS = (
    "crit_reg_alpha", "crit_reg_beta", "crit_target_coupling", "metabolic_gate", "metabolic_k", "metabolic_threshold",
    "metabolic_threshold_mode", "metabolic_score", "metabolic_noise_std", "generation_mode", "metabolic_mode",
    "mcts_horizon", "mcts_ucb_c", "consolidation_write", "latent_persistence", "cfr_enabled", "align_type",
    "align_weight", "sleep_enabled", "sleep_stages", "sleep_interval", "sleep_budget", "sleep_n2_budget",
    "sleep_rem_budget", "sleep_n2_batches", "sleep_rem_dreams", "sleep_rem_length", "sleep_merge_sim_threshold",
    "sleep_survival_floor", "sleep_rem_reactivate", "polyphasic_enabled", "polyphasic_n_partitions",
    "polyphasic_k_awake", "polyphasic_topology", "polyphasic_swap_interval", "buffer_mode", "wernicke_enabled")
_EVAL_KEYS = ("metabolic_gate", "metabolic_k", "metabolic_score", "metabolic_noise_std", "metabolic_mode",
              "generation_mode", "warmup_write_mode", "warmup_latent", "warmup_cold_start")


def run_experiment(config_path: str, *, data_path: str, budget_seconds: float = 300, checkpoint_dir: Optional[str] = None,
                   checkpoint_name: Optional[str] = None) -> dict[str, Any]:
    cfg = load_config(config_path, data_path=data_path, budget_seconds=budget_seconds)
    device = resolve_device(cfg.device)
    param_dtype = resolve_param_dtype(cfg.dtype, device)
    train_tokens, val_tokens, test_tokens = prepare_fineweb_splits(cfg.data_path, device=device)
    train_starts = build_lm_starts(int(train_tokens.numel()), cfg.seq_len, cfg.stride)
    eval_starts = choose_eval_starts(build_lm_starts(int(val_tokens.numel()), cfg.seq_len, cfg.stride),
                                     batch_size=cfg.batch_size, eval_batches=cfg.eval_batches, seed=cfg.seed)
    tokenizer = _build_tokenizer(cfg, device, param_dtype)
    model = build_model(cfg, device, param_dtype)
    params = sum(p.numel() for p in model.parameters()) + (sum(p.numel() for p in tokenizer.parameters())
                                                           if tokenizer else 0)
    print(f"Model: {cfg.model_type} | dim={cfg.model_dim} | params={params:,} | {model.artifact_bytes():,} bytes")
    tr = train_chaoscontrol_for_budget(
        model, train_tokens=train_tokens, train_starts=train_starts, seq_len=cfg.seq_len, batch_size=cfg.batch_size,
        device=device, param_dtype=param_dtype, budget_seconds=cfg.budget_seconds, base_lr=cfg.base_lr,
        weight_decay=cfg.weight_decay, grad_clip_norm=cfg.grad_clip_norm, seed=cfg.seed, tokenizer=tokenizer,
        **{k: getattr(cfg, k) for k in _TRAIN_KEYS})
    sp = tr.get("structured_proj")
    ev = evaluate_chaoscontrol_bpb(
        model, tokens=val_tokens, eval_starts=eval_starts, batch_size=cfg.batch_size, seq_len=cfg.seq_len,
        device=device, structured_proj=sp, warmup=cfg.eval_warmup, total_raw_bytes=int(val_tokens.numel()),
        tokenizer=tokenizer, **{k: getattr(cfg, k) for k in _EVAL_KEYS})
    print(f"Result: bpb={ev['bpb']:.4f}" + (f" bpb_gated={ev['bpb_gated']:.4f}" if "bpb_gated" in ev else "") +
          f" | steps={tr['steps']} | {tr['elapsed_s']:.1f}s")
    curve: dict[int, float] = {}
    if getattr(model, "outer_model", None) is not None:
        curve = evaluate_warming_curve(model, test_tokens if int(test_tokens.numel()) > 0 else val_tokens,
                                       score_tokens=1024, device=device)
        if curve:
            print("Warming curve: " + " ".join(f"{n}:{b:.3f}" for n, b in sorted(curve.items())))
    ckpt = None
    if checkpoint_dir is not None:
        ckpt = save_checkpoint(Path(checkpoint_dir), checkpoint_name or f"{Path(config_path).stem}_seed{cfg.seed}",
                               model, tokenizer, sp, cfg)
    tr_out = {k: v for k, v in tr.items() if k not in ("structured_proj", "regret_table")}
    return {"config": _cfg_dict(cfg), "train": tr_out, "eval": ev, "warming_curve": curve,
            "params": params + tr.get("extra_params", 0), "checkpoint_path": str(ckpt) if ckpt else None}


def main(argv: Optional[list[str]] = None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--config", required=True)
    p.add_argument("--data-path", "--enwik8-path", required=True, dest="data_path")
    p.add_argument("--budget", type=float, default=300)
    p.add_argument("--output-json", default=None)
    p.add_argument("--checkpoint-dir", default=None)
    p.add_argument("--checkpoint-name", default=None)
    a = p.parse_args(argv)
    res = run_experiment(a.config, data_path=a.data_path, budget_seconds=a.budget, checkpoint_dir=a.checkpoint_dir,
                         checkpoint_name=a.checkpoint_name)
    if a.output_json:
        out = Path(a.output_json)
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(res, indent=2, default=str))
        print(f"Saved to {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
