"""Single-file <= 16 MB model artifact: quantise, LZMA-compress, write; and the
inverse.  Payload keys, quantisation ladder (int8 -> int6 -> prune episodic
slots by survival) and the 16 000 000-byte budget follow
src/chaoscontrol/artifact.py:113-413, so artifacts are interchangeable.
"""
from __future__ import annotations

import copy
import io
import lzma
from dataclasses import asdict, is_dataclass
from pathlib import Path
from typing import Any, Optional

import torch
import torch.nn as nn

TARGET_BYTES = 16_000_000


def _quantize(t: torch.Tensor, qmax: int) -> dict[str, Any]:
    """Per-tensor symmetric quantisation to [-qmax-1, qmax] stored as int8."""
    scale = t.abs().max() / qmax
    if float(scale) == 0.0:
        scale = torch.tensor(1.0)
    return {"q": (t / scale).round().clamp(-qmax - 1, qmax).to(torch.int8), "scale": scale.float()}


def _dequantize(entry: dict[str, Any]) -> torch.Tensor:
    return entry["q"].float() * entry["scale"]


def _quantize_state_dict(sd: dict, *, use_int6: bool) -> dict:
    qmax = 31 if use_int6 else 127
    for k, v in list(sd.items()):
        if isinstance(v, torch.Tensor):
            sd[k] = _quantize(v.float(), qmax) if v.ndim == 2 else v.half()
    return sd


def _dequantize_state_dict(sd: dict) -> dict:
    for k, v in list(sd.items()):
        if isinstance(v, dict) and "q" in v and "scale" in v:
            sd[k] = _dequantize(v)
        elif isinstance(v, torch.Tensor):
            sd[k] = v.float()
    return sd


def _cpu_tree(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _cpu_tree(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_cpu_tree(v) for v in obj)
    return obj


def _config_dict(config) -> dict:
    if config is None:
        return {}
    if is_dataclass(config):
        return asdict(config)
    return dict(config)


def _collect_state(model: nn.Module, tokenizer, config, regret_table, online_eval_state,
                   replay_eviction_loop) -> dict:
    state: dict[str, Any] = {
        "model": {k: _cpu_tree(v) for k, v in model.state_dict().items()
                  if not str(k).endswith("._extra_state")},
        "tokenizer": ({k: _cpu_tree(v) for k, v in tokenizer.state_dict().items()}
                      if tokenizer is not None else None),
        "config": _config_dict(config),
        "episodic_slots": [], "episodic_survival": [], "episodic_buckets": [],
        "episodic_slot_event_ids": [], "episodic_table_state": None, "latent_traces": [],
        "semantic_bases": None, "regret_table": None,
    }
    om = getattr(model, "outer_model", None)
    if om is not None and hasattr(om, "_slots"):
        state["episodic_slots"] = [s.detach().cpu() for s in om._slots]
        state["episodic_survival"] = list(getattr(om, "_survival", []))
        state["episodic_buckets"] = list(getattr(om, "_slot_buckets", []))
        state["episodic_slot_event_ids"] = list(getattr(om, "_slot_event_ids", []))
        table = getattr(om, "table", None)
        if table is not None and hasattr(table, "state_dict"):
            state["episodic_table_state"] = {k: v for k, v in table.state_dict().items() if k != "slots"}
        state["latent_traces"] = [{"bucket_id": t["bucket_id"],
                                   "centroid_contrib": t["centroid_contrib"].detach().cpu()}
                                  for t in getattr(om, "_latent_traces", [])]
    st = getattr(model, "semantic_tier", None)
    if st is not None and hasattr(st, "bases"):
        state["semantic_bases"] = st.bases.detach().cpu()
    if regret_table is not None:
        state["regret_table"] = regret_table.cumulative_regret.detach().cpu()
    online: dict[str, Any] = {}
    if isinstance(getattr(model, "_online_eval_state", None), dict):
        online.update(_cpu_tree(model._online_eval_state))
    if isinstance(online_eval_state, dict):
        online.update(_cpu_tree(online_eval_state))
    if replay_eviction_loop is not None and hasattr(replay_eviction_loop, "state_dict"):
        online["replay_eviction"] = _cpu_tree(replay_eviction_loop.state_dict())
    state["online_eval_state"] = online
    return state


def _pack(state: dict, quantization: str, lzma_preset: int, slots_to_keep: Optional[int]):
    sd = copy.deepcopy(state)
    int6 = quantization == "int6"
    _quantize_state_dict(sd["model"], use_int6=int6)
    if sd["tokenizer"] is not None:
        _quantize_state_dict(sd["tokenizer"], use_int6=int6)
    if sd["episodic_slots"]:
        n = len(sd["episodic_slots"])
        if slots_to_keep is not None and slots_to_keep < n:
            surv = sd["episodic_survival"]
            keep = sorted(sorted(range(n), key=lambda i: surv[i])[n - slots_to_keep:])
            for key in ("episodic_slots", "episodic_survival", "episodic_buckets"):
                sd[key] = [sd[key][i] for i in keep]
            ids = sd.get("episodic_slot_event_ids") or [0] * n
            sd["episodic_slot_event_ids"] = [ids[i] for i in keep]
            sd["episodic_table_state"] = None
        qmax = 31 if int6 else 127
        sd["episodic_slots"] = [_quantize((s if s.ndim >= 2 else s.unsqueeze(0)).float(), qmax)
                                for s in sd["episodic_slots"]]
    for tr in sd["latent_traces"]:
        t = tr["centroid_contrib"]
        tr["centroid_contrib"] = _quantize((t if t.ndim >= 2 else t.unsqueeze(0)).float(), 31 if int6 else 127)
    for key in ("semantic_bases", "regret_table"):
        if sd[key] is not None:
            sd[key] = sd[key].half()
    buf = io.BytesIO()
    torch.save(sd, buf)
    return lzma.compress(buf.getvalue(), preset=lzma_preset), len(sd["episodic_slots"])


def serialize_artifact(model: nn.Module, tokenizer: Optional[nn.Module], config, path, *,
                       target_bytes: int = TARGET_BYTES, regret_table=None, lzma_preset: int = 6,
                       force_quantization: Optional[str] = None, online_eval_state: Optional[dict] = None,
                       replay_eviction_loop=None) -> dict[str, Any]:
    """Write the artifact and return ``{"path", "size_bytes", "quantization",
    "slots_kept", "slots_pruned", "online_eval_state"}``.  Raises if even int6 with
    all episodic slots pruned does not fit ``target_bytes``."""
    path = Path(path)
    state = _collect_state(model, tokenizer, config, regret_table, online_eval_state, replay_eviction_loop)
    n_slots = len(state["episodic_slots"])
    ladder = [force_quantization] if force_quantization else ["int8", "int6"]
    blob, quant, kept = None, None, n_slots
    for q in ladder:
        blob, kept = _pack(state, q, lzma_preset, None)
        quant = q
        if len(blob) <= target_bytes:
            break
    if len(blob) > target_bytes and n_slots > 0:
        for keep_n in range(n_slots - 1, -1, -1):
            blob, kept = _pack(state, quant, lzma_preset, keep_n)
            if len(blob) <= target_bytes:
                break
    if len(blob) > target_bytes:
        raise ValueError("Artifact too large after all compression attempts: "
                         f"{len(blob):,} bytes > {target_bytes:,} byte budget")
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_bytes(blob)
    return {"path": str(path), "size_bytes": len(blob), "quantization": quant, "slots_kept": kept,
            "slots_pruned": n_slots - kept, "online_eval_state": sorted(state["online_eval_state"].keys())}


def load_artifact(path, device: str = "cpu"):
    """Inverse of :func:`serialize_artifact`: ``(model, tokenizer_state_or_None, config_dict)``."""
    from .config import ChaosControlConfig
    from .models.model import CareStudentLM
    state = torch.load(io.BytesIO(lzma.decompress(Path(path).read_bytes())), map_location="cpu",
                       weights_only=False)
    cfg = state.get("config") or {}
    model_sd = _dequantize_state_dict(state["model"])
    try:
        kwargs = ChaosControlConfig.from_dict(cfg, strict=False).model_kwargs() if "data_path" in cfg else None
    except Exception:
        kwargs = None
    if kwargs is None:
        from .config import ssm_constructor_kwargs
        kwargs = ssm_constructor_kwargs(cfg) if "vocab_size" in cfg else _infer_kwargs(model_sd)
    model = CareStudentLM(**kwargs)
    model.load_state_dict(model_sd, strict=True)
    om = getattr(model, "outer_model", None)
    if om is not None and state.get("episodic_slots") and hasattr(om, "_slots"):
        om._slots = [_dequantize(e) for e in state["episodic_slots"]]
        om._survival = list(state.get("episodic_survival", []))
        om._slot_buckets = list(state.get("episodic_buckets", []))
    if state.get("semantic_bases") is not None and getattr(model, "semantic_tier", None) is not None:
        model.semantic_tier.bases.data.copy_(state["semantic_bases"].float())
    model._online_eval_state = state.get("online_eval_state", {})
    tok = _dequantize_state_dict(state["tokenizer"]) if state.get("tokenizer") is not None else None
    return model.to(device), tok, cfg


def _infer_kwargs(sd: dict) -> dict:
    V, D = sd["embed.weight"].shape
    layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("layers."))
    ff = sd["layers.0.ff.fc.weight"].shape[0] // D
    return dict(vocab_size=V, dim=D, num_layers=layers, ff_mult=ff)


def eval_artifact(path, tokens: torch.Tensor, device: str = "cpu", *, eval_batches: int = 32,
                  batch_size: int = 8, seq_len: int = 256, raw_bytes_per_token: float = 1.0,
                  seed: int = 0) -> dict:
    """Load an artifact and report mean CE / bits-per-byte on windows of ``tokens``."""
    from .data import batch_from_starts, build_lm_starts, choose_eval_starts
    from .scoring import compute_bpb
    model, _, _ = load_artifact(path, device=device)
    model.eval()
    starts = choose_eval_starts(build_lm_starts(tokens.numel(), seq_len, seq_len), batch_size=batch_size,
                                eval_batches=eval_batches, seed=seed)
    tot_ce, tot_tok = 0.0, 0
    with torch.no_grad():
        for i in range(0, len(starts), batch_size):
            inp, tgt = batch_from_starts(tokens, starts[i: i + batch_size], seq_len, torch.device(device))
            logits = model(inp)["logits"].float()
            tot_ce += float(torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]),
                                                              tgt.reshape(-1), reduction="sum"))
            tot_tok += tgt.numel()
    return {"mean_ce": tot_ce / max(tot_tok, 1), "tokens": tot_tok,
            "bpb": compute_bpb(tot_ce, tot_tok * raw_bytes_per_token),
            "artifact_bytes": Path(path).stat().st_size}
