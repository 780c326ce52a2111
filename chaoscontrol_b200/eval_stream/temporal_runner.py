"""Temporal-heads evaluation driver: per-document, chunked, state-carrying
scoring under one of several conditions, with per-document JSONL records, an
optional per-document analysis stream and a budget / provenance summary
(scripts/run_exp22_temporal_heads.py:1-582).

Conditions
    ``score_only``                 one pass, unshifted horizon
    ``single_horizon``             one head with one ``log_a`` shift
    ``temporal_heads``             H heads with different shifts, mixed in log-probability space
    ``identical_heads_uniform``    H identical heads, uniform mixer: must reproduce ``score_only``
    ``same_horizon_virtual_depth`` compute-matched control: the layers re-run
                                   ``depth_recurrence_count`` times instead of H heads
``gated_temporal_heads`` is refused, as in the reference: no pre-registered gate exists.

Documents come from a validation cache directory, or from JSONL files plus a
SentencePiece model.  The first token of every chunk after a document's first
is scored from the previous chunk's last-position distribution, so chunking
never drops a target.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Iterable, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

from ..scoring import compute_bpb
from .budget import BudgetTracker, EvalDeadline
from .temporal_heads import (TemporalHeadConfig, make_same_horizon_virtual_depth_config,
                             score_temporal_heads_chunk, update_online_exp_weighted_log_weights)

__all__ = ["CONDITIONS", "Exp22RunConfig", "run", "main"]

CONDITIONS = ("score_only", "single_horizon", "temporal_heads", "identical_heads_uniform",
              "gated_temporal_heads", "same_horizon_virtual_depth")


@dataclass
class Exp22RunConfig:
    condition: str = "temporal_heads"
    horizon_shifts: tuple[float, ...] = (-0.5, 0.0, 0.5)
    head_ids: Optional[tuple[str, ...]] = None
    chunk_size: int = 256
    max_docs: int = 50_000
    seed: int = 0
    budget_seconds: float = 600.0
    score_floor_seconds: float = 0.0
    safety_margin_seconds: float = 0.0
    checkpoint_path: str = ""
    output_path: str = ""
    summary_path: str = ""
    analysis_path: str = ""
    evidence_label: str = "exploratory"
    depth_recurrence_count: int = 3
    mixer: str = "uniform_logprob"
    mixer_weights: Optional[tuple[float, ...]] = None
    online_eta: float = 1.0
    online_initial_weights: Optional[tuple[float, ...]] = None


def _sha256_file(path: Path) -> Optional[str]:
    if not path.is_file():
        return None
    h = hashlib.sha256()
    with path.open("rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _hash_cfg(cfg: dict) -> str:
    return hashlib.sha256(json.dumps(cfg, sort_keys=True, default=str).encode()).hexdigest()[:16]


def _keyed(d: dict) -> dict[str, Any]:
    return {str(k): v for k, v in d.items()}


def _mean_layer_summaries(samples: dict) -> dict:
    """Per head: chunk-by-chunk lists of per-layer stat dicts -> one list of per-layer means."""
    out = {}
    for key, chunks in samples.items():
        if not chunks:
            continue
        layers = []
        for li in range(max(len(c) for c in chunks)):
            rows = [c[li] for c in chunks if li < len(c) and c[li] is not None]
            fields = sorted({f for r in rows for f in r})
            layers.append({f: (float(np.mean([r[f] for r in rows if r.get(f) is not None]))
                               if any(r.get(f) is not None for r in rows) else None) for f in fields})
        out[key] = layers
    return out


def _build_model(cfg: Exp22RunConfig, device: torch.device, model=None) -> tuple[torch.nn.Module, dict]:
    """The checkpoint's model; for the virtual-depth control the same weights in a model whose
    layers repeat (experiments/22: compute matched to H heads)."""
    if model is not None:
        return model.to(device).eval(), {}
    from ..models.model import CareStudentLM
    ck = torch.load(cfg.checkpoint_path, map_location="cpu", weights_only=False)
    mcfg = dict(ck.get("config") or {})
    if cfg.condition == "same_horizon_virtual_depth":
        mcfg = make_same_horizon_virtual_depth_config(mcfg, depth_recurrence_count=cfg.depth_recurrence_count)
    from ..runner_fast_path import build_model
    dtype = next(iter(ck["model"].values())).dtype
    m = build_model(mcfg, device, dtype) if mcfg else CareStudentLM(**ck["model_kwargs"]).to(device)
    m.load_state_dict(ck["model"], strict=False)
    return m.eval(), mcfg


def _docs(val_cache_dir: Optional[str], jsonl_paths: Optional[Sequence[str]], sp_model_path: Optional[str],
          max_docs: int) -> Iterable[tuple[int, np.ndarray, int]]:
    if val_cache_dir:
        from .io import load_val_cache
        vc = load_val_cache(Path(val_cache_dir))
        for i, doc in enumerate(vc.iter_docs()):
            if i >= max_docs:
                return
            yield int(doc.doc_id), np.asarray(vc.tokens_for_doc(doc)).astype(np.int64), int(doc.raw_bytes)
        return
    from .io import DocStreamer
    for rec in DocStreamer(jsonl_paths=[Path(p) for p in jsonl_paths or []], sp_model_path=Path(sp_model_path),
                           max_docs=max_docs):
        yield int(rec.doc_id), np.asarray(rec.tokens, dtype=np.int64), int(rec.raw_bytes)


def _boundary_nll(log_probs: torch.Tensor, target: torch.Tensor) -> float:
    return float(-log_probs.reshape(-1, log_probs.shape[-1])[0, int(target.reshape(-1)[0])])


@torch.no_grad()
def _direct_chunk(model, chunk: torch.Tensor, states):
    """Plain scoring of one chunk with carried state: ``(nll sum, targets, final states, last log-probs)``."""
    out = model(chunk, initial_states=states)
    logp = F.log_softmax(out["logits"][0].float(), dim=-1)
    n = chunk.shape[1] - 1
    nll = float(-logp[:-1].gather(-1, chunk[0, 1:, None]).sum()) if n > 0 else 0.0
    return nll, n, out.get("final_states"), logp[-1]


@torch.no_grad()
def run(cfg: Exp22RunConfig, *, val_cache_dir: Optional[str] = None, jsonl_paths: Optional[Sequence[str]] = None,
        sp_model_path: Optional[str] = None, model: Optional[torch.nn.Module] = None,
        device: Optional[torch.device] = None) -> dict[str, Any]:
    if cfg.condition not in CONDITIONS:
        raise ValueError(f"unknown condition {cfg.condition!r}; one of {CONDITIONS}")
    if cfg.condition == "gated_temporal_heads":
        raise NotImplementedError("gated_temporal_heads is not wired into this runner: run temporal_heads for "
                                  "always-on heads, or pre-register a previous-chunk gate first")
    torch.manual_seed(cfg.seed)
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model, ckpt_cfg = _build_model(cfg, device, model)
    shifts = tuple(float(x) for x in cfg.horizon_shifts)
    head_ids = tuple(str(x) for x in cfg.head_ids) if cfg.head_ids else None
    if cfg.condition == "identical_heads_uniform":
        if any(s != 0.0 for s in shifts):
            raise ValueError("identical_heads_uniform requires every horizon shift to be 0.0")
        if len(shifts) < 2:
            raise ValueError("identical_heads_uniform requires at least two heads")
        if cfg.mixer != "uniform_logprob":
            raise ValueError("identical_heads_uniform requires mixer='uniform_logprob'")
        head_ids = head_ids or tuple(f"same_{i}" for i in range(len(shifts)))
    if cfg.condition == "single_horizon" and len(shifts) != 1:
        raise ValueError("single_horizon requires exactly one horizon shift")
    tcfg = TemporalHeadConfig(
        horizon_shifts=shifts, head_ids=head_ids, mixer=cfg.mixer,
        mixer_weights=tuple(map(float, cfg.mixer_weights)) if cfg.mixer_weights else None,
        online_eta=float(cfg.online_eta),
        online_initial_weights=tuple(map(float, cfg.online_initial_weights)) if cfg.online_initial_weights else None)
    temporal = cfg.condition in ("single_horizon", "temporal_heads", "identical_heads_uniform")
    keys = tcfg.head_ids or tcfg.horizon_shifts
    budget = BudgetTracker(total_budget_seconds=cfg.budget_seconds, score_floor_seconds=cfg.score_floor_seconds,
                           safety_margin_seconds=cfg.safety_margin_seconds)
    deadline = EvalDeadline(cfg.budget_seconds)
    out_fh = analysis_fh = None
    if cfg.output_path:
        Path(cfg.output_path).parent.mkdir(parents=True, exist_ok=True)
        out_fh = open(cfg.output_path, "w")
    if cfg.analysis_path:
        Path(cfg.analysis_path).parent.mkdir(parents=True, exist_ok=True)
        analysis_fh = open(cfg.analysis_path, "w")
    tot = {"docs": 0, "chunks": 0, "tokens": 0, "loss": 0.0, "bytes": 0}
    winners_total = {k: 0 for k in keys}
    timed_out = False
    try:
        for doc_id, toks, raw_bytes in _docs(val_cache_dir, jsonl_paths, sp_model_path, cfg.max_docs):
            if deadline.is_expired():
                timed_out = True
                break
            t_doc = time.monotonic()
            loss, ntok, nchunks = 0.0, 0, 0
            head_loss = {k: 0.0 for k in keys}
            winners = {k: 0 for k in keys}
            half_life: dict = {k: [] for k in keys}
            divergence: dict = {}
            states_by = {k: None for k in keys}
            states = prev_mixed = prev_heads = online_w = prev_direct = None
            for lo in range(0, len(toks), cfg.chunk_size):
                chunk = torch.as_tensor(toks[lo:lo + cfg.chunk_size], device=device).unsqueeze(0)
                t0 = time.monotonic()
                first = chunk[:, 0]
                if temporal:
                    if prev_mixed is not None:
                        loss += _boundary_nll(prev_mixed, first)
                        ntok += 1
                        if prev_heads is not None:
                            per = {k: _boundary_nll(lp, first) for k, lp in prev_heads.items()}
                            for k, v in per.items():
                                head_loss[k] += v
                            winners[min(per, key=per.get)] += 1
                            if tcfg.mixer == "online_exp_weights_logprob" and online_w is not None:
                                online_w = update_online_exp_weighted_log_weights(
                                    online_w, [prev_heads[k] for k in keys], first, eta=tcfg.online_eta)
                    res = score_temporal_heads_chunk(model, chunk, states_by_shift=states_by, cfg=tcfg,
                                                     online_initial_log_weights=online_w)
                    states_by, prev_mixed = res.final_states_by_shift, res.last_mixed_log_probs
                    prev_heads, online_w = res.last_log_probs_by_shift, res.online_final_log_weights
                    loss += res.loss_nats
                    ntok += res.tokens_scored
                    for k, v in res.per_head_loss_nats.items():
                        head_loss[k] += v
                    for k, v in res.winner_counts_by_shift.items():
                        winners[k] = winners.get(k, 0) + v
                    for k, v in res.half_life_stats_by_shift.items():
                        half_life.setdefault(k, []).append(v)
                    for k, v in res.state_divergence_by_shift.items():
                        divergence.setdefault(k, []).append(v)
                else:
                    if prev_direct is not None:
                        loss += _boundary_nll(prev_direct, first)
                        ntok += 1
                    nll, n, states, prev_direct = _direct_chunk(model, chunk, states)
                    loss += nll
                    ntok += n
                nchunks += 1
                budget.add_score_time(time.monotonic() - t0)
            tot["docs"] += 1
            tot["chunks"] += nchunks
            tot["tokens"] += ntok
            tot["loss"] += loss
            tot["bytes"] += raw_bytes
            for k, v in winners.items():
                winners_total[k] = winners_total.get(k, 0) + v
            if out_fh is not None:
                rec = {"doc_id": doc_id, "condition": cfg.condition, "tokens": ntok, "chunks": nchunks,
                       "loss_nats": loss, "raw_bytes": raw_bytes, "bpb": compute_bpb(loss, raw_bytes),
                       "wall_seconds": time.monotonic() - t_doc}
                if temporal:
                    rec["per_head_loss_nats"] = _keyed(head_loss)
                out_fh.write(json.dumps(rec, sort_keys=True) + "\n")
            if analysis_fh is not None and temporal:
                analysis_fh.write(json.dumps({
                    "doc_id": doc_id, "mixer": tcfg.mixer, "horizon_shifts": list(shifts),
                    "head_ids": list(head_ids) if head_ids else None, "chunks": nchunks, "tokens": ntok,
                    "online_eta": tcfg.online_eta, "winner_counts_by_shift": _keyed(winners),
                    "half_life_stats_by_shift": _keyed(_mean_layer_summaries(half_life)),
                    "state_divergence_by_shift": _keyed(_mean_layer_summaries(divergence))},
                    sort_keys=True) + "\n")
    finally:
        for fh in (out_fh, analysis_fh):
            if fh is not None:
                fh.close()
    ck = Path(cfg.checkpoint_path) if cfg.checkpoint_path else None
    summary = budget.summary(
        docs_scored=tot["docs"], chunks_scored=tot["chunks"], tokens_scored=tot["tokens"], adapt_steps=0,
        timed_out=timed_out, collapsed=False, score_only_mode=cfg.condition == "score_only",
        elapsed_seconds=deadline.elapsed(), ckpt_sha256=_sha256_file(ck) if ck else None,
        ckpt_cfg_hash=_hash_cfg(ckpt_cfg), stream_seed=cfg.seed,
        gpu_name=torch.cuda.get_device_name(0) if device.type == "cuda" else None,
        torch_version=torch.__version__, cuda_version=torch.version.cuda, chunk_size=cfg.chunk_size,
        max_docs=cfg.max_docs)
    summary.update({
        "condition": cfg.condition, "evidence_label": cfg.evidence_label,
        "aggregate_bpb": compute_bpb(tot["loss"], tot["bytes"]), "aggregate_loss_nats": tot["loss"],
        "aggregate_raw_bytes": tot["bytes"], "horizon_shifts": list(shifts),
        "head_ids": list(head_ids) if head_ids else None, "mixer": tcfg.mixer,
        "mixer_weights": list(tcfg.mixer_weights) if tcfg.mixer_weights else None,
        "online_eta": tcfg.online_eta,
        "online_initial_weights": list(tcfg.online_initial_weights) if tcfg.online_initial_weights else None,
        "analysis_path": cfg.analysis_path or None, "temporal_head_count": len(keys) if temporal else 1,
        "depth_recurrence_count": cfg.depth_recurrence_count if cfg.condition == "same_horizon_virtual_depth" else 1,
        "winner_counts_by_shift": _keyed(winners_total) if temporal else None,
        "config": {k: (list(v) if isinstance(v, tuple) else v) for k, v in asdict(cfg).items()}})
    if cfg.summary_path:
        Path(cfg.summary_path).parent.mkdir(parents=True, exist_ok=True)
        Path(cfg.summary_path).write_text(json.dumps(summary, indent=2, sort_keys=True, default=str))
    return summary


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", type=Path, default=None, help="YAML with Exp22RunConfig fields")
    ap.add_argument("--condition", choices=CONDITIONS, default=None)
    ap.add_argument("--checkpoint-path", default=None)
    ap.add_argument("--val-cache-dir", default=None)
    ap.add_argument("--jsonl-paths", nargs="*", default=None)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--output-path", default=None)
    ap.add_argument("--summary-path", default=None)
    ap.add_argument("--analysis-path", default=None)
    ap.add_argument("--horizon-shifts", type=float, nargs="+", default=None)
    ap.add_argument("--mixer", default=None)
    ap.add_argument("--chunk-size", type=int, default=None)
    ap.add_argument("--max-docs", type=int, default=None)
    ap.add_argument("--budget-seconds", type=float, default=None)
    a = ap.parse_args(argv)
    fields: dict[str, Any] = {}
    if a.config:
        import yaml
        fields.update(yaml.safe_load(a.config.read_text()) or {})
    for k in ("condition", "checkpoint_path", "output_path", "summary_path", "analysis_path", "mixer",
              "chunk_size", "max_docs", "budget_seconds"):
        if getattr(a, k) is not None:
            fields[k] = getattr(a, k)
    if a.horizon_shifts is not None:
        fields["horizon_shifts"] = tuple(a.horizon_shifts)
    for k in ("horizon_shifts", "head_ids", "mixer_weights", "online_initial_weights"):
        if fields.get(k) is not None:
            fields[k] = tuple(fields[k])
    if not a.val_cache_dir and not (a.jsonl_paths and a.sp_model_path):
        ap.error("give --val-cache-dir, or --jsonl-paths with --sp-model-path")
    s = run(Exp22RunConfig(**fields), val_cache_dir=a.val_cache_dir, jsonl_paths=a.jsonl_paths,
            sp_model_path=a.sp_model_path)
    print(json.dumps({k: s[k] for k in ("condition", "aggregate_bpb", "docs_scored", "tokens_scored",
                                        "elapsed_seconds") if k in s}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
