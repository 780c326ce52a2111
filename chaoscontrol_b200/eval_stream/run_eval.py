"""Test-time-training evaluation driver: checkpoint + documents + `RunConfig`
-> per-document JSONL and a budget / provenance summary
(scripts/run_exp20_eval.py:1-398).

Documents come from a validation cache directory or from JSONL files plus a
SentencePiece model.  On a GPU the common setting (SGD, one step per chunk,
``reset`` persistence) runs through the CUDA-graph chunk runner; everything
else takes the eager score-then-adapt loop.  ``adapt_set: none`` is plain
chunked scoring with carried state.

``python -m chaoscontrol_b200.eval_stream.run_eval --config run.yaml
--val-cache-dir val/ [--adapt-set lm_head --steps-per-chunk 1 ...]``
"""
from __future__ import annotations

import argparse
import hashlib
import json
from dataclasses import asdict
from pathlib import Path
from typing import Any, Iterator, Optional, Sequence

import torch

from .types import DocRecord, RunConfig

__all__ = ["iter_docs", "run", "main"]


def iter_docs(*, val_cache_dir: Optional[str] = None, jsonl_paths: Optional[Sequence[str]] = None,
              sp_model_path: Optional[str] = None, max_docs: int = 50_000) -> Iterator[DocRecord]:
    if val_cache_dir:
        from .io import load_val_cache
        vc = load_val_cache(Path(val_cache_dir))
        for i, doc in enumerate(vc.iter_docs()):
            if i >= max_docs:
                return
            yield DocRecord(doc_id=int(doc.doc_id), tokens=vc.tokens_for_doc(doc).astype("int64").tolist(),
                            raw_bytes=int(doc.raw_bytes))
        return
    if not (jsonl_paths and sp_model_path):
        raise ValueError("give val_cache_dir, or jsonl_paths with sp_model_path")
    from .io import DocStreamer
    yield from DocStreamer(jsonl_paths=[Path(p) for p in jsonl_paths], sp_model_path=Path(sp_model_path),
                           max_docs=max_docs)


def _sha256(path: Path) -> Optional[str]:
    if not path.is_file():
        return None
    h = hashlib.sha256()
    with path.open("rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def run(cfg: RunConfig, *, val_cache_dir: Optional[str] = None, jsonl_paths: Optional[Sequence[str]] = None,
        sp_model_path: Optional[str] = None, model: Optional[torch.nn.Module] = None,
        device: Optional[torch.device] = None, optimizer: str = "sgd", use_graph: Optional[bool] = None,
        batched: Optional[bool] = None) -> dict[str, Any]:
    from ..scoring import run_ttt_eval, run_ttt_eval_graph
    torch.manual_seed(cfg.seed)
    device = device or torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    ckpt_cfg: dict = {}
    if model is None:
        from ..fast_score import _load_model
        model, ckpt_cfg = _load_model(cfg.checkpoint_path, device)
    model = model.to(device)
    if cfg.episodic_cache_enabled:
        raise ValueError("episodic_cache_enabled: the eval-time episodic cache runs as the packet_online_cache / "
                         "adaptive_carry evaluation passes (config key calc_types), not in this driver")
    metrics = None
    if cfg.output_path:
        from .io import MetricsCollector
        Path(cfg.output_path).parent.mkdir(parents=True, exist_ok=True)
        metrics = MetricsCollector(output_path=Path(cfg.output_path))
    docs = iter_docs(val_cache_dir=val_cache_dir, jsonl_paths=jsonl_paths, sp_model_path=sp_model_path,
                     max_docs=cfg.max_docs)
    graph_ok = (device.type == "cuda" and cfg.adapt_set != "none" and cfg.persistence_mode == "reset"
                and cfg.steps_per_chunk == 1 and optimizer == "sgd" and cfg.chunk_size > 0
                and cfg.delta_scale == 1.0 and cfg.log_a_shift == 0.0)
    if use_graph is None:
        use_graph = graph_ok
    if use_graph and not graph_ok:
        raise ValueError("the graph runner covers SGD, one step per chunk, reset persistence on a GPU only")
    driver = None
    try:
        from .batched_ttt import SUPPORTED_ADAPT_SETS, BatchedTTT, run_ttt_eval_batched
        if (use_graph and batched is not False and metrics is None and cfg.adapt_set in SUPPORTED_ADAPT_SETS
                and BatchedTTT.supported(model)):
            # many documents per step; per-document metric rows need the one-document-at-a-time drivers
            out = run_ttt_eval_batched(model, docs, adapt_set=cfg.adapt_set, chunk_size=cfg.chunk_size,
                                       eval_lr=cfg.eval_lr, max_docs=cfg.max_docs)
            out.pop("runner", None)
            driver = "batched"
        elif use_graph:
            out = run_ttt_eval_graph(model, docs, adapt_set=cfg.adapt_set, chunk_size=cfg.chunk_size,
                                     eval_lr=cfg.eval_lr, max_docs=cfg.max_docs, metrics=metrics)
        else:
            out = run_ttt_eval(model, docs, adapt_set=cfg.adapt_set, persistence_mode=cfg.persistence_mode,
                               chunk_size=cfg.chunk_size, steps_per_chunk=cfg.steps_per_chunk, eval_lr=cfg.eval_lr,
                               optimizer=optimizer, budget_seconds=cfg.budget_seconds,
                               score_floor_seconds=cfg.score_floor_seconds,
                               safety_margin_seconds=cfg.safety_margin_seconds, delta_scale=cfg.delta_scale,
                               log_a_shift=cfg.log_a_shift, metrics=metrics, max_docs=cfg.max_docs)
    finally:
        if metrics is not None and hasattr(metrics, "close"):
            metrics.close()
    summary = {k: v for k, v in out.items() if k != "per_doc_ce"}
    ck = Path(cfg.checkpoint_path) if cfg.checkpoint_path else None
    summary.update({
        "driver": driver or ("graph" if use_graph else "eager"), "config": asdict(cfg),
        "ckpt_sha256": _sha256(ck) if ck else None,
        "ckpt_cfg_hash": hashlib.sha256(json.dumps(ckpt_cfg, sort_keys=True, default=str).encode()).hexdigest()[:16],
        "gpu_name": torch.cuda.get_device_name(device) if device.type == "cuda" else None,
        "torch_version": torch.__version__, "cuda_version": torch.version.cuda})
    if cfg.summary_path:
        Path(cfg.summary_path).parent.mkdir(parents=True, exist_ok=True)
        Path(cfg.summary_path).write_text(json.dumps(summary, indent=2, sort_keys=True, default=str))
    return summary


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", type=Path, default=None, help="YAML with RunConfig fields")
    ap.add_argument("--val-cache-dir", default=None)
    ap.add_argument("--jsonl-paths", nargs="*", default=None)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--optimizer", choices=("sgd", "muon"), default="sgd")
    ap.add_argument("--eager", action="store_true", help="never use the CUDA-graph chunk runner")
    for name, typ in (("adapt_set", str), ("persistence_mode", str), ("chunk_size", int), ("steps_per_chunk", int),
                      ("eval_lr", float), ("max_docs", int), ("budget_seconds", float), ("checkpoint_path", str),
                      ("output_path", str), ("summary_path", str), ("seed", int)):
        ap.add_argument("--" + name.replace("_", "-"), type=typ, default=None)
    a = ap.parse_args(argv)
    fields: dict[str, Any] = {}
    if a.config:
        import yaml
        fields.update(yaml.safe_load(a.config.read_text()) or {})
        # matrix builders write a label and the data paths beside the run fields; flags win over them
        fields.pop("name", None)
        fields.pop("phase", None)
        for key in ("val_cache_dir", "jsonl_paths", "sp_model_path"):
            v = fields.pop(key, None)
            if getattr(a, key) is None and v:
                setattr(a, key, v)
    for k, v in vars(a).items():
        if v is not None and k not in ("config", "val_cache_dir", "jsonl_paths", "sp_model_path", "optimizer", "eager"):
            fields[k] = v
    s = run(RunConfig.from_dict(fields), val_cache_dir=a.val_cache_dir, jsonl_paths=a.jsonl_paths,
            sp_model_path=a.sp_model_path, optimizer=a.optimizer, use_graph=False if a.eager else None)
    print(json.dumps({k: s.get(k) for k in ("bpb", "docs_scored", "tokens_scored", "adapt_steps", "driver")}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
