"""Document-parallel score-only evaluation driver (behaviour of
scripts/run_exp20_fast_score.py:60-1494): document packing policies, rank assignment,
the forward-token budget, token-coverage validation, an optional CUDA-graph chunk
scorer, and the ``run`` entry point / command line.

    python -m chaoscontrol_b200.fast_score --cache-dir VAL --checkpoint-path CKPT --output-path out.json
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m chaoscontrol_b200.fast_score ...

Scoring itself is :func:`chaoscontrol_b200.scoring.score_docs`: length-sorted blocks of
documents run chunk by chunk through the kernel trunk with a native ``h0 -> hT`` carry and the
fused LM head (no logits, no per-token loop).

Where the reference finds its largest batch by running forwards until one no longer raises an
out-of-memory error (run_exp20_fast_score.py:486-525), the budget here is ARITHMETIC: bytes per
token of the scorer's live tensors against the free memory the device reports.  Nothing is ever
driven out of memory to find a limit.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Optional, Sequence

import numpy as np
import torch
import torch.nn as nn

from .eval_stream.io import CachedDoc, load_val_cache
from .scoring import _chunk_loss_rows, compute_bpb, score_docs

DEFAULT_MAX_FORWARD_TOKENS = 1 << 19
DOC_PACKINGS = ("source_order", "token_len_desc", "chunk_count_desc", "chunk_count_tail")

__all__ = ["chunk_count_for_doc", "padded_token_work", "resolve_doc_packing", "prepare_doc_work",
           "prepare_rank_doc_work", "doc_range_for_rank", "resolve_doc_batch_size", "resolve_max_forward_tokens",
           "estimate_max_forward_tokens", "expected_scored_tokens", "validate_doc_score_coverage",
           "record_order_safe_reason", "GraphChunkScorer", "run", "main", "DocWork"]


@dataclass
class DocWork:
    doc: CachedDoc
    output_index: int


# ---------------------------------------------------------------- packing
def chunk_count_for_doc(doc: CachedDoc, *, chunk_size: int) -> int:
    if chunk_size < 0:
        return 1 if int(doc.token_len) >= 2 else 0
    return max(1, -(-int(doc.token_len) // int(chunk_size)))


def padded_token_work(doc: CachedDoc, *, chunk_size: int) -> int:
    return int(doc.token_len) if chunk_size < 0 else chunk_count_for_doc(doc, chunk_size=chunk_size) * int(chunk_size)


def resolve_doc_packing(*, doc_packing: Optional[str], sort_docs_by_length: Optional[bool]) -> str:
    if doc_packing:
        return doc_packing
    if sort_docs_by_length is None:
        return "chunk_count_tail"
    return "token_len_desc" if sort_docs_by_length else "source_order"


def _packing_key(item: DocWork, packing: str, chunk_size: int) -> tuple:
    n = int(item.doc.token_len)
    chunks = chunk_count_for_doc(item.doc, chunk_size=chunk_size)
    # documents whose last chunk is similarly full sit together: less padding in the final block
    tail_bucket = 0 if chunk_size < 0 else (n % int(chunk_size)) // min(32, max(1, int(chunk_size)))
    keys = {"source_order": (item.output_index,), "token_len_desc": (-n, item.output_index),
            "chunk_count_desc": (-chunks, -n, item.output_index),
            "chunk_count_tail": (-chunks, tail_bucket, -n, item.output_index)}
    if packing not in keys:
        raise ValueError(f"unsupported doc_packing: {packing}")
    return keys[packing]


def prepare_doc_work(docs: Sequence[CachedDoc], *, sort_by_length: Optional[bool] = None,
                     doc_packing: Optional[str] = None, chunk_size: int = 256, start_index: int = 0) -> list[DocWork]:
    packing = resolve_doc_packing(doc_packing=doc_packing, sort_docs_by_length=sort_by_length)
    work = [DocWork(d, start_index + i) for i, d in enumerate(docs)]
    if packing == "source_order":
        return work
    return sorted(work, key=lambda w: _packing_key(w, packing, chunk_size))


def doc_range_for_rank(*, num_docs: int, rank: int, world_size: int) -> tuple[int, int]:
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank must be in [0, {world_size}), got {rank}")
    return num_docs * rank // world_size, num_docs * (rank + 1) // world_size


def prepare_rank_doc_work(docs: Sequence[CachedDoc], *, rank: int, world_size: int, doc_packing: str,
                          chunk_size: int, doc_batch_size: int) -> list[DocWork]:
    """This rank's share.  ``source_order`` gives contiguous ranges; every other policy packs the global
    order into batches of ``doc_batch_size`` and deals the batches out longest-work-first to the least
    loaded rank."""
    if doc_packing == "source_order":
        lo, hi = doc_range_for_rank(num_docs=len(docs), rank=rank, world_size=world_size)
        return prepare_doc_work(docs[lo:hi], doc_packing="source_order", chunk_size=chunk_size, start_index=lo)
    work = prepare_doc_work(docs, doc_packing=doc_packing, chunk_size=chunk_size)
    if world_size <= 1:
        return work
    bs = max(1, int(doc_batch_size))
    batches = [work[i:i + bs] for i in range(0, len(work), bs)]
    cost = [sum(padded_token_work(w.doc, chunk_size=chunk_size) for w in b) for b in batches]
    loads = [0] * world_size
    mine: list[DocWork] = []
    for bi in sorted(range(len(batches)), key=lambda i: -cost[i]):
        r = min(range(world_size), key=lambda k: (loads[k], k))
        loads[r] += cost[bi]
        if r == rank:
            mine.extend(batches[bi])
    return mine


# ---------------------------------------------------------------- batch budget
def resolve_doc_batch_size(*, requested_doc_batch_size: int, chunk_size: int, max_forward_tokens: int) -> int:
    want = max(1, int(requested_doc_batch_size))
    if chunk_size < 0 or max_forward_tokens <= 0:
        return want
    return min(want, max(1, int(max_forward_tokens) // max(1, int(chunk_size))))


def estimate_max_forward_tokens(model: nn.Module, *, device: torch.device, safety: float = 0.5) -> int:
    """Tokens per forward block that fit in the free device memory, from the scorer's per-token
    footprint: the kernel trunk keeps about ``(6 + 2 * ff_mult) * dim`` bf16 values per token alive
    inside a layer and the fused head adds a few floats; the PyTorch fallback also holds fp32 logits."""
    if device.type != "cuda":
        return DEFAULT_MAX_FORWARD_TOKENS
    free, _total = torch.cuda.mem_get_info(device)
    dim = int(getattr(model, "dim", 256))
    ff = int(model.layers[0].ff.fc.out_features) if hasattr(model, "layers") and len(model.layers) else 2 * dim
    per_token = 2 * (6 * dim + 2 * ff) + 64
    if not getattr(model, "kernel_trunk_supported", lambda: False)():
        per_token += 4 * int(model.lm_head.out_features) * 2
    return max(1, int(free * float(safety)) // per_token)


def resolve_max_forward_tokens(*, max_forward_tokens, requested_doc_batch_size: int, chunk_size: int,
                               device: torch.device, probe_fn: Optional[Callable[[int], int]] = None) -> int:
    """An explicit positive integer wins; ``"auto"`` asks ``probe_fn(requested_tokens)`` (the memory
    estimate) and never exceeds what the requested batch needs."""
    if isinstance(max_forward_tokens, int) or str(max_forward_tokens).lower() != "auto":
        value = int(max_forward_tokens)
        if value <= 0:
            raise ValueError(f"max_forward_tokens must be positive or 'auto', got {max_forward_tokens!r}")
        return value
    if chunk_size < 0:
        return 0
    want = max(1, int(requested_doc_batch_size)) * max(1, int(chunk_size))
    if device.type != "cuda":
        return want
    if probe_fn is None:
        return min(want, DEFAULT_MAX_FORWARD_TOKENS)
    return max(1, min(want, int(probe_fn(want))))


# ---------------------------------------------------------------- coverage
def expected_scored_tokens(*, token_len: int, chunk_size: int, score_boundary_targets: bool) -> int:
    """Targets a document must contribute: ``len - 1`` when chunk-boundary targets are scored (or the
    document is one chunk), else ``len - 1`` minus one per chunk boundary."""
    n = int(token_len)
    if n < 2:
        return 0
    if chunk_size < 0 or score_boundary_targets:
        return n - 1
    return sum(min(s + chunk_size, n) - s - 1 for s in range(0, n, chunk_size) if min(s + chunk_size, n) - s >= 2)


def validate_doc_score_coverage(*, doc: CachedDoc, tokens_scored: int, chunk_size: int,
                                score_boundary_targets: bool) -> None:
    want = expected_scored_tokens(token_len=doc.token_len, chunk_size=chunk_size,
                                  score_boundary_targets=score_boundary_targets)
    if int(tokens_scored) != want:
        raise RuntimeError(f"token coverage mismatch doc_id={doc.doc_id} expected={want} actual={tokens_scored} "
                           f"token_len={doc.token_len} chunk_size={chunk_size} "
                           f"score_boundary_targets={score_boundary_targets}")


def record_order_safe_reason(*, persistence_mode: str, score_only_mode: bool, doc_packing: str) -> str:
    if doc_packing == "source_order":
        return "source_order_preserved"
    if persistence_mode == "reset" and score_only_mode:
        return "reset_score_only_commutative_ce_reduction"
    return "not_order_safe_for_stateful_or_adaptive_eval"


# ---------------------------------------------------------------- CUDA-graph chunk scorer
class GraphChunkScorer:
    """Two captured graphs over static ``[batch, chunk + 1]`` token buffers: one that starts from a
    zero state and one that starts from ``static_prev_states``.  A replay copies the block (and the
    states) into the static buffers and returns per-position CE rows and the final states, which
    live in static outputs until the next replay."""

    def __init__(self, model: nn.Module, *, batch_size: int, chunk_size: int, device: torch.device) -> None:
        if device.type != "cuda":
            raise RuntimeError("graph scoring requires CUDA")
        if batch_size <= 0 or chunk_size < 1:
            raise ValueError("graph scoring requires batch_size > 0 and chunk_size >= 1")
        self.model, self.batch_size, self.chunk_size, self.device = model, int(batch_size), int(chunk_size), device
        self.static_block = torch.zeros(self.batch_size, self.chunk_size + 1, dtype=torch.long, device=device)
        with torch.no_grad():
            _rows, finals = self._forward(None)
        self.static_prev_states = [torch.zeros_like(f, dtype=torch.float32) for f in finals]
        self.zero_graph, self.carry_graph = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(3):
                self._forward(None)
                self._forward(self.static_prev_states)
        torch.cuda.current_stream(device).wait_stream(side)
        with torch.cuda.graph(self.zero_graph), torch.no_grad():
            self.zero_rows, self.zero_finals = self._forward(None)
        with torch.cuda.graph(self.carry_graph), torch.no_grad():
            self.carry_rows, self.carry_finals = self._forward(self.static_prev_states)

    def _forward(self, states):
        blk = self.static_block
        return _chunk_loss_rows(self.model, blk[:, :-1].contiguous(), blk[:, 1:].contiguous(), states)

    def replay(self, block: torch.Tensor, states: Optional[list] = None):
        if tuple(block.shape) != tuple(self.static_block.shape):
            raise ValueError(f"graph block shape {tuple(block.shape)} != {tuple(self.static_block.shape)}")
        self.static_block.copy_(block, non_blocking=True)
        if states is None:
            self.zero_graph.replay()
            return self.zero_rows, self.zero_finals
        if len(states) != len(self.static_prev_states):
            raise ValueError("graph initial state count mismatch")
        for dst, src in zip(self.static_prev_states, states):
            dst.copy_(src, non_blocking=True)
        self.carry_graph.replay()
        return self.carry_rows, self.carry_finals


# ---------------------------------------------------------------- run
def _sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for blk in iter(lambda: fh.read(1 << 20), b""):
            h.update(blk)
    return h.hexdigest()


def _load_model(checkpoint_path: str, device: torch.device) -> tuple[nn.Module, dict]:
    from .config import ssm_constructor_kwargs
    from .models.model import CareStudentLM
    blob = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
    cfg = dict(blob["config"])
    kwargs = cfg if "dim" in cfg else ssm_constructor_kwargs(cfg)
    model = CareStudentLM(**kwargs)
    model.load_state_dict(blob["model"], strict=True)
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    return model.to(device=device, dtype=dtype).eval(), cfg


def run(*, cache_dir: str, checkpoint_path: Optional[str], output_path: Optional[str], chunk_size: int = 512,
        doc_batch_size: int = 1024, max_forward_tokens="auto", doc_packing: Optional[str] = None,
        max_docs: Optional[int] = None, budget_seconds: float = 600.0, model: Optional[nn.Module] = None,
        device: Optional[torch.device] = None, summary_path: Optional[str] = None,
        safety_margin_seconds: float = 0.0, sort_docs_by_length: Optional[bool] = None,
        score_warmup_steps: int = 0, per_doc_path: Optional[str] = None,
        episodic_cache_source: str = "auto", allow_online_replay_checkpoint: bool = False) -> dict[str, Any]:
    """Scores a validation cache with documents sharded over the launched ranks and returns (rank 0
    also writes) the aggregate summary: bpb, tokens, documents, timing and provenance.

    ``summary_path`` receives the summary and ``per_doc_path`` one JSON line per document (doc id, scored
    tokens, summed CE, bytes) -- the reference's ``--summary-path`` / ``--output-path`` pair; without
    ``summary_path`` the summary goes to ``output_path``.  ``safety_margin_seconds`` is taken off the budget,
    ``score_warmup_steps`` scores that many leading batches once before the timed pass (kernel warm-up).
    ``episodic_cache_source`` (auto | fresh | checkpoint) and ``allow_online_replay_checkpoint`` only check
    the checkpoint's payload: frozen-weight scoring never consults the episodic cache, so cold and warm
    caches score identically and the summary says which one was asked for."""
    import torch.distributed as dist
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device is None:
        device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)
    if ws > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo")
    if episodic_cache_source not in ("auto", "fresh", "checkpoint"):
        raise ValueError(f"episodic_cache_source must be auto, fresh or checkpoint; got {episodic_cache_source!r}")
    ckpt_cfg: dict = {}
    cache_state = "none"
    if model is None:
        if not checkpoint_path:
            raise ValueError("run() needs a model or a checkpoint_path")
        blob = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
        has_cache = isinstance(blob, dict) and blob.get("episodic_cache") is not None
        online = isinstance(blob, dict) and isinstance(blob.get("online_eval_state"), dict) and \
            blob["online_eval_state"].get("replay_eviction") is not None
        if online and not allow_online_replay_checkpoint:
            raise ValueError("checkpoint carries online replay-eviction state; frozen-weight scoring does not run "
                             "the memory control plane: pass allow_online_replay_checkpoint to score it anyway")
        if episodic_cache_source == "checkpoint" and not has_cache:
            raise ValueError("--episodic-cache-source=checkpoint requires ckpt['episodic_cache']; payload absent")
        cache_state = ("fresh_forced" if episodic_cache_source == "fresh" and has_cache else
                       "loaded" if has_cache and episodic_cache_source != "fresh" else "fresh")
        del blob
        model, ckpt_cfg = _load_model(checkpoint_path, device)
    cache = load_val_cache(Path(cache_dir))
    docs = list(cache.iter_docs())
    if max_docs is not None:
        docs = docs[: int(max_docs)]
    packing = resolve_doc_packing(doc_packing=doc_packing, sort_docs_by_length=sort_docs_by_length)
    mft = resolve_max_forward_tokens(max_forward_tokens=max_forward_tokens, requested_doc_batch_size=doc_batch_size,
                                     chunk_size=chunk_size, device=device,
                                     probe_fn=lambda want: estimate_max_forward_tokens(model, device=device))
    bs = resolve_doc_batch_size(requested_doc_batch_size=doc_batch_size, chunk_size=chunk_size, max_forward_tokens=mft)
    work = prepare_rank_doc_work(docs, rank=rank, world_size=ws, doc_packing=packing, chunk_size=chunk_size,
                                 doc_batch_size=bs)
    tokens = torch.as_tensor(np.asarray(cache.tokens).astype(np.int32), device=device)
    starts = np.asarray([w.doc.token_start for w in work], dtype=np.int64)
    lens = np.asarray([w.doc.token_len for w in work], dtype=np.int64)
    rawb = np.asarray([w.doc.raw_bytes for w in work], dtype=np.int64)
    if int(score_warmup_steps) > 0 and len(work):
        n_warm = min(len(work), int(score_warmup_steps) * bs)
        score_docs(model, tokens, starts[:n_warm], lens[:n_warm], chunk_size=chunk_size, max_batch_tokens=bs * chunk_size)
    t0 = time.perf_counter()
    res = score_docs(model, tokens, starts, lens, chunk_size=chunk_size, max_batch_tokens=bs * chunk_size,
                     raw_bytes=rawb, deadline_s=max(0.0, float(budget_seconds) - float(safety_margin_seconds)))
    for w, n in zip(work, res.doc_tokens):
        if not res.extra.get("timed_out"):
            validate_doc_score_coverage(doc=w.doc, tokens_scored=int(n), chunk_size=chunk_size,
                                        score_boundary_targets=True)
    sums = torch.tensor([res.total_ce, float(res.total_tokens), float(res.total_bytes), float(len(work)),
                         float(sum(padded_token_work(w.doc, chunk_size=chunk_size) for w in work))],
                        dtype=torch.float64, device=device)
    maxes = torch.tensor([res.elapsed_s, time.perf_counter() - t0], dtype=torch.float64, device=device)
    if ws > 1:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        dist.all_reduce(maxes, op=dist.ReduceOp.MAX)
    ce, ntok, nbytes, ndocs, padded = (float(v) for v in sums.cpu())
    elapsed = float(maxes[0])
    summary = {
        "bpb": compute_bpb(ce, nbytes), "mean_ce_nats": ce / max(ntok, 1.0), "total_ce_nats": ce,
        "tokens_scored": int(ntok), "docs_scored": int(ndocs), "total_raw_bytes": int(nbytes),
        "padded_token_work": int(padded), "elapsed_s": elapsed, "tokens_per_s": ntok / elapsed if elapsed > 0 else 0.0,
        "world_size": ws, "chunk_size": int(chunk_size), "doc_batch_size": int(bs), "max_forward_tokens": int(mft),
        "doc_packing": packing, "timed_out": bool(res.extra.get("timed_out")),
        "record_order_safe": record_order_safe_reason(persistence_mode="reset", score_only_mode=True,
                                                      doc_packing=packing),
        "score_warmup_steps": int(score_warmup_steps), "safety_margin_seconds": float(safety_margin_seconds),
        "episodic_cache": {"source": episodic_cache_source, "state": cache_state, "consulted": False},
        "provenance": {"checkpoint_path": checkpoint_path,
                       "checkpoint_sha256": _sha256(Path(checkpoint_path)) if checkpoint_path else None,
                       "config_hash": hashlib.sha1(json.dumps(ckpt_cfg, sort_keys=True, default=str).encode()
                                                   ).hexdigest()[:12],
                       "gpu": torch.cuda.get_device_name(device) if device.type == "cuda" else "cpu",
                       "torch": torch.__version__, "cuda": torch.version.cuda}}
    if per_doc_path:
        # every rank writes its own documents; rank 0 keeps the plain name, the others add their rank
        pp = Path(per_doc_path)
        if ws > 1 and rank > 0:
            pp = pp.with_name(f"{pp.stem}.rank{rank}{pp.suffix}")
        pp.parent.mkdir(parents=True, exist_ok=True)
        with pp.open("w") as fh:
            for w, n, ce in zip(work, res.doc_tokens, res.doc_ce):
                fh.write(json.dumps({"doc_id": int(w.doc.doc_id), "tokens_scored": int(n), "ce_nats": float(ce),
                                     "raw_bytes": int(w.doc.raw_bytes)}) + "\n")
    target = summary_path or output_path
    if rank == 0 and target:
        out = Path(target)
        out.parent.mkdir(parents=True, exist_ok=True)
        tmp = out.with_suffix(out.suffix + ".tmp")
        tmp.write_text(json.dumps(summary, indent=2))
        tmp.rename(out)
    return summary


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="document-parallel score-only evaluation")
    ap.add_argument("--cache-dir", required=True)
    ap.add_argument("--checkpoint-path", required=True)
    ap.add_argument("--output-path", default=None)
    ap.add_argument("--chunk-size", type=int, default=512)
    ap.add_argument("--doc-batch-size", type=int, default=1024)
    ap.add_argument("--max-forward-tokens", default="auto")
    ap.add_argument("--doc-packing", default=None, choices=DOC_PACKINGS)
    ap.add_argument("--max-docs", type=int, default=None)
    ap.add_argument("--budget-seconds", type=float, default=600.0)
    # the reference scorer's flag set (scripts/run_exp20_fast_score.py:1398-1490): with --summary-path the
    # summary goes there and --output-path receives one JSON line per document
    ap.add_argument("--summary-path", default=None)
    ap.add_argument("--safety-margin-seconds", type=float, default=0.0)
    ap.add_argument("--persistence-mode", choices=["reset"], default="reset")
    ap.add_argument("--max-batch-tokens", dest="max_forward_tokens", help=argparse.SUPPRESS)
    ap.add_argument("--score-boundary-targets", action=argparse.BooleanOptionalAction, default=True)
    ap.add_argument("--sort-docs-by-length", action=argparse.BooleanOptionalAction, default=None)
    ap.add_argument("--torch-compile-mode", choices=["none", "default", "reduce-overhead", "max-autotune"], default="none",
                    help="accepted for command-line compatibility; there is no tracing compiler in this stack")
    ap.add_argument("--score-warmup-steps", type=int, default=0)
    ap.add_argument("--score-graph-mode", choices=["none", "cuda"], default="none",
                    help="accepted for compatibility: the chunk scorer is already one fused kernel sequence per batch")
    ap.add_argument("--score-through-packet-lane", action=argparse.BooleanOptionalAction, default=False,
                    help="accepted for compatibility: bare-SSM checkpoints have no side channel to bypass")
    ap.add_argument("--episodic-cache-enabled", action=argparse.BooleanOptionalAction, default=False)
    ap.add_argument("--episodic-cache-reset-per-doc", action=argparse.BooleanOptionalAction, default=False)
    for flag, default in (("--episodic-cache-capacity", 4096), ("--episodic-span-length", 4), ("--episodic-key-rep-dim", -1),
                          ("--episodic-grace-steps", 1000), ("--episodic-fingerprint-window", 8)):
        ap.add_argument(flag, type=int, default=default)
    ap.add_argument("--episodic-cache-source", choices=("auto", "fresh", "checkpoint"), default="auto")
    ap.add_argument("--allow-online-replay-checkpoint", action=argparse.BooleanOptionalAction, default=False)
    ap.add_argument("--device", default="auto")
    a = ap.parse_args(argv)
    if not a.score_boundary_targets:
        ap.error("--no-score-boundary-targets is not supported: every document contributes len - 1 targets")
    mft = a.max_forward_tokens if str(a.max_forward_tokens).lower() == "auto" else int(a.max_forward_tokens)
    dev = None if a.device == "auto" else torch.device(a.device)
    s = run(cache_dir=a.cache_dir, checkpoint_path=a.checkpoint_path,
            output_path=None if a.summary_path else a.output_path, summary_path=a.summary_path,
            per_doc_path=a.output_path if a.summary_path else None,
            chunk_size=a.chunk_size, doc_batch_size=a.doc_batch_size, max_forward_tokens=mft,
            doc_packing=a.doc_packing, max_docs=a.max_docs, budget_seconds=a.budget_seconds, device=dev,
            safety_margin_seconds=a.safety_margin_seconds, sort_docs_by_length=a.sort_docs_by_length,
            score_warmup_steps=a.score_warmup_steps, episodic_cache_source=a.episodic_cache_source,
            allow_online_replay_checkpoint=a.allow_online_replay_checkpoint)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({k: s[k] for k in ("bpb", "tokens_scored", "docs_scored", "elapsed_s", "tokens_per_s")}))
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
