"""Document sources and per-document metric logging for the streaming evaluator:
``DocStreamer`` (JSONL + SentencePiece), ``ValCache`` (pre-tokenised validation
set on disk: tokens.npy uint16, docs.npy struct array, manifest.json), synthetic
corpora for benchmarking, ``MetricsCollector`` with its collapse gate.
(cf. src/chaoscontrol/eval_stream/doc_stream.py, val_cache.py:14-231, metrics.py.)"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, Optional, Sequence

import numpy as np

from .types import DocRecord

DOC_DTYPE = np.dtype([("doc_id", "<i8"), ("token_start", "<i8"), ("token_len", "<i8"), ("raw_bytes", "<i8")])
CACHE_VERSION = 1


class DocStreamer:
    """Yields ``DocRecord``s by tokenising JSONL ``{"text": ...}`` lines.  Not
    re-iterable: every ``__iter__`` restarts ``doc_id`` at 0."""

    def __init__(self, *, jsonl_paths: Sequence[Path], sp_model_path: Path, max_docs: int = 50_000) -> None:
        import sentencepiece as spm
        self.jsonl_paths = [Path(p) for p in jsonl_paths]
        self.sp = spm.SentencePieceProcessor(model_file=str(sp_model_path))
        self.max_docs = max_docs

    def __iter__(self) -> Iterator[DocRecord]:
        doc_id = 0
        for p in self.jsonl_paths:
            with open(p, "r", encoding="utf-8") as fh:
                for line in fh:
                    line = line.strip()
                    if not line:
                        continue
                    try:
                        text = json.loads(line).get("text", "")
                    except json.JSONDecodeError:
                        continue
                    if not text:
                        continue
                    toks = self.sp.encode(text, out_type=int)
                    if not toks:
                        continue
                    yield DocRecord(doc_id=doc_id, tokens=toks, raw_bytes=len(text.encode("utf-8")))
                    doc_id += 1
                    if doc_id >= self.max_docs:
                        return


@dataclass
class CachedDoc:
    doc_id: int
    token_start: int
    token_len: int
    raw_bytes: int


@dataclass
class ValCache:
    cache_dir: Path
    manifest: dict
    tokens: np.ndarray      # uint16, all documents back to back
    docs: np.ndarray        # DOC_DTYPE

    @property
    def num_docs(self) -> int:
        return int(self.docs.shape[0])

    @property
    def total_tokens(self) -> int:
        return int(self.docs["token_len"].sum())

    @property
    def total_raw_bytes(self) -> int:
        return int(self.docs["raw_bytes"].sum())

    def iter_docs(self) -> Iterator[CachedDoc]:
        for r in self.docs:
            yield CachedDoc(int(r["doc_id"]), int(r["token_start"]), int(r["token_len"]), int(r["raw_bytes"]))

    def tokens_for_doc(self, doc: CachedDoc) -> np.ndarray:
        return self.tokens[doc.token_start: doc.token_start + doc.token_len]


def _sha256_file(path: Path, chunk: int = 1 << 20) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def _content_sha(tokens: np.ndarray, docs: np.ndarray) -> str:
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(tokens).tobytes())
    h.update(np.ascontiguousarray(docs).tobytes())
    return h.hexdigest()


def _save_cache(cache_dir: Path, tokens: np.ndarray, docs: np.ndarray, request: dict) -> dict:
    cache_dir.mkdir(parents=True, exist_ok=True)
    np.save(cache_dir / "tokens.npy", tokens)
    np.save(cache_dir / "docs.npy", docs)
    manifest = dict(request, cache_version=CACHE_VERSION, num_docs=int(docs.shape[0]),
                    total_tokens=int(docs["token_len"].sum()), total_raw_bytes=int(docs["raw_bytes"].sum()),
                    content_sha256=_content_sha(tokens, docs))
    tmp = cache_dir / "manifest.json.tmp"
    tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True))
    tmp.replace(cache_dir / "manifest.json")
    return manifest


def write_val_cache(*, jsonl_paths: Sequence[Path], sp_model_path: Path, cache_dir: Path,
                    max_docs: int = 50_000, force: bool = False) -> dict:
    """Tokenise once and store; a cache whose request (paths, tokenizer sha256,
    max_docs) matches is reused unless ``force``."""
    cache_dir = Path(cache_dir)
    request = {"jsonl_paths": [str(Path(p)) for p in jsonl_paths], "sp_model_sha256": _sha256_file(Path(sp_model_path)),
               "max_docs": int(max_docs)}
    mpath = cache_dir / "manifest.json"
    if not force and mpath.exists() and (cache_dir / "tokens.npy").exists() and (cache_dir / "docs.npy").exists():
        old = json.loads(mpath.read_text())
        if all(old.get(k) == v for k, v in request.items()) and old.get("cache_version") == CACHE_VERSION:
            return old
    toks: list[np.ndarray] = []
    rows = []
    pos = 0
    for rec in DocStreamer(jsonl_paths=jsonl_paths, sp_model_path=sp_model_path, max_docs=max_docs):
        arr = np.asarray(rec.tokens, dtype=np.uint16)
        rows.append((rec.doc_id, pos, arr.size, rec.raw_bytes))
        toks.append(arr)
        pos += arr.size
    tokens = np.concatenate(toks) if toks else np.zeros(0, np.uint16)
    return _save_cache(cache_dir, tokens, np.asarray(rows, dtype=DOC_DTYPE), request)


def write_synthetic_val_cache(cache_dir: Path, *, n_docs: int = 50_000, vocab: int = 16384,
                              median_len: float = 700.0, sigma: float = 1.0, min_len: int = 32,
                              max_len: int = 32768, zipf_s: float = 1.1, seed: int = 0,
                              bytes_per_token: float = 3.0) -> dict:
    """Same on-disk format, filled with Zipf tokens and lognormal document lengths."""
    from ..data import lognormal_doc_lengths, zipf_tokens
    lens = lognormal_doc_lengths(n_docs, median=median_len, sigma=sigma, lo=min_len, hi=max_len, seed=seed)
    tokens = zipf_tokens(int(lens.sum()), vocab, s=zipf_s, seed=seed + 1).numpy().astype(np.uint16)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    docs = np.zeros(n_docs, dtype=DOC_DTYPE)
    docs["doc_id"] = np.arange(n_docs)
    docs["token_start"] = starts
    docs["token_len"] = lens
    docs["raw_bytes"] = np.maximum(1, (lens * bytes_per_token).astype(np.int64))
    return _save_cache(Path(cache_dir), tokens, docs,
                       {"synthetic": True, "n_docs": n_docs, "vocab": vocab, "seed": seed,
                        "max_docs": n_docs, "jsonl_paths": [], "sp_model_sha256": None})


def load_val_cache(cache_dir: Path) -> ValCache:
    cache_dir = Path(cache_dir)
    manifest = json.loads((cache_dir / "manifest.json").read_text())
    tokens = np.load(cache_dir / "tokens.npy", mmap_mode="r")
    docs = np.load(cache_dir / "docs.npy", mmap_mode="r")
    if manifest.get("content_sha256") and int(manifest.get("num_docs", -1)) != int(docs.shape[0]):
        raise ValueError("val cache manifest does not match docs.npy")
    return ValCache(cache_dir=cache_dir, manifest=manifest, tokens=tokens, docs=docs)


class MetricsCollector:
    """Per-document JSONL log plus a collapse gate: the first ``stability_window``
    losses freeze a baseline (mean, sd); ``collapsed`` is raised when the loss
    stays more than ``stability_sd_threshold`` sd above it for
    ``stability_window // 2`` consecutive documents."""

    def __init__(self, *, output_path: Path, stability_window: int = 100,
                 stability_sd_threshold: float = 3.0) -> None:
        self.output_path = Path(output_path)
        self.output_path.parent.mkdir(parents=True, exist_ok=True)
        self._fh = self.output_path.open("w")
        self.stability_window = stability_window
        self.stability_sd_threshold = stability_sd_threshold
        self._warm: list[float] = []
        self._baseline: Optional[tuple[float, float]] = None
        self._drift = 0
        self.collapsed = False

    def record_doc(self, *, doc_id: int, bpb: float, tokens: int, loss_before: float,
                   loss_after: Optional[float], step_count: int, wall_ms: float, grad_norm: float,
                   state_norm: float) -> None:
        self._fh.write(json.dumps(dict(doc_id=doc_id, bpb=bpb, tokens=tokens, loss_before=loss_before,
                                       loss_after=loss_after, step_count=step_count, wall_ms=wall_ms,
                                       grad_norm=grad_norm, state_norm=state_norm)) + "\n")
        self._fh.flush()
        self._gate(loss_before)

    def _gate(self, loss: float) -> None:
        if self._baseline is None:
            self._warm.append(loss)
            if len(self._warm) >= self.stability_window:
                m = sum(self._warm) / len(self._warm)
                var = sum((x - m) ** 2 for x in self._warm) / len(self._warm)
                self._baseline = (m, var ** 0.5 if var > 0 else 1e-6)
            return
        m, sd = self._baseline
        self._drift = self._drift + 1 if loss - m > self.stability_sd_threshold * sd else 0
        if self._drift >= self.stability_window // 2:
            self.collapsed = True

    def close(self) -> None:
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
