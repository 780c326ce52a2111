"""Token data helpers: shard loading, LM window sampling, synthetic corpora.

``build_lm_starts`` / ``batch_from_starts`` / ``choose_eval_starts`` follow
src/chaoscontrol/data.py:316-347; ``load_fineweb_tokens`` reads the flat
little-endian uint16 shard format (data.py:120-145).  The synthetic generators
produce the Zipf / lognormal-length corpora used by the benchmarks when no
dataset is available.
"""
from __future__ import annotations

import json
import os
import random
import time
from concurrent.futures import ThreadPoolExecutor
from contextlib import nullcontext
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch


def build_lm_starts(num_tokens: int, seq_len: int, stride: int) -> list[int]:
    stop = num_tokens - seq_len - 1
    if stop <= 0:
        return []
    return list(range(0, stop, stride))


def batch_from_starts(tokens: torch.Tensor, starts: Sequence[int], seq_len: int,
                      device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    windows = [tokens[s: s + seq_len + 1] for s in starts]
    batch = torch.stack(windows).to(device=device, dtype=torch.long)
    return batch[:, :-1], batch[:, 1:]


def batch_from_start_tensor(tokens: torch.Tensor, starts: torch.Tensor, seq_len: int,
                            device: torch.device, *, vocab_size: Optional[int] = None,
                            pin: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Vectorised window gather: int32 inputs and int64 targets
    (cf. experiments/23_fast_path/fast_path.py:159-186)."""
    idx = starts.view(-1, 1).long() + torch.arange(seq_len + 1).view(1, -1)
    win = tokens[idx]
    if vocab_size is not None:
        win = win.clamp(0, vocab_size - 1)
    inputs = win[:, :-1].to(torch.int32)
    targets = win[:, 1:].to(torch.int64)
    if pin and torch.cuda.is_available():
        inputs, targets = inputs.pin_memory(), targets.pin_memory()
    return (inputs.to(device, non_blocking=True), targets.to(device, non_blocking=True))


def choose_eval_starts(starts: list[int], *, batch_size: int, eval_batches: int, seed: int) -> list[int]:
    needed = batch_size * eval_batches
    if not starts:
        return []
    if len(starts) <= needed:
        return starts[:needed]
    return random.Random(seed).sample(starts, needed)


# ---------------------------------------------------------------------------
# Device / dtype helpers (src/chaoscontrol/data.py:21-56)
# ---------------------------------------------------------------------------
def resolve_device(name: str) -> torch.device:
    if name == "auto":
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return torch.device(name)


def resolve_param_dtype(name: str, device: torch.device) -> torch.dtype:
    """``fp16`` / ``bf16`` / ``fp32``; anything off-GPU runs in fp32."""
    want = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[name]
    return want if device.type == "cuda" else torch.float32


def maybe_autocast(device: torch.device, dtype: torch.dtype):
    if device.type == "cuda" and dtype in (torch.float16, torch.bfloat16):
        return torch.autocast(device_type="cuda", dtype=dtype, enabled=True)
    return nullcontext()


def maybe_cache_tokens_on_device(tokens: torch.Tensor, *, device: torch.device, enabled: bool) -> torch.Tensor:
    if enabled and device.type == "cuda" and tokens.device != device:
        return tokens.to(device=device, dtype=torch.long)
    return tokens


def maybe_sync_cuda(device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize()


# ---------------------------------------------------------------------------
# Shard loading
# ---------------------------------------------------------------------------
def _concat_shards_mmap(shard_paths: list[Path], cache_path: Path) -> np.ndarray:
    """One flat uint16 cache file for a list of headerless uint16 shards,
    returned as a copy-on-write memory map (every process on the node shares the
    page cache).  The cache is filled by worker threads that each stream one shard
    straight into its slice of a pre-sized temporary map, so peak host memory is
    a few shard buffers rather than the whole corpus; the temporary is private to
    this PID and appears under the final name by an atomic rename, so concurrent
    ranks either win the rename or adopt the winner's file.
    (Role of src/chaoscontrol/data.py:60-117.)"""
    if cache_path.exists():
        return np.memmap(str(cache_path), dtype=np.uint16, mode="c")
    sizes = [p.stat().st_size for p in shard_paths]
    if any(sz % 2 for sz in sizes):
        raise ValueError("shard size not a multiple of 2 bytes (uint16)")
    counts = [sz // 2 for sz in sizes]
    offsets = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int64)
    tmp = cache_path.with_suffix(f".tmp.{os.getpid()}")
    try:
        dst = np.memmap(str(tmp), dtype=np.uint16, mode="w+", shape=(int(sum(counts)),))

        def _fill(i: int) -> None:
            dst[offsets[i]: offsets[i] + counts[i]] = np.memmap(str(shard_paths[i]), dtype=np.uint16, mode="r")

        with ThreadPoolExecutor(max_workers=min(32, max(1, len(shard_paths)))) as ex:
            list(ex.map(_fill, range(len(shard_paths))))
        dst.flush()
        del dst
        try:
            tmp.rename(cache_path)
        except OSError:
            tmp.unlink(missing_ok=True)
    except Exception:
        tmp.unlink(missing_ok=True)
        raise
    for _ in range(30):                      # another rank may still be renaming
        if cache_path.exists():
            break
        time.sleep(0.5)
    return np.memmap(str(cache_path), dtype=np.uint16, mode="c")


def _tokens_from_shards(data_dir, pattern: str, cache_name: str, what: str) -> torch.Tensor:
    root = Path(data_dir)
    shards = sorted(root.glob(pattern))
    if not shards:
        raise FileNotFoundError(f"No {what} shards found in {data_dir}")
    # int16 view of the uint16 map: same bits for ids < 32768, and zero-copy into torch
    return torch.from_numpy(_concat_shards_mmap(shards, root / cache_name).view(np.int16))


def load_fineweb_tokens(data_dir: str) -> tuple[torch.Tensor, torch.Tensor]:
    """``(train_tokens, val_tokens)`` from ``fineweb_train_*.bin`` / ``fineweb_val_*.bin``
    (flat little-endian uint16, no header), memory-mapped (data.py:120-145)."""
    return (_tokens_from_shards(data_dir, "fineweb_train_*.bin", ".train_cache.bin", "training"),
            _tokens_from_shards(data_dir, "fineweb_val_*.bin", ".val_cache.bin", "validation"))


def load_fineweb_val_tokens(data_dir: str) -> torch.Tensor:
    """Validation shards only: eval-only runs never build the training cache."""
    return _tokens_from_shards(data_dir, "fineweb_val_*.bin", ".val_cache.bin", "validation")


# ---------------------------------------------------------------------------
# Raw-byte corpora (data.py:163-309)
# ---------------------------------------------------------------------------
_COMPETITION_VAL_DOCS = 50_000


def _iter_jsonl_texts(jsonl_path: Path):
    bad = 0
    with open(jsonl_path, "r", encoding="utf-8") as fin:
        for line in fin:
            line = line.strip()
            if not line:
                continue
            try:
                yield json.loads(line).get("text", "")
            except json.JSONDecodeError:
                bad += 1
    if bad:
        print(f"  Skipped {bad} malformed JSONL lines")


def _extract_jsonl_to_raw(jsonl_path: Path, raw_path: Path) -> None:
    """All ``text`` fields, newline separated, as one flat UTF-8 file."""
    tmp = raw_path.with_suffix(".tmp")
    with open(tmp, "wb") as out:
        for text in _iter_jsonl_texts(jsonl_path):
            out.write(text.encode("utf-8") + b"\n")
    tmp.rename(raw_path)


def _extract_jsonl_split(jsonl_path: Path, val_path: Path, train_path: Path,
                         val_docs: int = _COMPETITION_VAL_DOCS) -> None:
    """First ``val_docs`` documents -> validation file, the rest -> training file."""
    vt, tt = val_path.with_suffix(".tmp"), train_path.with_suffix(".tmp")
    n = 0
    with open(vt, "wb") as fval, open(tt, "wb") as ftrain:
        for n, text in enumerate(_iter_jsonl_texts(jsonl_path), start=1):
            (fval if n <= val_docs else ftrain).write(text.encode("utf-8") + b"\n")
    vt.rename(val_path)
    tt.rename(train_path)
    print(f"  Split: {min(n, val_docs)} val docs, {max(n - val_docs, 0)} train docs")


def load_fineweb_raw_bytes(text_path: str) -> torch.Tensor:
    """A UTF-8 text file as a copy-on-write mmapped ``uint8`` tensor."""
    p = Path(text_path)
    if not p.exists() or p.stat().st_size == 0:
        raise ValueError(f"empty or missing text file: {text_path}")
    return torch.from_numpy(np.memmap(str(p), dtype=np.uint8, mode="c"))


def prepare_fineweb_splits(data_dir: str, *, device: torch.device, cache_on_device: bool = True,
                           train_fraction: float = 0.90) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(train, val, test)`` byte tensors (host resident).  Preference order: the
    document-aware pair ``docs_val_raw.txt`` / ``docs_train_raw.txt`` (built from
    ``docs_selected.jsonl`` when absent; the last 5 % of train is the held-out test),
    then the single-file ``docs_raw.txt`` with a percentage split."""
    root = Path(data_dir)
    val_raw, train_raw, jsonl = root / "docs_val_raw.txt", root / "docs_train_raw.txt", root / "docs_selected.jsonl"
    if not val_raw.exists() and jsonl.exists():
        _extract_jsonl_split(jsonl, val_raw, train_raw)
    if val_raw.exists() and train_raw.exists():
        val = load_fineweb_raw_bytes(str(val_raw))
        train_all = load_fineweb_raw_bytes(str(train_raw))
        cut = int(train_all.numel() * 0.95)
        return train_all[:cut], val, train_all[cut:]
    raw = root / "docs_raw.txt"
    if not raw.exists() and jsonl.exists():
        _extract_jsonl_to_raw(jsonl, raw)
    if not raw.exists():
        raise FileNotFoundError(f"No raw text found in {data_dir}. Need docs_selected.jsonl (preferred) "
                                f"or docs_raw.txt.")
    print("  WARNING: Using legacy percentage split — validation does not match the 50k-document set.")
    everything = load_fineweb_raw_bytes(str(raw))
    a, b = int(everything.numel() * train_fraction), int(everything.numel() * (train_fraction + 0.05))
    return everything[:a], everything[a:b], everything[b:]


def zipf_tokens(n: int, vocab: int, *, s: float = 1.1, seed: int = 0,
                dtype: torch.dtype = torch.int64) -> torch.Tensor:
    """``n`` iid tokens with ``P(k) ~ (k+1)^-s`` over ``vocab`` ids (inverse-CDF sampling)."""
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-s))
    cdf /= cdf[-1]
    rng = np.random.default_rng(seed)
    ids = np.searchsorted(cdf, rng.random(n), side="left").clip(0, vocab - 1)
    return torch.from_numpy(ids).to(dtype)


def lognormal_doc_lengths(n_docs: int, *, median: float = 700.0, sigma: float = 1.0,
                          lo: int = 32, hi: int = 32768, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    lens = rng.lognormal(mean=np.log(median), sigma=sigma, size=n_docs)
    return np.clip(lens, lo, hi).astype(np.int64)
