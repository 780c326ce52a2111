"""Input pipeline and loop arithmetic of the throughput trainer
(public surface of the reference's experiments/23_fast_path/fast_path.py:29-768).

* window gather: ``batch_from_start_tensor`` builds the ``[B, T+1]`` index in one
  shot (int32 inputs, int64 targets);
* start sampling without ever listing the starts: random, sequential-epoch and
  shuffled-epoch (an O(1)-memory permutation ``i -> (i * s + o) mod n`` with ``s``
  coprime to ``n``), all sharded by ``global_start_index % world_size == rank``;
* ``BatchPrefetcher``: the next batch is gathered by a worker thread straight
  into one of two PINNED staging buffers and copied on a dedicated copy stream;
  ``next()`` only makes the compute stream wait on that copy's event, so the
  host->device transfer and the host gather both overlap the running step
  (``Exp23BatchPrefetcher`` is the same class under the reference's name);
* loop arithmetic: steady-state step time, the CUDA-graph acceptance gate,
  throughput summary, the shared stop predicate.
"""
from __future__ import annotations

import copy
import json
import math
import random
import statistics
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

__all__ = ["build_token_buckets", "compute_per_bucket_val_ce", "batch_from_start_tensor", "steady_state_step_seconds", "summarize_cuda_graph_gate", "BatchPrefetcher",
           "Exp23BatchPrefetcher", "count_lm_starts", "count_sharded_lm_starts", "sample_sharded_lm_starts",
           "sequential_epoch_steps", "sequential_sharded_lm_starts", "shuffled_epoch_sharded_lm_starts",
           "SequentialShardedStartSampler", "ShuffledEpochShardedStartSampler", "choose_lm_starts_lazy",
           "summarize_train_timing", "should_stop_training_loop", "build_stage_a_matrix", "build_stage_b_matrix",
           "write_matrix", "read_speed_config"]

DEFAULT_STAGE_A_SEED = 1337
DEFAULT_STAGE_B_SEEDS = (1337, 2674, 4011)


# ---------------------------------------------------------------------------
# Window gather
# ---------------------------------------------------------------------------
def batch_from_start_tensor(*, tokens: torch.Tensor, starts: torch.Tensor, seq_len: int, device,
                            vocab_size: Optional[int] = None,
                            out: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``(inputs int32 [B, T], targets int64 [B, T])`` on ``device``.  ``out``, when
    given, is a ``[B, T+1]`` staging tensor in ``tokens``' dtype (pinned, typically)
    that receives the gathered windows."""
    if starts.ndim != 1:
        raise ValueError(f"starts must be 1D, got shape={tuple(starts.shape)}")
    idx = starts.to(device=tokens.device, dtype=torch.long).unsqueeze(1) + \
        torch.arange(seq_len + 1, dtype=torch.long, device=tokens.device).unsqueeze(0)
    if out is not None:
        torch.index_select(tokens, 0, idx.reshape(-1), out=out.view(-1))
        batch = out
    else:
        batch = torch.index_select(tokens, 0, idx.reshape(-1)).view(starts.numel(), seq_len + 1)
    if vocab_size is not None:
        batch.clamp_(0, int(vocab_size) - 1)
    return (batch[:, :-1].to(device=device, dtype=torch.int32, non_blocking=True),
            batch[:, 1:].to(device=device, dtype=torch.long, non_blocking=True))


# ---------------------------------------------------------------------------
# Start arithmetic
# ---------------------------------------------------------------------------
def count_lm_starts(num_tokens: int, seq_len: int, stride: int) -> int:
    """``len(range(0, num_tokens - seq_len - 1, stride))``."""
    if stride <= 0:
        raise ValueError(f"stride must be positive, got {stride}")
    stop = int(num_tokens) - int(seq_len) - 1
    return 0 if stop <= 0 else (stop - 1) // int(stride) + 1


def count_sharded_lm_starts(*, total_starts: int, rank: int, world_size: int) -> int:
    total_starts, rank, world_size = int(total_starts), int(rank), int(world_size)
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank must be in [0, {world_size}), got {rank}")
    return 0 if rank >= total_starts else (total_starts - 1 - rank) // world_size + 1


def _rank_starts(num_tokens, seq_len, stride, rank, world_size) -> int:
    n = count_sharded_lm_starts(total_starts=count_lm_starts(num_tokens, seq_len, stride), rank=rank,
                                world_size=world_size)
    if n <= 0:
        raise RuntimeError(f"rank {rank} has no train starts after world_size={world_size} sharding")
    return n


def _to_offsets(local_idx: torch.Tensor, rank: int, world_size: int, stride: int) -> torch.Tensor:
    return (int(rank) + local_idx * int(world_size)) * int(stride)


def sample_sharded_lm_starts(*, num_tokens: int, seq_len: int, stride: int, batch_size: int, rank: int,
                             world_size: int, generator: torch.Generator) -> torch.Tensor:
    """Uniform draws from this rank's starts, equivalent to sampling
    ``build_lm_starts(...)[rank::world_size]`` without building it."""
    n = _rank_starts(num_tokens, seq_len, stride, rank, world_size)
    local = torch.randint(0, n, (int(batch_size),), generator=generator, dtype=torch.long)
    return _to_offsets(local, rank, world_size, stride)


def sequential_epoch_steps(*, num_tokens: int, seq_len: int, stride: int, batch_size: int, world_size: int) -> int:
    """Fixed-shape steps that cover every start once: the longest rank shard,
    rounded up to whole batches (shorter shards repeat their last start)."""
    total = count_lm_starts(num_tokens, seq_len, stride)
    if total <= 0:
        return 0
    b, w = max(1, int(batch_size)), max(1, int(world_size))
    longest = max(count_sharded_lm_starts(total_starts=total, rank=r, world_size=w) for r in range(w))
    return (longest + b - 1) // b


def sequential_sharded_lm_starts(*, num_tokens: int, seq_len: int, stride: int, batch_size: int, rank: int,
                                 world_size: int, step: int) -> torch.Tensor:
    n = _rank_starts(num_tokens, seq_len, stride, rank, world_size)
    local = torch.arange(int(step) * int(batch_size), (int(step) + 1) * int(batch_size), dtype=torch.long)
    return _to_offsets(local.clamp_(max=n - 1), rank, world_size, stride)


def _coprime_stride(size: int, seed: int) -> int:
    size = int(size)
    if size <= 1:
        return 1
    s = (abs(int(seed)) % size) | 1
    while math.gcd(s, size) != 1:
        s += 2
        if s >= size:
            s = 1
    return s


def shuffled_epoch_sharded_lm_starts(*, num_tokens: int, seq_len: int, stride: int, batch_size: int, rank: int,
                                     world_size: int, step: int, seed: int) -> torch.Tensor:
    """Step ``step`` of a per-rank permutation held in O(1) memory."""
    n = _rank_starts(num_tokens, seq_len, stride, rank, world_size)
    raw = torch.arange(int(step) * int(batch_size), (int(step) + 1) * int(batch_size), dtype=torch.long)
    s = _coprime_stride(n, int(seed) + int(rank) * 104_729)
    o = (abs(int(seed)) + int(rank) * 65_537) % n
    return _to_offsets((raw * s + o) % n, rank, world_size, stride)


class _SteppedSampler:
    """Sampler callable with the prefetcher's signature and an internal step counter."""

    def __init__(self) -> None:
        self._step = 0
        self._lock = threading.Lock()

    def _take_step(self) -> int:
        with self._lock:
            s = self._step
            self._step += 1
        return s


class SequentialShardedStartSampler(_SteppedSampler):
    def __call__(self, *, num_tokens, seq_len, stride, batch_size, rank, world_size, generator=None):
        return sequential_sharded_lm_starts(num_tokens=num_tokens, seq_len=seq_len, stride=stride,
                                            batch_size=batch_size, rank=rank, world_size=world_size,
                                            step=self._take_step())


class ShuffledEpochShardedStartSampler(_SteppedSampler):
    def __init__(self, *, seed: int) -> None:
        super().__init__()
        self._seed = int(seed)

    def __call__(self, *, num_tokens, seq_len, stride, batch_size, rank, world_size, generator=None):
        return shuffled_epoch_sharded_lm_starts(num_tokens=num_tokens, seq_len=seq_len, stride=stride,
                                                batch_size=batch_size, rank=rank, world_size=world_size,
                                                step=self._take_step(), seed=self._seed)


def choose_lm_starts_lazy(*, num_tokens: int, seq_len: int, stride: int, batch_size: int, eval_batches: int,
                          seed: int) -> list[int]:
    need = int(batch_size) * int(eval_batches)
    total = count_lm_starts(num_tokens, seq_len, stride)
    if need <= 0 or total <= 0:
        return []
    picks = range(total) if total <= need else random.Random(int(seed)).sample(range(total), need)
    return [i * int(stride) for i in picks]


# ---------------------------------------------------------------------------
# Prefetcher
# ---------------------------------------------------------------------------
class BatchPrefetcher:
    """One-step-ahead batches.  ``prime()`` once, then ``next()`` per step.

    On a CUDA device with host-resident tokens the gather lands in one of two
    pinned ``[B, T+1]`` staging buffers and the copy runs on a private stream; the
    returned tensors are safe to use on the current stream (it waits on the copy
    event).  A staging buffer is reused two steps later, after its copy's event.
    With a custom ``batch_builder`` (or CPU device) it degrades to a plain
    worker-thread prefetch.
    """

    def __init__(self, *, tokens: torch.Tensor, seq_len: int, stride: int, batch_size: int, rank: int,
                 world_size: int, device, generator: torch.Generator, vocab_size: Optional[int] = None,
                 batch_sampler: Optional[Callable[..., torch.Tensor]] = None,
                 batch_builder: Callable[..., tuple[torch.Tensor, torch.Tensor]] = batch_from_start_tensor,
                 executor: Optional[ThreadPoolExecutor] = None) -> None:
        self._tokens, self._seq_len, self._stride = tokens, int(seq_len), int(stride)
        self._batch_size, self._rank, self._world_size = int(batch_size), int(rank), int(world_size)
        self._device = torch.device(device)
        self._generator = generator
        self._vocab_size = None if vocab_size is None else int(vocab_size)
        self._sampler = batch_sampler or sample_sharded_lm_starts
        self._builder = batch_builder
        self._executor = executor or ThreadPoolExecutor(max_workers=1)
        self._owns_executor = executor is None
        self._pending: Optional[Future] = None
        self._closed = False
        self._lock = threading.Lock()
        self._staged = (self._device.type == "cuda" and not tokens.is_cuda and
                        batch_builder is batch_from_start_tensor)
        if self._staged:
            self._stage = [torch.empty((self._batch_size, self._seq_len + 1), dtype=tokens.dtype).pin_memory()
                           for _ in range(2)]
            self._free = [torch.cuda.Event() for _ in range(2)]
            self._copy_stream = torch.cuda.Stream(device=self._device)
            self._slot = 0

    def _build(self):
        starts = self._sampler(num_tokens=int(self._tokens.numel()), seq_len=self._seq_len, stride=self._stride,
                               batch_size=self._batch_size, rank=self._rank, world_size=self._world_size,
                               generator=self._generator)
        if not self._staged:
            return self._builder(tokens=self._tokens, starts=starts, seq_len=self._seq_len, device=self._device,
                                 vocab_size=self._vocab_size), None
        slot = self._slot
        self._slot ^= 1
        self._free[slot].synchronize()                     # its previous copy has drained
        with torch.cuda.stream(self._copy_stream):
            pair = batch_from_start_tensor(tokens=self._tokens, starts=starts, seq_len=self._seq_len,
                                           device=self._device, vocab_size=self._vocab_size, out=self._stage[slot])
            done = torch.cuda.Event()
            done.record(self._copy_stream)
            self._free[slot] = done
        return pair, done

    def prime(self) -> "BatchPrefetcher":
        with self._lock:
            if self._closed:
                raise RuntimeError("prefetcher is closed")
            if self._pending is None:
                self._pending = self._executor.submit(self._build)
        return self

    def next(self) -> tuple[torch.Tensor, torch.Tensor]:
        with self._lock:
            if self._closed:
                raise RuntimeError("prefetcher is closed")
            pending, self._pending = self._pending, None
            pair, done = pending.result() if pending is not None else self._build()
            self._pending = self._executor.submit(self._build)
        if done is not None:
            torch.cuda.current_stream(self._device).wait_event(done)
            for t in pair:
                t.record_stream(torch.cuda.current_stream(self._device))
        return pair

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._closed = True
            pending, self._pending = self._pending, None
        if pending is not None:
            pending.cancel()
        if self._owns_executor:
            self._executor.shutdown(wait=True, cancel_futures=True)

    def __enter__(self) -> "BatchPrefetcher":
        return self.prime()

    def __exit__(self, exc_type, exc, tb) -> None:
        self.close()


Exp23BatchPrefetcher = BatchPrefetcher


# ---------------------------------------------------------------------------
# Loop arithmetic
# ---------------------------------------------------------------------------
def steady_state_step_seconds(step_times) -> float:
    """Median of the samples after the first (which pays one-time set-up costs)."""
    if not step_times:
        raise ValueError("step_times must be non-empty")
    if len(step_times) == 1:
        return float(step_times[0])
    return float(statistics.median(float(t) for t in step_times[1:]))


def summarize_cuda_graph_gate(*, budget_seconds: float, capture_seconds: float, warmup_seconds: float,
                              warmup_steps: int, eager_step_seconds: float, graph_step_seconds: float,
                              min_total_speedup: float = 0.05, max_capture_seconds: float = 30.0) -> dict[str, Any]:
    """Capture and warm-up are charged to the same budget as training: graph
    replay must raise the projected number of steps in the WHOLE budget by
    ``min_total_speedup``, not merely be faster per step."""
    budget = float(budget_seconds)
    capture, warmup = max(0.0, float(capture_seconds)), max(0.0, float(warmup_seconds))
    overhead = capture + warmup
    eager, graph = float(eager_step_seconds), float(graph_step_seconds)
    reasons = [msg for bad, msg in ((budget <= 0, "budget_seconds_must_be_positive"),
                                    (eager <= 0, "eager_step_seconds_must_be_positive"),
                                    (graph <= 0, "graph_step_seconds_must_be_positive")) if bad]
    eager_steps = budget / eager if budget > 0 and eager > 0 else 0.0
    graph_steps = 0.0
    if budget > overhead and graph > 0:
        graph_steps = (budget - overhead) / graph
    elif overhead >= budget:
        reasons.append("capture_overhead_exhausts_budget")
    speedup = graph_steps / eager_steps - 1.0 if eager_steps > 0 else float("-inf")
    saving = eager - graph
    if saving <= 0:
        reasons.append("graph_step_not_faster")
        be_steps = be_seconds = float("inf")
    else:
        be_steps = overhead / saving
        be_seconds = be_steps * eager
    if capture > float(max_capture_seconds):
        reasons.append("capture_seconds_exceeds_limit")
    if speedup < float(min_total_speedup):
        reasons.append("projected_speedup_below_minimum")
    return {"accepted": not reasons, "reasons": reasons, "budget_seconds": budget, "capture_seconds": capture,
            "warmup_seconds": warmup, "warmup_steps": int(warmup_steps), "overhead_seconds": overhead,
            "eager_step_seconds": eager, "graph_step_seconds": graph, "projected_eager_steps": eager_steps,
            "projected_graph_steps": graph_steps, "projected_total_speedup": speedup,
            "min_total_speedup": float(min_total_speedup), "max_capture_seconds": float(max_capture_seconds),
            "break_even_steps": be_steps, "break_even_seconds": be_seconds}


def summarize_train_timing(*, steps: int, elapsed_s: float, batch_size: int, seq_len: int, world_size: int,
                           episodic_enabled: bool = False) -> dict[str, float | int]:
    """With the episodic (N+1) topology the last rank consumes no training
    tokens, so throughput is counted over ``world_size - 1`` ranks."""
    consuming = max(int(world_size) - 1, 1) if episodic_enabled else int(world_size)
    per_step = int(batch_size) * int(seq_len) * consuming
    agg = int(steps) * per_step / max(float(elapsed_s), 1e-9)
    return {"tokens_per_step": per_step, "aggregate_tokens_per_sec": float(agg),
            "per_gpu_tokens_per_sec": float(agg / max(consuming, 1))}


def should_stop_training_loop(*, steps: int, elapsed_s: float, budget_seconds: float, stop_margin_seconds: float,
                              max_steps: Optional[int] = None) -> bool:
    if int(steps) <= 0:
        return False
    if max_steps is not None and int(steps) >= int(max_steps):
        return True
    return float(elapsed_s) >= max(0.0, float(budget_seconds) - float(stop_margin_seconds))


# ---------------------------------------------------------------------------
# Experiment matrices
# ---------------------------------------------------------------------------
def _base_fast_config(*, world_size: int, vocab_size: int) -> dict[str, Any]:
    return {
        "model_type": "ssm", "mode": "speed_sweep", "world_size": int(world_size), "vocab_size": int(vocab_size),
        "model_dim": 256, "num_layers": 4, "ff_mult": 2, "seq_len": 512, "stride": 256, "eval_batches": 0,
        "a_mode": "diag", "base_lr": 0.128, "weight_decay": 0.01, "grad_clip_norm": 1.0, "optimizer": "muon",
        "local_attn_window": 0, "local_attn_heads": 1, "local_attn_dim": 64, "device": "auto", "dtype": "bf16",
        "precision": "bf16", "fused_grad_clip": True, "fused_muon": True, "compile_full_path": False,
        "cuda_graph_mode": "none", "cuda_graph_min_total_speedup": 0.05, "cuda_graph_max_capture_seconds": 30.0,
        "train_sampling_mode": "random", "lm_head_backward_mode": "fused_streaming_v2", "lm_head_tile_size": 8192,
        "warmup_steps": 5, "restore_after_warmup": False, "stop_check_interval": 4, "stop_margin_seconds": 2.0,
        "prefetch_batches": True, "budget_seconds": 90.0,
    }


def build_stage_a_matrix(*, seeds=(DEFAULT_STAGE_A_SEED,), vocab_sizes=(16384,), batch_sizes=(1024, 2048, 4096),
                         chunk_sizes=(64, 128, 256, 512), activation_checkpoints=(True,), world_size: int = 8,
                         budget_seconds: float = 90.0, base_lr: float = 0.128) -> list[dict[str, Any]]:
    """Speed-ceiling sweep: short, no eval, one seed by default."""
    out = []
    for v in vocab_sizes:
        base = _base_fast_config(world_size=world_size, vocab_size=v)
        base.update(budget_seconds=float(budget_seconds), base_lr=float(base_lr))
        for b in batch_sizes:
            for c in chunk_sizes:
                for ck in activation_checkpoints:
                    for s in seeds:
                        e = copy.deepcopy(base)
                        e.update(name=f"stageA_v{v}_b{b}_c{c}_{'ckpt' if ck else 'nockpt'}_s{s}", seed=int(s),
                                 batch_size=int(b), chunk_size=int(c), activation_checkpoint=bool(ck))
                        out.append(e)
    return out


def build_stage_b_matrix(*, speed_config: dict[str, Any], seeds=DEFAULT_STAGE_B_SEEDS, vocab_sizes=(8192, 16384),
                         init_paths: Optional[dict[int, dict[str, str]]] = None, world_size: int = 8,
                         budget_seconds: float = 600.0) -> list[dict[str, Any]]:
    """Base-lock matrix built on a stage-A winner: embedding inits x seeds."""
    init_paths = init_paths or {}
    out = []
    for v in vocab_sizes:
        base = _base_fast_config(world_size=world_size, vocab_size=v)
        base.update(copy.deepcopy(speed_config))
        base.update(mode="base_lock", world_size=int(world_size), vocab_size=int(v),
                    eval_batches=int(speed_config.get("stage_b_eval_batches", 16)),
                    budget_seconds=float(budget_seconds), warmup_steps=int(speed_config.get("warmup_steps", 20)),
                    restore_after_warmup=bool(speed_config.get("restore_after_warmup", True)))
        for init in ("random", "meanstd", "fullcov"):
            path = None
            if init != "random":
                path = init_paths.get(int(v), {}).get(init)
                if path is None:
                    continue
            for s in seeds:
                e = copy.deepcopy(base)
                e.update(name=f"stageB_v{v}_{init}_s{s}", seed=int(s), embed_init=init, embed_init_path=path)
                out.append(e)
    return out


def write_matrix(path: Path, entries: list[dict[str, Any]]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(entries, indent=2, default=str))


def read_speed_config(path: Path) -> dict[str, Any]:
    text = path.read_text()
    if path.suffix.lower() in {".yaml", ".yml"}:
        import yaml
        data = yaml.safe_load(text)
    else:
        data = json.loads(text)
    return dict(data["config"]) if "config" in data else dict(data)


# ---------------------------------------------------------------------------
# validation CE by token-frequency bucket
# ---------------------------------------------------------------------------
def build_token_buckets(token_frequencies: torch.Tensor, num_buckets: int) -> torch.Tensor:
    """``[vocab]`` int64 bucket id per token from ``log1p(frequency)`` cut into
    ``num_buckets`` equal spans; bucket 0 holds the rarest tokens
    (runner_fast_path.py:427-458)."""
    if token_frequencies.ndim != 1:
        raise ValueError("token_frequencies must be 1D")
    if num_buckets < 1:
        raise ValueError(f"num_buckets must be >= 1, got {num_buckets}")
    lf = torch.log1p(token_frequencies.to(torch.float32).clamp_min(0.0))
    lo = float(lf.min())
    span = max(float(lf.max()) - lo, 1e-6)
    edges = torch.linspace(lo, lo + span + 1e-6, num_buckets + 1, device=lf.device, dtype=torch.float32)
    return torch.bucketize(lf, edges[1:-1]).clamp_(0, num_buckets - 1).to(torch.int64)


def compute_per_bucket_val_ce(*, model: Any, device: torch.device, tokens: torch.Tensor, num_tokens: int,
                              seq_len: int, stride: int, batch_size: int, vocab_size: int,
                              token_frequencies: Optional[torch.Tensor], num_buckets: int, rank: int = 0,
                              world_size: int = 1, precision: str = "bf16",
                              max_batches: Optional[int] = None) -> dict[str, Any]:
    """Deterministic no-grad pass over this rank's sequential validation windows;
    per-token CE is summed into the frequency buckets of the TARGET tokens
    (runner_fast_path.py:461-581).  Per-token CE comes from the chunked scorer
    (the fused head on a GPU), so ``[B, T, V]`` logits never exist; per-window
    sums stay on the device and come back in one transfer at the end."""
    from .cache_utility import chunked_nll_from_hidden
    from .precision import autocast_context
    if token_frequencies is None:
        raise ValueError("rare_bucket_ce_enabled=True requires rare_bucket_ce_token_frequencies")
    nb = int(num_buckets)
    bucket_of = build_token_buckets(token_frequencies, nb).to(device)
    total = count_lm_starts(num_tokens, seq_len, stride)
    mine = count_sharded_lm_starts(total_starts=total, rank=rank, world_size=world_size)
    empty = {"per_bucket_val_ce": [0.0] * nb, "rare_bucket_val_ce": 0.0, "val_bucket_num_buckets": nb,
             "val_bucket_token_counts": [0] * nb, "per_window_bucket_ce_sum": [], "per_window_bucket_count": []}
    if mine <= 0:
        return empty
    n_steps = (mine + batch_size - 1) // batch_size
    if max_batches is not None:
        n_steps = min(n_steps, int(max_batches))
    sums, counts = [], []
    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            for step in range(n_steps):
                starts = sequential_sharded_lm_starts(num_tokens=num_tokens, seq_len=seq_len, stride=stride,
                                                      batch_size=batch_size, rank=rank, world_size=world_size,
                                                      step=step)
                inputs, targets = batch_from_start_tensor(tokens=tokens, starts=starts, seq_len=seq_len,
                                                          device=device, vocab_size=vocab_size)
                with autocast_context(precision, device_type=inputs.device.type):
                    hidden = model.encode(inputs)
                ce = chunked_nll_from_hidden(model, hidden, targets).reshape(-1).to(torch.float64)
                idx = bucket_of[targets.reshape(-1).long()]
                sums.append(torch.zeros(nb, dtype=torch.float64, device=device).scatter_add_(0, idx, ce))
                counts.append(torch.zeros(nb, dtype=torch.int64, device=device).scatter_add_(
                    0, idx, torch.ones_like(idx)))
    finally:
        model.train(was_training)
    win_sum, win_cnt = torch.stack(sums), torch.stack(counts)
    b_sum, b_cnt = win_sum.sum(0), win_cnt.sum(0)
    if world_size > 1 and dist.is_available() and dist.is_initialized():
        dist.all_reduce(b_sum, op=dist.ReduceOp.SUM)
        dist.all_reduce(b_cnt, op=dist.ReduceOp.SUM)
    per = (b_sum / b_cnt.to(torch.float64).clamp_min(1.0)).cpu().tolist()
    k = max(1, nb // 4)
    return {"per_bucket_val_ce": [float(x) for x in per], "rare_bucket_val_ce": float(sum(per[:k]) / k),
            "val_bucket_num_buckets": nb, "val_bucket_token_counts": [int(x) for x in b_cnt.cpu().tolist()],
            "per_window_bucket_ce_sum": win_sum.cpu().tolist(), "per_window_bucket_count": win_cnt.cpu().tolist()}
