"""Tracing and timing helpers: NVTX ranges, CUDA-event section timers reduced as the
max over ranks, a scheduled ``torch.profiler`` capture with table / Chrome-trace export,
a one-shot topology snapshot and the SIGUSR1 stack dump.

The reference times sections with CUDA events + synchronize
(experiments/24_training_time_bundle/profile_event_sleep_arm.py:85-99), captures
``torch.profiler`` traces with ``schedule(wait=1, warmup=3, active=5)``
(experiments/19_phase1/profile_ssm_scan.py:238-295), dumps stacks on SIGUSR1 and records
the host topology (experiments/23_fast_path/runner_fast_path.py:67-93, 361-406); it has no
NVTX ranges.  Everything here degrades to a no-op / host clock on a machine without CUDA.
"""
from __future__ import annotations

import contextlib
import faulthandler
import json
import shutil
import signal
import subprocess
import sys
import time
from collections import defaultdict
from pathlib import Path
from typing import Any, Callable, Iterator, Optional

import torch

__all__ = ["nvtx_range", "nvtx_mark", "SectionTimer", "time_kernel", "profile_steps", "topology_snapshot",
           "enable_stack_dump_signal"]


def _cuda() -> bool:
    return torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    """Named range visible to Nsight tools (no-op without CUDA)."""
    if _cuda():
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if _cuda():
            torch.cuda.nvtx.range_pop()


def nvtx_mark(name: str) -> None:
    if _cuda():
        torch.cuda.nvtx.mark(name)


class SectionTimer:
    """``with timer.section("fwd"): ...`` records a CUDA-event pair on the current stream (host clock
    without CUDA) and an NVTX range; nothing synchronises until :meth:`summary`, which resolves all
    pairs after one synchronize and, in a process group, reports the MAX over ranks per section."""

    def __init__(self, *, nvtx: bool = True) -> None:
        self._pairs: dict[str, list] = defaultdict(list)
        self._nvtx = nvtx

    @contextlib.contextmanager
    def section(self, name: str) -> Iterator[None]:
        ctx = nvtx_range(name) if self._nvtx else contextlib.nullcontext()
        with ctx:
            if _cuda():
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                try:
                    yield
                finally:
                    b.record()
                    self._pairs[name].append((a, b))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._pairs[name].append((t0, time.perf_counter()))

    def summary(self, *, reduce_max: bool = True) -> dict[str, dict[str, float]]:
        """``{section: {"calls", "total_ms", "mean_ms"}}``."""
        if _cuda():
            torch.cuda.synchronize()
        out: dict[str, dict[str, float]] = {}
        for name, pairs in self._pairs.items():
            ms = [(a.elapsed_time(b) if _cuda() else (b - a) * 1e3) for a, b in pairs]
            out[name] = {"calls": float(len(ms)), "total_ms": float(sum(ms)), "mean_ms": float(sum(ms) / len(ms))}
        import torch.distributed as dist
        if reduce_max and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and out:
            names = sorted(out)
            dev = torch.device("cuda") if _cuda() and dist.get_backend() == "nccl" else torch.device("cpu")
            t = torch.tensor([out[n]["total_ms"] for n in names], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            for n, v in zip(names, t.tolist()):
                out[n]["total_ms"] = v
                out[n]["mean_ms"] = v / max(out[n]["calls"], 1.0)
        return out

    def reset(self) -> None:
        self._pairs.clear()


def time_kernel(fn: Callable[[], Any], *, warmup: int = 3, iters: int = 20, flush_l2_bytes: int = 256 << 20
                ) -> dict[str, float]:
    """Median / min milliseconds of ``fn`` with CUDA events on the launching stream, a synchronize on both
    sides and the L2 flushed between iterations by writing a buffer larger than it."""
    if not _cuda():
        ts = []
        for _ in range(warmup + iters):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
        ts = sorted(ts[warmup:])
        return {"ms_median": ts[len(ts) // 2], "ms_min": ts[0], "iters": float(iters)}
    flush = torch.empty(flush_l2_bytes, dtype=torch.uint8, device="cuda") if flush_l2_bytes else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return {"ms_median": ts[len(ts) // 2], "ms_min": ts[0], "iters": float(iters)}


def profile_steps(step_fn: Callable[[int], Any], *, out_dir: Path | str, wait: int = 1, warmup: int = 3,
                  active: int = 5, row_limit: int = 40) -> dict[str, Any]:
    """Runs ``wait + warmup + active`` calls of ``step_fn(i)`` under ``torch.profiler`` and writes
    ``cuda_table.txt`` / ``cpu_table.txt`` / ``trace.json`` / ``summary.json`` into ``out_dir``."""
    from torch.profiler import ProfilerActivity, profile, schedule
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if _cuda() else [])
    total = wait + warmup + active
    with profile(activities=acts, schedule=schedule(wait=wait, warmup=warmup, active=active, repeat=1)) as prof:
        for i in range(total):
            with nvtx_range(f"step{i}"):
                step_fn(i)
            prof.step()
    ka = prof.key_averages()
    (out / "cpu_table.txt").write_text(ka.table(sort_by="self_cpu_time_total", row_limit=row_limit))
    if _cuda():
        (out / "cuda_table.txt").write_text(ka.table(sort_by="self_cuda_time_total", row_limit=row_limit))
    prof.export_chrome_trace(str(out / "trace.json"))
    summary = {"steps_profiled": active, "events": len(ka), "cuda": _cuda(),
               "top_cpu": [e.key for e in sorted(ka, key=lambda e: -e.self_cpu_time_total)[:5]]}
    (out / "summary.json").write_text(json.dumps(summary, indent=2))
    return summary


def topology_snapshot() -> dict[str, str]:
    """Output of the host / GPU topology commands that exist on this machine (read-only queries)."""
    cmds = {"lscpu": ["lscpu"], "gpu_topo": ["nvidia-smi", "topo", "-m"], "numa": ["numactl", "-H"],
            "gpus": ["nvidia-smi", "--query-gpu=index,name,memory.total,clocks.max.sm", "--format=csv"]}
    out: dict[str, str] = {}
    for key, cmd in cmds.items():
        if shutil.which(cmd[0]) is None:
            continue
        try:
            out[key] = subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout
        except Exception as exc:  # noqa: BLE001
            out[key] = f"failed: {exc}"
    return out


def enable_stack_dump_signal(signum: int = signal.SIGUSR1) -> bool:
    """``kill -USR1 <pid>`` prints every thread's Python stack to stderr (for a run that looks stuck)."""
    try:
        faulthandler.register(signum, file=sys.stderr, all_threads=True, chain=False)
        return True
    except (AttributeError, ValueError, RuntimeError):
        return False
