"""Latency of the CPU controller: its vector kernels alone and the per-event hot path end to end.

Reference: experiments/25_controller_pretrain/bench_amx.py:52-300.  Two questions.

1. *Kernel level.*  Per-call time of the diagonal recurrence ``h = decay * h + x`` (512 lanes) through
   the scalar path and through the AVX-512 path, and of the bf16 matmul at the policy's layer-1 shape
   (16 x 32 x 16, one AMX tile) and at a tiled shape (64 x 64 x 32), each through the scalar path and
   through AMX.  A path the CPU or the build does not have is reported as ``{"available": false,
   "reason": ...}`` -- never timed under the accelerated label through a fallback.
2. *Per event.*  The controller process does, for every query event, ``forward`` (score the simplex),
   ``record_decision`` (keep what was chosen and why) and, when the replay outcome comes back,
   ``on_replay_outcome`` (credit assignment, REINFORCE gradient, SGD).  Three modes: ``forward_only``,
   ``decision_record``, ``full_replay_event`` (``sgd_interval = 1``: the worst case, an SGD apply on
   every event).  The producers emit about 6.7 K replay outcomes per second, so an event has about
   150 microseconds; ``within_event_budget`` says whether the full event fits.

The kernel timings call the shared library on preallocated buffers (no array construction in the
timed call); the per-event timings go through the same Python classes the runtime uses.
"""
from __future__ import annotations

import argparse
import json
import platform
import statistics
import time
from pathlib import Path
from typing import Any, Callable, Optional, Sequence

import numpy as np

from . import native as N

SIMPLEX = {"N": 16, "K_v": 16, "K_s": 4, "H": 32}
EVENT_BUDGET_US = 150.0


def time_us(fn: Callable[[], None], iterations: int, warmup: int) -> dict[str, float]:
    for _ in range(warmup):
        fn()
    samples = []
    for _ in range(iterations):
        t0 = time.perf_counter_ns()
        fn()
        samples.append((time.perf_counter_ns() - t0) / 1e3)
    samples.sort()
    return {"mean_us": statistics.fmean(samples), "median_us": statistics.median(samples),
            "p99_us": samples[min(len(samples) - 1, int(0.99 * len(samples)))]}


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def _simplex_inputs(seed: int):
    rng = np.random.default_rng(seed)
    V = rng.standard_normal((SIMPLEX["N"], SIMPLEX["K_v"])).astype(np.float32)
    raw = rng.standard_normal((SIMPLEX["N"], SIMPLEX["K_v"])).astype(np.float32)
    raw /= np.linalg.norm(raw, axis=1, keepdims=True)
    return V, np.clip(raw @ raw.T, -1.0, 1.0).astype(np.float32), (rng.standard_normal(SIMPLEX["K_s"]) * 0.5).astype(np.float32)


def _outcome(slot: int, gpu_step: int, selection_step: int) -> np.ndarray:
    ev = np.zeros((), dtype=N.REPLAY_OUTCOME)
    ev["event_type"], ev["slot_id"], ev["gpu_step"], ev["selection_step"] = 3, slot, gpu_step, selection_step
    ev["replay_id"], ev["policy_version"], ev["ce_delta_raw"] = 1, 1, 0.5
    ev["grad_cos_rare"] = ev["grad_cos_total"] = np.nan
    return ev


def bench_kernels(*, iterations: int, warmup: int, recurrence_dim: int, seed: int) -> dict[str, Any]:
    rng = np.random.default_rng(seed)
    lib, feats = N.lib(), N.cpu_features()
    out: dict[str, Any] = {}
    decay = (rng.random(recurrence_dim) * 0.1 + 0.9).astype(np.float32)
    x = rng.standard_normal(recurrence_dim).astype(np.float32)
    h = rng.standard_normal(recurrence_dim).astype(np.float32)
    dp, xp, hp = decay.ctypes.data, x.ctypes.data, h.ctypes.data
    out["generic_fp32_recurrence"] = time_us(lambda: lib.ccbc_diag_step(dp, xp, hp, recurrence_dim, 1), iterations, warmup)
    if feats["avx512f"]:
        out["avx512_recurrence"] = time_us(lambda: lib.ccbc_diag_step(dp, xp, hp, recurrence_dim, 0), iterations, warmup)
    else:
        out["avx512_recurrence"] = {"available": False, "reason": "this CPU has no AVX-512F"}
    for label, (M, K, Nn) in (("16x32x16", (16, 32, 16)), ("64x64x32_tiled", (64, 64, 32))):
        A = _bf16_bits(rng.standard_normal((M, K)))
        B = _bf16_bits(rng.standard_normal((K, Nn)))
        Cm = np.zeros((M, Nn), np.float32)
        ap, bp, cp = A.ctypes.data, B.ctypes.data, Cm.ctypes.data
        out[f"generic_bf16_matmul_{label}"] = time_us(lambda: lib.ccbc_bf16_matmul(ap, bp, cp, M, Nn, K, 1), iterations, warmup)
        if feats["amx_bf16"] and feats["amx_enabled"] and lib.ccbc_bf16_matmul(ap, bp, cp, M, Nn, K, 0):
            out[f"amx_bf16_matmul_{label}"] = time_us(lambda: lib.ccbc_bf16_matmul(ap, bp, cp, M, Nn, K, 0), iterations, warmup)
        else:
            out[f"amx_bf16_matmul_{label}"] = {"available": False,
                                               "reason": "this CPU has no AMX-BF16, or the kernel did not grant tile state"}
    return out


def bench_events(*, iterations: int, warmup: int, seed: int) -> dict[str, Any]:
    V, E, sf = _simplex_inputs(seed * 2)
    n = SIMPLEX["N"]
    out: dict[str, Any] = {}
    pol = N.SimplexPolicy(**SIMPLEX, seed=seed)
    out["forward_only"] = time_us(lambda: pol.forward(V, E, sf), iterations, warmup)

    def learner(sgd_interval: int):
        lrn = N.SimplexOnlineLearner(num_slots=8, max_entries_per_slot=4, gamma=0.995, learning_rate=1e-3,
                                     sgd_interval=sgd_interval, ema_interval=4096)
        p = N.SimplexPolicy(**SIMPLEX, seed=seed)
        lrn.initialize(p)
        return lrn, p

    for mode, sgd_interval in (("decision_record", 1024), ("full_replay_event", 1)):
        lrn, p = learner(sgd_interval)
        t = [0]

        def one(lrn=lrn, p=p, t=t, full=(mode == "full_replay_event")):
            i = t[0]
            slot, sel = i % 8, 2 * i
            probs, _ = p.forward(V, E, sf)
            lrn.record_decision(slot, sel, i % n, float(probs[i % n]), V, E, sf)
            if full:
                lrn.on_replay_outcome(_outcome(slot, sel + 1, sel))
            t[0] = i + 1
        try:
            out[mode] = time_us(one, iterations, warmup)
            if mode == "full_replay_event":
                tel = lrn.telemetry()
                out[mode]["sgd_steps"] = int(tel["sgd_steps"])
                out[mode]["credited_actions"] = int(tel["credited_actions"])
        finally:
            lrn.close()
    out["event_budget_us"] = EVENT_BUDGET_US
    out["within_event_budget"] = bool(out["full_replay_event"]["median_us"] <= EVENT_BUDGET_US)
    return out


def run_benchmark(*, iterations: int = 10_000, warmup: int = 1_000, recurrence_dim: int = 512, seed: int = 1337) -> dict[str, Any]:
    return {"host": {"platform": platform.platform(), "machine": platform.machine(), "python": platform.python_version()},
            "cpu_features": N.cpu_features(), "iterations": int(iterations), "warmup": int(warmup),
            "simplex_dims": dict(SIMPLEX), "recurrence_dim": int(recurrence_dim),
            "isolated_kernel": bench_kernels(iterations=iterations, warmup=warmup, recurrence_dim=recurrence_dim, seed=seed),
            "simplex_per_query": bench_events(iterations=iterations, warmup=warmup, seed=seed)}


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iterations", type=int, default=10_000)
    ap.add_argument("--warmup", type=int, default=1_000)
    ap.add_argument("--recurrence-dim", type=int, default=512)
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--output", type=Path, default=None)
    a = ap.parse_args(argv)
    res = run_benchmark(iterations=a.iterations, warmup=a.warmup, recurrence_dim=a.recurrence_dim, seed=a.seed)
    text = json.dumps(res, indent=2, sort_keys=True)
    if a.output is not None:
        a.output.parent.mkdir(parents=True, exist_ok=True)
        a.output.write_text(text + "\n")
    print(text)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
