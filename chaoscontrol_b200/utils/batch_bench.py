"""Batch-size sweep of one training step: which batch is the largest before tokens per second stop rising?

    python -m chaoscontrol_b200.utils.batch_bench [--batch-sizes 256,512,1024,2048] [--output-json F]

Same job as the reference's ``tools/benchmark_batch.py:88-200`` (sweep, per-size mean / std step time,
tokens per second, recommendation, table + optional JSON), on this framework's training step:
``train_ssm_step`` (forward + backward, fused LM head) followed by ``zero_grad``.  On a GPU each step is
timed with CUDA events on the launching stream after a synchronize; a size is *skipped*, not attempted,
when its estimated footprint (parameters, activations kept for backward, the logits tile) does not fit the
free device memory with the safety margin, and the sweep stops at the first size that runs out of memory
-- larger ones are not tried.  On a CPU the sweep runs (small sizes) only to show that the script works.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from typing import Any, Callable, Optional, Sequence

import torch

__all__ = ["estimate_step_bytes", "bench_one", "recommend", "sweep", "render", "main"]


def estimate_step_bytes(*, batch: int, seq_len: int, dim: int, num_layers: int, vocab: int, ff_mult: int = 2) -> int:
    """Upper estimate of device bytes one step holds: per layer the block input, the packed projection
    (4 D), the scan output, both MLP halves (2 F each kept for the SiLU backward) in bf16 plus fp32 row
    statistics; twice that for the gradients that live at the same time; a 1024-row logits tile pair in
    fp32; parameters with fp32 master copy and two optimizer moments."""
    rows, F = batch * seq_len, ff_mult * dim
    per_layer = rows * (dim + 4 * dim + dim + 2 * F + dim) * 2 + rows * 8
    acts = 2 * num_layers * per_layer + rows * dim * 2 * 4
    logits = 2 * 1024 * vocab * 4 + rows * 16
    params = (vocab * dim + num_layers * (4 * dim * dim + dim * dim + 2 * F * dim + 4 * dim)) * (2 + 4 + 8)
    return int(acts + logits + params)


def _oom(exc: BaseException) -> bool:
    return isinstance(exc, torch.cuda.OutOfMemoryError) or "out of memory" in str(exc).lower()


def bench_one(step: Callable[[], None], *, batch: int, seq_len: int, warmup: int, steps: int,
              device: torch.device) -> dict[str, Any]:
    """Time ``step`` ``steps`` times after ``warmup`` untimed calls."""
    row: dict[str, Any] = {"batch_size": int(batch), "oom": False, "skipped": None}
    try:
        for _ in range(warmup):
            step()
        times = []
        if device.type == "cuda":
            torch.cuda.synchronize(device)
            for _ in range(steps):
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record()
                step()
                t1.record()
                t1.synchronize()
                times.append(t0.elapsed_time(t1))
        else:
            for _ in range(steps):
                t0 = time.perf_counter()
                step()
                times.append((time.perf_counter() - t0) * 1e3)
        mean = statistics.fmean(times)
        row.update(mean_ms=round(mean, 3), std_ms=round(statistics.stdev(times), 3) if len(times) > 1 else 0.0,
                   tokens_per_sec=round(batch * seq_len / (mean / 1e3)))
    except (RuntimeError, torch.cuda.OutOfMemoryError) as exc:
        if not _oom(exc):
            raise
        row.update(mean_ms=None, std_ms=None, tokens_per_sec=None, oom=True)
        if device.type == "cuda":
            torch.cuda.empty_cache()
    return row


def recommend(rows: Sequence[dict[str, Any]], tolerance: float = 0.05) -> Optional[int]:
    """Largest batch of the leading run of sizes whose tokens per second did not fall by more than
    ``tolerance`` against the size before it (a larger batch that is not slower per token is free)."""
    ok = [r for r in rows if r.get("tokens_per_sec")]
    if not ok:
        return None
    best = ok[0]["batch_size"]
    for prev, cur in zip(ok, ok[1:]):
        if cur["tokens_per_sec"] >= prev["tokens_per_sec"] * (1.0 - tolerance):
            best = cur["batch_size"]
        else:
            break
    return int(best)


def sweep(*, batch_sizes: Sequence[int], dim: int = 256, num_layers: int = 4, seq_len: int = 512, vocab: int = 16384,
          ff_mult: int = 2, warmup: int = 3, steps: int = 10, device: Optional[str] = None,
          memory_fraction: float = 0.8, seed: int = 0) -> dict[str, Any]:
    from ..models.model import CareStudentLM
    from ..train_ssm import train_ssm_step
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    rows = []
    for bs in sorted(int(b) for b in batch_sizes):
        need = estimate_step_bytes(batch=bs, seq_len=seq_len, dim=dim, num_layers=num_layers, vocab=vocab, ff_mult=ff_mult)
        if dev.type == "cuda":
            free, _total = torch.cuda.mem_get_info(dev)
            if need > memory_fraction * free:
                rows.append({"batch_size": bs, "oom": False, "mean_ms": None, "std_ms": None, "tokens_per_sec": None,
                             "skipped": f"estimated {need / 2**30:.1f} GiB exceeds {memory_fraction:.0%} of the "
                                        f"{free / 2**30:.1f} GiB free"})
                continue
        torch.manual_seed(seed)
        model = CareStudentLM(vocab_size=vocab, dim=dim, num_layers=num_layers, ff_mult=ff_mult).to(dev)
        if dev.type == "cuda":
            model = model.to(torch.bfloat16)
        model.train()
        x = torch.randint(0, vocab, (bs, seq_len), device=dev)
        y = torch.roll(x, -1, dims=1)
        precision = "bf16" if dev.type == "cuda" else "fp32"

        def step(model=model, x=x, y=y, precision=precision):
            train_ssm_step(model, x, y, chunk_size=seq_len, precision=precision, lm_head_backward_mode="fused")
            model.zero_grad(set_to_none=False)
        row = bench_one(step, batch=bs, seq_len=seq_len, warmup=warmup, steps=steps, device=dev)
        row["estimated_gib"] = round(need / 2**30, 2)
        rows.append(row)
        del model, x, y, step
        if dev.type == "cuda":
            torch.cuda.empty_cache()
        if row["oom"]:
            break                                        # larger sizes are not attempted after the first failure
    return {"device": str(dev), "device_name": torch.cuda.get_device_name(dev) if dev.type == "cuda" else "cpu",
            "model": {"dim": dim, "num_layers": num_layers, "seq_len": seq_len, "vocab": vocab, "ff_mult": ff_mult},
            "warmup": warmup, "steps": steps, "results": rows, "recommended_batch_size": recommend(rows)}


def render(rep: dict[str, Any]) -> str:
    lines = [f"{'batch':>8}  {'mean_ms':>10}  {'std_ms':>8}  {'tok/sec':>12}  status"]
    for r in rep["results"]:
        if r.get("tokens_per_sec"):
            mark = " <- recommended" if r["batch_size"] == rep["recommended_batch_size"] else ""
            lines.append(f"{r['batch_size']:>8}  {r['mean_ms']:>10.3f}  {r['std_ms']:>8.3f}  {r['tokens_per_sec']:>12,}  ok{mark}")
        else:
            lines.append(f"{r['batch_size']:>8}  {'-':>10}  {'-':>8}  {'-':>12}  " + ("out of memory" if r["oom"] else f"skipped: {r['skipped']}"))
    return "\n".join(lines)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--num-layers", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--vocab-size", type=int, default=16384)
    ap.add_argument("--ff-mult", type=int, default=2)
    ap.add_argument("--batch-sizes", default="128,256,512,1024,2048")
    ap.add_argument("--warmup-steps", type=int, default=3)
    ap.add_argument("--measure-steps", type=int, default=10)
    ap.add_argument("--memory-fraction", type=float, default=0.8)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output-json", default=None)
    a = ap.parse_args(argv)
    rep = sweep(batch_sizes=[int(b) for b in a.batch_sizes.split(",") if b], dim=a.dim, num_layers=a.num_layers,
                seq_len=a.seq_len, vocab=a.vocab_size, ff_mult=a.ff_mult, warmup=a.warmup_steps, steps=a.measure_steps,
                device=a.device, memory_fraction=a.memory_fraction)
    print(f"[device] {rep['device_name']}")
    print(render(rep))
    print(f"recommended batch size: {rep['recommended_batch_size']}")
    if a.output_json:
        with open(a.output_json, "w") as fh:
            json.dump(rep, fh, indent=2)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
