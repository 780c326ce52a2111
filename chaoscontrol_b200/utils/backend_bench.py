"""Backend comparisons: the diagonal recurrence (serial loop / chunked tensor ops / the CUDA scan kernel) in
forward, backward and forward+backward, and one SSM block fused against unfused.

    python -m chaoscontrol_b200.utils.backend_bench scan  [--B 1024 --T 512 --D 256 --dtype bf16]
    python -m chaoscontrol_b200.utils.backend_bench block [--batch-sizes 32 128 512 --seq-len 512 --dim 256]

Same tables as the reference's ``benchmarks/bench_ssm_scan.py:60-324`` and
``benchmarks/bench_fused_block.py:60-232``.  ``fwd`` runs without gradients; ``bwd`` replays
``autograd.grad`` on one retained graph; ``fwd+bwd`` builds a fresh graph each iteration, which is what a
training step pays.  Timing: CUDA events on the launching stream on a GPU (wall clock on a CPU), mean
over the timed iterations after the warm-up.  The serial loop is skipped above ``--python-max-T`` steps
(it is there to show the gap, and a 512-step Python loop at full batch takes seconds per iteration).
"""
from __future__ import annotations

import argparse
import json
import time
from typing import Any, Callable, Optional, Sequence

import torch

from ..ops import scan as S

__all__ = ["time_ms", "bench_scan", "bench_block", "main"]

DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def time_ms(fn: Callable[[], Any], *, warmup: int, iters: int, device: torch.device) -> float:
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(iters):
            fn()
        t1.record()
        t1.synchronize()
        return t0.elapsed_time(t1) / iters
    t = time.perf_counter()
    for _ in range(iters):
        fn()
    return (time.perf_counter() - t) * 1e3 / iters


def scan_backends(device: torch.device) -> dict[str, Callable]:
    out = {"python": S.diag_recurrence_reference, "chunked": S.diag_recurrence_chunked}
    if device.type == "cuda":
        out["ssm_scan"] = S.ssm_scan
    return out


def bench_scan(*, B: int, T: int, D: int, dtype: str = "bf16", warmup: int = 5, iters: int = 20,
               device: Optional[str] = None, python_max_T: int = 128, seed: int = 0) -> dict[str, Any]:
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(seed)
    decay = (torch.rand(B, T, D, generator=g) * 0.2 + 0.8).to(dev, dt)
    update = torch.randn(B, T, D, generator=g).to(dev, dt)
    rows = []
    for name, fn in scan_backends(dev).items():
        if name == "python" and T > python_max_T:
            rows.append({"backend": name, "skipped": f"T = {T} > {python_max_T}"})
            continue

        def fwd(fn=fn):
            with torch.no_grad():
                fn(decay, update)
        d1, u1 = decay.clone().requires_grad_(True), update.clone().requires_grad_(True)
        out = fn(d1, u1)
        gout = torch.ones_like(out)

        def bwd(out=out, d1=d1, u1=u1, gout=gout):
            torch.autograd.grad(out, (d1, u1), gout, retain_graph=True)

        def both(fn=fn):
            d2, u2 = decay.detach().requires_grad_(True), update.detach().requires_grad_(True)
            o = fn(d2, u2)
            torch.autograd.grad(o, (d2, u2), torch.ones_like(o))
        row: dict[str, Any] = {"backend": name}
        for mode, f in (("fwd", fwd), ("bwd", bwd), ("fwd+bwd", both)):
            ms = time_ms(f, warmup=warmup, iters=iters, device=dev)
            row[mode] = {"ms": round(ms, 4), "tokens_per_sec": round(B * T / ms * 1e3)}
        rows.append(row)
    return {"device": str(dev), "shape": {"B": B, "T": T, "D": D}, "dtype": dtype, "warmup": warmup, "iters": iters,
            "results": rows}


def bench_block(*, batch_sizes: Sequence[int], seq_len: int = 512, dim: int = 256, ff_mult: int = 2, dtype: str = "bf16",
                warmup: int = 5, iters: int = 20, device: Optional[str] = None, seed: int = 0) -> dict[str, Any]:
    """One block, the same weights in both variants, forward + backward per iteration."""
    from ..models.core_fused import FusedCareSSMBlock, get_post_scan_backend
    from ..models.model import CareSSMBlock
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dt = DTYPES[dtype] if dev.type == "cuda" else torch.float32
    rows = []
    for bs in batch_sizes:
        torch.manual_seed(seed)
        plain = CareSSMBlock(dim, ff_mult).to(dev, dt)
        fused = FusedCareSSMBlock.from_unfused(plain)
        x = torch.randn(bs, seq_len, dim, device=dev, dtype=dt)

        def step(block):
            xi = x.detach().requires_grad_(True)
            block(xi).float().sum().backward()
            block.zero_grad(set_to_none=True)
        a = time_ms(lambda: step(plain), warmup=warmup, iters=iters, device=dev)
        b = time_ms(lambda: step(fused), warmup=warmup, iters=iters, device=dev)
        rows.append({"batch_size": int(bs), "unfused_ms": round(a, 4), "fused_ms": round(b, 4),
                     "unfused_tokens_per_sec": round(bs * seq_len / a * 1e3),
                     "fused_tokens_per_sec": round(bs * seq_len / b * 1e3), "speedup": round(a / b, 3)})
    return {"device": str(dev), "dtype": str(dt).replace("torch.", ""), "seq_len": seq_len, "dim": dim, "ff_mult": ff_mult,
            "backend": get_post_scan_backend(), "results": rows}


def _render_scan(rep: dict[str, Any]) -> str:
    lines = [f"{'backend':<10} {'mode':<8} {'ms/step':>10} {'tok/s':>14}"]
    for r in rep["results"]:
        if "skipped" in r:
            lines.append(f"{r['backend']:<10} skipped ({r['skipped']})")
            continue
        for mode in ("fwd", "bwd", "fwd+bwd"):
            lines.append(f"{r['backend']:<10} {mode:<8} {r[mode]['ms']:>10.4f} {r[mode]['tokens_per_sec']:>14,}")
    return "\n".join(lines)


def _render_block(rep: dict[str, Any]) -> str:
    lines = [f"{'batch':>6} {'unfused ms':>11} {'fused ms':>9} {'unfused tok/s':>14} {'fused tok/s':>12} {'speedup':>8}"]
    for r in rep["results"]:
        lines.append(f"{r['batch_size']:>6} {r['unfused_ms']:>11.4f} {r['fused_ms']:>9.4f} {r['unfused_tokens_per_sec']:>14,} "
                     f"{r['fused_tokens_per_sec']:>12,} {r['speedup']:>8.3f}")
    return "\n".join(lines)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("scan")
    s.add_argument("--B", type=int, default=1024)
    s.add_argument("--T", type=int, default=512)
    s.add_argument("--D", type=int, default=256)
    s.add_argument("--python-max-T", type=int, default=128)
    b = sub.add_parser("block")
    b.add_argument("--batch-sizes", type=int, nargs="+", default=[32, 128, 512])
    b.add_argument("--seq-len", type=int, default=512)
    b.add_argument("--dim", type=int, default=256)
    b.add_argument("--ff-mult", type=int, default=2)
    for p in (s, b):
        p.add_argument("--dtype", default="bf16", choices=sorted(DTYPES))
        p.add_argument("--warmup", type=int, default=5)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--device", default=None)
        p.add_argument("--output-json", default=None)
    a = ap.parse_args(argv)
    if a.cmd == "scan":
        rep = bench_scan(B=a.B, T=a.T, D=a.D, dtype=a.dtype, warmup=a.warmup, iters=a.iters, device=a.device,
                         python_max_T=a.python_max_T)
        print(_render_scan(rep))
    else:
        rep = bench_block(batch_sizes=a.batch_sizes, seq_len=a.seq_len, dim=a.dim, ff_mult=a.ff_mult, dtype=a.dtype,
                          warmup=a.warmup, iters=a.iters, device=a.device)
        print(f"post-scan backend: {rep['backend']}")
        print(_render_block(rep))
    if a.output_json:
        with open(a.output_json, "w") as fh:
            json.dump(rep, fh, indent=2)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
