"""Warm multi-run worker: one ``torchrun`` launch executes a whole matrix of
``(condition, seed)`` configs, keeping the processes, CUDA contexts, NCCL / peer-memory
set-up and the loaded token shards alive between entries (behaviour of
experiments/19_prereqs/runner_persistent_ddp.py:145-805 and the launcher-side checks of
run_persistent_launcher.py:84-350).

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node N \\
        -m chaoscontrol_b200.runner_persistent_ddp --data-path D --sp-model-path M \\
        --config-matrix matrix.json --output-dir out/ --budget 600

The matrix is a JSON list of complete config dicts, each with ``name`` and ``seed``; entry
``i`` writes ``{name}_s{seed}.json``.  Contracts:

* idempotent AND config-checked: an existing output is skipped only when its stored
  ``config`` equals the requested entry, otherwise the run stops (a stale file from an edited
  matrix must not pass as a result);
* per-entry error isolation: every rank learns through a MAX-reduced flag whether any rank
  failed, rank 0 writes an ``{"config", "error"}`` marker and all ranks move on together;
* warm-up / restore: optional warm-up steps run on a snapshot that is restored before the
  timed run, with a fresh optimizer (handled inside ``run_condition``).
"""
from __future__ import annotations

import argparse
import gc
import hashlib
import json
import os
import random
import subprocess
import sys
import time
import traceback
from pathlib import Path
from typing import Any, Callable, Optional

import numpy as np
import torch
import torch.distributed as dist

REQUIRED_ENTRY_FIELDS = ("name", "seed", "precision", "model_dim", "num_layers", "seq_len", "batch_size",
                         "vocab_size", "optimizer", "base_lr", "chunk_size")
BENIGN_ERROR_PATTERNS = ("skipped:",)
FP8_UNAVAILABLE_PATTERNS = ("fp8 unavailable",)

__all__ = ["config_hash", "require_config_match", "apply_seed", "write_result_json", "sync_error_flag",
           "warmup_and_restore", "run_one_seed", "run_matrix_worker", "check_output_integrity",
           "validate_matrix_world_size", "base_config", "build_default_matrix", "fp8_is_available",
           "reject_stale_skip_markers", "filter_matrix_for_fp8", "write_skip_markers", "launch_main", "main"]


# ---------------------------------------------------------------- worker-side helpers
def config_hash(config: dict[str, Any]) -> str:
    return hashlib.sha1(json.dumps(config, sort_keys=True, default=str).encode()).hexdigest()[:8]


def require_config_match(out_path: Path, requested: dict[str, Any]) -> None:
    """Raises unless the stored output answers exactly the requested config.  Every rank reads the
    same file and decides the same way, so no collective is needed."""
    try:
        stored = json.loads(Path(out_path).read_text())
    except Exception as exc:
        raise RuntimeError(f"idempotent skip aborted: could not read stored JSON at {out_path}: {exc}. "
                           f"Delete or fix the file to re-run.") from exc
    if stored.get("config") != requested:
        raise RuntimeError(f"idempotent skip aborted: config mismatch at {out_path}. Stored config "
                           f"hash={config_hash(stored.get('config') or {})} does not match requested "
                           f"hash={config_hash(requested)}. Delete the stale output or use a fresh --output-dir.")


def apply_seed(seed: int) -> None:
    """Re-seeds every generator the training path touches (the previous entry advanced them all)."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def write_result_json(out_path: Path, payload: dict[str, Any]) -> None:
    out_path = Path(out_path)
    out_path.parent.mkdir(parents=True, exist_ok=True)
    tmp = out_path.with_suffix(".tmp")
    tmp.write_text(json.dumps(payload, indent=2, default=str))
    tmp.rename(out_path)


def sync_error_flag(local_error: bool, device: torch.device, ddp_active: bool) -> bool:
    """True on every rank when any rank failed."""
    if not ddp_active:
        return bool(local_error)
    flag = torch.tensor([1.0 if local_error else 0.0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return bool(flag.item() > 0.5)


def warmup_and_restore(*, model: torch.nn.Module, warmup_call_fn: Callable[[], Any],
                       build_optimizer_fn: Callable[[], torch.optim.Optimizer], device: torch.device,
                       ddp_active: bool) -> torch.optim.Optimizer:
    """Snapshot -> warm-up -> restore -> gradients cleared -> fresh optimizer.  After it the model is
    byte-identical to its pre-warm-up state and nothing of the warm-up's optimizer state survives."""
    snap = {k: v.detach().clone() for k, v in model.state_dict().items()}
    warmup_call_fn()
    model.load_state_dict(snap, strict=True)
    model.zero_grad(set_to_none=True)
    if device.type == "cuda":
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
    if ddp_active:
        dist.barrier()
    return build_optimizer_fn()


def run_one_seed(*, config: dict[str, Any], out_path: Path, data_path: str, sp_model_path: Optional[str],
                 budget_seconds: float, world_size: Optional[int] = None) -> dict[str, Any]:
    """One matrix entry through the production train + eval entry point, process group kept."""
    from .runner_fast_path import run_condition
    apply_seed(int(config.get("seed", 0)))
    return run_condition(dict(config), data_path=data_path, sp_model_path=sp_model_path,
                         budget_seconds=float(budget_seconds), output_json=str(out_path), output_ckpt=None,
                         world_size_override=world_size, keep_process_group=True)


def _dry_run(entries: list[dict], matrix_path: Path, output_dir: Path) -> int:
    print(f"[dry-run] matrix={matrix_path} entries={len(entries)}\n[dry-run] output_dir={output_dir}")
    for i, e in enumerate(entries):
        name, seed = str(e.get("name", f"entry{i}")), int(e.get("seed", 0))
        out = output_dir / f"{name}_s{seed}.json"
        print(f"[dry-run] {i:3d}: name={name} seed={seed} precision={e.get('precision', 'bf16')} "
              f"hash={config_hash(e)} out={out} ({'existing' if out.exists() else 'new'})")
    for i, e in enumerate(entries):
        missing = sorted(set(REQUIRED_ENTRY_FIELDS) - set(e))
        if missing:
            raise ValueError(f"entry {i} (name={e.get('name')!r}) missing required fields: {missing}")
    print(f"[dry-run] all {len(entries)} entries have required fields")
    return 0


def run_matrix_worker(entries: list[dict[str, Any]], *, output_dir: Path, data_path: str,
                      sp_model_path: Optional[str], budget_seconds: float, world_size: Optional[int] = None,
                      run_entry: Optional[Callable[..., Any]] = None) -> dict[str, int]:
    """The per-process loop.  ``run_entry`` (default :func:`run_one_seed`) can be replaced in tests."""
    for key in ("device", "vocab_size"):
        vals = {str(e.get(key, "auto" if key == "device" else None)) for e in entries}
        if len(vals) > 1:
            raise ValueError(f"matrix entries disagree on {key}: {sorted(vals)}; one warm worker needs one value")
    run_entry = run_entry or run_one_seed
    ddp = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
    rank = dist.get_rank() if ddp else 0
    device = (torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
              if torch.cuda.is_available() and (not ddp or dist.get_backend() == "nccl") else torch.device("cpu"))
    counts = {"completed": 0, "skipped": 0, "errored": 0}
    t0 = time.monotonic()
    for i, entry in enumerate(entries):
        name, seed = str(entry.get("name") or ""), int(entry.get("seed", 0))
        if not name:
            raise ValueError(f"entry {i} missing 'name' field")
        out = Path(output_dir) / f"{name}_s{seed}.json"
        if sync_error_flag(out.exists(), device, ddp):        # MAX-reduce: any rank sees the file
            require_config_match(out, entry)
            if rank == 0:
                print(f"[rank 0] skip {name}_s{seed} (output exists at {out})", flush=True)
            counts["skipped"] += 1
            continue
        t_entry, err = time.monotonic(), None
        try:
            run_entry(config=entry, out_path=out, data_path=data_path, sp_model_path=sp_model_path,
                      budget_seconds=budget_seconds, world_size=world_size)
        except Exception as exc:  # noqa: BLE001 - isolation is the point
            err = f"{type(exc).__name__}: {exc}"
            if rank == 0:
                print(f"[rank 0] ERROR on {name}_s{seed}: {err}\n{traceback.format_exc()}", flush=True)
            gc.collect()
            if device.type == "cuda":
                torch.cuda.empty_cache()
        if sync_error_flag(err is not None, device, ddp):
            counts["errored"] += 1
            if rank == 0:
                write_result_json(out, {"config": entry, "error": err or "peer_rank_error"})
            if ddp:
                dist.barrier()
            continue
        counts["completed"] += 1
        if rank == 0:
            print(f"[rank 0] completed {name}_s{seed} in {time.monotonic() - t_entry:.1f}s "
                  f"(entry {i + 1}/{len(entries)})", flush=True)
    if rank == 0:
        print(f"[rank 0] matrix done: {counts} elapsed={time.monotonic() - t0:.1f}s", flush=True)
    return counts


# ---------------------------------------------------------------- launcher-side helpers
def check_output_integrity(output_dir: Path, entries: list[dict[str, Any]],
                           benign_error_patterns: tuple[str, ...] = BENIGN_ERROR_PATTERNS
                           ) -> tuple[int, int, list[str]]:
    """``(successes, benign skips, real errors)`` over the expected outputs: counting files is not
    enough, every file may be an error marker."""
    ok = benign = 0
    bad: list[str] = []
    for e in entries:
        tag = f"{e.get('name', '?')}_s{int(e.get('seed', 0))}"
        path = Path(output_dir) / f"{tag}.json"
        if not path.exists():
            bad.append(f"{tag}: missing output file")
            continue
        try:
            data = json.loads(path.read_text())
        except Exception as exc:  # noqa: BLE001
            bad.append(f"{tag}: malformed JSON ({exc})")
            continue
        if "error" in data:
            if any(p in str(data["error"]) for p in benign_error_patterns):
                benign += 1
            else:
                bad.append(f"{tag}: error={data['error']}")
        elif "eval" in data and "train" in data:
            ok += 1
        else:
            bad.append(f"{tag}: neither 'error' nor ('eval'+'train') keys present")
    return ok, benign, bad


def validate_matrix_world_size(entries: list[dict[str, Any]], cli_world_size: int) -> None:
    """The run uses the launcher's world size; an entry tagged with another one would mislabel results."""
    off = [(str(e.get("name", "?")), int(e.get("seed", 0)), e.get("world_size")) for e in entries
           if e.get("world_size") != cli_world_size]
    if off:
        more = f" (+{len(off) - 5} more)" if len(off) > 5 else ""
        raise ValueError(f"matrix entries' world_size disagrees with --world-size={cli_world_size}: {off[:5]}{more}")


def base_config(*, world_size: int, base_lr: float, precision: str, seed: int, name: str, **overrides: Any) -> dict:
    """One entry in the submission regime (4 x 256, V = 16384, seq 512, batch 1024 per rank, Muon)."""
    cfg = {"name": name, "seed": seed, "precision": precision, "model_type": "ssm", "vocab_size": 16384,
           "model_dim": 256, "num_layers": 4, "ff_mult": 2, "seq_len": 512, "stride": 256, "batch_size": 1024,
           "eval_batches": 16, "a_mode": "diag", "base_lr": base_lr, "activation_checkpoint": True,
           "optimizer": "muon", "chunk_size": 64, "world_size": world_size, "local_attn_window": 0,
           "local_attn_heads": 1, "local_attn_dim": 64, "grad_clip_norm": 1.0, "weight_decay": 0.01,
           "device": "auto", "dtype": "bf16"}
    cfg.update(overrides)
    return cfg


def build_default_matrix(world_size: int, base_lr: float, seeds: list[int], conditions: list[str]) -> list[dict]:
    """conditions x seeds, grouped by condition."""
    return [base_config(world_size=world_size, base_lr=base_lr, precision=p, seed=s, name=p)
            for p in conditions for s in seeds]


def fp8_is_available() -> bool:
    """The in-tree fp8 linears need a CUDA device and the kernel library."""
    try:
        from .ops import _lib
        return bool(torch.cuda.is_available() and _lib.available())
    except Exception:
        return False


def _fp8_entries(entries):
    return [e for e in entries if str(e.get("precision", "")).startswith("fp8")]


def reject_stale_skip_markers(entries: list[dict], output_dir: Path,
                              unavailable_patterns: tuple[str, ...] = FP8_UNAVAILABLE_PATTERNS,
                              probe: Callable[[], bool] = fp8_is_available) -> None:
    """When fp8 can run here, skip markers left by an earlier run on a host where it could not must be
    deleted first: honouring them would exit 0 with no fp8 result."""
    if not probe():
        return
    stale = []
    for e in _fp8_entries(entries):
        p = Path(output_dir) / f"{e.get('name', '?')}_s{int(e.get('seed', 0))}.json"
        try:
            err = str(json.loads(p.read_text()).get("error", ""))
        except Exception:
            continue
        if any(pat in err for pat in unavailable_patterns):
            stale.append(p)
    if stale:
        more = f"\n  (+{len(stale) - 5} more)" if len(stale) > 5 else ""
        raise RuntimeError(f"fp8 is available on this host, but {len(stale)} fp8 entries have stale skip markers "
                           "from a run where it was not. Delete them to re-run fp8:\n  " +
                           "\n  ".join(map(str, stale[:5])) + more)


def filter_matrix_for_fp8(entries: list[dict], output_dir: Path, probe: Callable[[], bool] = fp8_is_available
                          ) -> tuple[list[dict], list[dict]]:
    """``(runnable, skipped)``: fp8 entries are dropped when fp8 cannot run on this host."""
    fp8 = _fp8_entries(entries)
    if not fp8 or probe():
        return list(entries), []
    print(f"[launcher] fp8 unavailable on this host; dropping {len(fp8)} fp8 entries from the matrix.", flush=True)
    return [e for e in entries if e not in fp8], fp8


def write_skip_markers(skipped: list[dict], output_dir: Path) -> None:
    """A skipped entry gets a decisive marker, so downstream sees 'skipped', not 'absent'."""
    for e in skipped:
        write_result_json(Path(output_dir) / f"{e.get('name', '?')}_s{int(e.get('seed', 0))}.json",
                          {"config": e, "error": "skipped: fp8 unavailable on this host"})


# ---------------------------------------------------------------- CLI (launcher)
DEFAULT_LAUNCH_SEEDS = [1337, 2674, 4011, 5348]


def launch_main(argv: Optional[list[str]] = None, *, call=subprocess.call) -> int:
    """``python -m chaoscontrol_b200.runner_persistent_ddp launch ...``: builds (or reads) the matrix, runs
    the pre-flight checks, starts ONE torchrun job whose ranks walk the whole matrix in a warm process group
    (this module's worker), then fails closed on any real error among the expected outputs
    (experiments/19_prereqs/run_persistent_launcher.py:382-540 of the reference)."""
    ap = argparse.ArgumentParser(prog="runner_persistent_ddp launch", description="warm multi-seed launcher")
    ap.add_argument("--data-path", required=True)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--budget", type=float, default=600.0)
    ap.add_argument("--world-size", type=int, default=4)
    ap.add_argument("--base-lr", type=float, default=0.128)
    ap.add_argument("--seeds", type=int, nargs="+", default=DEFAULT_LAUNCH_SEEDS)
    ap.add_argument("--conditions", nargs="+", default=["bf16", "fp8"])
    ap.add_argument("--matrix-json", default=None, help="a pre-written matrix instead of conditions x seeds")
    ap.add_argument("--rdzv-port", type=int, default=29500)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    out = Path(a.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    if a.matrix_json:
        entries = json.loads(Path(a.matrix_json).read_text())
        if not isinstance(entries, list):
            raise ValueError(f"--matrix-json file must be a JSON list, got {type(entries).__name__}")
        print(f"[launcher] using external matrix: {a.matrix_json} ({len(entries)} entries)", flush=True)
    else:
        entries = build_default_matrix(a.world_size, a.base_lr, list(a.seeds), list(a.conditions))
        print(f"[launcher] built matrix: conditions={a.conditions} seeds={a.seeds} ws={a.world_size} lr={a.base_lr} "
              f"({len(entries)} entries)", flush=True)
    validate_matrix_world_size(entries, a.world_size)
    reject_stale_skip_markers(entries, out)
    runnable, skipped = filter_matrix_for_fp8(entries, out)
    if skipped:
        write_skip_markers(skipped, out)
    if not runnable:
        print(f"[launcher] FAIL: zero runnable entries of {len(entries)} after the pre-flight checks; an empty run "
              "is not a successful run", flush=True)
        return 1
    matrix_path = out / ".persistent_matrix.json"
    matrix_path.write_text(json.dumps(runnable, indent=2, default=str))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={int(a.world_size)}",
           "--master-addr", "127.0.0.1", "--master-port", str(int(a.rdzv_port)), "-m",
           "chaoscontrol_b200.runner_persistent_ddp", "--config-matrix", str(matrix_path), "--data-path", a.data_path,
           "--output-dir", str(out), "--budget", str(float(a.budget)), "--world-size", str(int(a.world_size))]
    if a.sp_model_path:
        cmd += ["--sp-model-path", a.sp_model_path]
    if a.dry_run:
        print("[launcher] dry-run; would execute:\n  " + " ".join(cmd))
        print("[launcher] first runnable entry:\n  " + json.dumps(runnable[0], indent=2, default=str))
        print(f"[launcher] matrix left at {matrix_path} for inspection")
        return 0
    print(f"[launcher] launching: {' '.join(cmd)}", flush=True)
    try:
        ret = call(cmd)
    finally:
        matrix_path.unlink(missing_ok=True)
    if ret != 0:
        print(f"[launcher] torchrun exited non-zero: {ret}", flush=True)
        return int(ret)
    ok, benign, bad = check_output_integrity(out, entries)
    print(f"[launcher] outputs: success={ok} benign_skip={benign} errors={len(bad)} total_expected={len(entries)}", flush=True)
    for err in bad:
        print(f"  - {err}", flush=True)
    return 1 if bad else 0


# ---------------------------------------------------------------- CLI (worker)
def main(argv: Optional[list[str]] = None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if args and args[0] == "launch":
        return launch_main(args[1:])
    argv = args
    ap = argparse.ArgumentParser(description="warm multi-run worker (or `launch ...` for the launcher)")
    ap.add_argument("--data-path", required=True)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--config-matrix", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--budget", type=float, default=600.0)
    ap.add_argument("--world-size", type=int, default=None)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    entries = json.loads(Path(a.config_matrix).read_text())
    if not isinstance(entries, list):
        raise ValueError(f"matrix JSON must be a list of entry dicts, got {type(entries).__name__}")
    if a.dry_run:
        return _dry_run(entries, Path(a.config_matrix), Path(a.output_dir))
    from .runner_fast_path import _init_distributed
    _init_distributed(a.world_size)
    try:
        run_matrix_worker(entries, output_dir=Path(a.output_dir), data_path=a.data_path,
                          sp_model_path=a.sp_model_path, budget_seconds=a.budget, world_size=a.world_size)
    finally:
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
