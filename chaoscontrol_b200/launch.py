"""Launch helpers: torchrun command lines for the runner, per-entry config
files, and the ranked summary of a results directory
(functions of experiments/23_fast_path/launch.py:16-200)."""
from __future__ import annotations

import json
import socket
import subprocess
import sys
from pathlib import Path
from typing import Any, Optional

__all__ = ["pick_free_port", "build_torchrun_cmd", "write_entry_config", "summarize_result_dir", "run_matrix",
           "DRY_RUN_RDZV_PORT"]

DRY_RUN_RDZV_PORT = 0       # obviously fake: a dry-run command pasted into a shell fails at rendezvous


def pick_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def build_torchrun_cmd(*, runner_path: Path | str = "chaoscontrol_b200.runner_fast_path", config_path: Path,
                       data_path: str, sp_model_path: Optional[str], output_json: Path, world_size: int,
                       rdzv_port: Optional[int] = None, output_ckpt: Optional[Path] = None,
                       budget_seconds: Optional[float] = None, val_cache_dir: Optional[Path | str] = None,
                       dry_run: bool = False) -> list[str]:
    """``python -m torch.distributed.run`` on 127.0.0.1 (container hostnames may not resolve).
    ``runner_path`` is a script path, or a dotted module name (run with ``-m``)."""
    if rdzv_port is None:
        rdzv_port = DRY_RUN_RDZV_PORT if dry_run else pick_free_port()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={int(world_size)}",
           "--master-addr", "127.0.0.1", "--master-port", str(rdzv_port)]
    rp = str(runner_path)
    cmd += [rp] if rp.endswith(".py") else ["-m", rp]
    cmd += ["--config", str(config_path), "--data-path", data_path, "--output-json", str(output_json)]
    if sp_model_path:
        cmd += ["--sp-model-path", sp_model_path]
    if output_ckpt is not None:
        cmd += ["--output-ckpt", str(output_ckpt)]
    if budget_seconds is not None:
        cmd += ["--budget", str(float(budget_seconds))]
    if val_cache_dir is not None:
        cmd += ["--val-cache-dir", str(val_cache_dir)]
    return cmd


def write_entry_config(entry: dict[str, Any], config_dir: Path) -> Path:
    import yaml
    config_dir.mkdir(parents=True, exist_ok=True)
    path = config_dir / f"{entry['name']}.yaml"
    path.write_text(yaml.safe_dump(entry, sort_keys=True))
    return path


def summarize_result_dir(results_dir: Path) -> dict[str, Any]:
    """``{"ranked": [...by aggregate tok/s, best first], "errors": [...]}`` over ``*.json`` results."""
    ranked: list[dict[str, Any]] = []
    errors: list[dict[str, str]] = []
    if not results_dir.exists():
        return {"ranked": ranked, "errors": errors}
    for path in sorted(results_dir.glob("*.json")):
        if path.name in {"matrix.json", "summary.json"}:
            continue
        try:
            data = json.loads(path.read_text())
        except json.JSONDecodeError as exc:
            errors.append({"name": path.stem, "error": f"unreadable: {exc}"})
            continue
        if not isinstance(data, dict):
            continue
        name = str((data.get("config") or {}).get("name", path.stem))
        if "error" in data:
            errors.append({"name": name, "error": str(data["error"])})
            continue
        tr, ev = data.get("train") or {}, data.get("eval") or {}
        ranked.append({"name": name, "aggregate_tokens_per_sec": float(tr.get("aggregate_tokens_per_sec", 0.0)),
                       "steps": int(tr.get("steps", 0)), "final_loss": tr.get("final_loss"), "bpb": ev.get("bpb"),
                       "peak_vram_mb": tr.get("peak_vram_mb")})
    ranked.sort(key=lambda r: r["aggregate_tokens_per_sec"], reverse=True)
    return {"ranked": ranked, "errors": errors}


def run_matrix(entries: list[dict[str, Any]], *, results_dir: Path, data_path: str, sp_model_path: Optional[str],
               world_size: int, dry_run: bool = False, val_cache_dir: Optional[str] = None,
               limit: Optional[int] = None, skip_existing: bool = True,
               checkpoint_dir: Optional[Path] = None) -> dict[str, Any]:
    """Runs the first ``limit`` entries (all by default).  With ``skip_existing`` an entry whose
    result file exists is left alone (idempotent re-runs); a failed entry leaves
    ``{"config", "error"}`` in its place so the sweep continues.  ``checkpoint_dir`` makes every
    run save ``<name>.pt`` there."""
    results_dir.mkdir(parents=True, exist_ok=True)
    if checkpoint_dir is not None and not dry_run:
        Path(checkpoint_dir).mkdir(parents=True, exist_ok=True)
    cmds = []
    for e in entries[:limit] if limit is not None else entries:
        out = results_dir / f"{e['name']}.json"
        if out.exists() and skip_existing:
            continue
        cfg = write_entry_config(e, results_dir / "configs")
        cmd = build_torchrun_cmd(config_path=cfg, data_path=data_path, sp_model_path=sp_model_path, output_json=out,
                                 world_size=world_size,
                                 budget_seconds=e.get("budget_seconds"), val_cache_dir=val_cache_dir,
                                 output_ckpt=None if checkpoint_dir is None else Path(checkpoint_dir) / f"{e['name']}.pt",
                                 dry_run=dry_run)
        cmds.append(cmd)
        if dry_run:
            continue
        if out.exists():
            out.unlink()
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0 and not out.exists():
            out.write_text(json.dumps({"config": e, "error": proc.stderr[-2000:]}, indent=2, default=str))
    summary = summarize_result_dir(results_dir)
    summary["commands"] = cmds if dry_run else []
    (results_dir / "summary.json").write_text(json.dumps(summary, indent=2, default=str))
    return summary
