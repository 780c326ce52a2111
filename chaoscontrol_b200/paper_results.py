"""Append-only JSONL registry of runs that may appear in a paper table, each tagged
``exploratory`` or ``confirmatory`` and stamped with the git commit that produced it
(API of src/chaoscontrol/paper_results.py:31-258: ``register / load / query / verify /
load_canonical_configs / is_canonical``; ``python -m chaoscontrol_b200.paper_results``
is the command-line face the reference keeps in ``scripts/paper_results.py``).

``verify`` rejects duplicate ``(experiment, condition, seed, status)`` keys and
confirmatory records written from a dirty working tree (their commit hash would not
pin the code that made the measurement).
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from collections import Counter
from dataclasses import asdict, dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Iterable, Literal, Optional

SCHEMA_VERSION = 1
Status = Literal["exploratory", "confirmatory"]
_STATUSES = ("confirmatory", "exploratory")
_REPO_ROOT = Path(__file__).resolve().parents[1]
DEFAULT_REGISTRY_PATH = _REPO_ROOT / "paper_results" / "registry.jsonl"
DEFAULT_CANONICAL_CONFIGS_PATH = _REPO_ROOT / "paper_results" / "canonical_configs.json"

__all__ = ["RunRecord", "Status", "SCHEMA_VERSION", "DEFAULT_REGISTRY_PATH", "DEFAULT_CANONICAL_CONFIGS_PATH",
           "register", "load", "query", "verify", "load_canonical_configs", "is_canonical", "main"]


@dataclass
class RunRecord:
    experiment: str
    condition: str
    seed: int
    status: Status
    metrics: dict
    config_hash: str
    git_sha: str = ""
    git_dirty: bool = False
    timestamp: str = ""
    artifacts: list = field(default_factory=list)
    extras: dict = field(default_factory=dict)
    schema_version: int = SCHEMA_VERSION

    def __post_init__(self) -> None:
        if self.status not in _STATUSES:
            raise ValueError(f"invalid status: {self.status!r} (expected one of {sorted(_STATUSES)})")
        if not self.timestamp:
            self.timestamp = datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")

    def key(self) -> tuple[str, str, int, str]:
        return (self.experiment, self.condition, self.seed, self.status)


def _git(*args: str) -> Optional[str]:
    try:
        return subprocess.run(["git", "-C", str(_REPO_ROOT), *args], capture_output=True, text=True,
                              check=True).stdout
    except (subprocess.CalledProcessError, FileNotFoundError):
        return None


def register(*, experiment: str, condition: str, seed: int, status: Status, metrics: dict, config_hash: str,
             artifacts: Iterable[str] = (), extras: Optional[dict] = None, registry_path=None,
             git_sha: Optional[str] = None, git_dirty: Optional[bool] = None) -> RunRecord:
    """Appends one record; commit hash / dirty flag / timestamp are filled in unless given."""
    if git_sha is None:
        out = _git("rev-parse", "HEAD")
        git_sha = out.strip() if out is not None else "unknown"
    if git_dirty is None:
        out = _git("status", "--porcelain")
        git_dirty = True if out is None else bool(out.strip())
    rec = RunRecord(experiment=experiment, condition=condition, seed=seed, status=status, metrics=dict(metrics),
                    config_hash=config_hash, git_sha=git_sha, git_dirty=git_dirty, artifacts=list(artifacts),
                    extras=dict(extras or {}))
    path = Path(registry_path) if registry_path is not None else DEFAULT_REGISTRY_PATH
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("a") as fh:
        fh.write(json.dumps(asdict(rec), sort_keys=True) + "\n")
    return rec


def load(registry_path=None) -> list[RunRecord]:
    path = Path(registry_path) if registry_path is not None else DEFAULT_REGISTRY_PATH
    if not path.exists():
        return []
    out = []
    for no, raw in enumerate(path.read_text().splitlines(), start=1):
        if not raw.strip():
            continue
        try:
            d = json.loads(raw)
        except json.JSONDecodeError as exc:
            raise ValueError(f"{path}:{no}: invalid JSON: {exc}") from exc
        d.pop("schema_version", None)
        out.append(RunRecord(**d))
    return out


def query(*, experiment: Optional[str] = None, condition: Optional[str] = None, status: Optional[Status] = None,
          registry_path=None) -> list[RunRecord]:
    want = {"experiment": experiment, "condition": condition, "status": status}
    return [r for r in load(registry_path)
            if all(v is None or getattr(r, k) == v for k, v in want.items())]


def verify(registry_path=None) -> dict:
    records = load(registry_path)
    first: dict[tuple, int] = {}
    dups = []
    for i, r in enumerate(records):
        if r.key() in first:
            dups.append(f"{r.key()} (lines {first[r.key()] + 1} and {i + 1})")
        else:
            first[r.key()] = i
    if dups:
        raise ValueError("duplicate registry keys: " + ", ".join(dups))
    dirty = [f"{r.experiment}/{r.condition} seed={r.seed} (line {i + 1})" for i, r in enumerate(records)
             if r.git_dirty and r.status == "confirmatory"]
    if dirty:
        raise ValueError("confirmatory records committed from dirty tree: " + ", ".join(dirty) +
                         ". Commit and re-register, or downgrade status to exploratory.")
    by_status = Counter(r.status for r in records)
    return {"n_records": len(records), "experiments": sorted({r.experiment for r in records}),
            "confirmatory": by_status["confirmatory"], "exploratory": by_status["exploratory"],
            "dirty_records": sum(r.git_dirty for r in records)}


def load_canonical_configs(path=None) -> dict[str, dict]:
    """``{config_hash: {experiment, condition, rationale, lineage}}``; ``{}`` when the file is absent."""
    p = Path(path) if path is not None else DEFAULT_CANONICAL_CONFIGS_PATH
    if not p.exists():
        return {}
    data = json.loads(p.read_text())
    return data["canonical"] if isinstance(data, dict) and "canonical" in data else data


def is_canonical(*, config_hash: str, experiment: str, condition: str, path=None) -> bool:
    """True only when the hash is declared canonical for this very (experiment, condition)."""
    entry = load_canonical_configs(path).get(config_hash)
    return entry is not None and entry.get("experiment") == experiment and entry.get("condition") == condition


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="paper_results")
    ap.add_argument("--registry", default=None)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("verify")
    ls = sub.add_parser("list")
    for k in ("experiment", "condition", "status"):
        ls.add_argument(f"--{k}", default=None)
    add = sub.add_parser("register")
    for k in ("experiment", "condition", "status", "config-hash"):
        add.add_argument(f"--{k}", required=True)
    add.add_argument("--seed", type=int, required=True)
    add.add_argument("--metrics", required=True, help="JSON object")
    add.add_argument("--artifact", action="append", default=[])
    add.add_argument("--artifacts", nargs="*", default=[], help="artifact paths, as one list")
    add.add_argument("--extras", default=None, help="JSON object stored with the record")
    a = ap.parse_args(argv)
    try:
        if a.cmd == "verify":
            print(json.dumps(verify(a.registry), indent=2))
        elif a.cmd == "list":
            for r in query(experiment=a.experiment, condition=a.condition, status=a.status, registry_path=a.registry):
                print(json.dumps(asdict(r), sort_keys=True))
        else:
            rec = register(experiment=a.experiment, condition=a.condition, seed=a.seed, status=a.status,
                           metrics=json.loads(a.metrics), config_hash=a.config_hash,
                           artifacts=[*a.artifact, *a.artifacts], extras=json.loads(a.extras) if a.extras else None,
                           registry_path=a.registry)
            print(json.dumps(asdict(rec), sort_keys=True))
    except ValueError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
