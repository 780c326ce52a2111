"""Throughput-lever screens (experiment 18): one table of tests, one launcher, one
set of decision gates.

The reference keeps one orchestrator script per test
(experiments/18_throughput_levers/run_exp18.py and run_exp18_test{3,4,4b,5,5b,6,7,8,10}.py,
shared helpers in _harness.py).  Each asks one question about the 4 x 256 / V 16384
recipe, varies one axis, and ends in a gate that later tests inherit from.  Here
every test is a :class:`LeverTest` row: the base envelope, the axis, the launch
pattern, and the gate; ``build_entries`` turns a row into the ``launch.run_matrix``
entry list and ``decide`` applies the gate to result files.

Learning-rate rule shared by all tests: the calibrated anchor is batch 32 at
2e-3; rates scale linearly with the global batch (``linear_lr``).  Tests 6, 7 and
8 do not carry a rate of their own: they read the winner of the rate screen
(test 5 / 5b) and refuse a missing or provisional one unless ``base_lr`` is given.
"""
from __future__ import annotations

import json
import math
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Optional, Sequence

from .analysis import paired_ttest

ANCHOR_BATCH, ANCHOR_LR = 32, 2e-3
SWEEP_SEEDS = [1337, 2674, 4011, 5348, 6685, 8022, 9359]
DEFAULT_SEEDS = SWEEP_SEEDS[:4]
UNIFORM_LOSS = {8192: math.log(8192), 16384: math.log(16384)}
STALL_MARGIN = 1.0          # a final loss within this many nats of ln(V) counts as a stall (ln 16384 = 9.70 -> 8.70)
NOISE_GAP_BPB = 0.006       # two conditions closer than this with p >= 0.05 are inside seed noise
DDP_PER_GPU_FLOOR = 0.85    # a DDP world must keep this share of the single-GPU per-GPU rate
FP8_SPEEDUP_FLOOR = 1.3     # fp8 must buy this much aggregate throughput to be worth the dtype risk
FP8_BPB_TOLERANCE = 0.02


def linear_lr(global_batch: int) -> float:
    return ANCHOR_LR * global_batch / ANCHOR_BATCH


def _envelope(**over: Any) -> dict[str, Any]:
    cfg = {"model_type": "ssm", "vocab_size": 16384, "model_dim": 256, "num_layers": 4, "ff_mult": 2,
           "seq_len": 512, "stride": 256, "batch_size": 512, "eval_batches": 16, "a_mode": "diag",
           "base_lr": ANCHOR_LR, "local_attn_window": 0, "local_attn_heads": 1, "local_attn_dim": 64}
    cfg.update(over)
    return cfg


_SUBMISSION = dict(batch_size=1024, optimizer="muon", chunk_size=64, activation_checkpoint=True)


@dataclass(frozen=True)
class LeverTest:
    key: str
    question: str
    pattern: str                                   # "parallel_single_gpu" | "ddp"
    conditions: Callable[[Optional[float]], dict[str, dict[str, Any]]]
    gate: str
    inherits_lr_from: Optional[str] = None
    seeds: Sequence[int] = field(default_factory=lambda: tuple(DEFAULT_SEEDS))
    budget_seconds: float = 600.0

    def world_size(self, cfg: dict[str, Any]) -> int:
        return int(cfg.get("world_size", 1 if self.pattern == "parallel_single_gpu" else 2))


def _need_lr(lr: Optional[float], key: str) -> float:
    if lr is None:
        raise ValueError(f"{key} inherits its learning rate from the rate screen: pass base_lr or run that screen first")
    return float(lr)


TESTS: dict[str, LeverTest] = {t.key: t for t in (
    LeverTest("test2", "does the 16384-entry tokenizer beat the 8192-entry one at a matched envelope?",
              "parallel_single_gpu",
              lambda lr: {f"bare_fast_ssm_sp{v}": _envelope(vocab_size=v, batch_size=32, crit_target_coupling=0.92)
                          for v in (8192, 16384)},
              "best_bpb", seeds=tuple(SWEEP_SEEDS)),
    LeverTest("test3", "does activation checkpointing turn memory headroom into lower bpb at matched wall clock?",
              "parallel_single_gpu",
              lambda lr: {"noctk_bs512": _envelope(batch_size=512, activation_checkpoint=False, crit_target_coupling=0.92),
                          "ckpt_bs1024": _envelope(batch_size=1024, activation_checkpoint=True, crit_target_coupling=0.92),
                          "ckpt_bs2048": _envelope(batch_size=2048, activation_checkpoint=True, crit_target_coupling=0.92)},
              "beats_first"),
    LeverTest("test4", "does data parallelism turn a second GPU into lower bpb at matched wall clock?", "ddp",
              lambda lr: {"ws1": _envelope(world_size=1, base_lr=linear_lr(512), crit_target_coupling=0.92),
                          "ws2_ddp": _envelope(world_size=2, base_lr=linear_lr(1024), crit_target_coupling=0.92)},
              "ddp_scaling"),
    LeverTest("test4b", "world-size screen in the submission regime (global batch 2048 / 4096)", "ddp",
              lambda lr: {"ws2": _envelope(world_size=2, base_lr=0.064, **_SUBMISSION),
                          "ws4": _envelope(world_size=4, base_lr=0.128, **_SUBMISSION)},
              "ddp_scaling"),
    LeverTest("test5", "which rate is stable and best at global batch 1024?", "ddp",
              lambda lr: {n: _envelope(world_size=2, base_lr=linear_lr(1024) / d, crit_target_coupling=0.92)
                          for n, d in (("lr_linear", 1), ("lr_half", 2), ("lr_quarter", 4))},
              "lr_screen"),
    LeverTest("test5b", "the same screen at global batch 2048 with Muon", "ddp",
              lambda lr: {n: _envelope(world_size=2, base_lr=linear_lr(2048) / d, batch_size=1024, optimizer="muon",
                                       chunk_size=64)
                          for n, d in (("lr_linear", 1), ("lr_half", 2), ("lr_quarter", 4))},
              "lr_screen"),
    LeverTest("test6", "do longer sequences buy bpb per wall clock?", "ddp",
              lambda lr: {f"seq{s}": _envelope(world_size=2, seq_len=s, stride=s // 2, base_lr=_need_lr(lr, "test6"),
                                               activation_checkpoint=True, crit_target_coupling=0.92)
                          for s in (512, 1024, 2048)},
              "best_bpb_vs_first", inherits_lr_from="test5"),
    LeverTest("test7", "AdamW, Muon or LAMB at the data-parallel batch?", "ddp",
              lambda lr: {n: _envelope(world_size=2, optimizer=o, base_lr=_need_lr(lr, "test7"), crit_target_coupling=0.92)
                          for n, o in (("adamw_baseline", "adamw"), ("muon", "muon"), ("lamb", "lamb"))},
              "pairwise", inherits_lr_from="test5"),
    LeverTest("test8", "sequence length again, checkpointing held on for every arm", "ddp",
              lambda lr: {f"seq{s}": _envelope(world_size=2, seq_len=s, stride=256, base_lr=_need_lr(lr, "test8"),
                                               **_SUBMISSION)
                          for s in (512, 1024, 2048)},
              "best_bpb_vs_first", inherits_lr_from="test5b"),
    LeverTest("test10", "is fp8 worth its risk at the submission regime?", "ddp",
              lambda lr: {p: _envelope(world_size=4, base_lr=0.128 if lr is None else lr, precision=p, **_SUBMISSION)
                          for p in ("bf16", "fp8")},
              "fp8_gate"),
)}


# ---------------------------------------------------------------------------
# matrix
# ---------------------------------------------------------------------------
def inherited_lr(test: LeverTest, results_root: Path, *, allow_provisional: bool = False) -> Optional[float]:
    """The winner's rate from the screen this test inherits from, or None when it has none.
    Raises when the screen has not run, emitted no winner, or only a provisional one."""
    if test.inherits_lr_from is None:
        return None
    path = Path(results_root) / f"results_{test.inherits_lr_from}" / f"{test.inherits_lr_from}_summary.json"
    if not path.exists():
        raise FileNotFoundError(f"{test.key} needs {path} (the rate screen's summary) or an explicit base_lr")
    dec = json.loads(path.read_text()).get("_decision", {})
    if dec.get("winner_base_lr") is None:
        raise ValueError(f"{path} names no winner: {test.key} cannot inherit a rate from it")
    if dec.get("winner_is_provisional") and not allow_provisional:
        raise ValueError(f"{path}: the winner is provisional (not cross-checked); pass base_lr to override")
    return float(dec["winner_base_lr"])


def build_entries(key: str, *, base_lr: Optional[float] = None, results_root: Optional[Path] = None,
                  seeds: Optional[Sequence[int]] = None, budget_seconds: Optional[float] = None) -> list[dict[str, Any]]:
    """Entries for ``launch.run_matrix``: ``<condition>_s<seed>`` names, one per condition and seed."""
    test = TESTS[key]
    if base_lr is None and test.inherits_lr_from is not None and results_root is not None:
        base_lr = inherited_lr(test, results_root)
    out = []
    for cname, cfg in test.conditions(base_lr).items():
        for s in (seeds or test.seeds):
            e = dict(cfg, name=f"{cname}_s{s}", condition=cname, seed=int(s), world_size=test.world_size(cfg),
                     budget_seconds=float(budget_seconds or test.budget_seconds), exp18_test=key)
            out.append(e)
    return out


def launch_plan(entries: Sequence[dict[str, Any]], num_gpus: int) -> list[list[dict[str, Any]]]:
    """Waves of entries that run at the same time on ``num_gpus`` GPUs: single-GPU entries
    fill every GPU, a data-parallel entry takes ``world_size`` of them."""
    waves: list[list[dict[str, Any]]] = []
    cur, used = [], 0
    for e in entries:
        ws = int(e.get("world_size", 1))
        if ws > num_gpus:
            raise ValueError(f"{e['name']} needs {ws} GPUs, the pod has {num_gpus}")
        if used + ws > num_gpus:
            waves.append(cur)
            cur, used = [], 0
        cur.append(e)
        used += ws
    if cur:
        waves.append(cur)
    return waves


def run_test(key: str, *, results_root: Path, data_path: str, sp_model_path: Optional[str], base_lr: Optional[float] = None,
             seeds: Optional[Sequence[int]] = None, budget_seconds: Optional[float] = None, dry_run: bool = False) -> dict:
    """Run every entry of a test through ``launch.run_matrix`` (one world size at a time) and decide."""
    from .launch import run_matrix
    entries = build_entries(key, base_lr=base_lr, results_root=results_root, seeds=seeds, budget_seconds=budget_seconds)
    rdir = Path(results_root) / f"results_{key}"
    cmds = []
    for ws in sorted({e["world_size"] for e in entries}):
        s = run_matrix([e for e in entries if e["world_size"] == ws], results_dir=rdir, data_path=data_path,
                       sp_model_path=sp_model_path, world_size=ws, dry_run=dry_run)
        cmds += s.get("commands", [])
    if dry_run:
        return {"commands": cmds, "entries": entries}
    summary = decide(key, rdir, base_lr=base_lr)
    (rdir / f"{key}_summary.json").write_text(json.dumps(summary, indent=2, default=str))
    return summary


# ---------------------------------------------------------------------------
# results and gates
# ---------------------------------------------------------------------------
def result_is_finite(data: dict[str, Any]) -> bool:
    try:
        vals = [float(data["eval"]["bpb"]), float(data["train"]["final_loss"])]
    except (KeyError, TypeError, ValueError):
        return False
    return all(math.isfinite(v) for v in vals)


def loss_is_stable(loss: float, vocab: int = 16384) -> bool:
    return math.isfinite(loss) and loss < UNIFORM_LOSS.get(vocab, math.log(vocab)) - STALL_MARGIN


def collect(results_dir: Path, conditions: Sequence[str]) -> tuple[dict[str, dict], list[str]]:
    """Per condition: bpb / final loss / aggregate tok/s by seed.  Non-finite files are listed, not used."""
    rows: dict[str, dict] = {}
    invalid: list[str] = []
    for c in conditions:
        pat = re.compile(rf"^{re.escape(c)}_s(\d+)\.json$")
        row = {"bpb": {}, "loss": {}, "tps": {}, "world_size": 1, "vocab": 16384}
        for f in sorted(Path(results_dir).glob(f"{c}_s*.json")):
            m = pat.match(f.name)
            if not m:
                continue
            data = json.loads(f.read_text())
            if not result_is_finite(data):
                invalid.append(f.stem)
                continue
            s = int(m.group(1))
            row["bpb"][s] = float(data["eval"]["bpb"])
            row["loss"][s] = float(data["train"]["final_loss"])
            row["tps"][s] = float(data["train"].get("aggregate_tokens_per_sec", 0.0))
            row["world_size"] = int((data.get("config") or {}).get("world_size", 1))
            row["vocab"] = int((data.get("config") or {}).get("vocab_size", 16384))
        if row["bpb"]:
            rows[c] = row
    return rows, invalid


def _mean(v) -> float:
    v = list(v)
    return sum(v) / len(v) if v else float("nan")


def _paired(a: dict[int, float], b: dict[int, float]) -> dict[str, Any]:
    """``a - b`` over shared seeds with the paired t-test's p (nan below two pairs)."""
    shared = sorted(set(a) & set(b))
    if len(shared) < 2:
        return {"n": len(shared), "delta": _mean(a[s] - b[s] for s in shared) if shared else float("nan"),
                "p": float("nan")}
    t, p = paired_ttest([a[s] for s in shared], [b[s] for s in shared])
    return {"n": len(shared), "delta": _mean(a[s] - b[s] for s in shared), "t": t, "p": p}


def _gate_best_bpb(rows: dict, order: list[str], **_) -> dict:
    ranked = sorted(rows, key=lambda c: _mean(rows[c]["bpb"].values()))
    out = {"winner": ranked[0] if ranked else None}
    if len(ranked) > 1:
        out["winner_vs_runner_up"] = _paired(rows[ranked[1]]["bpb"], rows[ranked[0]]["bpb"])
    return out


def _gate_vs_first(rows: dict, order: list[str], require_significance: bool, **_) -> dict:
    base = order[0]
    if base not in rows:
        return {"winner": None, "reason": f"baseline {base} has no finite results"}
    cmp_ = {c: _paired(rows[base]["bpb"], rows[c]["bpb"]) for c in order[1:] if c in rows}
    best = min(rows, key=lambda c: _mean(rows[c]["bpb"].values()))
    if require_significance:
        passing = [c for c, r in cmp_.items() if r["delta"] > 0 and r["p"] < 0.05]
        best = min(passing, key=lambda c: _mean(rows[c]["bpb"].values())) if passing else base
    return {"winner": best, "vs_baseline": cmp_}


def _gate_ddp(rows: dict, order: list[str], **_) -> dict:
    base = order[0]
    if base not in rows:
        return {"winner": None, "reason": f"{base} missing"}
    b = rows[base]
    per_gpu_base = _mean(b["tps"].values()) / max(b["world_size"], 1)
    verdicts = {}
    for c in order[1:]:
        if c not in rows:
            continue
        r = rows[c]
        per_gpu = _mean(r["tps"].values()) / max(r["world_size"], 1)
        pr = _paired(b["bpb"], r["bpb"])
        keeps_rate = per_gpu_base > 0 and per_gpu / per_gpu_base >= DDP_PER_GPU_FLOOR
        learns = pr["delta"] > 0 and pr["p"] < 0.05
        verdicts[c] = {"per_gpu_rate_ratio": per_gpu / per_gpu_base if per_gpu_base > 0 else float("nan"),
                       "keeps_rate": bool(keeps_rate), "bpb": pr, "learns_more": bool(learns),
                       "passes": bool(keeps_rate and learns)}
    passing = [c for c, v in verdicts.items() if v["passes"]]
    return {"winner": passing[-1] if passing else base, "verdicts": verdicts}


def _gate_lr(rows: dict, order: list[str], cfgs: dict, baseline_bpb: Optional[dict[int, float]] = None, **_) -> dict:
    ranked = sorted(rows, key=lambda c: _mean(rows[c]["bpb"].values()))
    stable = [c for c in ranked if all(loss_is_stable(l, rows[c]["vocab"]) for l in rows[c]["loss"].values())]
    cand = None
    if len(stable) >= 2:
        top, second = stable[0], stable[1]
        pr = _paired(rows[second]["bpb"], rows[top]["bpb"])
        clear = pr["n"] < 2 or pr["delta"] > NOISE_GAP_BPB or pr["p"] < 0.05
        cand = top if clear else min((top, second), key=lambda c: cfgs[c]["base_lr"])   # inside noise: the calmer rate
    elif stable:
        cand = stable[0]
    out: dict[str, Any] = {"stage1_candidate": cand, "stable_conditions": stable, "winner_lr_condition": None,
                           "winner_is_provisional": False, "winner_vs_baseline": None}
    if cand is not None:
        if not baseline_bpb:
            out.update(winner_lr_condition=cand, winner_is_provisional=True)
        else:
            pr = _paired(baseline_bpb, rows[cand]["bpb"])
            out["winner_vs_baseline"] = pr
            if pr["n"] < 2:
                out.update(winner_lr_condition=cand, winner_is_provisional=True)
            elif pr["delta"] > 0 and pr["p"] < 0.05:
                out["winner_lr_condition"] = cand
    w = out["winner_lr_condition"]
    out["winner_base_lr"] = cfgs[w]["base_lr"] if w else None
    out["winner"] = w
    return out


def _gate_pairwise(rows: dict, order: list[str], **_) -> dict:
    pairs = {f"{a}_vs_{b}": _paired(rows[a]["bpb"], rows[b]["bpb"])
             for i, a in enumerate(order) for b in order[i + 1:] if a in rows and b in rows}
    base = order[0]
    better = [c for c in order[1:] if c in rows and base in rows
              and (lambda r: r["delta"] > 0 and r["p"] < 0.05)(_paired(rows[base]["bpb"], rows[c]["bpb"]))]
    win = min(better, key=lambda c: _mean(rows[c]["bpb"].values())) if better else (base if base in rows else None)
    return {"winner": win, "pairs": pairs}


def _gate_fp8(rows: dict, order: list[str], **_) -> dict:
    if "bf16" not in rows or "fp8" not in rows:
        return {"winner": "bf16" if "bf16" in rows else None, "reason": "one precision has no finite results"}
    stable = all(loss_is_stable(l, rows["fp8"]["vocab"]) for l in rows["fp8"]["loss"].values())
    speed = _mean(rows["fp8"]["tps"].values()) / max(_mean(rows["bf16"]["tps"].values()), 1e-9)
    pr = _paired(rows["fp8"]["bpb"], rows["bf16"]["bpb"])                    # positive: fp8 worse
    degraded = pr["n"] >= 2 and pr["delta"] > FP8_BPB_TOLERANCE and pr["p"] < 0.05
    ok = stable and speed >= FP8_SPEEDUP_FLOOR and not degraded
    return {"winner": "fp8" if ok else "bf16", "fp8_stable": bool(stable), "speedup": speed,
            "fp8_minus_bf16_bpb": pr, "fp8_degraded": bool(degraded)}


_GATES = {"best_bpb": _gate_best_bpb,
          "beats_first": lambda rows, order, **k: _gate_vs_first(rows, order, True),
          "best_bpb_vs_first": lambda rows, order, **k: _gate_vs_first(rows, order, False),
          "ddp_scaling": _gate_ddp, "lr_screen": _gate_lr, "pairwise": _gate_pairwise, "fp8_gate": _gate_fp8}


def decide(key: str, results_dir: Path, *, base_lr: Optional[float] = None,
           baseline_bpb_by_seed: Optional[dict[int, float]] = None) -> dict[str, Any]:
    """Per-condition means plus the test's gate.  ``baseline_bpb_by_seed`` is the single-GPU
    cohort the rate screens cross-check their candidate against (absent: provisional winner)."""
    test = TESTS[key]
    cfgs = test.conditions(base_lr if base_lr is not None else (1.0 if test.inherits_lr_from else None))
    order = list(cfgs)
    rows, invalid = collect(results_dir, order)
    summary: dict[str, Any] = {c: {"mean_bpb": _mean(r["bpb"].values()), "n_seeds": len(r["bpb"]),
                                   "mean_aggregate_tokens_per_sec": _mean(r["tps"].values()),
                                   "stable_seed_count": sum(loss_is_stable(l, r["vocab"]) for l in r["loss"].values())}
                               for c, r in rows.items()}
    dec = _GATES[test.gate](rows, order, cfgs=cfgs, baseline_bpb=baseline_bpb_by_seed) if rows else {"winner": None}
    dec["invalid_result_files"] = invalid
    summary["_decision"] = dec
    summary["_test"] = {"key": key, "question": test.question, "gate": test.gate}
    return summary


def main(argv: Optional[Sequence[str]] = None) -> int:
    import argparse
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("test", choices=sorted(TESTS))
    ap.add_argument("--results-root", type=Path, default=Path("results_exp18"))
    ap.add_argument("--data-path", default=None)
    ap.add_argument("--sp-model-path", default=None)
    ap.add_argument("--base-lr", type=float, default=None)
    ap.add_argument("--budget", type=float, default=None)
    ap.add_argument("--seeds", type=int, nargs="*", default=None)
    ap.add_argument("--summarize-only", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    if a.summarize_only:
        out = decide(a.test, a.results_root / f"results_{a.test}", base_lr=a.base_lr)
    else:
        if not a.data_path and not a.dry_run:
            ap.error("--data-path is required to launch")
        out = run_test(a.test, results_root=a.results_root, data_path=a.data_path or "", sp_model_path=a.sp_model_path,
                       base_lr=a.base_lr, seeds=a.seeds, budget_seconds=a.budget, dry_run=a.dry_run)
    print(json.dumps(out, indent=2, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
