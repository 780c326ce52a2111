"""Phase-1 lever ablation (experiment 19): the leave-one-out matrix, a per-lever
micro-benchmark, and the summariser with its gates.

Reference: experiments/19_phase1/build_matrix_phase1.py:108-194 (matrix),
bench_phase1a.py:150-660 (2^3 lever micro-benchmark with warm-up/restore, timed
blocks, idempotent JSONL), summarize_phase1.py:153-675 (coverage gate, quality
gate, coherent pairs, SHIP / PARK / INCONCLUSIVE).

The three levers of this build are the native counterparts of the reference's
``fused_grad_clip`` / ``fused_muon`` / ``compile_full_path``:

* ``fused_grad_clip``  -- flat-arena clip kernels instead of ``clip_grad_norm_``;
* ``fused_muon``       -- batched Newton-Schulz over the arena's shape groups instead
  of one matrix at a time;
* ``compile_full_path`` -- the key name is kept because result files and matrices are
  keyed by it; here it switches the hand-scheduled kernel engine on (no tracing
  compiler is involved; off = module-by-module autograd).

Matrix entries are consumed by ``runner_persistent_ddp`` (same key names).
"""
from __future__ import annotations

import argparse
import copy
import itertools
import json
import math
import statistics
import time
from pathlib import Path
from typing import Any, Iterable, Optional, Sequence

from .analysis import paired_ttest
from .runner_persistent_ddp import BENIGN_ERROR_PATTERNS, check_output_integrity, config_hash

LEVERS: tuple[str, ...] = ("fused_grad_clip", "fused_muon", "compile_full_path")
LEAVE_OUT_LABEL = {"fused_grad_clip": "no_fused_clip", "fused_muon": "no_fused_muon", "compile_full_path": "no_compile"}
SHIP_P, SHIP_LOSS_TOL, SHIP_VRAM_FRAC = 0.05, 0.02, 0.05

#: world size 4 anchor of the submission regime (rate = 2 x the world-size-2 winner)
DEFAULT_BASE_CONFIG: dict[str, Any] = {
    "model_type": "ssm", "world_size": 4, "vocab_size": 16384, "model_dim": 256, "num_layers": 4, "ff_mult": 2,
    "seq_len": 512, "stride": 256, "batch_size": 1024, "eval_batches": 16, "a_mode": "diag", "base_lr": 0.128,
    "weight_decay": 0.01, "grad_clip_norm": 1.0, "activation_checkpoint": True, "optimizer": "muon", "chunk_size": 64,
    "local_attn_window": 0, "local_attn_heads": 1, "local_attn_dim": 64, "device": "auto", "dtype": "bf16",
    "warmup_steps": 20}


# ---------------------------------------------------------------------------
# matrix
# ---------------------------------------------------------------------------
def lever_combos() -> list[tuple[str, dict[str, bool]]]:
    """``stock`` (all off), ``all`` (all on) and one leave-one-out row per lever."""
    rows = [("stock", {k: False for k in LEVERS}), ("all", {k: True for k in LEVERS})]
    rows += [(LEAVE_OUT_LABEL[k], {j: j != k for j in LEVERS}) for k in LEVERS]
    return rows


def build_matrix_phase1(seeds: Sequence[int] = (1337, 2674, 4011), *, include_fp8: bool = False,
                        base_config: Optional[dict[str, Any]] = None) -> list[dict[str, Any]]:
    base = copy.deepcopy(base_config or DEFAULT_BASE_CONFIG)
    out = []
    for precision in ("bf16",) + (("fp8_fused",) if include_fp8 else ()):
        for label, combo in lever_combos():
            for s in seeds:
                e = copy.deepcopy(base)
                e.update(combo)
                e.update(name=f"{precision}_{label}", precision=precision, seed=int(s))
                out.append(e)
    return out


# ---------------------------------------------------------------------------
# summariser
# ---------------------------------------------------------------------------
class CoverageError(RuntimeError):
    pass


class QualityError(RuntimeError):
    pass


class PairingError(RuntimeError):
    pass


def load_run_json(runs_dir: Path, entry: dict[str, Any]) -> Optional[dict[str, Any]]:
    p = Path(runs_dir) / f"{entry['name']}_s{int(entry['seed'])}.json"
    if not p.exists():
        return None
    try:
        return json.loads(p.read_text())
    except json.JSONDecodeError:
        return None


def full_coverage_gate(matrix: Sequence[dict], runs_dir: Path, *, lenient: bool = False) -> list[str]:
    missing = [f"{e['name']}_s{int(e['seed'])}" for e in matrix if load_run_json(runs_dir, e) is None]
    if missing and not lenient:
        raise CoverageError(f"{len(missing)} expected result file(s) missing: {missing[:8]}")
    return missing


def quality_gate(matrix: Sequence[dict], runs_dir: Path, *, lenient: bool = False) -> tuple[int, int, list[str]]:
    ok, benign, bad = check_output_integrity(Path(runs_dir), list(matrix), BENIGN_ERROR_PATTERNS)
    real = [b for b in bad if not (lenient and b.endswith("missing output file"))]
    if real:
        raise QualityError(f"{len(real)} run(s) failed: {real[:5]}; no verdicts from a contaminated matrix")
    return ok, benign, bad


def _is_all_on(e: dict) -> bool:
    return all(bool(e.get(k)) for k in LEVERS)


def _is_lever_off(e: dict, lever: str) -> bool:
    return not bool(e.get(lever)) and all(bool(e.get(k)) for k in LEVERS if k != lever)


def resolve_coherent_pairs(matrix: Sequence[dict]) -> dict[tuple[str, str], list[tuple[dict, dict]]]:
    """``(precision, lever) -> [(all-on entry, lever-off entry)]`` matched by seed.  Two entries
    of one (precision, combination, seed) make the pairing ambiguous: that is an error."""
    by_prec: dict[str, list[dict]] = {}
    for e in matrix:
        by_prec.setdefault(str(e.get("precision", "bf16")), []).append(e)
    out: dict[tuple[str, str], list[tuple[dict, dict]]] = {}
    for prec, ents in by_prec.items():
        on: dict[int, dict] = {}
        for e in ents:
            if _is_all_on(e):
                if int(e["seed"]) in on:
                    raise PairingError(f"two all-on entries for {prec} seed {e['seed']}")
                on[int(e["seed"])] = e
        for lever in LEVERS:
            off: dict[int, dict] = {}
            for e in ents:
                if _is_lever_off(e, lever):
                    if int(e["seed"]) in off:
                        raise PairingError(f"two {lever}-off entries for {prec} seed {e['seed']}")
                    off[int(e["seed"])] = e
            pairs = [(on[s], off[s]) for s in sorted(set(on) & set(off))]
            if pairs:
                out[(prec, lever)] = pairs
    return out


def tokens_per_step(cfg: dict[str, Any]) -> int:
    return int(cfg.get("batch_size", 0)) * int(cfg.get("seq_len", 0)) * int(cfg.get("world_size", 1))


def extract_metrics(result: dict[str, Any]) -> dict[str, float]:
    tr, ev = result.get("train") or {}, result.get("eval") or {}
    tps = tr.get("aggregate_tokens_per_sec")
    if tps is None and tr.get("steps") and tr.get("elapsed_s"):
        tps = float(tr["steps"]) * tokens_per_step(result.get("config") or {}) / float(tr["elapsed_s"])
    f = lambda v: float(v) if v is not None else float("nan")      # noqa: E731
    return {"tokens_per_sec": f(tps), "final_loss": f(tr.get("final_loss")), "bpb": f(ev.get("bpb")),
            "peak_vram_mb": f(tr.get("peak_vram_mb"))}


def _mean(v: Iterable[float]) -> float:
    v = [x for x in v if math.isfinite(x)]
    return sum(v) / len(v) if v else float("nan")


def compute_lever_verdict(on: Sequence[dict[str, float]], off: Sequence[dict[str, float]]) -> dict[str, Any]:
    """Paired ``all-on minus lever-off`` deltas and the verdict ladder: throughput must rise,
    then loss and memory must hold, then the rise must be significant."""
    assert len(on) == len(off)
    n = len(on)
    d = {k: [a[k] - b[k] for a, b in zip(on, off)] for k in ("tokens_per_sec", "final_loss", "bpb", "peak_vram_mb")}
    m_tps, m_loss, m_vram = _mean(d["tokens_per_sec"]), _mean(d["final_loss"]), _mean(d["peak_vram_mb"])
    p = paired_ttest([a["tokens_per_sec"] for a in on], [b["tokens_per_sec"] for b in off])[1] if n >= 2 else float("nan")
    base_vram = _mean(b["peak_vram_mb"] for b in off)
    vram_frac = m_vram / base_vram if math.isfinite(base_vram) and base_vram > 0 else float("nan")
    mean_on = _mean(a["tokens_per_sec"] for a in on)
    if not math.isfinite(m_tps) or m_tps <= 0:
        verdict, reason = "PARK", "mean delta tok/s <= 0"
    elif math.isfinite(m_loss) and abs(m_loss) > SHIP_LOSS_TOL:
        verdict, reason = "PARK", f"|delta final_loss| {abs(m_loss):.4f} > {SHIP_LOSS_TOL}"
    elif math.isfinite(vram_frac) and abs(vram_frac) > SHIP_VRAM_FRAC:
        verdict, reason = "PARK", f"|delta peak_vram| / baseline {abs(vram_frac):.3f} > {SHIP_VRAM_FRAC}"
    elif math.isnan(p) or p >= SHIP_P:
        verdict, reason = "INCONCLUSIVE", f"positive but p = {p:.3f}: more seeds"
    else:
        verdict, reason = "SHIP", f"delta tok/s {m_tps:.0f} (p = {p:.3f}), quality gates hold"
    return {"n": n, "mean_delta_tokens_per_sec": m_tps,
            "marginal_tokens_per_sec_frac": m_tps / mean_on if mean_on and math.isfinite(mean_on) else float("nan"),
            "mean_delta_final_loss": m_loss, "mean_delta_bpb": _mean(d["bpb"]), "mean_delta_peak_vram_mb": m_vram,
            "delta_peak_vram_frac": vram_frac, "paired_t_p_value": p, "verdict": verdict, "reason": reason}


def render_markdown(verdicts: dict[tuple[str, str], dict], *, missing: Sequence[str] = (), counts=None) -> str:
    lines = ["# Phase 1 lever ablation", ""]
    if counts:
        lines += [f"runs: {counts[0]} ok, {counts[1]} benign skips, {len(missing)} missing", ""]
    lines += ["| precision | lever | n | delta tok/s | marginal | p | delta loss | delta VRAM | verdict |",
              "|---|---|---|---|---|---|---|---|---|"]
    for (prec, lever), v in sorted(verdicts.items()):
        lines.append(f"| {prec} | {lever} | {v['n']} | {v['mean_delta_tokens_per_sec']:+.0f} | "
                     f"{v['marginal_tokens_per_sec_frac']:+.3%} | {v['paired_t_p_value']:.3g} | "
                     f"{v['mean_delta_final_loss']:+.4f} | {v['delta_peak_vram_frac']:+.2%} | **{v['verdict']}** |")
    if missing:
        lines += ["", "missing: " + ", ".join(missing)]
    return "\n".join(lines) + "\n"


def summarize(matrix: Sequence[dict], runs_dir: Path, *, lenient: bool = False) -> dict[str, Any]:
    counts = quality_gate(matrix, runs_dir, lenient=lenient)
    missing = full_coverage_gate(matrix, runs_dir, lenient=lenient)
    verdicts: dict[tuple[str, str], dict] = {}
    for key, pairs in resolve_coherent_pairs(matrix).items():
        on, off = [], []
        for a, b in pairs:
            ra, rb = load_run_json(runs_dir, a), load_run_json(runs_dir, b)
            if ra is None or rb is None or "error" in ra or "error" in rb:
                continue
            on.append(extract_metrics(ra))
            off.append(extract_metrics(rb))
        if on:
            verdicts[key] = compute_lever_verdict(on, off)
    return {"verdicts": verdicts, "missing": missing, "counts": counts,
            "markdown": render_markdown(verdicts, missing=missing, counts=counts)}


# ---------------------------------------------------------------------------
# micro-benchmark: every combination of the levers, timed in blocks
# ---------------------------------------------------------------------------
def all_lever_combos() -> list[dict[str, bool]]:
    return [dict(zip(LEVERS, bits)) for bits in itertools.product((False, True), repeat=len(LEVERS))]


def combo_name(combo: dict[str, bool]) -> str:
    return "+".join(k for k in LEVERS if combo[k]) or "stock"


def split_steps(n_timed: int, n_blocks: int) -> list[int]:
    n_blocks = max(1, min(n_blocks, n_timed))
    q, r = divmod(n_timed, n_blocks)
    return [q + (1 if i < r else 0) for i in range(n_blocks)]


def run_one_measurement(combo: dict[str, bool], seed: int, *, model_cfg: Optional[dict[str, Any]] = None,
                        warmup_steps: int = 5, n_timed_steps: int = 20, n_blocks: int = 4,
                        device: Optional[str] = None) -> dict[str, Any]:
    """Warm-up on a snapshot that is restored afterwards (so warm-up never moves the optimizer
    state the timed steps start from), then ``n_timed_steps`` in ``n_blocks`` separately timed blocks."""
    import torch
    from .models.model import CareStudentLM
    from .optim.muon import Muon
    from .train_ssm import train_ssm_step
    cfg = dict(vocab_size=16384, dim=256, num_layers=4, ff_mult=2, batch_size=1024, seq_len=512, base_lr=0.064)
    cfg.update(model_cfg or {})
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    torch.manual_seed(seed)
    model = CareStudentLM(vocab_size=cfg["vocab_size"], dim=cfg["dim"], num_layers=cfg["num_layers"],
                          ff_mult=cfg["ff_mult"]).to(dev)
    if dev.type == "cuda":
        model = model.to(torch.bfloat16)
    if combo["compile_full_path"] and dev.type == "cuda":
        from .utils.arena import ParamArena
        ParamArena.install(model)
    opt = Muon(list(model.parameters()), lr=cfg["base_lr"], fused=bool(combo["fused_muon"]))
    opt.bind_param_names(list(model.named_parameters()))
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, cfg["vocab_size"], (cfg["batch_size"], cfg["seq_len"] + 1), generator=g).to(dev)

    from .parallel.distributed import clip_arena_grad_norm, clip_grad_norm_fused
    from .utils.arena import get_arena
    engine_on = bool(combo["compile_full_path"]) and dev.type == "cuda"
    params = [p for p in model.parameters()]

    def step() -> float:
        loss = train_ssm_step(model, tok[:, :-1], tok[:, 1:], 64, precision="bf16" if dev.type == "cuda" else "fp32",
                              lm_head_backward_mode="fused_streaming_cached" if engine_on else "chunked")
        arena = get_arena(model) if engine_on else None
        if arena is not None and combo["fused_grad_clip"]:
            clip_arena_grad_norm(arena, 1.0)
        elif combo["fused_grad_clip"]:
            clip_grad_norm_fused(params, 1.0)
        else:
            if arena is not None:
                arena.materialize_grads()
            torch.nn.utils.clip_grad_norm_(params, 1.0)
            if arena is not None:
                arena.pull_grads()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return float(loss)

    snap_m = {k: v.detach().clone() for k, v in model.state_dict().items()}
    snap_o = copy.deepcopy(opt.state_dict())
    for _ in range(warmup_steps):
        step()
    model.load_state_dict(snap_m)
    opt.load_state_dict(snap_o)
    sync = torch.cuda.synchronize if dev.type == "cuda" else (lambda: None)
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats()
    rates, loss = [], float("nan")
    for n in split_steps(n_timed_steps, n_blocks):
        sync()
        t0 = time.perf_counter()
        for _ in range(n):
            loss = step()
        sync()
        rates.append(n * cfg["batch_size"] * cfg["seq_len"] / (time.perf_counter() - t0))
    return {"combo": combo_name(combo), **{k: bool(v) for k, v in combo.items()}, "seed": int(seed),
            "tokens_per_sec": statistics.fmean(rates), "tokens_per_sec_std": statistics.pstdev(rates),
            "block_tokens_per_sec": rates, "final_loss": loss,
            "peak_vram_mb": torch.cuda.max_memory_allocated() / 2 ** 20 if dev.type == "cuda" else 0.0,
            "n_timed_steps": n_timed_steps, "warmup_steps": warmup_steps}


def read_existing_hashes(results_path: Path) -> set[str]:
    if not Path(results_path).exists():
        return set()
    out = set()
    for line in Path(results_path).read_text().splitlines():
        try:
            out.add(json.loads(line)["config_hash"])
        except (json.JSONDecodeError, KeyError):
            continue
    return out


def run_bench(output_dir: Path, *, seeds: Sequence[int] = (1337, 2674), combos: Optional[Sequence[dict]] = None,
              measure=run_one_measurement, **kw) -> Path:
    """Every (combination, seed) once; rows already in ``results.jsonl`` (same config hash) are skipped."""
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=True)
    res = output_dir / "results.jsonl"
    done = read_existing_hashes(res)
    for combo in (combos or all_lever_combos()):
        for s in seeds:
            h = config_hash({"combo": combo, "seed": int(s), **{k: v for k, v in kw.items() if k != "device"}})
            if h in done:
                continue
            row = measure(combo, int(s), **kw)
            row["config_hash"] = h
            with res.open("a") as f:
                f.write(json.dumps(row) + "\n")
            done.add(h)
    write_summary(res, output_dir / "summary.md")
    return res


def paired_deltas(rows: Sequence[dict], lever: str, metric: str) -> dict[str, Any]:
    """Lever on minus off, paired on (the other levers' setting, seed): 4 pairs per seed."""
    others = [k for k in LEVERS if k != lever]
    key = lambda r: (tuple(bool(r[k]) for k in others), int(r["seed"]))      # noqa: E731
    on = {key(r): float(r[metric]) for r in rows if r[lever]}
    off = {key(r): float(r[metric]) for r in rows if not r[lever]}
    shared = sorted(set(on) & set(off))
    d = [on[k] - off[k] for k in shared]
    p = paired_ttest([on[k] for k in shared], [off[k] for k in shared])[1] if len(shared) >= 2 else float("nan")
    return {"n": len(shared), "mean": _mean(d), "std": statistics.pstdev(d) if len(d) > 1 else 0.0, "p": p,
            "baseline": _mean(off[k] for k in shared)}


def write_summary(results_path: Path, summary_path: Path) -> str:
    rows = [json.loads(l) for l in Path(results_path).read_text().splitlines() if l.strip()]
    lines = ["# Lever micro-benchmark", "", "| lever | metric | n pairs | mean delta | relative | p |", "|---|---|---|---|---|---|"]
    for lever in LEVERS:
        for metric in ("tokens_per_sec", "peak_vram_mb", "final_loss"):
            d = paired_deltas(rows, lever, metric)
            rel = d["mean"] / d["baseline"] if d["baseline"] and math.isfinite(d["baseline"]) and d["baseline"] != 0 else float("nan")
            lines.append(f"| {lever} | {metric} | {d['n']} | {d['mean']:+.4g} | {rel:+.2%} | {d['p']:.3g} |")
    text = "\n".join(lines) + "\n"
    Path(summary_path).write_text(text)
    return text


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    m = sub.add_parser("matrix")
    m.add_argument("--output", type=Path, required=True)
    m.add_argument("--seeds", type=int, nargs="+", default=[1337, 2674, 4011])
    m.add_argument("--include-fp8", action="store_true")
    m.add_argument("--base-config", type=Path, default=None)
    s = sub.add_parser("summarize")
    s.add_argument("--matrix-json", type=Path, required=True)
    s.add_argument("--runs-dir", type=Path, required=True)
    s.add_argument("--output", type=Path, default=None)
    s.add_argument("--lenient", action="store_true")
    b = sub.add_parser("bench")
    b.add_argument("--output-dir", type=Path, required=True)
    b.add_argument("--seeds", type=int, nargs="+", default=[1337, 2674])
    b.add_argument("--warmup-steps", type=int, default=5)
    b.add_argument("--n-timed-steps", type=int, default=20)
    b.add_argument("--n-blocks", type=int, default=4)
    a = ap.parse_args(argv)
    if a.cmd == "matrix":
        base = json.loads(a.base_config.read_text()) if a.base_config else None
        a.output.write_text(json.dumps(build_matrix_phase1(a.seeds, include_fp8=a.include_fp8, base_config=base), indent=2))
        return 0
    if a.cmd == "bench":
        run_bench(a.output_dir, seeds=a.seeds, warmup_steps=a.warmup_steps, n_timed_steps=a.n_timed_steps,
                  n_blocks=a.n_blocks)
        return 0
    try:
        matrix = json.loads(a.matrix_json.read_text())
    except (OSError, json.JSONDecodeError) as exc:
        print(f"matrix unreadable: {exc}")
        return 4
    try:
        out = summarize(matrix, a.runs_dir, lenient=a.lenient)
    except QualityError as exc:
        print(exc)
        return 1
    except CoverageError as exc:
        print(exc)
        return 2
    except PairingError as exc:
        print(exc)
        return 3
    if a.output:
        a.output.write_text(out["markdown"])
    else:
        print(out["markdown"])
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
