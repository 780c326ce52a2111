"""Seeded versus empty episodic store under ``packet_online_cache``
(src/chaoscontrol/eval/packet_online_cache_compare.py:72-160): the same checkpoint is scored once with
the store it was trained with and once with the store cleared first; ``delta_bpb = empty - seeded`` is
what the trained-in memory is worth."""
from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Any, Optional

import torch

from .registry import evaluate_with_calc_types

__all__ = ["run_packet_online_cache_compare", "load_and_run_packet_online_cache_compare"]


def run_packet_online_cache_compare(*, model: torch.nn.Module, val_cache, device: torch.device,
                                    compare_config: Optional[dict[str, Any]] = None,
                                    output_json: Optional[str | Path] = None) -> dict[str, Any]:
    """The empty pass runs on a copy taken BEFORE the seeded pass writes to the store, so the two
    passes are independent."""
    cfg = dict(compare_config or {})
    twin = copy.deepcopy(model)

    def one(m, seeded: bool) -> dict[str, Any]:
        return evaluate_with_calc_types(model=m, val_cache=val_cache, device=device,
                                        calc_types=["packet_online_cache"],
                                        calc_type_configs={"packet_online_cache": {**cfg, "seeded": seeded}}
                                        )["packet_online_cache"]
    seeded, empty = one(model, True), one(twin, False)
    out = {"compare_type": "packet_online_cache", "artifact_path": getattr(model, "_compare_artifact_path", None),
           "val_cache_dir": str(getattr(val_cache, "cache_dir", "")), "compare_config": cfg, "seeded": seeded,
           "empty": empty, "delta_bpb": float(empty["bpb"]) - float(seeded["bpb"]),
           "delta_loss": float(empty["loss"]) - float(seeded["loss"])}
    if output_json is not None:
        path = Path(output_json)
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(path.suffix + ".tmp")
        tmp.write_text(json.dumps(out, indent=2, sort_keys=True, default=str))
        tmp.rename(path)
    return out


def load_and_run_packet_online_cache_compare(*, artifact_path: str | Path, val_cache_dir: str | Path,
                                             device: str | torch.device = "cpu",
                                             compare_config: Optional[dict[str, Any]] = None,
                                             output_json: Optional[str | Path] = None) -> dict[str, Any]:
    from ..artifact import load_artifact
    from ..eval_stream.io import load_val_cache
    dev = torch.device(device) if isinstance(device, str) else device
    model, _tok, _cfg = load_artifact(artifact_path, str(dev))
    model._compare_artifact_path = str(artifact_path)
    return run_packet_online_cache_compare(model=model, val_cache=load_val_cache(Path(val_cache_dir)), device=dev,
                                           compare_config=compare_config, output_json=output_json)


def main(argv: Optional[list[str]] = None) -> int:
    """``python -m chaoscontrol_b200.eval.packet_online_cache_compare --artifact-path A --val-cache-dir D
    --output-json O`` (scripts/run_packet_online_cache_compare.py:22-47)."""
    import argparse
    ap = argparse.ArgumentParser(description="Score one artifact with its trained-in episodic store and with the "
                                             "store emptied first, and keep the summary.")
    ap.add_argument("--artifact-path", required=True, type=Path)
    ap.add_argument("--val-cache-dir", required=True, type=Path)
    ap.add_argument("--output-json", required=True, type=Path)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--chunk-tokens", type=int, default=256)
    ap.add_argument("--write-tokens-per-chunk", type=int, default=16)
    ap.add_argument("--gate-value", type=float, default=1.0)
    ap.add_argument("--decay", type=float, default=1.0)
    a = ap.parse_args(argv)
    res = load_and_run_packet_online_cache_compare(
        artifact_path=a.artifact_path, val_cache_dir=a.val_cache_dir, device=a.device,
        compare_config={"chunk_tokens": a.chunk_tokens, "write_tokens_per_chunk": a.write_tokens_per_chunk,
                        "gate_value": a.gate_value, "decay": a.decay}, output_json=a.output_json)
    print(json.dumps(res, indent=2, sort_keys=True, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
