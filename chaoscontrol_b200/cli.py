"""Data-preparation and measurement commands that sit beside the runners:

``build-dataset``     JSONL text -> BPE tokenizer (trained on documents after the validation split, seeded,
                      byte fallback) -> shards -> ``build_manifest.json``      (scripts/build_sp_shards.py)
``build-shards``      JSONL text + SentencePiece model -> ``fineweb_{train,val}_NNNNNN.bin`` (flat little-endian
                      uint16, no header, no EOS appended, every shard ends on a document boundary)
``build-val-cache``   JSONL text -> ``tokens.npy`` / ``docs.npy`` / ``manifest.json``  (scripts/build_exp20_val_cache.py)
``verify-val-cache``  a validation shard against a cache built from the same text     (scripts/verify_sp16384_eval_cache.py)
``eval-quant``        bits-per-byte of a checkpoint before and after the int6 GPTQ + LZMA round trip
                                                                       (scripts/eval_quant.py)

``python -m chaoscontrol_b200.cli <command> --help``
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import time
from pathlib import Path
from typing import Optional, Sequence

import numpy as np
import torch

__all__ = ["main", "build_shards", "verify_val_cache", "eval_quant"]

ARTIFACT_LIMIT_BYTES = 16 * 1024 * 1024


# ---------------------------------------------------------------------------
# tokenizer + shards
# ---------------------------------------------------------------------------
SHARD_INDEX_WIDTH = 6            # fineweb_{train,val}_{NNNNNN}.bin
MAX_VOCAB_FOR_SHARDS = 32768     # the loaders map the uint16 files as int16: same bits below 2^15


def _jsonl_texts(paths: Sequence[Path]):
    for path in paths:
        with open(path, "r", encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                try:
                    text = json.loads(line).get("text", "")
                except json.JSONDecodeError:
                    continue
                if text:
                    yield text


def train_tokenizer(*, jsonl_paths: Sequence[Path], vocab_size: int, tokenizer_dir: Path, val_docs: int = 50_000,
                    sp_train_docs: int = 5_000_000, sp_seed: int = 1337, num_threads: int = 4,
                    force: bool = False) -> Path:
    """Trains the BPE tokenizer of the shard pipeline (scripts/build_sp_shards.py:140-218 of the reference) and
    returns ``<tokenizer_dir>/fineweb_<vocab>_bpe.model``.  The training text is the first ``sp_train_docs``
    documents AFTER the validation split, so the tokenizer never sees validation text; byte fallback keeps every
    string round-trippable; unk / bos / eos are ids 0 / 1 / 2 and there is no pad; the whole corpus is used in file
    order with input shuffling off, which leaves BPE training nothing random: the same input gives the same
    model (``sp_seed`` is recorded in the build manifest; this trainer has no seed field to hand it to).  An existing model is kept unless ``force``.  The
    model and its vocabulary file appear together (trained under a partial name, then renamed)."""
    import sentencepiece as spm
    if not 0 < int(vocab_size) <= MAX_VOCAB_FOR_SHARDS:
        raise ValueError(f"vocab_size must be in (0, {MAX_VOCAB_FOR_SHARDS}], got {vocab_size}")
    tokenizer_dir = Path(tokenizer_dir)
    tokenizer_dir.mkdir(parents=True, exist_ok=True)
    final = tokenizer_dir / f"fineweb_{int(vocab_size)}_bpe.model"
    if final.exists() and not force:
        return final
    corpus = tokenizer_dir / f".sp_train_{int(vocab_size)}.txt"
    n = 0
    with corpus.open("w", encoding="utf-8") as out:
        for i, text in enumerate(_jsonl_texts(jsonl_paths)):
            if i < int(val_docs):
                continue
            if n >= int(sp_train_docs):
                break
            out.write(text.replace("\n", " ") + "\n")
            n += 1
    if n == 0:
        corpus.unlink(missing_ok=True)
        raise ValueError("no training documents after the validation split: lower val_docs or supply more text")
    partial = tokenizer_dir / f".partial_fineweb_{int(vocab_size)}_bpe"
    for suf in (".model", ".vocab"):
        Path(str(partial) + suf).unlink(missing_ok=True)
    try:
        spm.SentencePieceTrainer.Train(
            input=str(corpus), model_prefix=str(partial), vocab_size=int(vocab_size), model_type="bpe",
            character_coverage=0.9995, byte_fallback=True, unk_id=0, bos_id=1, eos_id=2, pad_id=-1,
            num_threads=int(num_threads), input_sentence_size=0, shuffle_input_sentence=False, minloglevel=2)
    finally:
        corpus.unlink(missing_ok=True)
    os.replace(str(partial) + ".model", final)
    try:
        os.replace(str(partial) + ".vocab", final.with_suffix(".vocab"))
    except OSError:
        final.unlink(missing_ok=True)           # the pair stays consistent
        raise
    return final


def build_dataset(*, jsonl_paths: Sequence[Path], vocab_size: int, output_dir: Path, tokenizer_dir: Path,
                  val_docs: int = 50_000, sp_train_docs: int = 5_000_000, shard_size: int = 100_000_000,
                  sp_seed: int = 1337, num_threads: int = 4, skip_train: bool = False, skip_tokenize: bool = False,
                  force: bool = False, dry_run: bool = False) -> dict:
    """Tokenizer, then shards, then ``build_manifest.json`` describing both (the reference's one-command
    pipeline).  A finished build whose manifest matches the request is left alone unless ``force``."""
    output_dir, tokenizer_dir = Path(output_dir), Path(tokenizer_dir)
    request = {"vocab_size": int(vocab_size), "val_docs": int(val_docs), "sp_train_docs": int(sp_train_docs),
               "shard_size": int(shard_size), "sp_seed": int(sp_seed), "docs": [str(Path(p)) for p in jsonl_paths]}
    model_path = tokenizer_dir / f"fineweb_{int(vocab_size)}_bpe.model"
    plan = {"request": request, "tokenizer_model": str(model_path), "output_dir": str(output_dir),
            "train_tokenizer": not skip_train and (force or not model_path.exists()), "tokenize": not skip_tokenize}
    if dry_run:
        return {"dry_run": True, **plan}
    mpath = output_dir / "build_manifest.json"
    if mpath.exists() and not force:
        old = json.loads(mpath.read_text())
        if old.get("request") == request:
            return old
        raise ValueError(f"{mpath} describes another build ({old.get('request')}); use force=True or another "
                         "output directory")
    if not skip_train:
        train_tokenizer(jsonl_paths=jsonl_paths, vocab_size=vocab_size, tokenizer_dir=tokenizer_dir, val_docs=val_docs,
                        sp_train_docs=sp_train_docs, sp_seed=sp_seed, num_threads=num_threads, force=force)
    if not model_path.exists():
        raise FileNotFoundError(f"{model_path} not found: train the tokenizer first (skip_train was set)")
    out = dict(plan)
    if not skip_tokenize:
        if force and output_dir.exists():
            for f in output_dir.glob("fineweb_*_*.bin"):
                f.unlink()
        out["shards"] = build_shards(jsonl_paths=jsonl_paths, sp_model_path=model_path, out_dir=output_dir,
                                     val_docs=val_docs, shard_tokens=shard_size)
        out["tokenizer_sha256"] = hashlib.sha256(model_path.read_bytes()).hexdigest()
        output_dir.mkdir(parents=True, exist_ok=True)
        mpath.write_text(json.dumps(out, indent=2))
    return out


def build_shards(*, jsonl_paths: Sequence[Path], sp_model_path: Path, out_dir: Path, val_docs: int = 50_000,
                 shard_tokens: int = 100_000_000, max_docs: Optional[int] = None) -> dict:
    """The first ``val_docs`` documents become validation shards, the rest
    training shards; tokens are uint16 and a vocabulary above 65 536 is refused."""
    import sentencepiece as spm
    sp = spm.SentencePieceProcessor(model_file=str(sp_model_path))
    if sp.vocab_size() > MAX_VOCAB_FOR_SHARDS:
        raise ValueError(f"vocabulary {sp.vocab_size()} does not fit the shard format: readers view the uint16 "
                         f"shards as int16, so token ids must stay below {MAX_VOCAB_FOR_SHARDS}")
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    state = {"train": {"buf": [], "n": 0, "idx": 0, "tokens": 0, "docs": 0},
             "val": {"buf": [], "n": 0, "idx": 0, "tokens": 0, "docs": 0}}

    def flush(split: str) -> None:
        s = state[split]
        if not s["buf"]:
            return
        arr = np.concatenate(s["buf"]).astype("<u2")
        arr.tofile(out_dir / f"fineweb_{split}_{s['idx']:0{SHARD_INDEX_WIDTH}d}.bin")
        s["buf"], s["n"], s["idx"] = [], 0, s["idx"] + 1

    seen = 0
    for path in jsonl_paths:
        with open(path, "r", encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                try:
                    text = json.loads(line).get("text", "")
                except json.JSONDecodeError:
                    continue
                if not text:
                    continue
                if max_docs is not None and seen >= max_docs:
                    break
                split = "val" if seen < val_docs else "train"
                seen += 1
                ids = np.asarray(sp.encode(text, out_type=int), dtype=np.uint16)
                s = state[split]
                s["buf"].append(ids)
                s["n"] += ids.size
                s["tokens"] += int(ids.size)
                s["docs"] += 1
                if s["n"] >= shard_tokens:
                    flush(split)
    flush("train")
    flush("val")
    manifest = {"vocab_size": int(sp.vocab_size()), "append_eos": False, "dtype": "uint16-le", "header_bytes": 0,
                **{f"{k}_{f}": state[k][f] for k in state for f in ("tokens", "docs")},
                "train_shards": state["train"]["idx"], "val_shards": state["val"]["idx"]}
    (out_dir / "shards_manifest.json").write_text(json.dumps(manifest, indent=2))
    return manifest


# ---------------------------------------------------------------------------
# validation cache
# ---------------------------------------------------------------------------
def verify_val_cache(*, val_shard: Path, val_cache_dir: Path, expected_tokens: Optional[int] = None,
                     chunk_tokens: int = 1 << 22) -> dict:
    """Token-for-token comparison of a flat validation shard with a cache's
    ``tokens.npy``, streamed in chunks; reports the first mismatch."""
    from .eval_stream.io import load_val_cache
    cache = load_val_cache(Path(val_cache_dir))
    shard = np.memmap(val_shard, dtype="<u2", mode="r")
    toks = np.asarray(cache.tokens)
    n = min(shard.size, toks.size)
    first = None
    for s in range(0, n, int(chunk_tokens)):
        a, b = shard[s: s + chunk_tokens], toks[s: s + chunk_tokens]
        neq = np.nonzero(a[: b.size] != b[: a.size])[0]
        if neq.size:
            i = s + int(neq[0])
            first = {"index": i, "shard": int(shard[i]), "cache": int(toks[i])}
            break
    doc_sum = int(np.asarray(cache.docs["token_len"]).sum())
    out = {"shard_tokens": int(shard.size), "cache_tokens": int(toks.size), "doc_token_sum": doc_sum,
           "docs": int(len(cache.docs)), "first_mismatch": first,
           "ok": first is None and shard.size == toks.size == doc_sum and
           (expected_tokens is None or int(expected_tokens) == int(toks.size))}
    if expected_tokens is not None:
        out["expected_tokens"] = int(expected_tokens)
    return out


# ---------------------------------------------------------------------------
# quantisation round trip
# ---------------------------------------------------------------------------
def _score(model, cache, *, chunk_size: int, max_docs: Optional[int], device: torch.device) -> dict:
    from .scoring import score_val_cache
    model.eval()
    with torch.no_grad():
        return score_val_cache(model, cache, chunk_size=chunk_size, max_docs=max_docs, device=device)


def eval_quant(*, ckpt: Path, val_cache_dir: Optional[Path] = None, output_json: Path, device: str = "auto",
               chunk_size: int = 512, max_docs: Optional[int] = None, calibration_seqs: int = 16,
               calibration_seq_len: int = 128, seed: int = 0, eval_jsonl: Optional[Path] = None,
               sp_model_path: Optional[Path] = None) -> dict:
    """Score the validation cache with the checkpoint as trained, quantise
    (self-generated calibration text -> Hessians -> GPTQ int6 -> LZMA), write the
    blob beside the JSON, load it back into a fresh model, score the same
    documents again, and report both bits-per-byte figures and the artifact size
    against the 16 MiB limit."""
    from .eval_stream.io import load_val_cache
    from .quantization.gptq import GPTQQuantizer, ar_self_generated_calibration
    from .quantization.packaging import pack_int6_lzma, unpack_int6_lzma
    from .runner_exp21 import build_model
    torch.manual_seed(seed)
    dev = torch.device("cuda" if (device == "auto" and torch.cuda.is_available()) else
                       ("cpu" if device == "auto" else device))
    blob = torch.load(ckpt, map_location="cpu", weights_only=False)
    cfg = dict(blob["config"])
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = build_model(cfg, dev, dtype)
    model.load_state_dict(blob["model"], strict=True)
    if val_cache_dir is None:
        # the reference's input pair: raw validation text and the tokenizer; tokenised once into a cache
        # beside the output
        if eval_jsonl is None or sp_model_path is None:
            raise ValueError("eval_quant needs val_cache_dir, or eval_jsonl together with sp_model_path")
        from .eval_stream.io import write_val_cache
        val_cache_dir = Path(output_json).with_suffix(".valcache")
        write_val_cache(jsonl_paths=[Path(eval_jsonl)], sp_model_path=Path(sp_model_path), cache_dir=val_cache_dir,
                        max_docs=max_docs if max_docs is not None else 50_000)
    cache = load_val_cache(Path(val_cache_dir))
    t0 = time.perf_counter()
    before = _score(model, cache, chunk_size=chunk_size, max_docs=max_docs, device=dev)
    seqs = ar_self_generated_calibration(model, num_seqs=calibration_seqs, seq_len=calibration_seq_len,
                                         vocab_size=int(cfg["vocab_size"]), seed=seed, device=dev)
    q = GPTQQuantizer()
    q.calibrate(model, seqs, device=dev)
    quantized, meta = q.quantize_state_dict({k: v for k, v in model.state_dict().items() if torch.is_tensor(v)})
    packed = pack_int6_lzma(quantized, meta)
    output_json = Path(output_json)
    output_json.parent.mkdir(parents=True, exist_ok=True)
    blob_path = output_json.with_suffix(output_json.suffix + ".int6.ptz.lzma")
    blob_path.write_bytes(packed)
    del model
    result, meta2 = unpack_int6_lzma(packed)
    restored = build_model(cfg, dev, dtype)
    sd = GPTQQuantizer.dequantize_state_dict(result, meta2)
    missing = restored.load_state_dict({k: v.to(dtype) if v.is_floating_point() else v for k, v in sd.items()},
                                       strict=False)
    after = _score(restored, cache, chunk_size=chunk_size, max_docs=max_docs, device=dev)
    out = {"ckpt": str(ckpt), "bpb_bf16": before["bpb"], "bpb_int6": after["bpb"],
           "delta_bpb": after["bpb"] - before["bpb"], "artifact_bytes": len(packed),
           "artifact_margin_mb": (ARTIFACT_LIMIT_BYTES - len(packed)) / 2 ** 20,
           "docs_scored": before["docs_scored"], "tokens_scored": before["tokens_scored"],
           "int6_tensors": sum(1 for m in meta.values() if m["type"] == "int6"),
           "missing_keys": list(missing.missing_keys), "unexpected_keys": list(missing.unexpected_keys),
           "blob_path": str(blob_path), "elapsed_s": time.perf_counter() - t0,
           "pass_bf16": before, "pass_int6": after}
    output_json.write_text(json.dumps(out, indent=2, default=str))
    return out


# ---------------------------------------------------------------------------
# artifact headroom of a wider trunk
# ---------------------------------------------------------------------------
MEASURED_DIM256_COMPRESSED_BYTES = 7_375_816     # int6 + LZMA size of a trained 4 x 256, V 16384 trunk
ARTIFACT_LIMIT_BYTES = 16_000_000
DEFAULT_OVERHEAD_BYTES = 500_000


def artifact_headroom(*, dim: int = 384, vocab_size: int = 16_384, num_layers: int = 4, ff_mult: int = 2,
                      overhead_bytes: int = DEFAULT_OVERHEAD_BYTES, measure: bool = False) -> dict:
    """Will a ``dim``-wide bare-SSM trunk fit the 16 000 000-byte artifact?  The estimate scales the measured
    compressed size of the 256-wide trunk by the ratio of raw bf16 sizes
    (experiments/24_crct/validate_dim384_artifact.py:58-100).  ``measure`` additionally quantises a freshly
    initialised model of that shape to int6 and LZMA-packs it -- an upper bound in practice, since random
    weights compress worse than trained ones."""
    from .models.model import CareStudentLM

    def build(d: int):
        return CareStudentLM(vocab_size=vocab_size, dim=d, num_layers=num_layers, ff_mult=ff_mult, a_mode="diag",
                             rich_b_mode="none", outer_model_dim=0)
    model = build(dim)
    raw, base_raw = int(model.artifact_bytes()), int(build(256).artifact_bytes())
    compressed = int(round(raw * MEASURED_DIM256_COMPRESSED_BYTES / float(base_raw)))
    total = compressed + int(overhead_bytes)
    out = {"dim": int(dim), "vocab_size": int(vocab_size), "num_layers": int(num_layers), "raw_bf16_bytes": raw,
           "baseline_dim256_raw_bf16_bytes": base_raw, "estimated_compressed_model_bytes": compressed,
           "overhead_bytes": int(overhead_bytes), "estimated_total_bytes": total,
           "margin_bytes": ARTIFACT_LIMIT_BYTES - total, "controller_params": 0,
           "under_budget": total < ARTIFACT_LIMIT_BYTES}
    if measure:
        from .artifact import _collect_state, _pack
        state = _collect_state(model, None, {"dim": dim}, None, None, None)
        blob, _ = _pack(state, "int6", 6, None)
        out["measured_random_init_int6_bytes"] = len(blob)
    return out


# ---------------------------------------------------------------------------
def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="chaoscontrol_b200.cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("build-shards")
    s.add_argument("--jsonl-path", type=Path, nargs="+", required=True)
    s.add_argument("--sp-model-path", type=Path, required=True)
    s.add_argument("--out-dir", type=Path, required=True)
    s.add_argument("--val-docs", type=int, default=50_000)
    s.add_argument("--shard-tokens", type=int, default=100_000_000)
    s.add_argument("--max-docs", type=int, default=None)
    c = sub.add_parser("build-val-cache")
    c.add_argument("--jsonl-path", type=Path, nargs="+", required=True)
    c.add_argument("--sp-model-path", type=Path, required=True)
    c.add_argument("--cache-dir", type=Path, required=True)
    c.add_argument("--max-docs", type=int, default=50_000)
    c.add_argument("--force", action="store_true")
    v = sub.add_parser("verify-val-cache")
    v.add_argument("--val-shard", type=Path, required=True)
    v.add_argument("--val-cache-dir", type=Path, required=True)
    v.add_argument("--expected-tokens", type=int, default=None)
    v.add_argument("--chunk-tokens", type=int, default=1 << 22)
    e = sub.add_parser("eval-quant")
    e.add_argument("--ckpt", type=Path, required=True)
    e.add_argument("--val-cache-dir", type=Path, default=None)
    e.add_argument("--eval-jsonl", type=Path, default=None, help="raw validation text (with --sp-model-path) instead of a cache")
    e.add_argument("--sp-model-path", type=Path, default=None)
    e.add_argument("--budget-seconds", type=float, default=600.0, help="accepted for command-line compatibility")
    e.add_argument("--output-json", type=Path, required=True)
    e.add_argument("--device", default="auto")
    e.add_argument("--chunk-size", type=int, default=512)
    e.add_argument("--max-docs", type=int, default=None)
    e.add_argument("--calibration-seqs", type=int, default=16)
    e.add_argument("--calibration-seq-len", type=int, default=128)
    e.add_argument("--seed", type=int, default=0)
    d = sub.add_parser("build-dataset", help="train the BPE tokenizer, then write the uint16 shards")
    d.add_argument("--docs-path", "--jsonl-path", dest="docs_path", type=Path, nargs="+", required=True)
    d.add_argument("--vocab-size", type=int, required=True)
    d.add_argument("--output-dir", type=Path, required=True)
    d.add_argument("--tokenizer-dir", type=Path, required=True)
    d.add_argument("--sp-train-docs", type=int, default=5_000_000)
    d.add_argument("--val-docs", type=int, default=50_000)
    d.add_argument("--shard-size", type=int, default=100_000_000)
    d.add_argument("--sp-seed", type=int, default=1337)
    d.add_argument("--num-workers", type=int, default=max(1, (os.cpu_count() or 2) // 2))
    d.add_argument("--dry-run", action="store_true")
    d.add_argument("--skip-tokenize", action="store_true")
    d.add_argument("--skip-train", action="store_true")
    d.add_argument("--force", action="store_true")
    h = sub.add_parser("artifact-headroom")
    h.add_argument("--dim", type=int, default=384)
    h.add_argument("--vocab-size", type=int, default=16_384)
    h.add_argument("--num-layers", type=int, default=4)
    h.add_argument("--ff-mult", type=int, default=2)
    h.add_argument("--overhead-bytes", type=int, default=DEFAULT_OVERHEAD_BYTES)
    h.add_argument("--measure", action="store_true")
    h.add_argument("--output", type=Path, default=None)
    a = ap.parse_args(argv)
    if a.cmd == "artifact-headroom":
        out = artifact_headroom(dim=a.dim, vocab_size=a.vocab_size, num_layers=a.num_layers, ff_mult=a.ff_mult,
                                overhead_bytes=a.overhead_bytes, measure=a.measure)
        text = json.dumps(out, indent=2, sort_keys=True)
        if a.output is not None:
            a.output.write_text(text + "\n")
        else:
            print(text)
        return 0 if out["under_budget"] else 2
    if a.cmd == "build-dataset":
        out = build_dataset(jsonl_paths=a.docs_path, vocab_size=a.vocab_size, output_dir=a.output_dir,
                            tokenizer_dir=a.tokenizer_dir, val_docs=a.val_docs, sp_train_docs=a.sp_train_docs,
                            shard_size=a.shard_size, sp_seed=a.sp_seed, num_threads=a.num_workers,
                            skip_train=a.skip_train, skip_tokenize=a.skip_tokenize, force=a.force, dry_run=a.dry_run)
        print(json.dumps(out, indent=2, default=str))
        return 0
    if a.cmd == "build-shards":
        out = build_shards(jsonl_paths=a.jsonl_path, sp_model_path=a.sp_model_path, out_dir=a.out_dir,
                           val_docs=a.val_docs, shard_tokens=a.shard_tokens, max_docs=a.max_docs)
    elif a.cmd == "build-val-cache":
        from .eval_stream.io import write_val_cache
        out = write_val_cache(jsonl_paths=a.jsonl_path, sp_model_path=a.sp_model_path, cache_dir=a.cache_dir,
                              max_docs=a.max_docs, force=a.force)
    elif a.cmd == "verify-val-cache":
        out = verify_val_cache(val_shard=a.val_shard, val_cache_dir=a.val_cache_dir,
                               expected_tokens=a.expected_tokens, chunk_tokens=a.chunk_tokens)
        print(json.dumps(out, indent=2))
        return 0 if out["ok"] else 1
    else:
        out = eval_quant(ckpt=a.ckpt, val_cache_dir=a.val_cache_dir, output_json=a.output_json, device=a.device,
                         chunk_size=a.chunk_size, max_docs=a.max_docs, calibration_seqs=a.calibration_seqs,
                         calibration_seq_len=a.calibration_seq_len, seed=a.seed, eval_jsonl=a.eval_jsonl,
                         sp_model_path=a.sp_model_path)
        out = {k: v for k, v in out.items() if not k.startswith("pass_")}
    print(json.dumps(out, indent=2, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
