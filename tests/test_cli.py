"""Package command line: shard building, validation-cache verification, quantisation round trip."""
import json

import numpy as np
import pytest
import torch

from chaoscontrol_b200 import cli
from chaoscontrol_b200.eval_stream.io import write_synthetic_val_cache


def test_verify_val_cache_finds_the_first_mismatch(tmp_path):
    write_synthetic_val_cache(tmp_path / "cache", n_docs=20, vocab=64, median_len=40, min_len=8, max_len=80)
    toks = np.load(tmp_path / "cache" / "tokens.npy")
    shard = tmp_path / "fineweb_val_000000.bin"
    toks.astype("<u2").tofile(shard)
    ok = cli.verify_val_cache(val_shard=shard, val_cache_dir=tmp_path / "cache", expected_tokens=int(toks.size),
                              chunk_tokens=100)
    assert ok["ok"] and ok["first_mismatch"] is None and ok["docs"] == 20
    bad = toks.copy()
    bad[137] ^= 1
    bad.astype("<u2").tofile(shard)
    out = cli.verify_val_cache(val_shard=shard, val_cache_dir=tmp_path / "cache", chunk_tokens=100)
    assert not out["ok"] and out["first_mismatch"]["index"] == 137
    assert cli.main(["verify-val-cache", "--val-shard", str(shard), "--val-cache-dir", str(tmp_path / "cache")]) == 1


def test_eval_quant_round_trip(tmp_path):
    from chaoscontrol_b200.runner_exp21 import build_model
    cfg = dict(vocab_size=64, model_dim=32, num_layers=2, ff_mult=2, seq_len=32)
    torch.manual_seed(0)
    model = build_model(cfg, torch.device("cpu"), torch.float32)
    torch.save({"model": model.state_dict(), "config": cfg}, tmp_path / "m.pt")
    write_synthetic_val_cache(tmp_path / "cache", n_docs=12, vocab=64, median_len=40, min_len=8, max_len=80)
    out = cli.eval_quant(ckpt=tmp_path / "m.pt", val_cache_dir=tmp_path / "cache", output_json=tmp_path / "q.json",
                         device="cpu", chunk_size=16, calibration_seqs=2, calibration_seq_len=16)
    assert out["docs_scored"] == 12 and np.isfinite(out["bpb_bf16"]) and np.isfinite(out["bpb_int6"])
    assert abs(out["delta_bpb"]) < 0.2 and 0 < out["artifact_bytes"] < cli.ARTIFACT_LIMIT_BYTES
    assert not out["missing_keys"] and (tmp_path / "q.json.int6.ptz.lzma").stat().st_size == out["artifact_bytes"]
    assert json.loads((tmp_path / "q.json").read_text())["ckpt"].endswith("m.pt")


def test_build_shards_with_a_stub_tokenizer(tmp_path, monkeypatch):
    import sys
    import types

    class _SP:
        def __init__(self, model_file=None):
            pass

        def vocab_size(self):
            return 300

        def encode(self, text, out_type=int):
            return [ord(c) % 300 for c in text]

    monkeypatch.setitem(sys.modules, "sentencepiece", types.SimpleNamespace(SentencePieceProcessor=_SP))
    src = tmp_path / "docs.jsonl"
    src.write_text("\n".join(json.dumps({"text": "doc %d " % i * (i + 1)}) for i in range(10)) + "\n\nnot json\n")
    m = cli.build_shards(jsonl_paths=[src], sp_model_path=tmp_path / "sp.model", out_dir=tmp_path / "out", val_docs=3,
                         shard_tokens=40)
    assert m["val_docs"] == 3 and m["train_docs"] == 7 and m["append_eos"] is False
    val = np.concatenate([np.fromfile(p, dtype="<u2") for p in sorted((tmp_path / "out").glob("fineweb_val_*.bin"))])
    assert val.size == m["val_tokens"] and m["train_shards"] >= 2
    assert val[:6].tolist() == [ord(c) for c in "doc 0 "]
    from chaoscontrol_b200.data import load_fineweb_tokens
    tr, va = load_fineweb_tokens(str(tmp_path / "out"))
    assert tr.numel() == m["train_tokens"] and va.numel() == m["val_tokens"]
