"""The tokenising data paths with a real (tiny) SentencePiece model: document stream, validation cache,
shard builder, shard / cache verification (CPU)."""
import json

import numpy as np
import pytest

spm = pytest.importorskip("sentencepiece")

from chaoscontrol_b200 import cli  # noqa: E402
from chaoscontrol_b200.eval_stream import io as IO  # noqa: E402

WORDS = ("alpha beta gamma delta epsilon zeta eta theta iota kappa lambda mu nu xi omicron pi rho sigma tau "
         "upsilon phi chi psi omega").split()


@pytest.fixture(scope="module")
def corpus(tmp_path_factory):
    root = tmp_path_factory.mktemp("sp")
    rng = np.random.default_rng(0)
    docs = [" ".join(rng.choice(WORDS, size=int(rng.integers(5, 40)))) for _ in range(60)]
    (root / "train.txt").write_text("\n".join(docs))
    spm.SentencePieceTrainer.train(input=str(root / "train.txt"), model_prefix=str(root / "tok"), vocab_size=80,
                                   model_type="bpe", character_coverage=1.0, minloglevel=2)
    a, b = root / "a.jsonl", root / "b.jsonl"
    a.write_text("\n".join([json.dumps({"text": d}) for d in docs[:30]] + ["", "{broken json", json.dumps({"text": ""}),
                                                                          json.dumps({"other": 1})]) + "\n")
    b.write_text("\n".join(json.dumps({"text": d}) for d in docs[30:]) + "\n")
    return {"root": root, "model": root / "tok.model", "jsonl": [a, b], "docs": docs}


def test_doc_stream_skips_bad_lines_numbers_documents_and_counts_bytes(corpus):
    sp = spm.SentencePieceProcessor(model_file=str(corpus["model"]))
    recs = list(IO.DocStreamer(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"]))
    assert len(recs) == 60 and [r.doc_id for r in recs] == list(range(60))
    for r, text in zip(recs, corpus["docs"]):
        assert r.tokens == sp.encode(text, out_type=int) and r.raw_bytes == len(text.encode())


def test_doc_stream_stops_at_max_docs_and_restarts_numbering(corpus):
    s = IO.DocStreamer(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], max_docs=31)
    first, again = list(s), list(s)
    assert len(first) == 31 and first[-1].doc_id == 30 and [r.doc_id for r in again] == list(range(31))


def test_val_cache_layout_and_manifest(corpus, tmp_path):
    man = IO.write_val_cache(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], cache_dir=tmp_path / "vc", max_docs=50)
    cache = IO.load_val_cache(tmp_path / "vc")
    assert cache.num_docs == man["num_docs"] == 50 and cache.tokens.dtype == np.uint16
    assert cache.total_tokens == man["total_tokens"] == cache.tokens.size and cache.total_raw_bytes == man["total_raw_bytes"]
    starts = cache.docs["token_start"]
    assert starts[0] == 0 and np.array_equal(starts[1:], np.cumsum(cache.docs["token_len"])[:-1])
    sp = spm.SentencePieceProcessor(model_file=str(corpus["model"]))
    d7 = list(cache.iter_docs())[7]
    assert cache.tokens_for_doc(d7).tolist() == sp.encode(corpus["docs"][7], out_type=int)
    assert len(man["sp_model_sha256"]) == 64 and man["cache_version"] == IO.CACHE_VERSION and len(man["content_sha256"]) == 64


def test_val_cache_is_reused_until_the_request_changes(corpus, tmp_path, monkeypatch):
    kw = dict(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], cache_dir=tmp_path / "vc")
    first = IO.write_val_cache(max_docs=20, **kw)
    calls = []
    real = IO.DocStreamer.__iter__
    monkeypatch.setattr(IO.DocStreamer, "__iter__", lambda self: (calls.append(1), real(self))[1])
    assert IO.write_val_cache(max_docs=20, **kw) == first and calls == []           # reused
    IO.write_val_cache(max_docs=20, force=True, **kw)
    assert calls == [1]                                                             # forced rebuild
    other = IO.write_val_cache(max_docs=25, **kw)
    assert other["num_docs"] == 25 and len(calls) == 2                              # another request


def test_load_refuses_a_manifest_that_disagrees_with_the_documents(corpus, tmp_path):
    IO.write_val_cache(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], cache_dir=tmp_path / "vc", max_docs=10)
    m = json.loads((tmp_path / "vc" / "manifest.json").read_text())
    m["num_docs"] = 11
    (tmp_path / "vc" / "manifest.json").write_text(json.dumps(m))
    with pytest.raises(ValueError, match="does not match"):
        IO.load_val_cache(tmp_path / "vc")


def test_shards_split_validation_first_and_roll_over_by_size(corpus, tmp_path):
    man = cli.build_shards(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], out_dir=tmp_path / "sh",
                           val_docs=10, shard_tokens=300)
    assert man["val_docs"] == 10 and man["train_docs"] == 50 and man["vocab_size"] == 80 and man["append_eos"] is False
    assert man["dtype"] == "uint16-le" and man["header_bytes"] == 0 and man["train_shards"] >= 2
    files = sorted(p.name for p in (tmp_path / "sh").glob("*.bin"))
    assert files[0] == "fineweb_train_000000.bin" and "fineweb_val_000000.bin" in files
    train = np.concatenate([np.fromfile(p, dtype="<u2") for p in sorted((tmp_path / "sh").glob("fineweb_train_*.bin"))])
    val = np.concatenate([np.fromfile(p, dtype="<u2") for p in sorted((tmp_path / "sh").glob("fineweb_val_*.bin"))])
    sp = spm.SentencePieceProcessor(model_file=str(corpus["model"]))
    want_val = np.concatenate([sp.encode(t, out_type=int) for t in corpus["docs"][:10]])
    want_train = np.concatenate([sp.encode(t, out_type=int) for t in corpus["docs"][10:]])
    assert np.array_equal(val, want_val) and np.array_equal(train, want_train)      # no header, no separators
    assert man["train_tokens"] == train.size and man["val_tokens"] == val.size
    assert json.loads((tmp_path / "sh" / "shards_manifest.json").read_text()) == man


def test_shards_respect_max_docs(corpus, tmp_path):
    man = cli.build_shards(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], out_dir=tmp_path / "sh",
                           val_docs=5, max_docs=12)
    assert man["val_docs"] == 5 and man["train_docs"] == 7


def test_validation_shard_and_cache_agree_token_for_token(corpus, tmp_path):
    cli.build_shards(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], out_dir=tmp_path / "sh", val_docs=60)
    IO.write_val_cache(jsonl_paths=corpus["jsonl"], sp_model_path=corpus["model"], cache_dir=tmp_path / "vc", max_docs=60)
    shard = tmp_path / "sh" / "fineweb_val_000000.bin"
    ok = cli.verify_val_cache(val_shard=shard, val_cache_dir=tmp_path / "vc", chunk_tokens=97)
    assert ok["ok"] and ok["first_mismatch"] is None and ok["docs"] == 60 and ok["shard_tokens"] == ok["cache_tokens"] == ok["doc_token_sum"]
    assert not cli.verify_val_cache(val_shard=shard, val_cache_dir=tmp_path / "vc", expected_tokens=ok["cache_tokens"] + 1)["ok"]
    arr = np.fromfile(shard, dtype="<u2")
    arr[123] ^= 1
    arr.tofile(shard)
    bad = cli.verify_val_cache(val_shard=shard, val_cache_dir=tmp_path / "vc", chunk_tokens=50)
    assert not bad["ok"] and bad["first_mismatch"]["index"] == 123
    assert cli.main(["verify-val-cache", "--val-shard", str(shard), "--val-cache-dir", str(tmp_path / "vc")]) == 1


def test_cli_builds_shards_and_cache(corpus, tmp_path, capsys):
    args = ["--jsonl-path", *map(str, corpus["jsonl"]), "--sp-model-path", str(corpus["model"])]
    assert cli.main(["build-shards", *args, "--out-dir", str(tmp_path / "sh"), "--val-docs", "8"]) == 0
    assert json.loads(capsys.readouterr().out)["val_docs"] == 8
    assert cli.main(["build-val-cache", *args, "--cache-dir", str(tmp_path / "vc"), "--max-docs", "9"]) == 0
    assert json.loads(capsys.readouterr().out)["num_docs"] == 9


def test_tokenizer_training_is_seeded_skips_validation_text_and_keeps_the_pair_together(corpus, tmp_path):
    kw = dict(jsonl_paths=corpus["jsonl"], vocab_size=300, val_docs=10, sp_train_docs=40, num_threads=1)
    a = cli.train_tokenizer(tokenizer_dir=tmp_path / "t1", **kw)
    b = cli.train_tokenizer(tokenizer_dir=tmp_path / "t2", **kw)
    # the model file records its own input path, so compare what matters: the learned pieces and their scores
    assert a.name == "fineweb_300_bpe.model" and a.with_suffix(".vocab").read_text() == b.with_suffix(".vocab").read_text()
    assert not list((tmp_path / "t1").glob(".partial*")) and not list((tmp_path / "t1").glob(".sp_train*"))
    sp = spm.SentencePieceProcessor(model_file=str(a))
    assert (sp.unk_id(), sp.bos_id(), sp.eos_id(), sp.pad_id()) == (0, 1, 2, -1) and sp.vocab_size() == 300
    assert sp.decode(sp.encode("alpha \u2603 beta")) == "alpha \u2603 beta"          # byte fallback round-trips a rare character
    stamp = a.stat().st_mtime_ns
    assert cli.train_tokenizer(tokenizer_dir=tmp_path / "t1", **kw) == a and a.stat().st_mtime_ns == stamp   # kept
    with pytest.raises(ValueError, match="no training documents"):
        cli.train_tokenizer(tokenizer_dir=tmp_path / "t3", **{**kw, "val_docs": 1000})
    with pytest.raises(ValueError, match="vocab_size"):
        cli.train_tokenizer(tokenizer_dir=tmp_path / "t3", **{**kw, "vocab_size": 40000})


def test_one_command_dataset_build_is_idempotent_and_guards_its_folder(corpus, tmp_path, capsys):
    args = ["build-dataset", "--docs-path", *map(str, corpus["jsonl"]), "--vocab-size", "300", "--output-dir",
            str(tmp_path / "ds"), "--tokenizer-dir", str(tmp_path / "tok"), "--val-docs", "10", "--sp-train-docs", "40",
            "--shard-size", "400", "--num-workers", "1"]
    assert cli.main(args + ["--dry-run"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["dry_run"] and plan["train_tokenizer"] and plan["tokenize"] and not (tmp_path / "ds").exists()
    assert cli.main(args) == 0
    man = json.loads(capsys.readouterr().out)
    assert man["shards"]["val_docs"] == 10 and man["shards"]["train_docs"] == 50 and man["shards"]["vocab_size"] == 300
    assert len(man["tokenizer_sha256"]) == 64 and (tmp_path / "ds" / "build_manifest.json").exists()
    files = {p.name: p.stat().st_mtime_ns for p in (tmp_path / "ds").glob("*.bin")}
    assert cli.main(args) == 0                                            # same request: nothing is rewritten
    capsys.readouterr()
    assert files == {p.name: p.stat().st_mtime_ns for p in (tmp_path / "ds").glob("*.bin")}
    other = [x if x != "300" else "280" for x in args]
    with pytest.raises(ValueError, match="another build"):
        cli.main(other)
    with pytest.raises(FileNotFoundError):
        cli.build_dataset(jsonl_paths=corpus["jsonl"], vocab_size=290, output_dir=tmp_path / "ds2", tokenizer_dir=tmp_path / "tok",
                          skip_train=True)


def test_eval_quant_takes_raw_text_and_a_tokenizer(corpus, tmp_path):
    import torch

    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.runner_exp21 import save_output_ckpt
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=80, dim=16, num_layers=1)
    save_output_ckpt(str(tmp_path / "m.pt"), model, dict(vocab_size=80, model_dim=16, num_layers=1))
    rc = cli.main(["eval-quant", "--ckpt", str(tmp_path / "m.pt"), "--eval-jsonl", str(corpus["jsonl"][0]), "--sp-model-path",
                   str(corpus["model"]), "--output-json", str(tmp_path / "q.json"), "--device", "cpu", "--chunk-size", "16",
                   "--max-docs", "6", "--calibration-seqs", "2", "--calibration-seq-len", "16", "--budget-seconds", "5"])
    out = json.loads((tmp_path / "q.json").read_text())
    assert rc == 0 and out["docs_scored"] == 6 and out["bpb_bf16"] > 0 and out["artifact_bytes"] > 0
    assert (tmp_path / "q.valcache" / "manifest.json").exists()
    with pytest.raises(ValueError, match="val_cache_dir, or eval_jsonl"):
        cli.eval_quant(ckpt=tmp_path / "m.pt", output_json=tmp_path / "q2.json", device="cpu")
