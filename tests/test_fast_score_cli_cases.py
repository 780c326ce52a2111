"""Score-only driver: the reference scorer's command-line flags and the checkpoint payload checks (CPU)."""
import json

import pytest
import torch

from chaoscontrol_b200 import fast_score as FS
from chaoscontrol_b200.episodic.cache import EpisodicCache
from chaoscontrol_b200.eval_stream.io import write_synthetic_val_cache
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.runner_exp21 import save_output_ckpt


@pytest.fixture()
def setup(tmp_path):
    torch.manual_seed(0)
    write_synthetic_val_cache(tmp_path / "val", n_docs=10, vocab=48, median_len=40.0, sigma=0.6, min_len=8, max_len=100, seed=3)
    model = CareStudentLM(vocab_size=48, dim=16, num_layers=2)
    save_output_ckpt(str(tmp_path / "m.pt"), model, dict(vocab_size=48, model_dim=16, num_layers=2))
    return tmp_path


def _args(root, *extra):
    return ["--cache-dir", str(root / "val"), "--checkpoint-path", str(root / "m.pt"), "--chunk-size", "16", "--device", "cpu",
            *extra]


def test_summary_and_per_document_outputs(setup):
    out, summ = setup / "o" / "docs.jsonl", setup / "o" / "summary.json"
    assert FS.main(_args(setup, "--output-path", str(out), "--summary-path", str(summ), "--doc-batch-size", "4")) == 0
    s = json.loads(summ.read_text())
    rows = [json.loads(x) for x in out.read_text().splitlines()]
    assert len(rows) == s["docs_scored"] == 10 and sorted(r["doc_id"] for r in rows) == list(range(10))
    assert sum(r["tokens_scored"] for r in rows) == s["tokens_scored"]
    assert sum(r["ce_nats"] for r in rows) == pytest.approx(s["total_ce_nats"], rel=1e-9)
    assert sum(r["raw_bytes"] for r in rows) == s["total_raw_bytes"]


def test_output_path_alone_still_receives_the_summary(setup):
    out = setup / "only.json"
    assert FS.main(_args(setup, "--output-path", str(out))) == 0
    assert json.loads(out.read_text())["docs_scored"] == 10


def test_reference_flags_are_accepted_and_the_inert_ones_change_nothing(setup):
    a, b = setup / "a.json", setup / "b.json"
    FS.main(_args(setup, "--summary-path", str(a)))
    FS.main(_args(setup, "--summary-path", str(b), "--persistence-mode", "reset", "--torch-compile-mode", "max-autotune",
                  "--score-graph-mode", "none", "--score-through-packet-lane", "--no-episodic-cache-enabled",
                  "--episodic-cache-capacity", "128", "--episodic-span-length", "4", "--episodic-key-rep-dim", "-1",
                  "--episodic-grace-steps", "10", "--episodic-fingerprint-window", "8", "--episodic-cache-reset-per-doc",
                  "--score-boundary-targets", "--score-warmup-steps", "2", "--safety-margin-seconds", "1.5",
                  "--max-batch-tokens", "256"))
    sa, sb = json.loads(a.read_text()), json.loads(b.read_text())
    assert sa["total_ce_nats"] == pytest.approx(sb["total_ce_nats"], rel=1e-6) and sa["tokens_scored"] == sb["tokens_scored"]
    assert sb["score_warmup_steps"] == 2 and sb["safety_margin_seconds"] == 1.5 and sb["max_forward_tokens"] == 256
    with pytest.raises(SystemExit):
        FS.main(_args(setup, "--no-score-boundary-targets"))
    with pytest.raises(SystemExit):
        FS.main(_args(setup, "--persistence-mode", "carry_state"))


def test_sort_flag_selects_the_packing(setup):
    s1 = FS.run(cache_dir=str(setup / "val"), checkpoint_path=str(setup / "m.pt"), output_path=None, chunk_size=16,
                device=torch.device("cpu"), sort_docs_by_length=False)
    s2 = FS.run(cache_dir=str(setup / "val"), checkpoint_path=str(setup / "m.pt"), output_path=None, chunk_size=16,
                device=torch.device("cpu"), sort_docs_by_length=True)
    assert s1["doc_packing"] == "source_order" and s2["doc_packing"] != "source_order"
    assert s1["total_ce_nats"] == pytest.approx(s2["total_ce_nats"], rel=1e-6)


def test_episodic_cache_source_is_checked_against_the_checkpoint(setup):
    kw = dict(cache_dir=str(setup / "val"), output_path=None, chunk_size=16, device=torch.device("cpu"))
    plain = str(setup / "m.pt")
    assert FS.run(checkpoint_path=plain, **kw)["episodic_cache"] == {"source": "auto", "state": "fresh", "consulted": False}
    with pytest.raises(ValueError, match="requires ckpt"):
        FS.run(checkpoint_path=plain, episodic_cache_source="checkpoint", **kw)
    with pytest.raises(ValueError, match="auto, fresh or checkpoint"):
        FS.run(checkpoint_path=plain, episodic_cache_source="warm", **kw)
    blob = torch.load(plain, weights_only=False)
    blob["episodic_cache"] = EpisodicCache(capacity=4, span_length=2, key_rep_dim=4).to_dict()
    warm = str(setup / "warm.pt")
    torch.save(blob, warm)
    assert FS.run(checkpoint_path=warm, **kw)["episodic_cache"]["state"] == "loaded"
    assert FS.run(checkpoint_path=warm, episodic_cache_source="checkpoint", **kw)["episodic_cache"]["state"] == "loaded"
    cold = FS.run(checkpoint_path=warm, episodic_cache_source="fresh", **kw)
    assert cold["episodic_cache"]["state"] == "fresh_forced"
    assert cold["total_ce_nats"] == FS.run(checkpoint_path=warm, **kw)["total_ce_nats"]     # the cache is never consulted


def test_online_maintenance_state_needs_an_explicit_yes(setup):
    blob = torch.load(str(setup / "m.pt"), weights_only=False)
    blob["online_eval_state"] = {"replay_eviction": {"version": 1}}
    path = str(setup / "online.pt")
    torch.save(blob, path)
    kw = dict(cache_dir=str(setup / "val"), checkpoint_path=path, output_path=None, chunk_size=16, device=torch.device("cpu"))
    with pytest.raises(ValueError, match="allow_online_replay_checkpoint"):
        FS.run(**kw)
    assert FS.run(allow_online_replay_checkpoint=True, **kw)["docs_scored"] == 10
    assert FS.main(["--cache-dir", str(setup / "val"), "--checkpoint-path", path, "--chunk-size", "16", "--device", "cpu",
                    "--allow-online-replay-checkpoint"]) == 0
