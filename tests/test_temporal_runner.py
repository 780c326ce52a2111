"""Temporal-heads evaluation driver on a tiny CPU model and a synthetic validation cache."""
import json

import pytest
import torch

from chaoscontrol_b200.eval_stream import load_val_cache, write_synthetic_val_cache
from chaoscontrol_b200.eval_stream.temporal_runner import Exp22RunConfig, main, run
from chaoscontrol_b200.models.model import CareStudentLM


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    d = tmp_path_factory.mktemp("vc")
    write_synthetic_val_cache(d, n_docs=5, vocab=64, median_len=40, sigma=0.3, min_len=20, max_len=60, seed=4)
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2).eval(), d


def _run(setup, **kw):
    model, d = setup
    return run(Exp22RunConfig(chunk_size=16, max_docs=5, **kw), val_cache_dir=str(d), model=model,
               device=torch.device("cpu"))


def test_chunking_never_drops_a_target_and_matches_whole_document_scoring(setup):
    model, d = setup
    vc = load_val_cache(d)
    s = _run(setup, condition="score_only")
    assert s["docs_scored"] == 5 and s["tokens_scored"] == vc.total_tokens - vc.num_docs
    whole = 0.0
    for doc in vc.iter_docs():
        ids = torch.as_tensor(vc.tokens_for_doc(doc).astype("int64")).unsqueeze(0)
        logits = model(ids)["logits"][0, :-1].float()
        whole += float(torch.nn.functional.cross_entropy(logits, ids[0, 1:], reduction="sum").detach())
    assert s["aggregate_loss_nats"] == pytest.approx(whole, rel=1e-4)      # carried state == one long pass
    assert s["temporal_head_count"] == 1 and s["condition"] == "score_only"


def test_identical_heads_reproduce_score_only_and_shifts_change_it(setup, tmp_path):
    base = _run(setup, condition="score_only")
    same = _run(setup, condition="identical_heads_uniform", horizon_shifts=(0.0, 0.0, 0.0))
    assert same["aggregate_loss_nats"] == pytest.approx(base["aggregate_loss_nats"], rel=1e-5)
    assert same["head_ids"] == ["same_0", "same_1", "same_2"]
    single = _run(setup, condition="single_horizon", horizon_shifts=(0.0,))
    assert single["aggregate_loss_nats"] == pytest.approx(base["aggregate_loss_nats"], rel=1e-5)
    heads = _run(setup, condition="temporal_heads", horizon_shifts=(-1.0, 0.0, 1.0),
                 mixer="online_exp_weights_logprob", output_path=str(tmp_path / "docs.jsonl"),
                 analysis_path=str(tmp_path / "an.jsonl"), summary_path=str(tmp_path / "s" / "sum.json"))
    assert heads["tokens_scored"] == base["tokens_scored"] and heads["temporal_head_count"] == 3
    assert abs(heads["aggregate_loss_nats"] - base["aggregate_loss_nats"]) > 1e-6
    assert sum(heads["winner_counts_by_shift"].values()) == heads["tokens_scored"]
    rows = [json.loads(x) for x in (tmp_path / "docs.jsonl").read_text().splitlines()]
    assert len(rows) == 5 and set(rows[0]["per_head_loss_nats"]) == {"-1.0", "0.0", "1.0"}
    assert sum(r["tokens"] for r in rows) == heads["tokens_scored"]
    an = [json.loads(x) for x in (tmp_path / "an.jsonl").read_text().splitlines()]
    assert len(an) == 5 and "half_life_stats_by_shift" in an[0]
    assert json.loads((tmp_path / "s" / "sum.json").read_text())["aggregate_bpb"] == heads["aggregate_bpb"]


def test_condition_validation(setup):
    with pytest.raises(NotImplementedError):
        _run(setup, condition="gated_temporal_heads")
    with pytest.raises(ValueError, match="every horizon shift"):
        _run(setup, condition="identical_heads_uniform", horizon_shifts=(0.0, 0.5))
    with pytest.raises(ValueError, match="at least two"):
        _run(setup, condition="identical_heads_uniform", horizon_shifts=(0.0,))
    with pytest.raises(ValueError, match="exactly one"):
        _run(setup, condition="single_horizon", horizon_shifts=(0.0, 0.5))
    with pytest.raises(ValueError, match="unknown condition"):
        _run(setup, condition="nope")


def test_budget_expiry_stops_between_documents(setup):
    s = _run(setup, condition="score_only", budget_seconds=0.0)
    assert s["docs_scored"] == 0 and s["timed_out"]


def test_cli_from_checkpoint(setup, tmp_path, capsys):
    model, d = setup
    cfg = dict(vocab_size=64, model_dim=16, num_layers=2, ff_mult=2, dtype="fp32")
    torch.save({"model": model.state_dict(), "config": cfg}, tmp_path / "ck.pt")
    for cond in ("temporal_heads", "same_horizon_virtual_depth"):
        assert main(["--condition", cond, "--checkpoint-path", str(tmp_path / "ck.pt"), "--val-cache-dir", str(d),
                     "--chunk-size", "16", "--max-docs", "2", "--summary-path", str(tmp_path / f"{cond}.json")]) == 0
        out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
        assert out["condition"] == cond and out["docs_scored"] == 2
    assert json.loads((tmp_path / "same_horizon_virtual_depth.json").read_text())["depth_recurrence_count"] == 3
