"""Test-time-training evaluation driver on a tiny CPU model."""
import json

import pytest
import torch

from chaoscontrol_b200.eval_stream import write_synthetic_val_cache
from chaoscontrol_b200.eval_stream.run_eval import iter_docs, main, run
from chaoscontrol_b200.eval_stream.types import RunConfig
from chaoscontrol_b200.models.model import CareStudentLM


@pytest.fixture(scope="module")
def cache(tmp_path_factory):
    d = tmp_path_factory.mktemp("vc")
    write_synthetic_val_cache(d, n_docs=6, vocab=64, median_len=40, sigma=0.3, min_len=20, max_len=60, seed=4)
    return d


def _model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2)


def test_docs_from_cache_and_argument_check(cache):
    docs = list(iter_docs(val_cache_dir=str(cache), max_docs=4))
    assert len(docs) == 4 and all(len(d.tokens) >= 20 and d.raw_bytes > 0 for d in docs)
    with pytest.raises(ValueError):
        list(iter_docs())


def test_score_only_then_adaptation_changes_the_score_and_restores_weights(cache, tmp_path):
    model = _model()
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    base = run(RunConfig(adapt_set="none", chunk_size=16, max_docs=6), val_cache_dir=str(cache), model=model,
               device=torch.device("cpu"))
    ttt = run(RunConfig(adapt_set="lm_head", chunk_size=16, max_docs=6, eval_lr=0.5, steps_per_chunk=1,
                        output_path=str(tmp_path / "o" / "docs.jsonl"), summary_path=str(tmp_path / "s.json")),
              val_cache_dir=str(cache), model=model, device=torch.device("cpu"))
    assert base["docs_scored"] == ttt["docs_scored"] == 6 and base["tokens_scored"] == ttt["tokens_scored"]
    assert base["driver"] == ttt["driver"] == "eager" and base["adapt_steps"] == 0 and ttt["adapt_steps"] > 0
    assert ttt["bpb"] != base["bpb"]
    for n, p in model.named_parameters():                       # reset persistence: nothing leaks out
        assert torch.equal(p, before[n]), n
    rows = [json.loads(x) for x in (tmp_path / "o" / "docs.jsonl").read_text().splitlines()]
    assert len(rows) == 6
    assert json.loads((tmp_path / "s.json").read_text())["config"]["adapt_set"] == "lm_head"
    with pytest.raises(ValueError, match="graph runner"):
        run(RunConfig(adapt_set="lm_head", chunk_size=16), val_cache_dir=str(cache), model=model,
            device=torch.device("cpu"), use_graph=True)
    with pytest.raises(ValueError, match="calc_types"):
        run(RunConfig(episodic_cache_enabled=True), val_cache_dir=str(cache), model=model,
            device=torch.device("cpu"))


def test_cli_from_checkpoint(cache, tmp_path, capsys):
    model = _model()
    torch.save({"model": model.state_dict(),
                "config": dict(vocab_size=64, model_dim=16, num_layers=2, ff_mult=2, dtype="fp32")}, tmp_path / "ck.pt")
    cfg = tmp_path / "run.yaml"
    cfg.write_text("adapt_set: lm_head\nchunk_size: 16\neval_lr: 0.1\n")
    assert main(["--config", str(cfg), "--val-cache-dir", str(cache), "--checkpoint-path", str(tmp_path / "ck.pt"),
                 "--max-docs", "3", "--summary-path", str(tmp_path / "sum.json"), "--eager"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["docs_scored"] == 3 and out["driver"] == "eager"
    s = json.loads((tmp_path / "sum.json").read_text())
    assert s["ckpt_sha256"] and s["config"]["max_docs"] == 3
    with pytest.raises(ValueError, match="unknown RunConfig keys"):
        RunConfig.from_dict({"nope": 1})
