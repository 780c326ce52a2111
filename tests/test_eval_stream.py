"""Streaming evaluation on CPU: batched carried-state scorer vs whole-document
scoring, LPT sharding, legality / leak detection, state persistence modes,
delta modulation, budget accounting, val-cache round trip, TTT driver."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200.eval_stream import (BudgetTracker, DeltaModulator, LeakDetectedError,
                                           LegalityController, MetricsCollector, RunConfig, StateManager,
                                           attach_trainable_h0, detach_trainable_h0, load_val_cache,
                                           select_adapt_params, write_synthetic_val_cache)
from chaoscontrol_b200.eval_stream.types import DocRecord
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.scoring import assign_docs_lpt, compute_bpb, run_ttt_eval, score_docs, score_val_cache


def _model(seed=0):
    torch.manual_seed(seed)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2)


def test_chunked_carried_state_scoring_equals_whole_doc():
    m = _model().eval()
    rng = np.random.default_rng(0)
    lens = [37, 5, 64, 2, 19, 100]
    toks = torch.tensor(rng.integers(0, 64, sum(lens)), dtype=torch.long)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    res = score_docs(m, toks, starts, lens, chunk_size=16, max_batch_tokens=48, raw_bytes=[3 * n for n in lens])
    for i, (s, n) in enumerate(zip(starts, lens)):
        doc = toks[s:s + n].view(1, -1)
        with torch.no_grad():
            logits = m(doc)["logits"]
        ref = F.cross_entropy(logits[0, :-1], doc[0, 1:], reduction="sum").item()
        assert res.doc_ce[i] == pytest.approx(ref, rel=1e-4, abs=1e-4), i
        assert res.doc_tokens[i] == n - 1
    assert res.total_tokens == sum(n - 1 for n in lens)
    assert res.bpb == pytest.approx(compute_bpb(res.total_ce, 3 * sum(lens)))


def test_lpt_assignment_balances_and_covers():
    lens = [1000, 900, 50, 40, 30, 20, 10, 5]
    shards = assign_docs_lpt(lens, 3, 16)
    assert sorted(i for s in shards for i in s) == list(range(len(lens)))
    loads = [sum(math.ceil((lens[i] - 1) / 16) * 16 for i in s) for s in shards]
    assert max(loads) - min(loads) <= 1008
    assert compute_bpb(math.log(2.0) * 8, 8) == pytest.approx(1.0)


def test_val_cache_roundtrip_and_scoring(tmp_path):
    man = write_synthetic_val_cache(tmp_path / "vc", n_docs=20, vocab=64, median_len=40, sigma=0.5,
                                    min_len=4, max_len=90, seed=1)
    vc = load_val_cache(tmp_path / "vc")
    assert vc.num_docs == 20 and vc.total_tokens == man["total_tokens"] and vc.tokens.dtype == np.uint16
    d = next(vc.iter_docs())
    assert len(vc.tokens_for_doc(d)) == d.token_len
    out = score_val_cache(_model(), vc, chunk_size=16)
    assert out["docs_scored"] == 20 and out["tokens_scored"] == vc.total_tokens - 20
    assert math.isfinite(out["bpb"]) and out["bpb"] > 0


def test_legality_controller_and_leak_detection():
    m = _model()
    ctl = LegalityController(m, leak_detection=True)
    chunk = torch.randint(0, 64, (1, 12))
    loss, finals = ctl.score_chunk(chunk)
    assert loss > 0 and len(finals) == 2
    opt = torch.optim.SGD(select_adapt_params(m, adapt_set="log_a+delta_proj"), lr=0.1)
    after = ctl.adapt_on_chunk(chunk, optimizer=opt, steps=2)
    assert after is not None
    with pytest.raises(LeakDetectedError):
        ctl.score_chunk(chunk)
    ctl.mark_new_epoch()
    ctl.score_chunk(chunk)
    with pytest.raises(ValueError):
        ctl.score_chunk(chunk[:, :1])
    assert ctl.adapt_on_chunk(chunk, optimizer=opt, steps=0) is None


def test_state_manager_modes_and_trainable_h0():
    m = _model()
    sm = StateManager(m, persistence_mode="reset")
    sm.start_doc(doc_id=0, batch_size=3)
    assert len(sm.get_state()) == 2 and sm.get_state()[0].shape == (3, 16)
    sm.set_state([torch.ones(3, 16), torch.ones(3, 16)])
    sm.start_doc(doc_id=1, batch_size=3)
    assert float(sm.get_state()[0].sum()) == 0.0
    sc = StateManager(m, persistence_mode="carry_state")
    sc.start_doc(doc_id=0, batch_size=1)
    sc.set_state([torch.ones(1, 16), torch.ones(1, 16)])
    sc.start_doc(doc_id=1, batch_size=1)
    assert float(sc.get_state()[0].sum()) == 16.0
    attach_trainable_h0(m)
    assert len(select_adapt_params(m, adapt_set="trainable_h0")) == 2
    sh = StateManager(m, persistence_mode="trainable_h0")
    sh.start_doc(doc_id=0, batch_size=2)
    out = m(torch.randint(0, 64, (2, 6)), initial_states=sh.get_state())
    out["logits"].sum().backward()
    assert m.layers[0].core._trainable_h0.grad is not None
    detach_trainable_h0(m)
    assert not any("_trainable_h0" in k for k in m.state_dict())
    with pytest.raises(ValueError):
        StateManager(m, persistence_mode="bogus")
    with pytest.raises(ValueError):
        select_adapt_params(m, adapt_set="bogus")
    assert len(select_adapt_params(m, adapt_set="all")) == len(list(m.parameters()))
    assert select_adapt_params(m, adapt_set="none") == []


def test_delta_modulator_restores():
    m = _model().eval()
    tok = torch.randint(0, 64, (1, 10))
    base = m(tok)["logits"]
    la = m.layers[0].core.log_a.detach().clone()
    with DeltaModulator(m, delta_scale=2.0, log_a_shift=0.5):
        mod = m(tok)["logits"]
        assert not torch.allclose(mod, base)
    assert torch.equal(m.layers[0].core.log_a, la)
    assert torch.allclose(m(tok)["logits"], base)
    with pytest.raises(ValueError):
        with DeltaModulator(m, log_a_shift=0.1, adapt_set_hint="log_a"):
            pass


def test_budget_tracker_summary():
    b = BudgetTracker(total_budget_seconds=600, score_floor_seconds=100, safety_margin_seconds=50)
    assert b.usable_ttt_budget_seconds == 450 and b.can_adapt()
    b.add_adapt_time(460)
    assert not b.can_adapt()
    s = b.summary(docs_scored=10, chunks_scored=50, tokens_scored=1000, adapt_steps=5, timed_out=False,
                  collapsed=False, score_only_mode=False, elapsed_seconds=20.0, max_docs=10)
    assert s["result_status"] == "exploratory_prefix_complete" and s["slack_remaining_seconds"] == 0.0
    s2 = BudgetTracker(total_budget_seconds=600).summary(
        docs_scored=50_000, chunks_scored=1, tokens_scored=1, adapt_steps=0, timed_out=False,
        collapsed=False, score_only_mode=True, elapsed_seconds=85.0, max_docs=50_000)
    assert s2["result_status"] == "record_eligible" and s2["score_floor_seconds"] == 85.0
    assert RunConfig.from_dict({"adapt_set": "all"}).adapt_set == "all"
    with pytest.raises(ValueError):
        RunConfig.from_dict({"nope": 1})


def test_ttt_eval_scores_then_adapts_and_restores(tmp_path):
    m = _model(3)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    docs = [DocRecord(i, list(np.random.default_rng(i).integers(0, 64, 40)), 120) for i in range(4)]
    with MetricsCollector(output_path=tmp_path / "m.jsonl", stability_window=2) as mc:
        out = run_ttt_eval(m, docs, adapt_set="log_a+delta_proj", chunk_size=16, eval_lr=0.05, metrics=mc)
    assert out["docs_scored"] == 4 and out["adapt_steps"] > 0 and math.isfinite(out["bpb"])
    for n, p in m.named_parameters():
        assert torch.equal(p, before[n]), n          # restored after every document
    score_only = run_ttt_eval(m, docs, adapt_set="none", chunk_size=16)
    assert score_only["adapt_steps"] == 0 and score_only["score_only_mode"]
    kept = run_ttt_eval(m, docs, adapt_set="log_a", persistence_mode="carry_both", chunk_size=16, eval_lr=0.05)
    assert kept["adapt_steps"] > 0
    assert not torch.equal(m.layers[0].core.log_a, before["layers.0.core.log_a"])
    assert (tmp_path / "m.jsonl").read_text().count("\n") == 4
