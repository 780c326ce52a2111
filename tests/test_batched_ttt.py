"""Batched score-then-adapt evaluation against the per-document loop.

CPU: fp32 model, ``run_ttt_eval`` (autograd, one document at a time) is the oracle
for ``run_ttt_eval_batched`` (hand-written backward, several documents per step,
slots refilled as documents end).  GPU: bf16 kernels against the graph-replayed
per-document runner.
"""
import numpy as np
import pytest
import torch

from chaoscontrol_b200.eval_stream.batched_ttt import BatchedTTT, build_plan, plan_slots, run_ttt_eval_batched
from chaoscontrol_b200.eval_stream.types import DocRecord
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.scoring import run_ttt_eval, run_ttt_eval_graph


def _docs(lens, vocab, seed=0):
    rng = np.random.default_rng(seed)
    return [DocRecord(doc_id=100 + i, tokens=rng.integers(0, vocab, n).tolist(), raw_bytes=4 * n)
            for i, n in enumerate(lens)]


def test_plan_covers_every_chunk_once_and_keeps_order_inside_a_document():
    lens = [5, 40, 17, 2, 1, 33, 64, 65, 16, 90, 0]
    C, slots = 16, 3
    toks = [list(range(1, n + 1)) for n in lens]
    plan = build_plan(toks, slots, C)
    start, slot, steps = plan_slots(lens, slots, C)
    assert plan.shape == (steps, slots, C + 4)
    seen = {}
    for s in range(steps):
        for b in range(slots):
            d = int(plan[s, b, C + 3])
            if d == len(lens):
                assert plan[s, b, C + 1] == 0 and plan[s, b, C + 2] == 0
                continue
            seen.setdefault(d, []).append((s, b))
    for d, n in enumerate(lens):
        if n < 2:
            assert d not in seen
            continue
        k = (n - 1 + C - 1) // C
        cells = seen[d]
        assert len(cells) == k and len({b for _, b in cells}) == 1          # one slot, k consecutive steps
        assert [s for s, _ in cells] == list(range(cells[0][0], cells[0][0] + k))
        got = []
        for j, (s, b) in enumerate(cells):
            row = plan[s, b]
            assert row[C + 2] == (1 if j == 0 else 0)
            v = int(row[C + 1])
            assert v == min(C, n - 1 - j * C)
            got.extend(row[1: v + 1].tolist())                              # the targets of this chunk
            assert row[0] == j * C + 1                                      # chunk j starts at token j*C
        assert got == list(range(2, n + 1))                                  # every target exactly once
    # no two documents share a cell, and a slot starts a new document only after the previous one ended
    assert sum(len(v) for v in seen.values()) == len({c for v in seen.values() for c in v})


@pytest.mark.parametrize("adapt_set", ["log_a+delta_proj", "log_a", "delta_proj"])
def test_batched_matches_per_document_loop_cpu(adapt_set):
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=128, dim=64, num_layers=2, ff_mult=2)
    docs = _docs([5, 40, 17, 2, 1, 33, 64, 65, 16, 90], 128)
    lr = 5.0                                      # large on purpose: the adaptation must move the scores
    ref = run_ttt_eval(m, docs, adapt_set=adapt_set, persistence_mode="reset", chunk_size=16, steps_per_chunk=1,
                       eval_lr=lr, optimizer="sgd", budget_seconds=3600.0)
    plain = run_ttt_eval(m, docs, adapt_set="none", persistence_mode="reset", chunk_size=16, budget_seconds=3600.0)
    effect = abs(ref["total_ce_nats"] - plain["total_ce_nats"])
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    for slots in (1, 3, 16):
        out = run_ttt_eval_batched(m, docs, adapt_set=adapt_set, chunk_size=16, eval_lr=lr, slots=slots)
        assert out["tokens_scored"] == ref["tokens_scored"] and out["chunks_scored"] == ref["chunks_scored"]
        assert out["docs_scored"] == ref["docs_scored"]
        err = abs(out["total_ce_nats"] - ref["total_ce_nats"])
        assert effect > 2e-3 and err < 0.02 * effect + 2e-4, (effect, err)
    for n, p in m.named_parameters():              # the model's own weights are never touched
        assert torch.equal(p, before[n])


def test_batched_per_document_scores_do_not_depend_on_the_slot_count_cpu():
    torch.manual_seed(1)
    m = CareStudentLM(vocab_size=64, dim=32, num_layers=2, ff_mult=2)
    docs = _docs([50, 3, 20, 20, 9, 70], 64, seed=3)
    a = run_ttt_eval_batched(m, docs, chunk_size=8, eval_lr=1.0, slots=2)["per_doc_ce"]
    b = run_ttt_eval_batched(m, docs, chunk_size=8, eval_lr=1.0, slots=5)["per_doc_ce"]
    assert a.keys() == b.keys() == {100, 101, 102, 103, 104, 105}
    for k in a:
        assert a[k] == pytest.approx(b[k], rel=1e-5, abs=1e-4)


def test_batched_rejects_other_adapt_sets():
    m = CareStudentLM(vocab_size=64, dim=32, num_layers=1, ff_mult=2)
    with pytest.raises(ValueError):
        BatchedTTT(m, adapt_set="lm_head", chunk_size=8, slots=2)


@pytest.mark.gpu
@pytest.mark.parametrize("use_graph", [False, True])
def test_batched_matches_graph_runner_gpu(use_graph):
    torch.manual_seed(0)
    dev = torch.device("cuda")
    m = CareStudentLM(vocab_size=16384, dim=256, num_layers=2, ff_mult=2).to(dev).to(torch.bfloat16)
    docs = _docs([300, 40, 700, 2, 257, 256, 513, 90, 1200, 31], 16384)
    lr = 0.5
    ref = run_ttt_eval_graph(m, docs, adapt_set="log_a+delta_proj", chunk_size=256, eval_lr=lr)
    plain = run_ttt_eval_graph(m, docs, adapt_set="none", chunk_size=256, eval_lr=lr)
    out = run_ttt_eval_batched(m, docs, chunk_size=256, eval_lr=lr, slots=4, use_graph=use_graph)
    assert out["tokens_scored"] == ref["tokens_scored"]
    effect = abs(ref["total_ce_nats"] - plain["total_ce_nats"])
    err = abs(out["total_ce_nats"] - ref["total_ce_nats"])
    assert err < 0.25 * effect + 2e-3 * abs(ref["total_ce_nats"]), (effect, err)
    for k, v in ref["per_doc_ce"].items():
        assert out["per_doc_ce"][k] == pytest.approx(v, rel=5e-3, abs=0.05)
    # a second pass over the same documents reuses the captured graph and gives the same bits
    again = run_ttt_eval_batched(m, docs, chunk_size=256, eval_lr=lr, slots=4, runner=out["runner"])
    assert again["per_doc_ce"] == out["per_doc_ce"]
    assert out["runner"].captures == (1 if use_graph else 0)
