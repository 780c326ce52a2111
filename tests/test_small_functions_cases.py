"""Small pure functions and thin glue that the end-to-end tests pass by: split-K choice, dW row chunks,
window gather, the legality controller's cache replay, the legacy 24-cell matrix runner (CPU)."""
import json
import types

import pytest
import torch

from chaoscontrol_b200 import data as D
from chaoscontrol_b200 import training as T
from chaoscontrol_b200.episodic.cache import EpisodicCache, fingerprint_tokens
from chaoscontrol_b200.eval_stream.legality import LeakDetectedError, LegalityController
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.ops.gemm import pick_splits
from chaoscontrol_b200.ops.lm_head import default_row_chunks


# ---------------------------------------------------------------- split-K / row chunks
@pytest.mark.parametrize("m,n,k", [(256, 256, 524288), (1024, 256, 524288), (512, 256, 4096), (256, 512, 64), (16384, 256, 32768)])
def test_split_k_fills_the_sms_with_non_empty_exact_splits(m, n, k):
    s = pick_splits(m, n, k)
    kblocks = (k + 63) // 64
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    assert 1 <= s <= kblocks and s * tiles <= max(148, tiles)
    kper = (kblocks + s - 1) // s
    assert (kblocks + kper - 1) // kper == s                              # every split gets at least one k-block


def test_split_k_is_one_when_tiles_already_fill_the_machine():
    assert pick_splits(128 * 148, 256, 4096) == 1 and pick_splits(256, 256, 64) == 1


@pytest.mark.parametrize("R,V", [(524288, 16384), (32768, 16384), (4096, 8192), (128, 16384), (100, 256)])
def test_row_chunks_divide_the_row_tiles_exactly(R, V):
    c = default_row_chunks(R, V)
    mt = (R + 127) // 128
    per = (mt + c - 1) // c
    assert 1 <= c <= min(mt, 64) and (mt + per - 1) // per == c


def test_row_chunks_balance_the_work_items_over_the_sms():
    c = default_row_chunks(524288, 16384)
    items = (16384 // 128) * c
    waves = (items + 147) // 148
    assert items / (waves * 148) > 0.97


# ---------------------------------------------------------------- window gather
def test_window_gather_matches_slicing_and_types():
    tokens = torch.arange(100, dtype=torch.int16)
    starts = torch.tensor([0, 7, 90])
    x, y = D.batch_from_start_tensor(tokens, starts, 9, torch.device("cpu"))
    assert x.dtype == torch.int32 and y.dtype == torch.int64 and x.shape == y.shape == (3, 9)
    ref_x, ref_y = D.batch_from_starts(tokens, starts.tolist(), 9, torch.device("cpu"))
    assert torch.equal(x.long(), ref_x) and torch.equal(y, ref_y)


def test_window_gather_can_clamp_to_the_vocabulary():
    tokens = torch.tensor([5, 70, 3, 999, 1, 2], dtype=torch.int32)
    x, y = D.batch_from_start_tensor(tokens, torch.tensor([0]), 4, torch.device("cpu"), vocab_size=64)
    assert x.tolist() == [[5, 63, 3, 63]] and y.tolist() == [[63, 3, 63, 1]]


# ---------------------------------------------------------------- legality controller with a cache
def _lm():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=32, dim=16, num_layers=1)


def _cache_with(span, key_tokens, window=4):
    c = EpisodicCache(capacity=4, span_length=len(span), key_rep_dim=4, fingerprint_window=window)
    c.append(key_fp=fingerprint_tokens(torch.tensor(key_tokens)), key_rep=torch.zeros(4),
             value_tok_ids=torch.tensor(span), value_anchor_id=0, current_step=0, embedding_version=0)
    return c


def test_cache_hit_on_the_chunk_tail_is_replayed_once_after_adaptation():
    model = _lm()
    chunk = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8]])
    cache = _cache_with([9, 10, 11, 12, 13], [5, 6, 7, 8])
    ctl = LegalityController(model, cache=cache, fingerprint_window=4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    steps = []
    real = opt.step
    opt.step = lambda *a, **k: (steps.append(1), real(*a, **k))[1]
    ctl.score_chunk(chunk)
    assert len(ctl._pending_cache_hits) == 1 and int(cache.last_fired_step[0]) == -1
    ctl.adapt_on_chunk(chunk, optimizer=opt, steps=2)
    assert len(steps) == 3 and ctl._pending_cache_hits == []            # two chunk steps + one replay
    ctl.adapt_on_chunk(chunk, optimizer=opt, steps=0)
    assert len(steps) == 3                                              # nothing pending, zero steps: no-op


def test_cache_miss_short_chunk_and_disabled_window_give_no_hits():
    model = _lm()
    cache = _cache_with([9, 10, 11], [5, 6, 7, 8])
    ctl = LegalityController(model, cache=cache, fingerprint_window=4)
    ctl.score_chunk(torch.tensor([[1, 2, 3, 4, 5, 6, 7, 9]]))
    assert ctl._pending_cache_hits == []
    assert ctl._query_cache(torch.tensor([[7, 8]])) == [] and ctl._query_cache(torch.tensor([5, 6, 7, 8])) == []
    off = LegalityController(model, cache=cache, fingerprint_window=0)
    assert off._query_cache(torch.tensor([[5, 6, 7, 8]])) == []
    assert LegalityController(model)._query_cache(torch.tensor([[5, 6, 7, 8]])) == []


def test_replay_budget_and_document_boundary():
    model = _lm()
    chunk = torch.tensor([[1, 2, 3, 4, 5, 6, 7, 8]])
    cache = _cache_with([9, 10, 11], [5, 6, 7, 8])
    ctl = LegalityController(model, cache=cache, fingerprint_window=4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ctl.score_chunk(chunk)
    before = [p.detach().clone() for p in model.parameters()]
    ctl.adapt_on_chunk(chunk, optimizer=opt, steps=0, cache_replay_steps=0)      # replay budget 0: nothing runs
    assert all(torch.equal(a, b) for a, b in zip(before, model.parameters())) and ctl._pending_cache_hits == []
    ctl.score_chunk(chunk)
    ctl.mark_new_epoch()
    assert ctl._pending_cache_hits == []


def test_single_token_span_is_not_replayed():
    model = _lm()
    cache = _cache_with([9], [5, 6, 7, 8])
    ctl = LegalityController(model, cache=cache, fingerprint_window=4)
    entry = cache.query(fingerprint_tokens(torch.tensor([5, 6, 7, 8])))
    assert ctl._replay(entry, torch.optim.SGD(model.parameters(), lr=0.1)) is None


def test_leak_detection_and_short_chunks():
    model = _lm()
    ctl = LegalityController(model, leak_detection=True)
    chunk = torch.tensor([[1, 2, 3, 4]])
    ctl.score_chunk(chunk)
    ctl.adapt_on_chunk(chunk, optimizer=torch.optim.SGD(model.parameters(), lr=0.1))
    with pytest.raises(LeakDetectedError):
        ctl.score_chunk(chunk)
    ctl.mark_new_epoch()
    ctl.score_chunk(chunk)
    with pytest.raises(ValueError, match="length >= 2"):
        ctl.score_chunk(torch.tensor([[1]]))


# ---------------------------------------------------------------- the legacy matrix runner
def test_matrix_runner_trains_every_cell_and_rewrites_the_results_file(tmp_path, monkeypatch):
    cells = T.build_chaoscontrol_matrix()
    assert len(cells) == 24 and {c["a_mode"] for c in cells} == {"diag", "paired", "full"}
    assert sum(c["outer_model_dim"] == 64 for c in cells) == 9 and cells[0]["label"] == "base"
    monkeypatch.setattr(T, "build_chaoscontrol_matrix", lambda: cells[:2] + cells[5:6])
    cfg = T.parse_chaoscontrol_args(["--data-path", "x", "--model-dim", "16", "--num-layers", "1", "--seq-len", "8",
                                     "--batch-size", "2", "--budget-seconds", "0.2", "--dtype", "fp32", "--matrix",
                                     "--output-json", str(tmp_path / "out" / "m.json")])
    for k, v in dict(vocab_size=32, metabolic_gate=False, metabolic_k=2, metabolic_threshold=0.1,
                     metabolic_threshold_mode="fixed", metabolic_score="ensemble_agreement", metabolic_noise_std=0.01,
                     generation_mode="noise", metabolic_mode="fork", mcts_horizon=2, mcts_ucb_c=1.4,
                     consolidation_write="last", latent_persistence=False, cfr_enabled=False, eval_warmup=False).items():
        if not hasattr(cfg, k):
            setattr(cfg, k, v)
    tokens = torch.randint(0, 32, (400,), generator=torch.Generator().manual_seed(0))
    res = T.run_chaoscontrol_matrix(cfg, device=torch.device("cpu"), param_dtype=torch.float32, train_tokens=tokens,
                                    train_starts=list(range(0, 300, 8)), eval_tokens=tokens, eval_starts=list(range(0, 64, 8)))
    assert [r["label"] for r in res] == ["base", "+nn", "+outer"] and all(r["train_steps"] >= 1 and r["bpb"] > 0 for r in res)
    assert res[2]["params"] > res[0]["params"] and res[0]["artifact_bytes"] == 2 * res[0]["params"]
    assert json.loads((tmp_path / "out" / "m.json").read_text())[2]["label"] == "+outer"
