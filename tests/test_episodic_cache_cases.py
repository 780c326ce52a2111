"""Episodic cache: storage, lookup, eviction policy, feedback, persistence -- one property per test (CPU)."""
import json

import pytest
import torch

from chaoscontrol_b200.episodic.cache import CacheEntry, EpisodicCache, fingerprint_tokens, fingerprint_tokens_batch


def _cache(**kw):
    base = dict(capacity=4, span_length=3, key_rep_dim=5, grace_steps=10, utility_ema_decay=0.5)
    base.update(kw)
    return EpisodicCache(**base)


def _put(c, fp, step=0, **kw):
    return c.append(key_fp=fp, key_rep=torch.full((c.key_rep_dim,), float(fp)), value_tok_ids=torch.arange(c.span_length) + fp,
                    value_anchor_id=fp * 10, current_step=step, embedding_version=7, **kw)


def test_new_cache_is_empty_with_typed_zeroed_storage():
    c = _cache()
    assert len(c) == 0 and not c.is_full and c.key_rep.shape == (4, 5) and c.value_tok_ids.shape == (4, 3)
    assert c.key_rep.dtype == torch.float32 and c.value_tok_ids.dtype == torch.int64 and c.occupied.dtype == torch.bool
    assert c.last_fired_step.tolist() == [-1] * 4 and c.write_step.tolist() == [-1] * 4 and float(c.utility_u.sum()) == 0.0


@pytest.mark.parametrize("kw", [dict(capacity=0), dict(span_length=0), dict(key_rep_dim=-1), dict(fingerprint_window=0),
                                dict(utility_ema_decay=0.0), dict(utility_ema_decay=1.0), dict(slot_state_dim=-1),
                                dict(simplex_k_max=-2)])
def test_bad_construction_arguments_are_refused(kw):
    with pytest.raises(ValueError):
        _cache(**kw)


def test_append_then_query_returns_the_entry():
    c = _cache()
    slot = _put(c, 42, step=3, pressure_at_write=0.7, source_write_id=99, write_bucket=2, protection_score=0.25)
    e = c.query(42)
    assert isinstance(e, CacheEntry) and e.slot == slot == 0 and e.key_fp == 42 and e.value_anchor_id == 420
    assert e.utility_u == 1.0 and e.last_fired_step == -1 and e.write_step == 3 and e.birth_embedding_version == 7
    assert e.pressure_at_write == pytest.approx(0.7) and e.source_write_id == 99 and e.write_bucket == 2
    assert e.protection_score == 0.25 and e.value_tok_ids.tolist() == [42, 43, 44] and len(c) == 1


def test_query_miss_and_returned_tensors_are_copies():
    c = _cache()
    _put(c, 1)
    assert c.query(2) is None
    e = c.query(1)
    e.key_rep.fill_(9.0)
    assert float(c.key_rep[0, 0]) == 1.0


def test_append_checks_shapes():
    c = _cache()
    with pytest.raises(ValueError, match="key_rep"):
        c.append(key_fp=1, key_rep=torch.zeros(4), value_tok_ids=torch.zeros(3, dtype=torch.long), value_anchor_id=0,
                 current_step=0, embedding_version=0)
    with pytest.raises(ValueError, match="value_tok_ids"):
        c.append(key_fp=1, key_rep=torch.zeros(5), value_tok_ids=torch.zeros(2, dtype=torch.long), value_anchor_id=0,
                 current_step=0, embedding_version=0)


def test_free_slots_fill_in_order_then_capacity_forces_an_eviction():
    c = _cache()
    assert [_put(c, fp, step=fp) for fp in (1, 2, 3, 4)] == [0, 1, 2, 3] and c.is_full
    slot = _put(c, 5, step=5)                                           # within grace: the oldest write goes
    assert slot == 0 and c.query(1) is None and c.query(5).slot == 0 and len(c) == 4


def test_past_grace_the_lowest_utility_goes():
    c = _cache()
    for fp in (1, 2, 3, 4):
        _put(c, fp, step=0)
    c.utility_u[:] = torch.tensor([0.9, 0.1, 0.5, 0.7])
    assert _put(c, 5, step=100) == 1 and c.query(2) is None


def test_protection_score_shields_a_low_utility_entry():
    c = _cache()
    for fp in (1, 2, 3, 4):
        _put(c, fp, step=0, protection_score=5.0 if fp == 2 else 0.0)
    c.utility_u[:] = torch.tensor([0.9, 0.1, 0.5, 0.7])
    assert _put(c, 5, step=100) == 2                                   # 0.1 + 5 is no longer the minimum


def test_only_entries_past_grace_compete_on_utility():
    c = _cache()
    for fp, step in ((1, 0), (2, 95), (3, 96), (4, 97)):
        _put(c, fp, step=step)
    c.utility_u[:] = torch.tensor([0.9, 0.0, 0.0, 0.0])
    assert _put(c, 5, step=100) == 0                                   # the young zero-utility entries are protected


def test_utility_is_an_ema_and_feedback_for_an_empty_slot_is_dropped():
    c = _cache()
    s = _put(c, 1)
    c.update_utility(s, 3.0)
    assert float(c.utility_u[s]) == pytest.approx(0.5 * 1.0 + 0.5 * 3.0)
    c.update_utility(s, -2.0)
    assert float(c.utility_u[s]) == pytest.approx(0.0)
    c.update_utility(3, 5.0)
    assert float(c.utility_u[3]) == 0.0
    with pytest.raises(IndexError):
        c.update_utility(4, 1.0)


def test_mark_fired_touches_only_the_fired_step():
    c = _cache()
    s = _put(c, 1, step=2)
    before = c.to_dict()
    c.mark_fired(s, 9)
    assert int(c.last_fired_step[s]) == 9
    after = c.to_dict()
    assert all(torch.equal(before[k], after[k]) for k in c._TENSOR_FIELDS if k != "last_fired_step")
    with pytest.raises(ValueError, match="not occupied"):
        c.mark_fired(1, 9)
    with pytest.raises(IndexError):
        c.mark_fired(-1, 9)


def test_evict_frees_the_slot_and_the_index():
    c = _cache()
    s = _put(c, 1)
    c.evict(s)
    assert len(c) == 0 and c.query(1) is None and int(c.write_step[s]) == -1 and float(c.utility_u[s]) == 0.0
    c.evict(s)                                                          # evicting an empty slot is a no-op
    with pytest.raises(IndexError):
        c.evict(17)
    assert _put(c, 2) == s


def test_a_repeated_fingerprint_takes_a_new_slot_and_lookup_follows_the_newest():
    c = _cache()
    a, b = _put(c, 7, step=0), _put(c, 7, step=1)
    assert a != b and c.query(7).slot == b and len(c) == 2
    c.evict(b)
    assert c.query(7) is None                                           # the index pointed at the newer copy


def test_snapshot_is_a_dict_of_tensors_on_the_device():
    c = _cache(slot_state_dim=2, simplex_k_max=3)
    _put(c, 1)
    snap = c.snapshot_to(torch.device("cpu"))
    assert set(snap) == set(c._TENSOR_FIELDS) and snap["slot_state"].shape == (4, 2) and snap["simplex_edge_slot"].shape == (4, 3)
    assert snap["simplex_edge_slot"].tolist()[0] == [-1, -1, -1] and bool(snap["occupied"][0])


def test_reset_returns_to_the_constructed_state_and_keeps_the_shape():
    c = _cache()
    for fp in (1, 2):
        _put(c, fp, step=fp)
    c.reset()
    fresh = _cache()
    assert len(c) == 0 and c.query(1) is None and c.capacity == 4 and c.grace_steps == 10
    assert all(torch.equal(getattr(c, n), getattr(fresh, n)) for n in c._TENSOR_FIELDS)


def test_round_trip_preserves_state_and_lookup():
    c = _cache(slot_state_dim=2, simplex_k_max=2)
    for fp in (1, 2, 3):
        _put(c, fp, step=fp, write_bucket=fp)
    c.update_utility(1, 4.0)
    c.mark_fired(2, 8)
    c.slot_state[0] = torch.tensor([0.5, -0.5], dtype=torch.float16)
    c.simplex_edge_slot[0] = torch.tensor([2, 1])
    d = EpisodicCache.from_dict(c.to_dict())
    assert all(torch.equal(getattr(c, n), getattr(d, n)) for n in c._TENSOR_FIELDS)
    assert all(getattr(c, n) == getattr(d, n) for n in c._CONFIG_FIELDS) and d.query(3).last_fired_step == 8      # slot 2 holds fingerprint 3
    assert _put(d, 4, step=9) == 3


def test_saved_blob_holds_clones_and_missing_keys_are_errors():
    c = _cache()
    _put(c, 1)
    blob = c.to_dict()
    blob["utility_u"].fill_(77.0)
    assert float(c.utility_u[0]) == 1.0
    for key in ("capacity", "occupied", "fp_index"):
        bad = c.to_dict()
        del bad[key]
        with pytest.raises(KeyError, match=key):
            EpisodicCache.from_dict(bad)


def test_every_displacement_writes_one_trace_row_in_schema_order(tmp_path):
    path = tmp_path / "evict.ndjson"
    c = _cache(capacity=2, eviction_trace_path=str(path))
    _put(c, 1, step=0)
    _put(c, 2, step=1)
    assert not path.exists()                                            # filling free slots displaces nothing
    _put(c, 3, step=2, displacing_candidate_id=55)
    rows = [json.loads(x) for x in path.read_text().splitlines()]
    assert len(rows) == 1 and list(rows[0]) == ["evicted_slot_id", "evicted_key_fp", "evicted_utility_at_eviction",
                                                "evicted_write_step", "evicted_last_fired_step", "evicted_protection_score",
                                                "gpu_step", "displacing_candidate_id", "displacing_key_fp"]
    assert rows[0]["evicted_key_fp"] == 1 and rows[0]["gpu_step"] == 2 and rows[0]["displacing_candidate_id"] == 55
    assert rows[0]["displacing_key_fp"] == 3 and rows[0]["evicted_utility_at_eviction"] == 1.0


def test_fingerprints_scalar_and_batch_agree_and_depend_on_order():
    torch.manual_seed(0)
    t = torch.randint(0, 16384, (5, 8))
    batch = fingerprint_tokens_batch(t)
    assert batch == [fingerprint_tokens(row) for row in t] and len(set(batch)) == 5
    assert fingerprint_tokens(t[0]) != fingerprint_tokens(t[0].flip(0)) and all(0 <= f < 2 ** 63 for f in batch)
