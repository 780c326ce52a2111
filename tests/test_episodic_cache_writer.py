"""Episodic cache, write selection, fingerprints, and the device record packer."""
import json

import numpy as np
import pytest
import torch

from chaoscontrol_b200.episodic import writer as W
from chaoscontrol_b200.episodic.cache import (FINGERPRINT_BASE, FINGERPRINT_MODULUS, EpisodicCache,
                                              fingerprint_tokens, fingerprint_tokens_batch)
from chaoscontrol_b200.episodic.native import WRITE_EVENT


def test_fingerprint_scalar_batch_and_known_value():
    toks = torch.tensor([5, 0, 65535, 123456789])
    h = 0
    for t in toks.tolist():
        h = (h * FINGERPRINT_BASE + t + 1) % FINGERPRINT_MODULUS
    assert fingerprint_tokens(toks) == h
    torch.manual_seed(0)
    big = torch.randint(0, 2 ** 31, (64, 30))
    assert fingerprint_tokens_batch(big) == [fingerprint_tokens(r) for r in big]
    with pytest.raises(ValueError):
        fingerprint_tokens(big)
    with pytest.raises(ValueError):
        fingerprint_tokens_batch(toks)


def _entry(i, D=4, S=2):
    return dict(key_fp=100 + i, key_rep=torch.full((D,), float(i)), value_tok_ids=torch.tensor([i, i + 1]),
                value_anchor_id=i, embedding_version=0)


def test_cache_append_query_evict_policy(tmp_path):
    trace = tmp_path / "evict.ndjson"
    c = EpisodicCache(capacity=3, span_length=2, key_rep_dim=4, grace_steps=10, eviction_trace_path=str(trace))
    for i in range(3):
        assert c.append(**_entry(i), current_step=i) == i
    assert c.is_full and len(c) == 3
    e = c.query(101)
    assert e.slot == 1 and e.value_anchor_id == 1 and e.utility_u == 1.0 and c.query(999) is None
    # warm-up (nobody past grace): FIFO by write step
    assert c.append(**_entry(3), current_step=5) == 0 and c.query(100) is None
    # past grace: lowest utility + protection goes
    c.update_utility(1, -50.0)
    c.protection_score[2] = 5.0
    assert c.append(**_entry(4), current_step=100) == 1
    rows = [json.loads(l) for l in trace.read_text().splitlines()]
    assert [r["evicted_slot_id"] for r in rows] == [0, 1] and rows[1]["displacing_key_fp"] == 104
    assert list(rows[0]) == ["evicted_slot_id", "evicted_key_fp", "evicted_utility_at_eviction", "evicted_write_step",
                             "evicted_last_fired_step", "evicted_protection_score", "gpu_step",
                             "displacing_candidate_id", "displacing_key_fp"]
    c.mark_fired(2, 77)
    assert int(c.last_fired_step[2]) == 77
    c.evict(2)
    assert c.query(102) is None and len(c) == 2
    with pytest.raises(ValueError):
        c.mark_fired(2, 1)
    c.update_utility(2, 1.0)                     # feedback for an evicted slot is ignored
    with pytest.raises(IndexError):
        c.evict(9)
    with pytest.raises(ValueError):
        c.append(**{**_entry(9), "key_rep": torch.zeros(5)}, current_step=0)


def test_cache_round_trip_and_reset():
    c = EpisodicCache(capacity=4, span_length=2, key_rep_dim=4, slot_state_dim=3, simplex_k_max=2)
    for i in range(3):
        c.append(**_entry(i), current_step=i, write_bucket=i)
    blob = c.to_dict()
    d = EpisodicCache.from_dict(blob)
    assert d.query(102).write_bucket == 2 and torch.equal(d.key_rep, c.key_rep) and d.slot_state.shape == (4, 3)
    blob.pop("write_bucket")
    with pytest.raises(KeyError):
        EpisodicCache.from_dict(blob)
    snap = c.snapshot_to(torch.device("cpu"))
    assert set(snap) == set(EpisodicCache._TENSOR_FIELDS)
    c.reset()
    assert len(c) == 0 and c.query(100) is None and int(c.write_step[0]) == -1
    with pytest.raises(ValueError):
        EpisodicCache(capacity=0)


class _Ring:
    def __init__(self, cap):
        self.cap, self.items = cap, []

    def push(self, ev):
        if len(self.items) >= self.cap:
            return False
        self.items.append(ev)
        return True


def _batch(B=3, T=20, D=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1000, (B, T), generator=g)
    tgt = torch.randint(0, 1000, (B, T), generator=g)
    return ids, tgt, torch.rand(B, T, generator=g), torch.rand(B, T, generator=g) * 5, torch.randn(B, T, D, generator=g)


def test_select_writes_matches_per_position_builder(tmp_path):
    W._reset_admission_trace_seq()
    ids, tgt, pr, ce, rep = _batch()
    ring, drops = _Ring(3), [0]
    trace = tmp_path / "adm.ndjson"
    out = W.select_writes(input_ids=ids, target_ids=tgt, pressure=pr, per_token_ce=ce, key_rep_per_position=rep,
                          top_p=0.2, fingerprint_window=4, span_length=3, source_rank=2, gpu_step=9, write_bucket=1,
                          admission_trace_path=str(trace), write_ring=ring, write_ring_drops=drops)
    pos = W.select_top_p_positions(pr * ce, 0.2)
    assert pos.shape == (12, 2)
    want = [W.build_write_payload(batch_index=int(b), position=int(t), input_ids=ids, target_ids=tgt,
                                  key_rep_per_position=rep, fingerprint_window=4, span_length=3) for b, t in pos]
    want = [w for w in want if w is not None]
    assert len(out) == len(want) > 0
    for a, b in zip(out, want):
        assert (a.batch_index, a.position, a.key_fp, a.value_anchor_id) == (b.batch_index, b.position, b.key_fp,
                                                                            b.value_anchor_id)
        assert torch.equal(a.key_rep, b.key_rep) and torch.equal(a.value_tok_ids, b.value_tok_ids)
    rows = [json.loads(l) for l in trace.read_text().splitlines()]
    assert len(rows) == 12 and sum(r["decision"] for r in rows) == len(out)
    assert rows[0]["candidate_id"] == (2 << 56) and rows[5]["candidate_id"] == (2 << 56) | 5
    assert len(ring.items) == min(3, len(out)) and drops[0] == max(0, len(out) - 3)
    ev = ring.items[0]
    assert len(ev["key_rep"]) == 256 and len(ev["value_tok_ids"]) == 4 and ev["gpu_step"] == 9
    assert list(ev)[:6] == ["event_type", "source_rank", "write_bucket", "candidate_id", "gpu_step", "key_fp"]
    with pytest.raises(ValueError):
        W.select_writes(input_ids=ids, target_ids=tgt, pressure=pr[:, :5], per_token_ce=ce, key_rep_per_position=rep,
                        top_p=0.1, fingerprint_window=4, span_length=3)
    with pytest.raises(ValueError):
        W.select_top_p_positions(pr, 0.0)


def test_pack_reference_layout_round_trips_through_wire_dtype():
    ids, tgt, pr, ce, rep = _batch(D=8)
    pos = torch.tensor([[0, 10], [1, 2], [2, 19], [1, 8]])
    raw = W.pack_write_events(input_ids=ids, target_ids=tgt, key_rep_per_position=rep, per_token_ce=ce,
                              positions=pos, candidate_base=torch.tensor([40]), pressure=pr, gpu_step=7,
                              source_rank=3, write_bucket=2, fingerprint_window=4, span_length=3)
    assert raw.shape == (4, 568) and raw.dtype == torch.uint8
    rec = raw.numpy().view(WRITE_EVENT).reshape(-1)
    assert rec["event_type"].tolist() == [1, 0, 0, 1]               # edge-trimmed candidates are zero records
    assert int(rec[3]["candidate_id"]) == (3 << 56) | 43 and int(rec[0]["gpu_step"]) == 7
    assert int(rec[0]["key_fp"]) == fingerprint_tokens(ids[0, 6:10])
    assert rec[0]["value_tok_ids"].tolist() == tgt[0, 10:13].tolist() + [0]
    got = torch.from_numpy(rec[0]["key_rep"][:8].copy()).view(torch.float16)
    assert torch.equal(got, rep[0, 10].to(torch.float16))
    assert float(rec[0]["pre_write_ce"]) == pytest.approx(float(ce[0, 10]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_pack_write_events_kernel_matches_host(dtype):
    torch.manual_seed(0)
    B, T, D = 8, 96, 256
    ids = torch.randint(0, 2 ** 31 - 1, (B, T))
    tgt = torch.randint(0, 65536, (B, T))
    ce = torch.rand(B, T) * 6
    pr = torch.rand(B, T)
    rep = torch.randn(B, T, D).to(dtype)
    pos = torch.stack([torch.randint(0, B, (300,)), torch.randint(0, T, (300,))], 1)
    for Wn, span, rd, pressure in ((8, 4, 256, pr), (40, 2, 100, None)):
        want = W.pack_write_events_reference(
            input_ids=ids, target_ids=tgt, key_rep_per_position=rep, per_token_ce=ce, positions=pos,
            candidate_base=1000, pressure=pressure, gpu_step=5, source_rank=6, write_bucket=9,
            fingerprint_window=Wn, span_length=span, key_rep_dim=rd)
        got = W.pack_write_events(
            input_ids=ids.cuda(), target_ids=tgt.cuda(), key_rep_per_position=rep.cuda(), per_token_ce=ce.cuda(),
            positions=pos.cuda(), candidate_base=torch.tensor([1000], device="cuda"),
            pressure=None if pressure is None else pressure.cuda(), gpu_step=5, source_rank=6, write_bucket=9,
            fingerprint_window=Wn, span_length=span, key_rep_dim=rd)
        torch.cuda.synchronize()
        assert torch.equal(got.cpu(), want)
        assert int((got[:, 0] == 1).sum()) > 100


# --------------------------------------------------------------------------- slot tensor / query
def test_gpu_slot_row_and_batched_round_trip():
    from chaoscontrol_b200.episodic import gpu_slot as G
    S, D = 3, 6
    assert G.slot_dim(span_length=4, key_rep_dim=256) == 528
    slots = G.make_slot_tensor(k_max=5, span_length=S, key_rep_dim=D, device="cpu")
    big = 2 ** 63 - 1
    G.pack_payload(slots[1], valid_mask=1.0, pressure=0.5, key_fp=big, value_anchor_id=7,
                   value_tok_ids=torch.tensor([7, 8, 9]), key_rep=torch.arange(6.0), residual=-torch.arange(6.0),
                   span_length=S, key_rep_dim=D, pre_write_ce=2.5, protection_score=0.25)
    u = G.unpack_payload(slots[1], span_length=S, key_rep_dim=D)
    assert u["key_fp"] == big and u["value_anchor_id"] == 7 and u["value_tok_ids"].tolist() == [7, 8, 9]
    assert u["pre_write_ce"] == 2.5 and u["protection_score"] == 0.25 and u["residual"][2] == -2.0
    assert G.unpack_payload(slots[0], span_length=S, key_rep_dim=D)["valid_mask"] == 0.0
    n = G.pack_payload_rows(slots, pressure=torch.tensor([1.0, 2.0]), key_fp=torch.tensor([big, 5]),
                            value_anchor_id=torch.tensor([1, 2]), value_tok_ids=torch.tensor([[1, 2, 3], [4, 5, 6]]),
                            key_rep=torch.ones(2, D), residual=torch.zeros(2, D))
    assert n == 2
    one = G.unpack_payload(slots[0], span_length=S, key_rep_dim=D)
    assert one["key_fp"] == big and one["valid_mask"] == 1.0 and one["pre_write_ce"] != one["pre_write_ce"]
    rows = G.unpack_payload_rows(slots, span_length=S, key_rep_dim=D)
    assert rows["key_fp"].tolist() == [big, 5] and rows["value_tok_ids"].tolist() == [[1, 2, 3], [4, 5, 6]]
    with pytest.raises(ValueError):
        G.make_slot_tensor(k_max=2, span_length=S, key_rep_dim=D, device="cpu", dtype=torch.float16)
    with pytest.raises(ValueError):
        G.pack_payload(slots[0][:5], valid_mask=1, pressure=0, key_fp=0, value_anchor_id=0,
                       value_tok_ids=torch.zeros(S), key_rep=torch.zeros(D), residual=torch.zeros(D),
                       span_length=S, key_rep_dim=D)


def test_query_topk_modes():
    from chaoscontrol_b200.episodic.query import query_topk, query_topk_batch
    c = EpisodicCache(capacity=6, span_length=2, key_rep_dim=4)
    assert query_topk(torch.ones(4), c, 3).numel() == 0
    reps = torch.eye(4)
    for i in range(4):
        c.append(key_fp=i + 1, key_rep=reps[i], value_tok_ids=torch.tensor([0, 0]), value_anchor_id=0,
                 current_step=i, embedding_version=0, pressure_at_write=float(10 - i))
    c.utility_u[2] = 5.0
    q = torch.tensor([0.9, 0.1, 0.5, 0.0])
    assert query_topk(q, c, 2).tolist() == [2, 0]                     # 0.5*5 beats 0.9*1
    assert query_topk(q, c, 9, score_mode="pressure_only").tolist() == [0, 1, 2, 3]
    c.evict(2)
    assert query_topk(q, c, 2).tolist() == [0, 1]
    idx, sc = query_topk_batch(torch.stack([q, reps[3]]), c.snapshot_to(torch.device("cpu")), 5)
    assert idx[0].tolist() == [0, 1, 3, -1, -1] and idx[1, 0] == 3 and torch.isinf(sc[0, 3])
    with pytest.raises(ValueError):
        query_topk(q, c, 2, score_mode="bogus")
    from chaoscontrol_b200.episodic.payload_dtypes import make_query_candidate_dtype, make_write_payload_dtype
    assert make_write_payload_dtype(span_length=4, key_rep_dim=8).itemsize == 8 + 32 + 32 + 8
    assert make_query_candidate_dtype(key_rep_dim=8).itemsize == 8 + 8 + 4 + 32
