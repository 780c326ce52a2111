"""Dream replay buffer and replay backward passes (cf. tests/test_exp24_dreamworld.py of the reference)."""
import math

import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200 import dreamworld as dw
from chaoscontrol_b200.episodic.cache import EpisodicCache
from chaoscontrol_b200.models.model import CareStudentLM


def _model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=40, dim=16, num_layers=2)


def test_buffer_bounds_and_diagnostics():
    buf = dw.DreamReplayBuffer(max_entries=3, max_age_steps=10)
    g = torch.Generator().manual_seed(0)
    assert buf.sample(g, 0) is None
    x = torch.ones(2, 4, requires_grad=True)
    for step in range(5):
        buf.add(step=step, states=[x * step], replay_tokens=torch.arange(6).view(2, 3))
    assert len(buf) == 3 and buf.drop_count == 2 and not buf._entries[0].states[0].requires_grad
    assert {buf.sample(g, 5).step for _ in range(20)} <= {2, 3, 4}
    d = buf.diagnostics(13)
    assert d["size"] == 2 and d["age_min"] == 9 and d["age_max"] == 10 and d["drop_count"] == 3
    assert buf.diagnostics(100)["size"] == 0 and buf.sample(g, 100) is None
    with pytest.raises(ValueError):
        dw.DreamReplayBuffer(0, 1)
    with pytest.raises(ValueError):
        dw.DreamReplayBuffer(1, 0)


def test_replay_window():
    inp = torch.arange(20).view(2, 10)
    assert dw.build_dream_replay_tokens(inp, 3, 4).tolist() == [[2, 3, 4, 5, 6], [12, 13, 14, 15, 16]]
    for bad in ((0, 1), (1, 0), (8, 4)):
        with pytest.raises(ValueError):
            dw.build_dream_replay_tokens(inp, *bad)
    with pytest.raises(ValueError):
        dw.build_dream_replay_tokens(inp[0], 2, 2)


def test_capture_then_replay_equals_continuing_the_sequence():
    model = _model()
    inp = torch.randint(0, 40, (3, 12))
    entry = dw.capture_dream_entry(model, inp, step=5, prefix_tokens=4, replay_tokens=6)
    assert entry.replay_tokens.shape == (3, 7) and len(entry.states) == 2
    with pytest.raises(ValueError):
        dw.capture_dream_entry(model, inp, step=5, prefix_tokens=1, replay_tokens=2)
    loss = dw.dreamworld_replay_backward(model, entry, 0.5)
    g_replay = [p.grad.clone() for p in model.parameters() if p.grad is not None]
    # the same loss from a full forward over the prefix + window
    model.zero_grad(set_to_none=True)
    out = model(inp[:, :9])["logits"][:, 3:9]
    ref = F.cross_entropy(out.reshape(-1, 40), inp[:, 4:10].reshape(-1))
    assert torch.allclose(loss, ref.detach(), atol=1e-5)
    assert dw.replay_grad_norm(model) == 0.0
    assert math.isclose(math.sqrt(sum(float(g.pow(2).sum()) for g in g_replay)),
                        float(torch.linalg.vector_norm(torch.cat([g.reshape(-1) for g in g_replay]))), rel_tol=1e-5)
    # row sub-sampling
    model.zero_grad(set_to_none=True)
    l2 = dw.dreamworld_replay_backward(model, entry, 1.0, replay_batch_size=1, generator=torch.Generator().manual_seed(1))
    assert math.isfinite(float(l2)) and dw.replay_grad_norm(model) > 0


def test_replay_from_cache_slots():
    model = _model()
    cache = EpisodicCache(capacity=4, span_length=5, key_rep_dim=4)
    for i in range(3):
        cache.append(key_fp=i + 1, key_rep=torch.randn(4), value_tok_ids=torch.randint(0, 40, (5,)), value_anchor_id=0,
                     current_step=i, embedding_version=0)
    assert dw.dreamworld_replay_from_cache_entry(model=model, cache=cache, slot=3, current_step=9) is None
    with pytest.raises(IndexError):
        dw.dreamworld_replay_from_cache_entry(model=model, cache=cache, slot=7, current_step=9)
    one = dw.dreamworld_replay_from_cache_entry(model=model, cache=cache, slot=1, current_step=9, weight=2.0)
    assert math.isnan(one["replay_grad_cos_rare"]) and one["utility_signal_transformed"] == 0.0
    row = cache.value_tok_ids[1].view(1, 5)
    ref = F.cross_entropy(model(row[:, :-1])["logits"].reshape(-1, 40), row[:, 1:].reshape(-1))
    assert one["replay_loss"] == pytest.approx(float(ref.detach()), abs=1e-5) and one["replay_grad_norm"] > 0
    model.zero_grad(set_to_none=True)
    many = dw.dreamworld_replay_from_cache_slots(model=model, cache=cache, slots=[0, 1, 3, 2])
    assert many["slots"] == [0, 1, 2]
    rows = cache.value_tok_ids[:3]
    refb = F.cross_entropy(model(rows[:, :-1])["logits"].reshape(-1, 40), rows[:, 1:].reshape(-1))
    assert many["replay_loss"] == pytest.approx(float(refb.detach()), abs=1e-5)
    assert dw.compute_utility_signal(-0.4) == (-0.4, 0.0) and dw.compute_utility_signal(0.3) == (0.3, 0.3)
    short = EpisodicCache(capacity=2, span_length=1, key_rep_dim=4)
    short.append(key_fp=1, key_rep=torch.randn(4), value_tok_ids=torch.zeros(1, dtype=torch.long), value_anchor_id=0,
                 current_step=0, embedding_version=0)
    assert dw.dreamworld_replay_from_cache_entry(model=model, cache=short, slot=0, current_step=1) is None
