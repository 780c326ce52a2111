"""Posterior corrections, fatigue dynamics and the regret table, one property per test (CPU)."""
import pytest
import torch

from chaoscontrol_b200.fatigue import FatigueTracker
from chaoscontrol_b200.models.posterior import BucketDelta, GlobalDelta, ResidualCache
from chaoscontrol_b200.regret import RegretTable


# ---------------------------------------------------------------- global / bucket deltas
def test_global_delta_starts_at_zero_and_expands_over_the_batch():
    g = GlobalDelta(8)
    assert g.read(5).shape == (5, 8) and float(g.read(5).abs().sum()) == 0.0


def test_global_delta_update_accumulates_with_lr_and_takes_2d_gradients():
    g = GlobalDelta(4, lr=0.5)
    g.update(torch.ones(4))
    g.update(torch.ones(1, 4) * 2)
    assert torch.allclose(g.delta, torch.full((1, 4), 1.5))
    small = GlobalDelta(4, lr=0.01)
    small.update(torch.ones(4))
    assert torch.allclose(small.delta, torch.full((1, 4), 0.01))


def test_global_delta_is_detached_and_reset_clears():
    g = GlobalDelta(4)
    g.update(torch.ones(4, requires_grad=True) * 2)
    assert not g.delta.requires_grad and "delta" in g.state_dict()
    g.reset()
    assert float(g.delta.abs().sum()) == 0.0


def test_bucket_delta_touches_only_its_bucket():
    b = BucketDelta(3, 4, lr=1.0)
    b.update(1, torch.ones(4))
    b.update(1, torch.ones(1, 4))
    assert torch.allclose(b.read(1, 2), torch.full((2, 4), 2.0))
    assert float(b.read(0, 2).abs().sum()) == 0.0 and float(b.read(2, 1).abs().sum()) == 0.0
    b.reset()
    assert float(b.deltas.abs().sum()) == 0.0 and b.deltas.shape == (3, 4)


# ---------------------------------------------------------------- residual cache
def test_empty_cache_reads_zeros_in_the_query_dtype():
    c = ResidualCache(4)
    out = c.read(torch.randn(3, 4, dtype=torch.float64))
    assert out.shape == (3, 4) and out.dtype == torch.float64 and float(out.abs().sum()) == 0.0


def test_single_entry_is_returned_whole():
    c = ResidualCache(4, k=4)
    c.store(torch.tensor([1.0, 0, 0, 0]), torch.tensor([0.5, 0.5, 0.5, 0.5]))
    assert torch.allclose(c.read(torch.tensor([[0.3, 0.1, 0.0, 0.0]])), torch.full((1, 4), 0.5))


def test_similar_query_weights_its_match_highest():
    c = ResidualCache(2, k=2)
    c.store(torch.tensor([1.0, 0.0]), torch.tensor([10.0, 0.0]))
    c.store(torch.tensor([0.0, 1.0]), torch.tensor([0.0, 10.0]))
    out = c.read(torch.tensor([[1.0, 0.05]]))
    assert out[0, 0] > out[0, 1] > 0
    w = torch.softmax(torch.tensor([1.0, 0.05]) / torch.tensor([1.0, 0.05]).norm(), 0)
    assert torch.allclose(out[0], 10.0 * w, atol=1e-5)


def test_top_k_limits_the_mixture_and_may_exceed_the_cache():
    c = ResidualCache(2, k=1)
    c.store(torch.tensor([1.0, 0.0]), torch.tensor([1.0, 0.0]))
    c.store(torch.tensor([0.0, 1.0]), torch.tensor([0.0, 1.0]))
    assert torch.allclose(c.read(torch.tensor([[0.9, 0.1]])), torch.tensor([[1.0, 0.0]]))
    big = ResidualCache(2, k=16)
    big.store(torch.tensor([1.0, 0.0]), torch.tensor([2.0, 2.0]))
    assert torch.allclose(big.read(torch.tensor([[0.0, 1.0]])), torch.tensor([[2.0, 2.0]]))


def test_cache_is_fifo_bounded_takes_2d_and_resets():
    c = ResidualCache(2, max_entries=3)
    for i in range(5):
        c.store(torch.tensor([[float(i), 1.0]]), torch.full((1, 2), float(i)))
    assert len(c._keys) == len(c._values) == 3 and float(c._values[0][0, 0]) == 2.0
    c.reset()
    assert c._keys == [] and float(c.read(torch.ones(1, 2)).abs().sum()) == 0.0


def test_batch_of_queries_reads_row_by_row():
    c = ResidualCache(2, k=1)
    c.store(torch.tensor([1.0, 0.0]), torch.tensor([1.0, 0.0]))
    c.store(torch.tensor([0.0, 1.0]), torch.tensor([0.0, 1.0]))
    out = c.read(torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.7, 0.6]]))
    assert out.tolist() == [[1.0, 0.0], [0.0, 1.0], [1.0, 0.0]]


def test_cache_does_not_track_gradients():
    c = ResidualCache(2)
    c.store(torch.ones(2, requires_grad=True), torch.ones(2, requires_grad=True))
    q = torch.ones(1, 2, requires_grad=True)
    assert not c.read(q).requires_grad


# ---------------------------------------------------------------- fatigue
def test_fatigue_defaults():
    f = FatigueTracker()
    assert f.score == 0.0 and (f.accumulation_rate, f.wake_decay_rate, f.sleep_decay_rate, f.surprise_suppression) == \
        (0.02, 0.005, 0.3, 1.0)


def test_fatigue_accumulates_under_stagnation_faster_with_pressure():
    lo, hi = FatigueTracker(), FatigueTracker()
    for _ in range(20):
        lo.step(0.0, 0.0, 0.2)
        hi.step(0.0, 0.0, 1.0)
    assert 0 < lo.score < hi.score


def test_improvement_removes_the_pressure():
    f = FatigueTracker()
    for _ in range(20):
        f.step(0.0, 1.0, 1.0)
    assert f.score == 0.0


def test_surprise_suppresses_and_drives_fatigue_down():
    calm, startled = FatigueTracker(), FatigueTracker()
    for _ in range(30):
        calm.step(0.0, 0.0, 1.0)
        startled.step(0.5, 0.0, 1.0)
    assert startled.score < calm.score
    before = calm.score
    calm.step(0.9, 0.0, 0.0)
    assert calm.score < 0.2 * before


def test_fatigue_stays_in_the_unit_interval():
    f = FatigueTracker(accumulation_rate=5.0)
    for _ in range(10):
        f.step(0.0, 0.0, 10.0)
    assert f.score <= 1.0
    f.step(100.0, 0.0, 0.0)
    assert f.score == 0.0
    f.apply_sleep_recovery(5.0)
    assert f.score == 0.0


def test_soft_ceiling_slows_accumulation():
    f = FatigueTracker(wake_decay_rate=0.0)
    steps = []
    for _ in range(100):
        a = f.score
        steps.append(f.step(0.0, 0.0, 1.0) - a)
    assert steps[0] > steps[50] > steps[99] > 0


def test_sleep_recovery_scales_with_quality():
    def after(q):
        f = FatigueTracker()
        f._fatigue = 0.8
        return f.apply_sleep_recovery(q)
    assert after(0.0) == 0.8 and after(1.0) == pytest.approx(0.5) and after(0.5) == pytest.approx(0.65)


def test_sleep_duration_runs_from_half_to_double_the_base():
    f = FatigueTracker()
    assert f.sleep_steps(128) == 64
    f._fatigue = 1.0
    assert f.sleep_steps(128) == 256
    f._fatigue = 0.5
    assert f.sleep_steps(100) == 125


def test_step_returns_the_new_score():
    f = FatigueTracker()
    assert f.step(0.0, 0.0, 1.0) == f.score == pytest.approx(0.02)


# ---------------------------------------------------------------- regret matching
def test_regret_accumulates_the_gap_to_each_alternative():
    r = RegretTable(2, 3)
    r.update(0, action_taken=1, counterfactual_values=[2.0, 9.0, 0.5], actual_value=1.0)
    assert r.get_regrets(0).tolist() == [1.0, 0.0, -0.5] and float(r.get_regrets(1).abs().sum()) == 0.0
    r.update(0, 0, [0.0, 3.0, 0.0], 1.0)
    assert r.get_regrets(0).tolist() == [1.0, 2.0, -1.5]


def test_strategy_is_the_positive_part_normalised():
    r = RegretTable(1, 3)
    r.cumulative_regret[0] = torch.tensor([1.0, 3.0, -5.0])
    s = r.get_strategy(0)
    assert s.tolist() == [0.25, 0.75, 0.0] and float(s.sum()) == pytest.approx(1.0)


def test_unknown_or_all_negative_bucket_plays_uniform():
    r = RegretTable(2, 4)
    assert r.get_strategy(1).tolist() == [0.25] * 4
    r.cumulative_regret[0] = -torch.ones(4)
    assert r.get_strategy(0).tolist() == [0.25] * 4


def test_reset_bucket_clears_only_that_row_and_views_are_copies():
    r = RegretTable(2, 2)
    r.cumulative_regret += 1.0
    view = r.get_regrets(0)
    view += 5.0
    assert r.cumulative_regret[0].tolist() == [1.0, 1.0]
    r.reset_bucket(0)
    assert r.cumulative_regret.tolist() == [[0.0, 0.0], [1.0, 1.0]]
