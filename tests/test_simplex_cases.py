"""Native simplex policy and its online learner, one property per test (CPU, the C++ control library)."""
import json

import numpy as np
import pytest

from chaoscontrol_b200.episodic import native as N

DIMS = dict(N=16, K_v=16, K_s=4, H=32)


def _inputs(seed=2):
    rng = np.random.default_rng(seed)
    V = rng.standard_normal((16, 16)).astype(np.float32)
    raw = rng.standard_normal((16, 16)).astype(np.float32)
    raw /= np.linalg.norm(raw, axis=1, keepdims=True)
    return V, (raw @ raw.T).astype(np.float32), (rng.standard_normal(4) * 0.5).astype(np.float32)


def _outcome(slot, gpu_step, reward, *, status=0, selection_step=None):
    ev = np.zeros((), N.REPLAY_OUTCOME)
    ev["event_type"], ev["slot_id"], ev["gpu_step"], ev["outcome_status"] = 3, slot, gpu_step, status
    ev["selection_step"] = gpu_step if selection_step is None else selection_step
    ev["reward_shaped"] = ev["ce_delta_raw"] = reward
    return ev


def _learner(pol=None, **kw):
    base = dict(num_slots=8, max_entries_per_slot=4, gamma=1.0, learning_rate=0.1, sgd_interval=1, ema_interval=4,
                ema_alpha=0.5, gerber_c=0.0)
    base.update(kw)
    L = N.SimplexOnlineLearner(**base)
    if pol is not None:
        L.initialize(pol)
    return L


# ---------------------------------------------------------------- policy forward
def test_forward_shapes_and_normalisation():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    p, logits = pol.forward(*_inputs())
    assert p.shape == logits.shape == (16,) and p.dtype == np.float32
    assert abs(float(p.sum()) - 1.0) < 1e-5 and float(p.min()) > 0


def test_forward_softmax_survives_huge_logits():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    pol.flat *= 200.0
    V, E, f = _inputs()
    p, logits = pol.forward(V * 50, E, f)
    assert np.isfinite(p).all() and abs(float(p.sum()) - 1.0) < 1e-4


def test_temperature_sharpens_and_flattens():
    V, E, f = _inputs()
    cold, warm, hot = (N.SimplexPolicy(**DIMS, temperature=t, seed=1).forward(V, E, f)[0] for t in (0.1, 1.0, 10.0))
    assert cold.max() > warm.max() > hot.max() and hot.max() - hot.min() < 0.05
    assert int(cold.argmax()) == int(warm.argmax()) == int(hot.argmax())


def test_forward_is_deterministic_and_depends_on_every_input():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    V, E, f = _inputs()
    p0, _ = pol.forward(V, E, f)
    assert np.array_equal(p0, pol.forward(V, E, f)[0])
    V2 = V.copy()
    V2[3] += 1.0
    assert not np.allclose(p0, pol.forward(V2, E, f)[0])
    assert not np.allclose(pol.forward(V, E * 0, f)[1], pol.forward(V, E, f)[1])


def test_simplex_bias_shifts_all_logits_equally():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    V, E, f = _inputs()
    p0, l0 = pol.forward(V, E, f)
    p1, l1 = pol.forward(V, E, f + 3.0)
    assert np.allclose(p0, p1, atol=1e-6)                              # a shared bias cancels in the softmax
    assert np.allclose(l0, l1, atol=1e-6)                              # and is not part of the per-vertex logits


def test_alpha_zero_makes_the_edges_irrelevant():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    pol.flat[-1] = 0.0                                                 # alpha is the last base weight
    V, E, f = _inputs()
    assert np.allclose(pol.forward(V, E, f)[0], pol.forward(V, -E, f)[0], atol=1e-7)


def test_bad_shapes_are_refused():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    assert int(N.lib().ccbc_simplex_flat_size(16, 4, 32)) == pol.flat.size == 16 * 32 + 32 + 32 + 1 + 4 + 1
    bad = N.SimplexPolicy(N=16, K_v=16, K_s=4, H=32, temperature=0.0, seed=1)
    with pytest.raises(ValueError, match="temperature"):
        bad.forward(*_inputs())


def test_residual_heads_change_logits_only_when_lambda_is_nonzero():
    V, E, f = _inputs()
    v3 = N.SimplexPolicyV3(N=16, K_v=16, K_e=1, K_s=4, H=32, n_heads=2, seed=1)
    base_n = int(N.lib().ccbc_simplex_flat_size(16, 4, 32))
    p_on, l_on, branch = v3.forward(V, E[..., None] if E.ndim == 2 else E, f, with_branch=True)
    assert float(np.abs(branch).sum()) > 0
    v3.flat[base_n] = 0.0                                              # lambda
    p_off, l_off = v3.forward(V, E, f)
    plain = N.SimplexPolicy(**DIMS, seed=1)
    plain.flat[:] = v3.flat[:base_n]
    assert np.allclose(l_off, plain.forward(V, E, f)[1], atol=1e-6) and not np.allclose(l_on, l_off)


# ---------------------------------------------------------------- gradient
def test_gradient_is_zero_for_zero_advantage_and_flips_with_its_sign():
    pol = N.SimplexPolicy(**DIMS, seed=1)
    V, E, f = _inputs()
    assert float(np.abs(pol.grad(V, E, f, chosen=3, advantage=0.0)).sum()) == 0.0
    g_pos, g_neg = pol.grad(V, E, f, 3, 1.0), pol.grad(V, E, f, 3, -1.0)
    assert np.allclose(g_pos, -g_neg, atol=1e-7) and np.allclose(pol.grad(V, E, f, 3, 2.0), 2 * g_pos, atol=1e-6)


def test_gradient_matches_central_differences():
    pol = N.SimplexPolicy(**DIMS, temperature=0.8, seed=5)
    V, E, f = _inputs(7)
    g = pol.grad(V, E, f, chosen=9, advantage=1.0)

    def loss(flat):
        q = N.SimplexPolicy(**DIMS, temperature=0.8, seed=5)
        q.flat = flat.astype(np.float32)
        return -np.log(float(q.forward(V, E, f)[0][9]))
    rng = np.random.default_rng(0)
    for i in rng.choice(pol.flat.size, 12, replace=False):
        d = np.zeros_like(pol.flat, dtype=np.float64)
        d[i] = 1e-2
        num = (loss(pol.flat + d) - loss(pol.flat - d)) / 2e-2
        assert g[i] == pytest.approx(num, abs=3e-3, rel=5e-2), i


def test_entropy_bonus_pushes_toward_uniform():
    pol = N.SimplexPolicy(**DIMS, temperature=0.3, seed=1)
    V, E, f = _inputs()
    p0, _ = pol.forward(V, E, f)
    ent0 = -(p0 * np.log(p0)).sum()
    g = pol.grad(V, E, f, chosen=0, advantage=0.0, entropy_beta=1.0)
    pol.flat -= 0.05 * g
    p1, _ = pol.forward(V, E, f)
    assert -(p1 * np.log(p1)).sum() > ent0


# ---------------------------------------------------------------- learner
def test_decisions_are_recorded_with_a_bounded_history():
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(pol)
    V, E, f = _inputs()
    for step in range(7):
        L.record_decision(2, step, chosen=1, p_chosen=0.1, V=V, E=E, feats=f)
    t = L.telemetry()
    assert t["history_appends"] == 7 and L.history_size(2) == 4 and L.history_size(3) == 0 and t["replay_outcomes"] == 0
    L.record_decision(99, 0, 1, 0.1, V, E, f)
    assert L.telemetry()["invalid_slot_skips"] == 1 and L.telemetry()["history_appends"] == 7
    L.close()


@pytest.mark.parametrize("setup,key", [("no_weights", "skipped_missing_state"), ("no_decision", "skipped_missing_state"),
                                      ("bad_status", None), ("bad_slot", "invalid_slot_skips")])
def test_outcomes_that_cannot_be_credited_are_skipped(setup, key):
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(None if setup == "no_weights" else pol)
    V, E, f = _inputs()
    if setup == "no_weights":
        with pytest.raises(ValueError, match="not initialised"):
            L.record_decision(1, 5, 2, 0.1, V, E, f)
    if setup == "bad_status":
        L.record_decision(1, 5, 2, 0.1, V, E, f)
    ev = _outcome(99 if setup == "bad_slot" else 1, 6, 1.0, status=1 if setup == "bad_status" else 0)
    L.on_replay_outcome(ev)
    t = L.telemetry()
    assert t["replay_outcomes"] == 1 and t["credited_actions"] == 0 and t["sgd_steps"] == 0
    if key:
        assert t[key] == 1
    L.close()


def test_non_finite_reward_is_dropped():
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(pol)
    V, E, f = _inputs()
    L.record_decision(1, 5, 2, 0.1, V, E, f)
    L.on_replay_outcome(_outcome(1, 6, float("nan")))
    assert L.telemetry()["credited_actions"] == 0 and np.array_equal(L.weights(), pol.flat)
    L.close()


@pytest.mark.parametrize("sign", [1.0, -1.0])
def test_reinforce_moves_the_chosen_probability_with_the_advantage(sign):
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(pol, learning_rate=0.5)
    V, E, f = _inputs()
    p0 = float(pol.forward(V, E, f)[0][7])
    # first outcome sets the reward mean (advantage 0); the second is above / below it
    for step, r in ((0, 0.0), (1, sign * 1.0)):
        L.record_decision(step, step, 7, p0, V, E, f)
        L.on_replay_outcome(_outcome(step, step, r))
    cur = N.SimplexPolicy(**DIMS, seed=3)
    cur.flat = L.weights()
    p1 = float(cur.forward(V, E, f)[0][7])
    assert (p1 > p0) if sign > 0 else (p1 < p0)
    assert L.telemetry()["credited_actions"] == 2
    L.close()


def test_gerber_gate_rejects_when_the_margin_changed_sign():
    pol = N.SimplexPolicy(**DIMS, temperature=0.2, seed=3)
    V, E, f = _inputs()
    p = pol.forward(V, E, f)[0]
    best, worst = int(p.argmax()), int(p.argmin())
    L = _learner(pol, gerber_c=0.5)
    # the margin spread is seeded by a few agreeing observations
    for step in range(3):
        L.record_decision(0, step, best, float(p[best]), V, E, f)
        L.on_replay_outcome(_outcome(0, step, 1.0 + step))
    acc0 = L.telemetry()["gerber_accepted"]
    # recorded as "was likelier than uniform", but the current policy makes it much less likely than uniform
    L.record_decision(1, 10, worst, 0.9, V, E, f)
    L.on_replay_outcome(_outcome(1, 10, 5.0))
    t = L.telemetry()
    assert t["gerber_rejected"] >= 1 and t["last_gerber_weight"] == 0.0 and t["gerber_accepted"] == acc0
    L.close()


def test_recency_decay_scales_the_credit():
    V, E, f = _inputs()
    norms = []
    for gamma in (1.0, 0.5):
        pol = N.SimplexPolicy(**DIMS, seed=3)
        L = _learner(pol, gamma=gamma, learning_rate=1.0)
        L.record_decision(0, 0, 3, 0.1, V, E, f)
        L.on_replay_outcome(_outcome(0, 0, 0.0))                          # seeds the reward mean
        L.record_decision(1, 0, 3, 0.1, V, E, f)
        w0 = L.weights().copy()
        L.on_replay_outcome(_outcome(1, 4, 2.0, selection_step=0))       # four steps after the decision
        norms.append(float(np.linalg.norm(L.weights() - w0)))
        L.close()
    assert norms[1] == pytest.approx(norms[0] * 0.5 ** 4, rel=0.05)


def test_sgd_and_slow_copy_cadences():
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(pol, sgd_interval=3, ema_interval=4, ema_alpha=0.5, max_entries_per_slot=1)
    V, E, f = _inputs()
    for step in range(8):
        L.record_decision(step % 8, step, 2, 0.1, V, E, f)
        L.on_replay_outcome(_outcome(step % 8, step, float(step % 3)))
    t = L.telemetry()
    assert t["credited_actions"] == 8 and t["sgd_steps"] == 8 // 3 and t["ema_blends"] == 8 // 4
    fast, slow = L.weights(), L.weights(slow=True)
    assert not np.allclose(fast, pol.flat) and not np.allclose(slow, fast) and not np.allclose(slow, pol.flat)
    L.close()


def test_trace_rows_cover_decisions_credits_skips_and_outcomes(tmp_path):
    pol = N.SimplexPolicy(**DIMS, seed=3)
    L = _learner(pol)
    path = tmp_path / "trace.ndjson"
    L.set_trace_path(str(path))
    V, E, f = _inputs()
    L.record_decision(1, 5, 2, 0.1, V, E, f)
    L.on_replay_outcome(_outcome(1, 6, 1.0))
    L.on_replay_outcome(_outcome(2, 7, 1.0))                              # no decision for slot 2
    L.set_trace_path("")
    rows = [json.loads(x) for x in path.read_text().splitlines()]
    kinds = [r["row_type"] for r in rows]
    assert kinds == ["decision", "credit", "replay_outcome", "skip"]
    assert rows[0]["chosen_idx"] == 2 and rows[1]["slot_id"] == 1 and rows[3]["status_reason"] == "missing_decision"
    assert {"advantage_raw", "gerber_weight", "p_current_chosen", "current_entropy"} <= set(rows[1])
    n = len(rows)
    L.on_replay_outcome(_outcome(1, 8, 1.0))                              # tracing is off again
    assert len(path.read_text().splitlines()) == n
    L.close()
