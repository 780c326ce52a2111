"""Episodic controller periphery: NDJSON loggers, replay-log analytics, the CPU SSM controller ABI
and the bounded learned action space."""
import json
import math

import numpy as np
import pytest
import torch

from chaoscontrol_b200.episodic import analytics, cpu_ssm_controller as csc, diagnostics as dg
from chaoscontrol_b200.episodic import learned_action_space as las


def _row(**over):
    row = {c: 0 for c in dg.REPLAY_LOG_SCHEMA}
    row.update(outcome_status="ok", arm="a", feature_manifest_hash="h", p_behavior=[0.5, 0.5],
               candidate_slot_ids=[1, 2], candidate_scores=[0.1, 0.2], logits=[0.0, 1.0])
    row.update(over)
    return row


def test_replay_logger_schema_and_nan(tmp_path):
    path = tmp_path / "run" / "episodic_replay_log_rank0.ndjson"
    with dg.DiagnosticsLogger(path) as log:
        log.write_row(_row(step=3, replay_loss=float("nan"), utility_post=torch.tensor(0.25),
                           entropy=np.float32(0.5), logits=torch.tensor([1.0, float("inf")])))
        with pytest.raises(KeyError):
            log.write_row({k: v for k, v in _row().items() if k != "slot"})
        with pytest.raises(KeyError):
            log.write_row(_row(extra=1))
    with dg.DiagnosticsLogger(path) as log:        # append, not truncate
        log.write_row(_row(step=4))
    rows = [json.loads(l) for l in path.read_text().splitlines()]
    assert [r["step"] for r in rows] == [3, 4]
    assert list(rows[0]) == list(dg.REPLAY_LOG_SCHEMA)
    assert rows[0]["replay_loss"] is None and rows[0]["utility_post"] == 0.25 and rows[0]["logits"] == [1.0, None]


def test_action_trace_logger(tmp_path):
    path = tmp_path / "trace.ndjson"
    with dg.ActionSpaceTraceLogger(path) as log:
        space = las.ConstrainedActionSpace(selection_readiness=1.0, selection_max_delta=0.5, trace_log=log)
        space.effective_scores(heuristic_scores=[1.0, 2.0], learned_scores=[10.0, -10.0], gpu_step=7,
                               reward_context={"pressure": float("nan")})
        with pytest.raises(KeyError):
            log.append({"gpu_step": 1})
    row = json.loads(path.read_text().splitlines()[0])
    assert list(row) == list(dg.ACTION_SPACE_TRACE_SCHEMA) and row["gpu_step"] == 7
    assert json.loads(row["bounded_action_json"]) == pytest.approx([0.5, -0.5], abs=1e-6)
    assert json.loads(row["reward_context_json"]) == {"pressure": None}


def test_replay_log_queries(tmp_path):
    with pytest.raises(FileNotFoundError):
        analytics.ReplayLogQuery.open(tmp_path)
    rng = np.random.default_rng(0)
    for rank in range(2):
        with dg.DiagnosticsLogger(tmp_path / f"episodic_replay_log_rank{rank}.ndjson") as log:
            for i in range(40):
                cos = float(rng.uniform(-1, 1))
                log.write_row(_row(step=i * 10, slot=i % 4, key_fp=100 + i % 4, write_step=i % 4,
                                   write_bucket=i % 2, write_pressure=1.0 + (i % 2), query_cosine=cos,
                                   replay_loss=2.0 - 0.5 * (i % 2), replay_grad_cos_rare=0.8 * cos + 0.01 * i,
                                   reward_shaped=cos, utility_post=0.1 * (i // 4)))
    with analytics.ReplayLogQuery.open(tmp_path) as q:
        assert len(q.table) == 80 and set(q.table["rank"]) == {0, 1}
        cohort = q.cohort_replay_utility().set_index("write_bucket")
        assert cohort.loc[0, "n_replays"] == 40 and cohort.loc[1, "mean_replay_loss"] == pytest.approx(1.5)
        drift = q.drift_trajectory_per_entry(window_steps=1000)
        assert len(drift) == 4 and (drift["drift_norm_avg"] >= 0).all()
        front = q.surprise_frontier(bucket_steps=100)
        assert {"step_bucket", "write_bucket", "frontier"} <= set(front.columns)
        assert front[front.write_bucket == 1]["frontier"].iloc[0] == pytest.approx(2.0 * 1.5)
        corr = q.retrieval_utility_correlation()
        assert corr["reward_shaped"] == pytest.approx(1.0) and corr["replay_grad_cos_rare"] > 0.8


def _weights(F=6, G=5, S=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return csc.CpuSsmControllerWeights(r(G, F), r(S, F), torch.rand(G, generator=g), torch.rand(S, generator=g),
                                       r(G), r(S), torch.tensor(0.3))


def test_cpu_ssm_controller_native_matches_torch(tmp_path):
    w = _weights()
    assert (w.feature_dim, w.global_dim, w.slot_dim) == (6, 5, 4)
    with pytest.raises(ValueError):
        csc.CpuSsmControllerWeights(w.w_global_in, w.w_slot_in[:, :3], w.decay_global, w.decay_slot,
                                    w.w_global_out, w.w_slot_out, w.bias)
    w.save(tmp_path / "c" / "w.pt")
    w2 = csc.CpuSsmControllerWeights.load(tmp_path / "c" / "w.pt")
    assert all(torch.equal(a, b) for a, b in zip(w.to_dict().values(), w2.to_dict().values()))
    with pytest.raises(KeyError):
        csc.CpuSsmControllerWeights.from_dict({"bias": 0.0})
    rt_c = csc.CpuSsmControllerRuntime(w, capacity=3, prefer_cpp=True)
    rt_t = csc.CpuSsmControllerRuntime(w, capacity=3, prefer_cpp=False)
    g = torch.Generator().manual_seed(1)
    for i in range(6):
        f = torch.randn(6, generator=g)
        a = rt_c.score_slot_with_snapshot(f, slot=i % 3)
        b = rt_t.score_slot_with_snapshot(f, slot=i % 3)
        assert torch.allclose(a.logit, b.logit, atol=1e-5) and torch.allclose(a.slot_state, b.slot_state, atol=1e-6)
    assert torch.allclose(rt_c.global_state, rt_t.global_state, atol=1e-5)
    assert torch.allclose(rt_c.slot_state, rt_t.slot_state, atol=1e-5)
    # snapshot carries the PRE-step state
    first = csc.CpuSsmControllerRuntime(w, capacity=1, prefer_cpp=False).score_slot_with_snapshot(torch.ones(6), slot=0)
    assert float(first.global_state.abs().sum()) == 0.0
    with pytest.raises(IndexError):
        rt_t.score_slot(torch.zeros(6), slot=9)
    with pytest.raises(ValueError):
        csc.CpuSsmControllerRuntime(w, capacity=0)


def test_bounded_scalar_spec():
    s = las.BoundedScalarSpec("t", 0.25, 4.0, transform="softplus")
    assert s.map(float("nan")) == 0.25 and 0.25 < s.map(0.0) < 4.0 and s.map(1e6) == pytest.approx(4.0, rel=1e-4)
    sig = las.BoundedScalarSpec("a", 0.0, 1.0)
    assert sig.map(0.0) == pytest.approx(0.5) and sig.map(-1e4) == pytest.approx(0.0) and sig.map(1e4) == pytest.approx(1.0)
    assert las.BoundedScalarSpec("c", 2.0, 2.0).map(3.0) == 2.0
    with pytest.raises(ValueError):
        las.BoundedScalarSpec("x", 1.0, 0.0)
    with pytest.raises(ValueError):
        las.BoundedScalarSpec("x", 0.0, 1.0, transform="relu")


def test_shared_event_ssm_is_stable_and_learns():
    ssm = las.SharedEventSsm(hidden_dim=16, seed=3)
    d = ssm.diagnostics()
    assert d["top_log_sv"] <= -0.02 + 1e-5 and d["controller_work_units"] == 17 * 16 + 256 + 160
    for i in range(500):
        out = ssm.observe({"pressure": 100.0, "ce": float(i), "score": float("nan")})
    assert set(out) == set(las.DEFAULT_HEADS) and all(math.isfinite(v) for v in out.values())
    assert ssm.diagnostics()["state_norm"] <= 8.0 + 1e-4
    same = las.SharedEventSsm(hidden_dim=16, seed=3)
    assert torch.equal(same.A, ssm.A) and torch.equal(same.W_in, ssm.W_in)
    before = ssm.head_output("eviction")
    hid = ssm.hidden
    ssm.update_head_from_hidden(head_name="eviction", hidden=hid, reward=100.0, learning_rate=0.01)
    after = ssm.head_output("eviction")
    assert after - before == pytest.approx(0.05 * (sum(h * h for h in hid) + 1.0), rel=1e-4)   # reward clipped to 5
    ssm.update_head_from_hidden(head_name="nope", hidden=hid, reward=1.0, learning_rate=0.01)
    assert ssm.work_ratio_vs_bare_ssm() < 1e-5
    assert las.make_shared_event_ssm_from_config({"episodic_controller_ssm_hidden_dim": 8}).hidden_dim == 8


def test_constrained_action_space_contract():
    trace = las.ActionSpaceTrace()
    off = las.ConstrainedActionSpace(trace_only=True, selection_readiness=1.0, selection_max_delta=1.0, trace_log=trace)
    h = [0.3, 0.1, 0.2]
    assert off.effective_scores(heuristic_scores=h, learned_scores=[9, 9, 9], gpu_step=0) == h and not trace.rows
    assert off.scalar_value(head_name="temperature", raw_value=3.0, gpu_step=0, fallback=1.5) == 1.5
    on = las.ConstrainedActionSpace(selection_readiness=0.5, selection_max_delta=0.2, max_tags_per_query=2,
                                    head_readiness={"temperature": 0.5}, trace_log=trace)
    eff = on.effective_scores(heuristic_scores=h, learned_scores=[0.0, 50.0, float("nan")], gpu_step=1)
    assert eff == pytest.approx([0.3, 0.2, 0.2])
    with pytest.raises(ValueError):
        on.effective_scores(heuristic_scores=h, learned_scores=[1.0], gpu_step=1)
    assert on.selected_indices(effective_scores=eff, gpu_step=1, requested_budget=3) == [0, 1]
    assert trace.rows[-1]["event_type"] == "action_space_clamp" and trace.rows[-1]["clamp_amount"] == 1.0
    assert on.selected_indices(effective_scores=eff, gpu_step=1, requested_budget=-4) == []
    t = on.scalar_value(head_name="temperature", raw_value=0.0, gpu_step=2, fallback=1.0)
    assert t == pytest.approx(0.5 * 1.0 + 0.5 * on.scalar_specs["temperature"].map(0.0))
    with pytest.raises(KeyError):
        las.ConstrainedActionSpace(head_readiness={"zzz": 1.0}).scalar_value(head_name="zzz", raw_value=0.0,
                                                                             gpu_step=0, fallback=0.0)
    with pytest.raises(ValueError):
        las.ConstrainedActionSpace(selection_max_delta=-1.0)
    # learned residual from the shared state, delayed credit
    ssm = las.SharedEventSsm(seed=1)
    learn = las.ConstrainedActionSpace(selection_readiness=1.0, selection_max_delta=1.0, event_ssm=ssm,
                                       online_learning_rate=0.1, trace_log=trace)
    eff2 = learn.effective_scores(heuristic_scores=h, learned_scores=None, gpu_step=3, reward_context={"pressure": 2.0})
    assert len(eff2) == 3 and all(abs(a - b) <= 1.0 for a, b in zip(eff2, h))
    learn.record_credit_assignment(key=42, head_names=["selection_rank", "bogus"], gpu_step=3)
    w0 = torch.tensor(ssm.head_weights["selection_rank"])
    assert learn.apply_reward(key=42, reward=1.0, gpu_step=4) == 1
    assert not torch.equal(w0, torch.tensor(ssm.head_weights["selection_rank"]))
    assert learn.apply_reward(key=42, reward=1.0, gpu_step=5) == 0
    assert las.coerce_action_space(None) is None and las.coerce_action_space(False) is None
    assert isinstance(las.coerce_action_space({"trace_only": True}), las.ConstrainedActionSpace)
    with pytest.raises(TypeError):
        las.coerce_action_space(3)


def test_numpy_shm_ring(tmp_path):
    import os
    from chaoscontrol_b200.episodic.ipc import ShmRing
    name = f"ccb_t_{os.getpid()}"
    ring = ShmRing.create(name=name, slot_shape=(3,), dtype=np.float32, capacity=4)
    try:
        with pytest.raises(FileExistsError):
            ShmRing.create(name=name, slot_shape=(3,), dtype=np.float32, capacity=4)
        for bad in (dict(slot_shape=(2,), dtype=np.float32, capacity=4), dict(slot_shape=(3,), dtype=np.float64, capacity=4),
                    dict(slot_shape=(3,), dtype=np.float32, capacity=5)):
            with pytest.raises(ValueError):
                ShmRing.attach(name=name, **bad)
        reader = ShmRing.attach(name=name, slot_shape=(3,), dtype=np.float32, capacity=4)
        assert reader.try_read() is None
        for i in range(6):
            ring.try_write(np.full(3, i, np.float32))
        assert ring.dropped_count() == 2 and len(reader) == 4
        got = [int(reader.try_read()[0]) for _ in range(4)]
        assert got == [2, 3, 4, 5] and reader.try_read() is None
        with pytest.raises(ValueError):
            ring.try_write(np.zeros(4, np.float32))
        with pytest.raises(ValueError):
            ring.try_write(np.zeros(3, np.float64))
        with pytest.raises(ValueError):
            ring.try_write([0, 0, 0])
        reader.close()
        reader.close_and_unlink()      # non-owner: no unlink
        again = ShmRing.attach(name=name, slot_shape=(3,), dtype=np.float32, capacity=4)
        again.close()
    finally:
        ring.close_and_unlink()
        ring.close_and_unlink()
    with pytest.raises(FileNotFoundError):
        ShmRing.attach(name=name, slot_shape=(3,), dtype=np.float32, capacity=4)
    with pytest.raises(ValueError):
        ShmRing.create(name=name + "x", slot_shape=(1,) * 9, dtype=np.float32, capacity=1)


def _filled_cache(n=6, dim=8):
    from chaoscontrol_b200.episodic.cache import EpisodicCache
    torch.manual_seed(0)
    cache = EpisodicCache(capacity=16, span_length=2, key_rep_dim=dim)
    for i in range(n):
        cache.append(key_fp=100 + i, key_rep=torch.randn(dim), value_tok_ids=torch.tensor([i, i + 1]),
                     value_anchor_id=i, current_step=10 * i, embedding_version=0, pressure_at_write=0.1 * i,
                     source_write_id=1000 + i, write_bucket=i % 4)
        cache.utility_u[i] = 0.5 + 0.1 * i
    return cache


def test_controller_cycle_heuristic_and_per_slot_runtime():
    from collections import deque
    from chaoscontrol_b200.episodic.controller import run_controller_cycle
    from chaoscontrol_b200.episodic.query import query_topk
    cache = _filled_cache()
    q = [{"step": 70, "rank": 1, "k": i, "pressure": 0.3, "residual": torch.randn(8)} for i in range(3)]
    residuals = [c["residual"].clone() for c in q]
    tags: list = []
    assert run_controller_cycle(controller_query_queue=deque(), tagged_replay_queue=tags, cache=cache) == 0
    n = run_controller_cycle(controller_query_queue=q, tagged_replay_queue=tags, cache=cache, k=4, selected_at=5,
                             policy_version=2)
    assert n == 3 and not q and len(tags) == 12
    for qi in range(3):
        mine = [t["slot"] for t in tags[4 * qi: 4 * qi + 4]]
        assert mine == query_topk(residuals[qi], cache, 4).tolist()
    t0 = tags[0]
    assert t0["query_event_id"] == (1 << 56) and t0["replay_id"] == ((1 << 56) & ((1 << 56) - 1)) << 8
    assert t0["source_write_id"] == 1000 + t0["slot"] and t0["selected_at"] == 5 and t0["policy_version"] == 2
    assert not any(isinstance(v, torch.Tensor) for t in tags for v in t.values())
    assert tags[1]["replay_id"] & 0xFF == 1 and t0["outcome_status"] == "pending"
    # learned per-slot runtime + bounded action space with a 2-tag budget
    rt = csc.CpuSsmControllerRuntime(_weights(F=4), capacity=16, prefer_cpp=False)
    recorded = []

    class Rec:
        def record_replay_selection(self, **kw):
            recorded.append(kw)

    tags2: list = []
    q2 = deque([{"step": 80, "query_event_id": 77, "pressure": 0.1, "residual": residuals[0]}])
    run_controller_cycle(controller_query_queue=q2, tagged_replay_queue=tags2, cache=cache, k=4,
                         controller_runtime=rt, action_recorder=Rec(),
                         action_space={"selection_readiness": 1.0, "selection_max_delta": 5.0, "max_tags_per_query": 2})
    assert len(tags2) == 2 and len(recorded) == 2 and tags2[0]["query_event_id"] == 77
    assert {"heuristic_rank", "action_space_score", "controller_features", "controller_slot_state"} <= set(tags2[0])
    assert tags2[0]["action_space_score"] >= tags2[1]["action_space_score"]
    empty = type(cache)(capacity=4, span_length=2, key_rep_dim=8)
    tags3: list = []
    assert run_controller_cycle(controller_query_queue=[{"step": 1, "residual": torch.randn(8)}],
                                tagged_replay_queue=tags3, cache=empty) == 1 and not tags3


def test_controller_cycle_simplex_runtime_and_thread():
    import threading
    from chaoscontrol_b200.episodic import controller as ctl
    cache = _filled_cache()
    rt = ctl.SimplexRuntime(num_slots=16)
    space = las.ConstrainedActionSpace(head_readiness={"temperature": 1.0}, event_ssm=las.SharedEventSsm(),
                                       online_learning_rate=0.1)
    tags: list = []
    q = [{"step": 90, "rank": 0, "k": 3, "pressure": 0.2, "residual": torch.randn(8), "arm": "c"}]
    ctl.run_controller_cycle(controller_query_queue=q, tagged_replay_queue=tags, cache=cache, k=16,
                             controller_runtime=rt, action_recorder=rt, simplex_selection_mode="sample",
                             simplex_generator=torch.Generator().manual_seed(0), action_space=space)
    assert len(tags) == 1
    t = tags[0]
    assert t["simplex_n_actual"] == 6 and len(t["p_behavior"]) == 6 and abs(sum(t["p_behavior"]) - 1) < 1e-5
    assert t["slot"] == t["candidate_slot_ids"][t["simplex_chosen_idx"]] and t["arm"] == "c"
    assert t["feature_manifest_hash"] == ctl.FEATURE_MANIFEST_HASH and 0 <= t["entropy"] <= math.log(6) + 1e-6
    assert rt.decisions and rt.decisions[0]["selection_mode"] == "sample"
    assert rt.learner.history_size(t["slot"]) == 1
    assert 0.25 <= rt.policy.temperature <= 4.0 and t["replay_id"] in space.credit_history
    assert space.apply_reward(key=t["replay_id"], reward=1.0, gpu_step=91) == 1
    V, E, sf, ids = ctl.build_simplex_inputs(cache_view=cache.snapshot_to(torch.device("cpu")),
                                             slots=torch.tensor([2, 4]), scores=torch.tensor([0.9, 0.1]),
                                             current_step=100)
    assert V.shape == (16, 16) and E.shape == (16, 16) and ids[:3] == [2, 4, 0]
    assert V[0, 0] == pytest.approx(0.7) and V[1, 2] == pytest.approx((100 - 40) / 1000) and E[0, 0] == pytest.approx(1.0)
    assert sf.tolist() == pytest.approx([0.9, 0.8, 0.9, 0.8])
    assert ctl.choose_simplex_vertex([0.1, 0.7, 0.2, 9.0], 3)[0] == 1
    assert ctl.choose_simplex_vertex([0.0, 0.0], 2)[1] == 0.5
    with pytest.raises(ValueError):
        ctl.choose_simplex_vertex([1.0], 1, mode="nope")
    rt.learner.close()
    # thread: starts, processes, stops
    stop, beat, lock = threading.Event(), [0], threading.Lock()
    queue, out = [], []
    th = threading.Thread(target=ctl.controller_main, daemon=True,
                          kwargs=dict(controller_query_queue=queue, tagged_replay_queue=out, cache=cache,
                                      stop_event=stop, queue_lock=lock, k=2, heartbeat=beat))
    th.start()
    with lock:
        queue.append({"step": 1, "rank": 0, "k": 0, "residual": torch.randn(8)})
    import time
    t0 = time.time()
    while len(out) < 2 and time.time() - t0 < 10:
        time.sleep(0.01)
    stop.set()
    th.join(timeout=10)
    assert not th.is_alive() and len(out) == 2 and beat[0] > 0
