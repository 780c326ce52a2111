"""Episodic runtime: the run config's controller options reach the objects they configure (CPU, one rank)."""
import json

import pytest
import torch

from chaoscontrol_b200.episodic.learned_action_space import (ACTION_SPACE_HEADS, ConstrainedActionSpace,
                                                            build_action_space_from_config)
from chaoscontrol_b200.episodic.runtime import EpisodicRuntime
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget

CFG = dict(model_dim=16, episodic_capacity=64, episodic_writes_per_step=4, episodic_fingerprint_window=2, seed=0)


def _rt(**cfg):
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    return model, EpisodicRuntime(model=model, config=dict(CFG, **cfg), rank=0, world_size=1, device=torch.device("cpu"))


# ---------------------------------------------------------------- the builder
def test_action_space_is_off_unless_enabled():
    assert build_action_space_from_config({}) is None
    assert build_action_space_from_config({"episodic_controller_action_space_enabled": False,
                                           "episodic_controller_selection_readiness": 1.0}) is None


def test_action_space_defaults_are_inert_but_carry_the_shared_recurrence():
    sp = build_action_space_from_config({"episodic_controller_action_space_enabled": True})
    assert isinstance(sp, ConstrainedActionSpace) and not sp.trace_only and sp.selection_readiness == 0.0
    assert sp.selection_max_delta == 0.0 and sp.max_tags_per_query is None and sp.event_ssm is not None
    assert set(sp.head_readiness) == set(ACTION_SPACE_HEADS) and all(v == 0.0 for v in sp.head_readiness.values())
    assert sp.online_learning_rate == 0.0 and sp.reward_clip == 5.0


def test_head_tables_flat_keys_and_the_selection_pair():
    sp = build_action_space_from_config({
        "episodic_controller_action_space_enabled": True, "episodic_controller_action_space_trace_only": True,
        "episodic_controller_head_readiness": {"eviction": 0.4, "temperature": 0.9},
        "episodic_controller_eviction_readiness": 0.1,                    # the table wins over the flat key
        "episodic_controller_replay_budget_max_delta": 2.0, "episodic_controller_selection_readiness": 0.75,
        "episodic_controller_selection_max_delta": 3.0, "episodic_controller_max_tags_per_query": 2,
        "episodic_controller_shared_event_ssm_enabled": False, "episodic_controller_action_learning_rate": 0.05,
        "episodic_controller_action_reward_clip": 2.5})
    assert sp.trace_only and sp.head_readiness["eviction"] == 0.4 and sp.head_readiness["temperature"] == 0.9
    assert sp.head_max_delta["replay_budget"] == 2.0 and sp.readiness("selection_rank") == 0.75
    assert sp.selection_max_delta == 3.0 and sp.head_max_delta["selection_rank"] == 3.0 and sp.max_tags_per_query == 2
    assert sp.event_ssm is None and sp.online_learning_rate == 0.05 and sp.reward_clip == 2.5


def test_recurrence_options_are_read():
    sp = build_action_space_from_config({"episodic_controller_action_space_enabled": True,
                                         "episodic_controller_ssm_hidden_dim": 8, "episodic_controller_ssm_decay": 0.5,
                                         "episodic_controller_ssm_seed": 3})
    assert sp.event_ssm.hidden_dim == 8 and sp.event_ssm.decay == 0.5


@pytest.mark.parametrize("bad", [{"episodic_controller_selection_max_delta": -1.0}, {"episodic_controller_max_tags_per_query": -2},
                                 {"episodic_controller_action_learning_rate": -0.1}])
def test_builder_refuses_impossible_bounds(bad):
    with pytest.raises(ValueError):
        build_action_space_from_config({"episodic_controller_action_space_enabled": True, **bad})


# ---------------------------------------------------------------- the runtime
def test_runtime_options_reach_cache_learner_and_generator():
    _, rt = _rt(episodic_utility_ema_decay=0.8, episodic_grace_steps=7, episodic_write_ring_max_drain_per_step=3,
                episodic_controller_runtime="simplex", episodic_controller_gerber_c=0.0,
                episodic_controller_selection_seed=123)
    try:
        assert rt.cache.utility_ema_decay == 0.8 and rt.cache.grace_steps == 7 and rt.max_drain == 3
        assert rt.action_space is None and rt.action_trace is None
        want = torch.Generator().manual_seed(123)
        assert torch.equal(rt._sel_gen.get_state(), want.get_state())
    finally:
        rt.close()


def test_drain_cap_limits_what_one_step_takes(tmp_path):
    model, rt = _rt(episodic_write_ring_max_drain_per_step=1)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, episodic=rt,
                                    stride=8, seq_len=16, batch_size=4, device=torch.device("cpu"), budget_seconds=600.0,
                                    precision="fp32", stop_check_interval=1, max_steps=5, lm_head_backward_mode="fused",
                                    prefetch_batches=False)
    finally:
        rt.close()
    e = res["episodic"]
    assert e["write_events_emitted"] > 5 >= e["write_events_ingested"] > 0                  # one per step at most


def test_enabled_action_space_runs_in_the_loop_and_traces(tmp_path):
    trace = tmp_path / "actions.ndjson"
    model, rt = _rt(episodic_controller_action_space_enabled=True, episodic_controller_selection_readiness=1.0,
                    episodic_controller_selection_max_delta=4.0, episodic_controller_max_tags_per_query=1,
                    episodic_controller_action_trace_path=str(trace))
    assert rt.action_space is not None and rt.action_space.max_tags_per_query == 1 and rt.action_trace is not None
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, episodic=rt,
                                    stride=8, seq_len=16, batch_size=4, device=torch.device("cpu"), budget_seconds=600.0,
                                    precision="fp32", stop_check_interval=1, max_steps=8, lm_head_backward_mode="fused",
                                    prefetch_batches=False)
    finally:
        rt.close()
    e = res["episodic"]
    assert e["action_space"] == {"trace_only": False, "selection_readiness": 1.0, "selection_max_delta": 4.0,
                                 "max_tags_per_query": 1, "shared_event_ssm": True, "online_learning_rate": 0.0}
    assert e["replays"] >= 1 and e["replays"] <= e["queries_ingested"]        # one tag per query at most
    rows = [json.loads(x) for x in trace.read_text().splitlines()]
    assert rows and {"gpu_step", "head_name", "bounded_action_json", "accepted", "readiness"} <= set(rows[0])
    assert any(r["head_name"] == "selection_rank" for r in rows)


def test_cache_side_tables_take_their_sizes_from_the_config():
    _, rt = _rt(episodic_slot_state_dim=6, episodic_simplex_k_max=3)
    try:
        assert rt.cache.slot_state.shape == (64, 6) and rt.cache.simplex_edge_slot.shape == (64, 3)
    finally:
        rt.close()
