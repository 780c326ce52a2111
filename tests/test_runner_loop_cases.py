"""The budgeted training loop: option validation, accounting, stop rules, graph gate -- one property per test (CPU)."""
import math

import pytest
import torch

from chaoscontrol_b200 import fast_path as FP
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.runner_fast_path import _build_optimizer, _loop_kwargs, train_fast_for_budget

CPU = torch.device("cpu")


def _run(model=None, opt="adamw", weight_decay=0.01, **kw):
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (2000,), dtype=torch.int16)
    model = model or CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    optim = _build_optimizer(dict(optimizer=opt, base_lr=1e-3, weight_decay=weight_decay), model)
    base = dict(train_tokens=tokens, train_num_tokens=2000, stride=8, seq_len=16, batch_size=4, device=CPU,
                optimizer=optim, budget_seconds=600.0, precision="fp32", stop_check_interval=1, max_steps=3,
                lm_head_backward_mode="chunked", prefetch_batches=False)
    base.update(kw)
    return train_fast_for_budget(model, **base), model


# ---------------------------------------------------------------- result block
def test_result_serialises_the_loss_trajectory_and_throughput():
    res, _ = _run(max_steps=4)
    assert res["steps"] == 4 and len(res["loss_history"]) == 4
    assert res["initial_loss"] == res["loss_history"][0] and res["final_loss"] == res["loss_history"][-1]
    assert res["tokens_per_step"] == 4 * 16 and res["aggregate_tokens_per_sec"] > 0
    assert res["per_gpu_tokens_per_sec"] == pytest.approx(res["aggregate_tokens_per_sec"])
    assert res["train_sampling_mode"] == "random" and res["cuda_graph_mode"] == "none" and res["peak_vram_mb"] == 0.0
    assert res["steady_state_step_seconds"] > 0 and res["distributed_muon"] is False
    import json
    json.dumps(res)


def test_same_seed_gives_the_same_trajectory_and_another_seed_does_not():
    a, _ = _run(seed=5)
    b, _ = _run(seed=5)
    c, _ = _run(seed=6)
    assert a["loss_history"] == b["loss_history"] and a["loss_history"] != c["loss_history"]


def test_max_steps_and_budget_both_stop_the_loop():
    res, _ = _run(max_steps=2)
    assert res["steps"] == 2
    clock = iter(range(0, 10_000, 10))                               # every reading is 10 s later
    res2, _ = _run(max_steps=None, budget_seconds=35.0, stop_margin_seconds=0.0, time_fn=lambda: float(next(clock)))
    assert 1 <= res2["steps"] <= 4


def test_prefetcher_on_and_off_see_the_same_batches():
    a, _ = _run(prefetch_batches=False, seed=2)
    b, _ = _run(prefetch_batches=True, seed=2)
    assert a["loss_history"] == pytest.approx(b["loss_history"], abs=1e-6)


@pytest.mark.parametrize("mode", ["fused", "chunked", "single", "fused_streaming_cached"])
def test_lm_head_modes_agree_on_the_first_loss(mode):
    ref, _ = _run(max_steps=1, lm_head_backward_mode="chunked")
    res, _ = _run(max_steps=1, lm_head_backward_mode=mode)
    assert res["loss_history"][0] == pytest.approx(ref["loss_history"][0], abs=1e-4)
    assert res["lm_head_backward_mode"] == mode


def test_embed_freeze_keeps_the_table_for_the_first_steps():
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    before = model.embed.weight.detach().clone()
    _run(model=model, max_steps=2, embed_freeze_steps=2, weight_decay=0.0)      # the freeze zeroes the gradient
    assert torch.equal(model.embed.weight.detach(), before)
    _run(model=model, max_steps=3, embed_freeze_steps=2, weight_decay=0.0)
    assert not torch.equal(model.embed.weight.detach(), before)


def test_grad_clip_bounds_the_update():
    m1 = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    m2 = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    m2.load_state_dict(m1.state_dict())
    start = torch.cat([p.detach().flatten() for p in m1.parameters()])
    _run(model=m1, max_steps=1, grad_clip_norm=1e-6)
    _run(model=m2, max_steps=1, grad_clip_norm=1e6)
    d1 = torch.cat([p.detach().flatten() for p in m1.parameters()]) - start
    d2 = torch.cat([p.detach().flatten() for p in m2.parameters()]) - start
    assert float(d1.norm()) > 0 and float(d2.norm()) > 0                # Adam normalises magnitude; both move
    assert torch.isfinite(d1).all() and torch.isfinite(d2).all()


# ---------------------------------------------------------------- validation
@pytest.mark.parametrize("kw,exc,match", [
    (dict(train_sampling_mode="nope"), ValueError, "train_sampling_mode"),
    (dict(cuda_graph_mode="always"), ValueError, "cuda_graph_mode"),
    (dict(replay_eviction_enabled=True), ValueError, "crct_enabled"),
    (dict(event_sleep_enabled=True), ValueError, "dreamworld_enabled"),
    (dict(dreamworld_enabled=True, crct_enabled=True), ValueError, "cannot be combined"),
])
def test_contradictory_options_are_refused(kw, exc, match):
    with pytest.raises(exc, match=match):
        _run(**kw)


def test_criticality_is_single_rank_only():
    class Hook:
        pass
    with pytest.raises(ValueError, match="single-rank"):
        _run(criticality=Hook(), world_size=2)


def test_predictive_aux_refuses_memory_rank_topologies():
    with pytest.raises(ValueError, match="predictive_aux_weight"):
        _run(predictive_aux_weight=0.1, predictive_aux_horizon=2, crct_enabled=True)


def test_scopt_refuses_foreign_loops():
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    optim = _build_optimizer(dict(optimizer="scopt", base_lr=1e-3), model)
    tokens = torch.randint(0, 64, (500,), dtype=torch.int16)
    with pytest.raises(ValueError, match="scopt"):
        train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=500, stride=8, seq_len=16, batch_size=4,
                              device=CPU, optimizer=optim, budget_seconds=1.0, dreamworld_enabled=True)


def test_cuda_graph_probe_on_cpu_runs_eagerly_and_says_why():
    res, _ = _run(cuda_graph_mode="probe")
    g = res["cuda_graph"]
    assert res["steps"] == 3 and g["accepted"] is False and g["reasons"]
    res2, _ = _run(cuda_graph_mode="probe", predictive_aux_weight=0.1, predictive_aux_horizon=2, predictive_aux_dim=16)
    assert "auxiliary_loss_not_supported" in res2["cuda_graph"]["reasons"]


def test_loop_kwargs_pass_only_known_keys():
    kw = _loop_kwargs({"chunk_size": 32, "train_sampling_mode": "random", "model_dim": 16, "dreamworld_weight": 0.1,
                       "scopt_split_interval": 8, "name": "x"})
    assert kw == {"chunk_size": 32, "train_sampling_mode": "random", "dreamworld_weight": 0.1, "scopt_split_interval": 8}


# ---------------------------------------------------------------- accounting helpers
def test_token_accounting_counts_training_ranks_only():
    a = FP.summarize_train_timing(steps=10, elapsed_s=2.0, batch_size=8, seq_len=16, world_size=4)
    assert a["tokens_per_step"] == 8 * 16 * 4 and a["aggregate_tokens_per_sec"] == pytest.approx(10 * 512 / 2.0)
    assert a["per_gpu_tokens_per_sec"] == pytest.approx(a["aggregate_tokens_per_sec"] / 4)
    e = FP.summarize_train_timing(steps=10, elapsed_s=2.0, batch_size=8, seq_len=16, world_size=4, episodic_enabled=True)
    assert e["tokens_per_step"] == 8 * 16 * 3 and e["per_gpu_tokens_per_sec"] == pytest.approx(e["aggregate_tokens_per_sec"] / 3)
    one = FP.summarize_train_timing(steps=1, elapsed_s=0.0, batch_size=1, seq_len=1, world_size=1, episodic_enabled=True)
    assert one["tokens_per_step"] == 1 and math.isfinite(one["aggregate_tokens_per_sec"])


def test_stop_rule():
    stop = FP.should_stop_training_loop
    assert stop(steps=0, elapsed_s=1e9, budget_seconds=1.0, stop_margin_seconds=0.0) is False       # always one step
    assert stop(steps=5, elapsed_s=0.0, budget_seconds=100.0, stop_margin_seconds=0.0, max_steps=5) is True
    assert stop(steps=4, elapsed_s=0.0, budget_seconds=100.0, stop_margin_seconds=0.0, max_steps=5) is False
    assert stop(steps=1, elapsed_s=98.0, budget_seconds=100.0, stop_margin_seconds=2.0) is True
    assert stop(steps=1, elapsed_s=97.9, budget_seconds=100.0, stop_margin_seconds=2.0) is False
    assert stop(steps=1, elapsed_s=0.0, budget_seconds=1.0, stop_margin_seconds=5.0) is True          # margin > budget


def test_steady_state_drops_the_first_step():
    assert FP.steady_state_step_seconds([9.0, 1.0, 3.0, 2.0]) == 2.0
    assert FP.steady_state_step_seconds([4.0]) == 4.0
    with pytest.raises(ValueError):
        FP.steady_state_step_seconds([])


def test_graph_gate_charges_capture_to_the_budget():
    ok = FP.summarize_cuda_graph_gate(budget_seconds=600, capture_seconds=5, warmup_seconds=1, warmup_steps=3,
                                      eager_step_seconds=0.010, graph_step_seconds=0.005)
    assert ok["accepted"] and ok["projected_total_speedup"] == pytest.approx((594 / 0.005) / (600 / 0.010) - 1)
    assert ok["break_even_steps"] == pytest.approx(6 / 0.005)
    short = FP.summarize_cuda_graph_gate(budget_seconds=10, capture_seconds=6, warmup_seconds=1, warmup_steps=3,
                                         eager_step_seconds=0.010, graph_step_seconds=0.005)
    assert not short["accepted"] and "projected_speedup_below_minimum" in short["reasons"]
    slow = FP.summarize_cuda_graph_gate(budget_seconds=600, capture_seconds=1, warmup_seconds=1, warmup_steps=3,
                                        eager_step_seconds=0.010, graph_step_seconds=0.010)
    assert not slow["accepted"] and "graph_step_not_faster" in slow["reasons"] and math.isinf(slow["break_even_steps"])
    long = FP.summarize_cuda_graph_gate(budget_seconds=6000, capture_seconds=40, warmup_seconds=1, warmup_steps=3,
                                        eager_step_seconds=0.010, graph_step_seconds=0.001)
    assert not long["accepted"] and "capture_seconds_exceeds_limit" in long["reasons"]
    dead = FP.summarize_cuda_graph_gate(budget_seconds=5, capture_seconds=6, warmup_seconds=0, warmup_steps=0,
                                        eager_step_seconds=0.010, graph_step_seconds=0.005)
    assert "capture_overhead_exhausts_budget" in dead["reasons"]
    bad = FP.summarize_cuda_graph_gate(budget_seconds=0, capture_seconds=0, warmup_seconds=0, warmup_steps=0,
                                       eager_step_seconds=0, graph_step_seconds=0)
    assert {"budget_seconds_must_be_positive", "eager_step_seconds_must_be_positive",
            "graph_step_seconds_must_be_positive"} <= set(bad["reasons"])


def test_predictive_aux_dim_must_match_the_model():
    with pytest.raises(ValueError, match="predictive_aux_dim"):
        _run(predictive_aux_weight=0.1, predictive_aux_horizon=2, predictive_aux_dim=8)


# ---------------------------------------------------------------- optional result blocks
def test_topology_snapshot_only_when_asked():
    res, _ = _run(max_steps=1)
    assert "topology_snapshot" not in res
    res, _ = _run(max_steps=1, emit_topology_snapshot=True)
    snap = res["topology_snapshot"]
    assert isinstance(snap, dict) and all(isinstance(v, str) for v in snap.values())
    assert "lscpu" in snap or snap == {}                                 # whatever query tools this host has


def test_scopt_interval_traces():
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    res, _ = _run(model=model, opt="scopt", max_steps=4, lm_head_backward_mode="fused", scopt_trace_interval_steps=2,
                  scopt_split_interval=2)
    tr = res["scopt"]["interval_traces"]
    assert [t["step"] for t in tr] == [2, 4] and all("scarcity_enabled" in t for t in tr)
    res2, _ = _run(model=CareStudentLM(vocab_size=64, dim=16, num_layers=1), opt="scopt", max_steps=2,
                   lm_head_backward_mode="fused")
    assert "interval_traces" not in res2["scopt"]
