"""Production runner end to end on CPU (tiny model, synthetic shards), the training
hooks, and the launch helpers."""
import json

import numpy as np
import pytest
import torch

from chaoscontrol_b200 import launch
from chaoscontrol_b200 import training_hooks as TH
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.utils.arena import ParamArena
from chaoscontrol_b200.runner_fast_path import run_condition, train_fast_for_budget, _build_optimizer


def _shards(tmp_path, vocab=64, n=20000):
    rng = np.random.default_rng(0)
    rng.integers(0, vocab, n, dtype=np.uint16).tofile(tmp_path / "fineweb_train_000.bin")
    rng.integers(0, vocab, n // 4, dtype=np.uint16).tofile(tmp_path / "fineweb_val_000.bin")


def _config(**kw):
    cfg = dict(name="tiny", vocab_size=64, model_dim=16, num_layers=2, ff_mult=2, seq_len=16, stride=8, batch_size=4,
               dtype="fp32", precision="fp32", device="cpu", optimizer="muon", base_lr=0.02, warmup_steps=2,
               restore_after_warmup=True, max_steps=6, eval_batches=2, lm_head_backward_mode="fused",
               stop_check_interval=2, fast_slow_enabled=True, fast_slow_interval=2, fast_slow_alpha=0.5,
               weight_ema_decay=0.9, seed=3)
    cfg.update(kw)
    return cfg


class _FakeSP:
    """Four control tokens, byte tokens, then pieces (some with the leading-space marker)."""

    def vocab_size(self):
        return 64

    def is_control(self, t):
        return t < 2

    def is_unknown(self, t):
        return t == 2

    def is_unused(self, t):
        return t == 3

    def is_byte(self, t):
        return 4 <= t < 10

    def id_to_piece(self, t):
        return ("▁" if t % 2 else "") + "ab"[: 1 + t % 2]


def test_sentencepiece_luts_and_byte_counts():
    from chaoscontrol_b200.sp_eval import build_sentencepiece_luts, token_byte_counts
    base, lead, boundary = build_sentencepiece_luts(_FakeSP(), 70, "cpu")
    assert base.shape == (70,) and boundary[:4].all() and not boundary[4:64].any() and boundary[64:].all()
    assert base[5] == 1 and base[11] == 2 and lead[11] and base[12] == 1 and not lead[12]
    prev = torch.tensor([0, 12, 12])
    tgt = torch.tensor([11, 11, 12])
    # leading space counts unless the previous token is a boundary token
    assert token_byte_counts(prev, tgt, base, lead, boundary).tolist() == [2, 3, 1]


def test_run_condition_cpu_end_to_end(tmp_path, monkeypatch):
    _shards(tmp_path)
    import chaoscontrol_b200.runner_fast_path as R
    import sys
    import types
    fake = types.ModuleType("sentencepiece")

    class _Proc(_FakeSP):
        def Load(self, path):
            return True
    fake.SentencePieceProcessor = _Proc
    monkeypatch.setitem(sys.modules, "sentencepiece", fake)
    out_json, out_ckpt = tmp_path / "res" / "tiny.json", tmp_path / "res" / "tiny.pt"
    res = run_condition(_config(), data_path=str(tmp_path), sp_model_path="fake.model", budget_seconds=30.0,
                        output_json=str(out_json), output_ckpt=str(out_ckpt), world_size_override=None)
    tr = res["train"]
    assert tr["steps"] == 6 and len(tr["loss_history"]) == 6 and np.isfinite(tr["final_loss"])
    assert tr["tokens_per_step"] == 64 and tr["aggregate_tokens_per_sec"] > 0
    assert tr["fast_slow"]["sync_count"] == 3 and tr["spectral"]["log_a_param_count"] == 2
    assert 0 < res["eval"]["bpb"] < 20 and res["eval"]["tokens"] == 2 * 4 * 16
    saved = json.loads(out_json.read_text())
    assert saved["params"] == res["params"] and saved["artifact"]["artifact_bytes_estimate"] == 2 * res["params"]
    ck = torch.load(out_ckpt, weights_only=False)
    m = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    m.load_state_dict(ck["model"])
    # eval-only pass from that checkpoint reproduces the evaluation
    ev = run_condition(_config(eval_only=True, checkpoint_path=str(out_ckpt), fast_slow_enabled=False),
                       data_path=str(tmp_path), sp_model_path="fake.model", budget_seconds=1.0, output_json=None,
                       output_ckpt=None, world_size_override=None)
    assert ev["train"]["steps"] == 0 and np.isfinite(ev["eval"]["bpb"])
    epi_ckpt = tmp_path / "epi.pt"
    epi = run_condition(_config(episodic_enabled=True, warmup_steps=0, episodic_capacity=64, episodic_writes_per_step=4,
                                episodic_fingerprint_window=2, fast_slow_enabled=False, weight_ema_decay=0.0,
                                eval_batches=0),
                        data_path=str(tmp_path), sp_model_path=None, budget_seconds=60.0, output_json=None,
                        output_ckpt=str(epi_ckpt), world_size_override=None)
    e = epi["train"]["episodic"]
    assert e["role"] == "solo" and e["write_events_ingested"] > 0 and e["cache_entries"] > 0 and e["replays"] > 0
    assert "episodic_cache" in torch.load(epi_ckpt, weights_only=False)
    with pytest.raises(ValueError):                                 # the teacher needs an episodic store
        run_condition(_config(crct_enabled=True, warmup_steps=0), data_path=str(tmp_path), sp_model_path=None,
                      budget_seconds=1.0, output_json=None, output_ckpt=None, world_size_override=None)
    mem = run_condition(_config(crct_enabled=True, replay_eviction_enabled=True, warmup_steps=1, outer_model_dim=8,
                                outer_model_type="multislot", outer_max_slots=0, buffer_mode="append_only",
                                crct_memory_write_tokens_per_step=4, fast_slow_enabled=False, weight_ema_decay=0.0),
                        data_path=str(tmp_path), sp_model_path="fake.model", budget_seconds=60.0, output_json=None,
                        output_ckpt=None, world_size_override=None)
    assert mem["train"]["steps"] == 6 and mem["train"]["crct"]["teacher_payloads"] == 6
    assert mem["train"]["crct"]["transport_mode"] == "inline" and np.isfinite(mem["eval"]["bpb"])
    with pytest.raises(ValueError):
        run_condition(_config(), data_path=str(tmp_path), sp_model_path=None, budget_seconds=1.0, output_json=None,
                      output_ckpt=None, world_size_override=4)


@pytest.mark.parametrize("mode,opt", [("sequential_epoch", "adamw"), ("shuffled_epoch", "lamb")])
def test_train_loop_epoch_modes_stop_after_one_epoch(tmp_path, mode, opt):
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (600,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    optim = _build_optimizer(dict(optimizer=opt, base_lr=1e-3), model)
    res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=600, stride=8, seq_len=16, batch_size=8,
                                device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0, precision="fp32",
                                stop_check_interval=1, train_sampling_mode=mode, lm_head_backward_mode="chunked",
                                prefetch_batches=False)
    assert res["steps"] == 10                       # ceil(73 starts / 8)
    with pytest.raises(ValueError):
        train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=600, stride=8, seq_len=16, batch_size=8,
                              device=torch.device("cpu"), optimizer=optim, budget_seconds=1.0,
                              train_sampling_mode="nope")


class _Heads:
    def __init__(self):
        self.rewards, self.credits = [], []

    def readiness(self, head):
        return 1.0

    def scalar_value(self, *, head_name, gpu_step, fallback, reward_context):
        return 0.5 if head_name == "consolidation" else 0.4

    def record_credit_assignment(self, **kw):
        self.credits.append(kw)

    def apply_reward(self, *, key, reward, gpu_step, reward_context):
        self.rewards.append((key, reward))
        return 1


def test_fast_slow_consolidator_interval_learned_and_eval_copy():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=8, num_layers=1)
    c = TH.FastSlowConsolidator.from_config(m, dict(fast_slow_enabled=True, fast_slow_interval=2, fast_slow_alpha=0.25))
    w0 = m.embed.weight.detach().clone()
    with torch.no_grad():
        m.embed.weight.add_(1.0)
    assert c.after_optimizer_step(m, step=1).mode == "hold" and not c.should_copy_slow_to_model_for_eval()
    d = c.after_optimizer_step(m, step=2)
    assert d.mode == "interval" and d.accepted
    assert torch.allclose(c.slow_state["embed.weight"], w0 + 0.25)
    heads = _Heads()
    d = c.after_optimizer_step(m, step=3, action_space=heads, loss_value=2.0)
    assert d.mode == "learned" and d.effective_alpha == pytest.approx(0.2) and heads.credits[0]["key"] == 3
    c.after_optimizer_step(m, step=4, action_space=heads, loss_value=1.5)
    assert heads.rewards == [(3, 0.5)] and c.last_reward == 0.5
    diag = c.diagnostics(m)
    assert diag["sync_count"] == 3 and diag["learned_sync_count"] == 2 and diag["fast_slow_l2"] > 0
    c.copy_slow_to_model(m)
    assert c.diagnostics(m)["fast_slow_l2"] == pytest.approx(0.0, abs=1e-6)
    rt = TH.fast_slow_decision_from_dict(TH.fast_slow_decision_to_dict(d))
    assert rt == d and TH.fast_slow_decision_from_dict("x") is None
    off = TH.FastSlowConsolidator.from_config(m, {})
    assert off.after_optimizer_step(m, step=2).mode == "disabled"


def test_spectral_predictive_and_freeze_hooks():
    m = CareStudentLM(vocab_size=32, dim=8, num_layers=2)
    with torch.no_grad():
        m.layers[0].core.log_a.fill_(-6.0)            # a ~ 0.0025: dead
        m.layers[1].core.log_a.fill_(6.0)             # a ~ 0.9975: sticky
    loss = TH.spectral_regularization_loss(m, 1.0, 2.0, 0.05, 0.95)
    a0, a1 = torch.sigmoid(torch.tensor(-6.0)), torch.sigmoid(torch.tensor(6.0))
    assert float(loss.detach()) == pytest.approx(float(((0.05 - a0) ** 2 + 2 * (a1 - 0.95) ** 2) / 2), rel=1e-5)
    s = TH.spectral_summary(m)
    assert s["log_a_param_count"] == 2 and s["a_min"] < 0.01 < 0.99 < s["a_max"]
    h = torch.randn(2, 10, 8)
    proj = torch.nn.Linear(8, 8)
    assert TH.predictive_auxiliary_loss(h, projection=proj, horizon=3) > 0
    assert TH.predictive_auxiliary_loss(h, projection=proj, horizon=10) is None
    m.embed.weight.grad = torch.ones_like(m.embed.weight)
    TH.zero_embedding_grad_until(m, step=5, freeze_steps=5)
    assert m.embed.weight.grad.sum() > 0
    TH.zero_embedding_grad_until(m, step=4, freeze_steps=5)
    assert m.embed.weight.grad.sum() == 0


def test_launch_helpers(tmp_path):
    cmd = launch.build_torchrun_cmd(config_path=tmp_path / "c.yaml", data_path="/d", sp_model_path="/sp",
                                    output_json=tmp_path / "o.json", world_size=8, dry_run=True, budget_seconds=90,
                                    output_ckpt=tmp_path / "o.pt", val_cache_dir="/vc")
    assert cmd[1:3] == ["-m", "torch.distributed.run"] and "--nproc-per-node=8" in cmd and "127.0.0.1" in cmd
    assert cmd[cmd.index("--master-port") + 1] == "0" and "-m" in cmd[3:] and "--val-cache-dir" in cmd
    p = launch.write_entry_config({"name": "e1", "batch_size": 4}, tmp_path / "cfg")
    assert p.name == "e1.yaml"
    (tmp_path / "r").mkdir()
    (tmp_path / "r" / "a.json").write_text(json.dumps({"config": {"name": "a"}, "train": {
        "aggregate_tokens_per_sec": 5.0, "steps": 3, "final_loss": 1.0}, "eval": {"bpb": 1.5}}))
    (tmp_path / "r" / "b.json").write_text(json.dumps({"config": {"name": "b"}, "train": {
        "aggregate_tokens_per_sec": 9.0, "steps": 3, "final_loss": 1.0}}))
    (tmp_path / "r" / "c.json").write_text(json.dumps({"config": {"name": "c"}, "error": "boom"}))
    s = launch.summarize_result_dir(tmp_path / "r")
    assert [r["name"] for r in s["ranked"]] == ["b", "a"] and s["errors"] == [{"name": "c", "error": "boom"}]
    dry = launch.run_matrix([{"name": "x", "budget_seconds": 5}], results_dir=tmp_path / "m", data_path="/d",
                            sp_model_path=None, world_size=2, dry_run=True)
    assert len(dry["commands"]) == 1 and (tmp_path / "m" / "configs" / "x.yaml").exists()
    assert 1024 < launch.pick_free_port() < 65536


def test_cuda_graph_probe_is_rejected_with_reasons_on_cpu():
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (600,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=600, stride=8, seq_len=16, batch_size=8,
                                device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0, precision="fp32",
                                max_steps=3, lm_head_backward_mode="chunked", cuda_graph_mode="probe",
                                prefetch_batches=False)
    assert res["steps"] == 3
    g = res["cuda_graph"]
    assert g["accepted"] is False and g["mode"] == "probe"
    assert "cuda_required" in g["reasons"] and "fused_lm_head_required" in g["reasons"]
    with pytest.raises(ValueError):
        train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=600, stride=8, seq_len=16, batch_size=8,
                              device=torch.device("cpu"), optimizer=optim, budget_seconds=1.0,
                              cuda_graph_mode="always", prefetch_batches=False)


@pytest.mark.gpu
def test_cuda_graph_loop_matches_eager_trajectory():
    """Same seed, same batches: the replayed step gives the eager loop's losses."""
    dev = torch.device("cuda:0")
    tokens = torch.randint(0, 512, (1 << 18,), dtype=torch.int16, generator=torch.Generator().manual_seed(1))

    def run(mode):
        torch.manual_seed(0)
        model = CareStudentLM(vocab_size=512, dim=256, num_layers=2).to(dev).to(torch.bfloat16)
        ParamArena.install(model)
        optim = _build_optimizer(dict(optimizer="muon", base_lr=0.02), model)
        return train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=tokens.numel(), stride=64,
                                     seq_len=256, batch_size=16, device=dev, optimizer=optim, budget_seconds=600.0,
                                     precision="bf16", max_steps=12, stop_check_interval=1, seed=5,
                                     lm_head_backward_mode="fused_streaming_cached", cuda_graph_mode=mode,
                                     cuda_graph_warmup_steps=3, vocab_size=512)

    eager, graph = run("none"), run("probe")
    assert graph["steps"] == 12 and eager["steps"] == 12
    g = graph["cuda_graph"]
    assert g["replay_steps"] == 8 and g["optimizer_step_captured"] is False
    a, b = torch.tensor(eager["loss_history"]), torch.tensor(graph["loss_history"])
    assert a.shape == b.shape and torch.allclose(a, b, atol=2e-2, rtol=0), (a, b)
    assert b[-1] < b[0]


def test_dreamworld_replay_and_event_sleep_in_the_loop():
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    kw = dict(train_tokens=tokens, train_num_tokens=4000, stride=8, seq_len=16, batch_size=4,
              device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0, precision="fp32",
              stop_check_interval=1, lm_head_backward_mode="fused", prefetch_batches=False, max_steps=12)
    res = train_fast_for_budget(model, dreamworld_enabled=True, dreamworld_cache_interval=2, dreamworld_interval=3,
                                dreamworld_weight=0.5, dreamworld_prefix_tokens=4, dreamworld_replay_tokens=4,
                                dreamworld_replay_batch_size=2, dreamworld_min_size=2, event_sleep_enabled=True,
                                event_sleep_loss_ratio=0.0, event_sleep_pressure_threshold=0.0,
                                event_sleep_warmup_steps=2, event_sleep_min_interval=4, event_sleep_weight=0.25, **kw)
    d = res["dreamworld"]
    assert res["steps"] == 12 and d["buffer"]["add_count"] == 6
    ev = d["event_sleep"]
    # the ratio threshold of zero fires on every decision; the minimum interval spaces the replays
    assert ev["decision_count"] >= 8 and 2 <= ev["replay_count"] <= 3 and ev["trigger_count"] == ev["replay_count"]
    assert d["replays"] >= ev["replay_count"] and ev["last_decision"]["triggered"] is True
    assert all(v == v for v in res["loss_history"])
    with pytest.raises(ValueError):
        train_fast_for_budget(model, event_sleep_enabled=True, **kw)


def _aux_run(**mech):
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    with torch.no_grad():
        for _, log_a in TH.iter_log_a_params(model):
            log_a.fill_(6.0)                          # a = sigmoid(6) = 0.9975: "sticky" channels
    optim = torch.optim.SGD(model.parameters(), lr=0.5)
    res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, stride=8, seq_len=16,
                                batch_size=4, device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0,
                                precision="fp32", stop_check_interval=1, lm_head_backward_mode="fused",
                                prefetch_batches=False, max_steps=8, grad_clip_norm=0.0, **mech)
    return model, res


def test_spectral_and_predictive_aux_losses_act_in_the_loop():
    base, res0 = _aux_run()
    spec, res1 = _aux_run(spectral_reg_lambda_sticky=1e4, spectral_reg_max_a=0.9)
    a0 = torch.cat([torch.sigmoid(p).reshape(-1) for _, p in TH.iter_log_a_params(base)])
    a1 = torch.cat([torch.sigmoid(p).reshape(-1) for _, p in TH.iter_log_a_params(spec)])
    assert res1["spectral"]["regularized_steps"] == 8 and "regularized_steps" not in res0["spectral"]
    assert a1.mean() < a0.mean() - 1e-4                 # the hinge pulls the decay back under max_a
    # identical data and seed: the predictive loss reaches the trunk through the second encoder pass
    pred, res2 = _aux_run(predictive_aux_weight=5.0, predictive_aux_horizon=2)
    assert res2["predictive_aux"]["steps"] == 8 and res2["predictive_aux"]["projection_norm"] > 0
    assert not torch.allclose(pred.embed.weight, base.embed.weight)
    assert torch.allclose(_aux_run()[0].embed.weight, base.embed.weight)          # the harness is deterministic
    with pytest.raises(ValueError, match="predictive_aux_dim"):
        _aux_run(predictive_aux_weight=1.0, predictive_aux_horizon=2, predictive_aux_dim=7)
    with pytest.raises(ValueError, match="predictive_aux_weight"):
        _aux_run(predictive_aux_weight=1.0, predictive_aux_horizon=2, crct_enabled=True)


@pytest.mark.gpu
def test_aux_losses_on_the_kernel_engine_path():
    """With the flat arena installed the main gradients come from the kernel engine; the auxiliary
    losses add theirs through autograd and must end up in the same flat buffer."""
    dev = torch.device("cuda:0")
    tokens = torch.randint(0, 512, (1 << 18,), dtype=torch.int16, generator=torch.Generator().manual_seed(1))

    def run(**mech):
        torch.manual_seed(0)
        model = CareStudentLM(vocab_size=512, dim=256, num_layers=2).to(dev).to(torch.bfloat16)
        with torch.no_grad():
            for _, log_a in TH.iter_log_a_params(model):
                log_a.fill_(6.0)
        ParamArena.install(model)
        optim = _build_optimizer(dict(optimizer="muon", base_lr=0.02), model)
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=tokens.numel(), stride=64,
                                    seq_len=256, batch_size=16, device=dev, optimizer=optim, budget_seconds=600.0,
                                    precision="bf16", max_steps=8, stop_check_interval=1, seed=5,
                                    lm_head_backward_mode="fused_streaming_cached", vocab_size=512, **mech)
        a = torch.cat([torch.sigmoid(p.float()).reshape(-1) for _, p in TH.iter_log_a_params(model)])
        return res, a.mean().item(), model.embed.weight.detach().float().clone()

    r0, a0, e0 = run()
    r1, a1, _ = run(spectral_reg_lambda_sticky=1e5, spectral_reg_max_a=0.9)
    r2, _, e2 = run(predictive_aux_weight=5.0, predictive_aux_horizon=4)
    assert r1["spectral"]["regularized_steps"] == 8 and a1 < a0 - 1e-4
    assert r2["predictive_aux"]["steps"] == 8 and not torch.allclose(e2, e0)
    assert all(v == v for v in r1["loss_history"] + r2["loss_history"])


def test_loss_triggered_replay_gate():
    from chaoscontrol_b200.dreamworld import LossTriggeredReplayEMA
    g = LossTriggeredReplayEMA(decay=0.5, warmup_steps=2)
    assert g.update(torch.tensor(2.0)) is None and g.update(torch.tensor(2.0)) is None
    calm = g.update(torch.tensor(2.0), threshold=1.1, pressure_threshold=0.05)
    assert calm.ready() and not calm.triggered and calm.fire_count == 0 and abs(calm.local_ratio - 1.0) < 1e-6
    spike = g.update(torch.tensor(3.0), threshold=1.1, pressure_threshold=0.05)
    assert spike.triggered and spike.local_fire and abs(spike.local_pressure - 0.4) < 1e-6
    assert abs(spike.ema_loss - 2.0) < 1e-6 and abs(float(g.value) - 2.5) < 1e-6
    with pytest.raises(ValueError):
        LossTriggeredReplayEMA(decay=1.0)


def test_criticality_distillation_hook_in_the_loop():
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    cfg = dict(criticality_distill_enabled=True, criticality_distill_num_layers=2, criticality_distill_dim=16,
               criticality_distill_seat_refresh_interval=2, criticality_distill_min_weighted_events_per_layer=0.0,
               criticality_distill_horizon_H=2, criticality_distill_event_frac=0.25, criticality_distill_weight=1.0,
               criticality_distill_trace_ttl_steps=16)
    hook = TH.CriticalityDistillHook.from_config(model, cfg)
    assert TH.CriticalityDistillHook.from_config(model, {}) is None
    with pytest.raises(ValueError):
        TH.CriticalityDistillHook.from_config(model, dict(criticality_distill_enabled=True))
    with pytest.raises(ValueError):
        TH.CriticalityDistillHook.from_config(model, dict(cfg, criticality_distill_num_layers=3))
    kw = dict(train_tokens=tokens, train_num_tokens=4000, stride=8, seq_len=16, batch_size=4,
              device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0, precision="fp32",
              stop_check_interval=1, lm_head_backward_mode="fused", prefetch_batches=False, max_steps=8)
    res = train_fast_for_budget(model, criticality=hook, **kw)
    d = res["criticality_distillation"]
    k = max(1, round(16 * 0.15))
    assert d["ingests"] == 8 and d["seat_refreshes"] == 3 and d["seats"] == 2 * k
    assert len(d["loss_trajectory"]) >= 5 and all(t["cd_loss"] > 0 for t in d["loss_trajectory"])
    assert len(d["snapshots"]) == 3
    # the loss only touches log_a of seated channels
    model.zero_grad(set_to_none=True)
    hook.cd.criticality_loss([c.log_a for c in hook.cores]).backward()
    g = model.layers[0].core.log_a.grad
    assert int((g != 0).sum()) == k and model.lm_head.weight.grad is None
    with pytest.raises(ValueError):
        train_fast_for_budget(model, criticality=hook, world_size=2, **kw)


def test_token_buckets_and_per_bucket_val_ce(tmp_path):
    from chaoscontrol_b200 import fast_path as FP
    freq = torch.tensor([0, 1, 10, 100, 1000, 10000])
    b = FP.build_token_buckets(freq, 3)
    assert b.tolist() == sorted(b.tolist()) and b[0] == 0 and b[-1] == 2
    with pytest.raises(ValueError):
        FP.build_token_buckets(freq.reshape(2, 3), 3)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    val = torch.randint(0, 64, (600,), dtype=torch.int16)
    freq = torch.bincount(val.long(), minlength=64)
    out = FP.compute_per_bucket_val_ce(model=model, device=torch.device("cpu"), tokens=val, num_tokens=600, seq_len=16,
                                       stride=8, batch_size=8, vocab_size=64, token_frequencies=freq, num_buckets=4,
                                       precision="fp32")
    n_steps = -(-FP.count_lm_starts(600, 16, 8) // 8)
    assert sum(out["val_bucket_token_counts"]) == n_steps * 8 * 16
    assert len(out["per_window_bucket_ce_sum"]) == n_steps
    # weighted mean of the bucket means is the plain mean CE over the same windows
    xs, ys = [], []
    for step in range(n_steps):
        st = FP.sequential_sharded_lm_starts(num_tokens=600, seq_len=16, stride=8, batch_size=8, rank=0,
                                             world_size=1, step=step)
        a, b2 = FP.batch_from_start_tensor(tokens=val, starts=st, seq_len=16, device=torch.device("cpu"),
                                           vocab_size=64)
        xs.append(a)
        ys.append(b2)
    x, y = torch.cat(xs), torch.cat(ys)
    with torch.no_grad():
        logits = model.lm_head(model.final_norm(model.encode(x.to(torch.int32))))
        ce = torch.nn.functional.cross_entropy(logits.reshape(-1, 64), y.reshape(-1).long())
    cnt = torch.tensor(out["val_bucket_token_counts"], dtype=torch.float64)
    mean = (torch.tensor(out["per_bucket_val_ce"], dtype=torch.float64) * cnt).sum() / cnt.sum()
    assert abs(float(mean) - float(ce)) < 1e-4
    assert abs(out["rare_bucket_val_ce"] - out["per_bucket_val_ce"][0]) < 1e-12
    _shards(tmp_path)
    res = run_condition(_config(rare_bucket_ce_enabled=True, rare_bucket_ce_max_batches=3, warmup_steps=0,
                                fast_slow_enabled=False, eval_batches=0),
                        data_path=str(tmp_path), sp_model_path=None, budget_seconds=60.0, output_json=None,
                        output_ckpt=None, world_size_override=None)
    assert len(res["train"]["per_bucket_val_ce"]) == 4 and res["train"]["val_bucket_num_buckets"] == 4
