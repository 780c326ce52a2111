"""Thin glue that whole-path tests pass by: study decisions and CLIs, lever gates, config projection, slot picking,
router feedback, criticality bookkeeping, fake quantisation (CPU)."""
import json

import pytest
import torch

from chaoscontrol_b200 import exp18, studies
from chaoscontrol_b200.config import ChaosControlConfig
from chaoscontrol_b200.eval_stream.batched_ttt import pick_slots
from chaoscontrol_b200.models.wernicke import WernickeLayer
from chaoscontrol_b200.optim.criticality import CriticalityDistillation
from chaoscontrol_b200.optim.schedule import _fake_quant_per_tensor_


# ---------------------------------------------------------------- study decisions and CLIs
def _c(delta, sig):
    return {"mean_delta": delta, "significant": sig}


def test_polyphasic_decision_ladder():
    d = studies._decide_polyphasic
    assert d({}) == "no data" and d({"polyphasic_vs_none": _c(-1, True)}) == "no data"
    assert d({"polyphasic_vs_none": _c(-0.1, False), "polyphasic_vs_offline": _c(0, False)}) == "POLYPHASIC NOT HELPFUL YET"
    assert d({"polyphasic_vs_none": _c(0.1, True), "polyphasic_vs_offline": _c(0, False)}) == "POLYPHASIC NOT HELPFUL YET"
    assert d({"polyphasic_vs_none": _c(-0.1, True), "polyphasic_vs_offline": _c(0.05, True)}) == \
        "POLYPHASIC HELPS BUT OFFLINE STILL BETTER"
    assert d({"polyphasic_vs_none": _c(-0.1, True), "polyphasic_vs_offline": _c(0.05, False)}) == "ADOPT POLYPHASIC"


def test_sleep_decision_ladder():
    d = studies._decide_sleep
    assert d({}) == "no data" and d({"sleep_vs_none": _c(-0.1, True)}) == "ADOPT FULL CYCLE"
    assert d({"sleep_vs_none": _c(-0.1, False)}) == "CAUTIOUS ADOPTION" and d({"sleep_vs_none": _c(0.1, True)}) == "SLEEP NOT HELPFUL YET"


def test_studies_cli_prints_matrix_layers_and_scaling(capsys, tmp_path):
    assert studies.main(["exp11_sleep_cycle"]) == 0
    ents = json.loads(capsys.readouterr().out)
    assert isinstance(ents, list) and ents and {"name", "seed"} <= set(ents[0])
    assert studies.main(["exp09_layers"]) == 0
    layers = json.loads(capsys.readouterr().out)
    assert list(layers)[0] == studies.LAYERS[0].tag and all(isinstance(v, list) for v in layers.values())
    assert studies.main(["exp10_scaling"]) == 0
    assert isinstance(json.loads(capsys.readouterr().out), dict)
    assert studies.main(["exp11_sleep_cycle", "--results-dir", str(tmp_path)]) == 0
    assert isinstance(json.loads(capsys.readouterr().out), dict)          # an empty results folder still analyses


# ---------------------------------------------------------------- lever gates
def _rows(**bpb):
    return {c: {"bpb": dict(enumerate(v)), "tps": {}, "loss": {}, "vocab": 16384} for c, v in bpb.items()}


def test_best_bpb_gate_ranks_and_compares_with_the_runner_up():
    g = exp18._gate_best_bpb(_rows(a=[1.50, 1.51, 1.49], b=[1.40, 1.41, 1.42], c=[1.60, 1.61, 1.62]), ["a", "b", "c"])
    assert g["winner"] == "b" and g["winner_vs_runner_up"]["n"] == 3 and g["winner_vs_runner_up"]["delta"] == pytest.approx(0.09)
    assert exp18._gate_best_bpb(_rows(a=[1.5]), ["a"]) == {"winner": "a"}
    assert exp18._gate_best_bpb({}, [])["winner"] is None


def test_beats_first_gate_needs_significance_only_when_asked():
    rows = _rows(base=[1.50, 1.52, 1.51, 1.49], better=[1.40, 1.41, 1.42, 1.40], noisy=[1.30, 1.70, 1.35, 1.69])
    order = ["base", "better", "noisy"]
    strict = exp18._gate_vs_first(rows, order, True)
    assert strict["winner"] == "better" and strict["vs_baseline"]["better"]["p"] < 0.05 and strict["vs_baseline"]["noisy"]["p"] > 0.05
    loose = exp18._gate_vs_first(_rows(base=[1.5, 1.5], lucky=[1.48, 1.51], best=[1.2, 1.9]), ["base", "lucky", "best"], False)
    assert loose["winner"] == "lucky"                                  # lowest mean, no test required
    nothing = exp18._gate_vs_first(_rows(base=[1.5, 1.5, 1.5], worse=[1.6, 1.61, 1.62]), ["base", "worse"], True)
    assert nothing["winner"] == "base"
    assert exp18._gate_vs_first(_rows(x=[1.0]), ["base", "x"], True)["winner"] is None


def test_exp18_cli_dry_run_and_summary(tmp_path, capsys):
    key = sorted(exp18.TESTS)[0]
    assert exp18.main([key, "--results-root", str(tmp_path), "--dry-run", "--base-lr", "0.064"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["entries"] and all(isinstance(c, list) for c in out["commands"])
    assert exp18.main([key, "--results-root", str(tmp_path), "--summarize-only", "--base-lr", "0.064"]) == 0
    s = json.loads(capsys.readouterr().out)
    assert s["_test"]["key"] == key and s["_decision"]["winner"] is None
    with pytest.raises(SystemExit):
        exp18.main([key, "--results-root", str(tmp_path)])              # launching needs a data path


# ---------------------------------------------------------------- config projection
def test_config_from_dict_is_strict_unless_told_otherwise_and_projects_onto_the_model():
    cfg = ChaosControlConfig.from_dict({"data_path": "d", "model_dim": 32, "num_layers": 3, "vocab_size": 100})
    kw = cfg.model_kwargs()
    assert kw["dim"] == 32 and kw["num_layers"] == 3 and kw["vocab_size"] == 100 and "model_dim" not in kw
    with pytest.raises(ValueError, match="unknown config keys"):
        ChaosControlConfig.from_dict({"data_path": "d", "model_dim": 32, "no_such_key": 1})
    assert ChaosControlConfig.from_dict({"data_path": "d", "model_dim": 48, "no_such_key": 1}, strict=False).model_dim == 48
    with pytest.raises(ValueError, match="buffer_mode"):
        ChaosControlConfig.from_dict({"data_path": "d", "buffer_mode": "nonsense"})


def test_config_from_yaml_takes_overrides(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("data_path: shards\nmodel_dim: 24\nnum_layers: 2\n")
    cfg = ChaosControlConfig.from_yaml(p, num_layers=5)
    assert cfg.model_dim == 24 and cfg.num_layers == 5


# ---------------------------------------------------------------- slot picking
def test_slot_count_keeps_the_batch_full_but_bounded():
    assert pick_slots([], 256) == 8 and pick_slots([1, 1], 256) == 8
    assert pick_slots([257] * 1000, 256) == 128                         # many one-chunk documents: the cap
    assert pick_slots([256 * 32 + 1] + [257] * 32, 256) == 8            # one long document dominates: 64 / 32 -> floor
    assert pick_slots([2561] * 20 + [257] * 100, 256) == 32             # (200 + 100) / 10 = 30 -> next multiple of 8
    assert pick_slots([257] * 1000, 256, hi=64) == 64 and pick_slots([300], 256, lo=16) == 16


# ---------------------------------------------------------------- router feedback
@pytest.mark.parametrize("router", ["moe", "vq"])
def test_compression_feedback_only_acts_on_damage(router):
    torch.manual_seed(0)
    w = WernickeLayer(dim=8, k_max=4, router_type=router)
    param = w.router.weight if router == "moe" else w.codebook
    before = param.detach().clone()
    w.compression_consequence_update(1, quality_delta=0.5)
    assert torch.equal(param.detach(), before)                          # an improvement teaches nothing
    w.compression_consequence_update(1, quality_delta=-2.0, lr=0.1)
    changed = (param.detach() != before).any(dim=-1)
    assert changed.tolist() == [False, True, False, False]
    if router == "moe":
        assert torch.allclose(param.detach()[1], before[1] * 1.2)
    else:
        d0 = torch.cdist(before, before)[1]
        d0[1] = float("inf")
        nearest = int(d0.argmin())
        assert (param.detach()[1] - before[nearest]).norm() > (before[1] - before[nearest]).norm()


# ---------------------------------------------------------------- criticality bookkeeping
def _cd():
    return CriticalityDistillation(num_layers=2, dim=3, trace_half_life_steps=2.0)


def test_quiet_baseline_folds_only_event_free_positions():
    cd = _cd()
    fe = torch.tensor([[[1.0, 2.0, 3.0], [100.0, 100.0, 100.0]]])
    mask = torch.tensor([[False, True]])
    cd.update_baseline_ema(layer=0, future_energy=fe, event_mask=mask)
    assert cd.baseline_future_energy[0].tolist() == [1.0, 2.0, 3.0] and bool(cd.baseline_initialized[0]) and not bool(cd.baseline_initialized[1])
    cd.update_baseline_ema(layer=0, future_energy=torch.zeros(1, 2, 3), event_mask=torch.zeros(1, 2, dtype=torch.bool))
    assert cd.baseline_future_energy[0].tolist() == pytest.approx([0.99, 1.98, 2.97])
    cd.update_baseline_ema(layer=1, future_energy=fe, event_mask=torch.ones(1, 2, dtype=torch.bool))
    assert not bool(cd.baseline_initialized[1])                         # nothing quiet: nothing learned
    with pytest.raises(ValueError, match="last dim"):
        cd.update_baseline_ema(layer=0, future_energy=torch.zeros(1, 2, 4), event_mask=mask)


def test_contribution_added_then_expired_leaves_nothing():
    cd = _cd()
    ev = torch.tensor([0.5, 0.25, 0.0])
    cd._add_contribution(layer=1, evidence=ev, event_count=4.0)
    assert cd.score_num[1].tolist() == [2.0, 1.0, 0.0] and float(cd.score_den[1]) == 4.0 and float(cd.event_mass[1]) == 4.0
    assert cd.score_from_accumulators()[1].tolist() == [0.5, 0.25, 0.0] and float(cd.score_from_accumulators()[0].abs().sum()) == 0.0
    cd._step_decay_accumulators(0)
    cd._step_decay_accumulators(2)                                      # one half-life later
    assert float(cd.score_den[1]) == pytest.approx(2.0)
    cd._subtract_expired_contribution(layer=1, evicted_step=0, current_step=2, evicted_evidence=ev, evicted_event_count=4.0)
    assert float(cd.score_den[1]) == pytest.approx(0.0, abs=1e-6) and float(cd.score_num[1].abs().sum()) == pytest.approx(0.0, abs=1e-6)
    cd._step_decay_accumulators(1)                                      # going back in time is ignored
    assert int(cd.last_decay_step) == 2


# ---------------------------------------------------------------- fake quantisation
def test_fake_quant_snaps_to_a_symmetric_grid():
    t = torch.tensor([-1.0, -0.34, 0.0, 0.26, 0.9, 1.0])
    q = t.clone()
    _fake_quant_per_tensor_(q, bits=3)                                   # levels: k / 3 for k in -3..3
    assert torch.allclose(q * 3, (q * 3).round(), atol=1e-6) and float(q.abs().max()) == 1.0
    assert float((q - t).abs().max()) <= 1.0 / 6 + 1e-6
    same = t.clone()
    _fake_quant_per_tensor_(same, bits=0)
    z = torch.zeros(4)
    _fake_quant_per_tensor_(z, bits=4)
    assert torch.equal(same, t) and float(z.abs().sum()) == 0.0
    fine = t.clone()
    _fake_quant_per_tensor_(fine, bits=16)
    assert torch.allclose(fine, t, atol=1e-4)
