"""Calc-type registry and the built-in passes on a tiny synthetic validation cache."""
import math

import pytest
import torch

from chaoscontrol_b200.eval import (calc_type_metadata, dispatch_eval_for_config, evaluate_with_calc_types,
                                    list_registered_calc_types, register_calc_type)
from chaoscontrol_b200.eval_stream import load_val_cache, write_synthetic_val_cache
from chaoscontrol_b200.models.model import CareStudentLM


@pytest.fixture(scope="module")
def setup(tmp_path_factory):
    d = tmp_path_factory.mktemp("vc")
    write_synthetic_val_cache(d, n_docs=6, vocab=64, median_len=24, sigma=0.4, min_len=4, max_len=40, seed=2)
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2), load_val_cache(d)


def test_registry_contents_and_metadata():
    names = list_registered_calc_types()
    assert {"score_only_reset", "carry_state", "adaptive_carry", "dreamworld_eval",
            "packet_online_cache"} <= set(names)
    assert calc_type_metadata("carry_state")["requires_source_order"]
    assert calc_type_metadata("dreamworld_eval")["requires_grad"]
    with pytest.raises(ValueError):
        calc_type_metadata("nope")
    with pytest.raises(ValueError):
        register_calc_type("score_only_reset")(lambda ctx: None)


def test_calc_types_run_and_relate(setup):
    model, vc = setup
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    out = evaluate_with_calc_types(
        model=model, val_cache=vc, device=torch.device("cpu"),
        calc_types=["score_only_reset", "carry_state", "adaptive_carry", "dreamworld_eval",
                    "packet_online_cache"],
        calc_type_configs={"carry_state": {"decay": 0.0}, "score_only_reset": {"chunk_size": 8},
                           "packet_online_cache": {"decay": 0.0},
                           "dreamworld_eval": {"K": 2, "L": 4, "lr": 1e-3},
                           "adaptive_carry": {"horizon_shifts": [-0.5, 0.0, 0.5]}})
    ntok = vc.total_tokens - vc.num_docs
    for name, e in out.items():
        assert e["tokens_scored"] == ntok and e["docs_scored"] == vc.num_docs, name
        assert math.isfinite(e["bpb"]) and e["bpb"] > 0
    # carry with decay 0 is exactly a reset; no memory and no carried state => the cache pass is a reset too
    assert out["carry_state"]["loss"] == pytest.approx(out["score_only_reset"]["loss"], rel=1e-4)
    assert out["packet_online_cache"]["loss"] == pytest.approx(out["score_only_reset"]["loss"], rel=1e-4)
    # exponential weights with eta = 1: the mixture loses at most log(n_experts) in total against its best head
    ac = out["adaptive_carry"]
    assert ac["loss"] <= min(ac["per_head_loss"].values()) + math.log(3) / ntok + 1e-6
    assert sum(ac["winner_counts"].values()) == ntok and abs(sum(ac["final_online_weights"]) - 1) < 1e-9
    # one unshifted head with full carry is the carried-state pass
    one = evaluate_with_calc_types(model=model, val_cache=vc, device=torch.device("cpu"),
                                   calc_types=["adaptive_carry", "carry_state"],
                                   calc_type_configs={"adaptive_carry": {"horizon_shifts": "0.0",
                                                                         "online_episodic_chunk_tokens": 7}})
    assert one["adaptive_carry"]["loss"] == pytest.approx(one["carry_state"]["loss"], rel=1e-4)
    assert one["adaptive_carry"]["final_online_weights"] is None
    for n, p in model.named_parameters():
        assert torch.equal(p, before[n]), n            # dreamworld restored every document
    with pytest.raises(ValueError):
        evaluate_with_calc_types(model=model, val_cache=vc, calc_types=["carry_state"],
                                 device=torch.device("cpu"), source_order_preserved=False)
    with pytest.raises(ValueError):
        evaluate_with_calc_types(model=model, val_cache=vc, calc_types=["bogus"], device=torch.device("cpu"))


def test_dispatch(setup):
    model, vc = setup
    res = dispatch_eval_for_config({"calc_types": ["carry_state", "score_only_reset"]}, model=model,
                                   val_cache=vc, device=torch.device("cpu"))
    assert res["headline_calc_type"] == "score_only_reset" and res["bpb"] == res["calc_types"]["score_only_reset"]["bpb"]
    res2 = dispatch_eval_for_config({"calc_types": ["carry_state"], "headline_calc_type": "carry_state"},
                                    model=model, val_cache=vc, device=torch.device("cpu"))
    assert res2["headline_calc_type"] == "carry_state"
    with pytest.raises(ValueError):
        dispatch_eval_for_config({"calc_types": ["carry_state"], "headline_calc_type": "x"}, model=model,
                                 val_cache=vc, device=torch.device("cpu"))
    with pytest.raises(ValueError):
        dispatch_eval_for_config({"calc_types": ["carry_state"]}, model=model, val_cache=None,
                                 device=torch.device("cpu"))
    legacy = dispatch_eval_for_config({}, model=model, val_cache=None, device=torch.device("cpu"),
                                      legacy_evaluate_fn=lambda m, **kw: {"bpb": 1.0, "loss": 2.0})
    assert legacy == {"bpb": 1.0, "loss": 2.0}


def _memory_model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                         outer_max_slots=0, buffer_mode="append_only")


def test_packet_online_cache_reads_then_writes(setup):
    _, vc = setup
    model = _memory_model()
    run = lambda **cfg: evaluate_with_calc_types(                                       # noqa: E731
        model=model, val_cache=vc, device=torch.device("cpu"), calc_types=["packet_online_cache"],
        calc_type_configs={"packet_online_cache": cfg})["packet_online_cache"]
    ntok = vc.total_tokens - vc.num_docs
    a = run(chunk_tokens=8, write_tokens_per_chunk=2, seeded=False)
    x = a                                           # extras are merged into the result entry
    assert a["tokens_scored"] == ntok and a["docs_scored"] == vc.num_docs
    assert x["slot_count_initial"] == 0 and x["slot_count_final"] == 2 * x["episodic_writes"] > 0
    # the very first chunk has nothing to read; every later chunk (and every document tail) reads
    assert x["episodic_reads"] == x["chunks_scored"] - 1 + vc.num_docs
    # seeded: the store left by the previous pass is read from the first chunk on and keeps growing
    b = run(chunk_tokens=8, write_tokens_per_chunk=2, seeded=True, controller_read_enabled=True, controller_topk_k=3)
    y = b
    assert y["slot_count_initial"] == x["slot_count_final"] and y["slot_count_final"] > y["slot_count_initial"]
    assert y["episodic_reads"] == y["chunks_scored"] + vc.num_docs
    assert y["controller_reads"] == y["episodic_reads"] and y["controller_selected_slots"] == 3 * y["controller_reads"]
    assert b["loss"] != pytest.approx(a["loss"], rel=1e-6)
    # gate 0 switches the residual off entirely; writes still happen
    c = run(chunk_tokens=8, write_tokens_per_chunk=1, gate_value=0.0, seeded=False)
    assert c["episodic_reads"] == 0 and c["episodic_writes"] > 0
    # microbatches of whole documents: one read and one commit per group
    d = run(batch_docs=4, write_tokens_per_chunk=2, seeded=False)
    z = d
    assert d["tokens_scored"] == ntok and z["chunks_scored"] == math.ceil(vc.num_docs / 4)
    assert z["episodic_reads"] == z["chunks_scored"] - 1 and z["slot_count_final"] == 2 * vc.num_docs
    for bad in (dict(chunk_tokens=0), dict(write_tokens_per_chunk=-1), dict(gate_value=-1.0), dict(batch_docs=0),
                dict(controller_read_enabled=True, controller_score_mode="nope")):
        with pytest.raises(ValueError):
            run(**bad)
    # a store that grows between the cue read and the score is refused
    real = model.encode

    def leaky(ids, **kw):
        out = real(ids, **kw)
        model.append_memory_from_hidden(out[0].detach(), max_tokens=1)
        return out
    model.encode = leaky
    try:
        with pytest.raises(RuntimeError, match="score-before-write"):
            run(chunk_tokens=8, seeded=False)
    finally:
        model.encode = real


def test_online_mixer_matches_the_per_token_loop():
    from chaoscontrol_b200.eval.calc_types import _online_mix
    torch.manual_seed(0)
    nll = torch.rand(3, 11, dtype=torch.float64) * 3
    lw = torch.log_softmax(torch.randn(3, dtype=torch.float64), 0)
    mixed, lw_end = _online_mix(nll, lw, eta=0.7)
    w, want = lw.clone(), []
    for t in range(11):
        want.append(-torch.logsumexp(w - nll[:, t], 0))
        w = torch.log_softmax(w - 0.7 * nll[:, t], 0)
    assert torch.allclose(mixed, torch.stack(want)) and torch.allclose(lw_end, w)


def test_dreamworld_eval_modes(setup):
    model, vc = setup
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    run = lambda **cfg: evaluate_with_calc_types(                                       # noqa: E731
        model=model, val_cache=vc, device=torch.device("cpu"), calc_types=["dreamworld_eval"],
        calc_type_configs={"dreamworld_eval": dict(K=2, L=4, lr=0.05, **cfg)})["dreamworld_eval"]
    a, b = run(), run(dream_target_mode="softmax", dream_temperature=0.7, seed=3)
    c = run(per_doc_reset=False)
    assert a["hyperparams"]["dream_target_mode"] == "argmax" and b["hyperparams"]["prefix_len"] == 16
    assert a["loss"] != pytest.approx(b["loss"], rel=1e-9)          # different dreams, different step
    assert c["loss"] != pytest.approx(a["loss"], rel=1e-9)          # adaptation carried across documents
    for n, p in model.named_parameters():
        assert torch.equal(p, before[n]), n                          # both modes leave the weights as found
    with pytest.raises(ValueError):
        run(dream_target_mode="beam")


def test_seeded_versus_empty_store_compare(setup, tmp_path):
    from chaoscontrol_b200.eval.packet_online_cache_compare import run_packet_online_cache_compare
    _, vc = setup
    model = _memory_model()
    # give the model a trained-in store
    with torch.no_grad():
        model.append_memory_from_hidden(torch.randn(1, 6, 16), max_tokens=6)
    n0 = model.outer_model.table.n_active
    out = run_packet_online_cache_compare(model=model, val_cache=vc, device=torch.device("cpu"),
                                          compare_config={"chunk_tokens": 8, "write_tokens_per_chunk": 1},
                                          output_json=tmp_path / "cmp.json")
    assert out["seeded"]["slot_count_initial"] == n0 and out["empty"]["slot_count_initial"] == 0
    assert out["seeded"]["tokens_scored"] == out["empty"]["tokens_scored"]
    assert out["delta_bpb"] == pytest.approx(out["empty"]["bpb"] - out["seeded"]["bpb"])
    assert (tmp_path / "cmp.json").exists() and out["compare_type"] == "packet_online_cache"


def test_seeded_versus_empty_compare_command_line(setup, tmp_path, monkeypatch, capsys):
    import json
    from chaoscontrol_b200.eval import packet_online_cache_compare as P
    _, vc = setup
    seen = {}

    def fake(**kw):
        seen.update(kw)
        return P.run_packet_online_cache_compare(model=_memory_model(), val_cache=vc, device=torch.device("cpu"),
                                                 compare_config=kw["compare_config"], output_json=kw["output_json"])
    monkeypatch.setattr(P, "load_and_run_packet_online_cache_compare", fake)
    assert P.main(["--artifact-path", "a.ccb", "--val-cache-dir", "vc", "--output-json", str(tmp_path / "o.json"),
                   "--device", "cpu", "--chunk-tokens", "8", "--write-tokens-per-chunk", "1", "--decay", "0.9"]) == 0
    assert seen["compare_config"] == {"chunk_tokens": 8, "write_tokens_per_chunk": 1, "gate_value": 1.0, "decay": 0.9}
    printed = json.loads(capsys.readouterr().out)
    assert printed["compare_type"] == "packet_online_cache" and json.loads((tmp_path / "o.json").read_text())["delta_bpb"] == printed["delta_bpb"]
