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
                           "dreamworld_eval": {"K": 2, "L": 4, "lr": 1e-3},
                           "adaptive_carry": {"decays": [0.0, 1.0]}})
    ntok = vc.total_tokens - vc.num_docs
    for name, e in out.items():
        assert e["tokens_scored"] == ntok and e["docs_scored"] == vc.num_docs, name
        assert math.isfinite(e["bpb"]) and e["bpb"] > 0
    # carry with decay 0 is exactly a reset; no memory => the cache pass is a reset too
    assert out["carry_state"]["loss"] == pytest.approx(out["score_only_reset"]["loss"], rel=1e-4)
    assert out["packet_online_cache"]["loss"] == pytest.approx(out["score_only_reset"]["loss"], rel=1e-4)
    # the mixture can only lose log(n_experts) per document against its best expert
    assert out["adaptive_carry"]["loss"] <= out["score_only_reset"]["loss"] + math.log(2) * vc.num_docs / ntok + 1e-6
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
