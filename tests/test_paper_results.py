import json

import pytest

from chaoscontrol_b200 import paper_results as pr


def test_registry_round_trip_query_verify(tmp_path, capsys):
    reg = tmp_path / "p" / "registry.jsonl"
    kw = dict(registry_path=reg, git_sha="abc", git_dirty=False, config_hash="h1")
    a = pr.register(experiment="e1", condition="c", seed=0, status="confirmatory", metrics={"bpb": 1.5}, **kw)
    pr.register(experiment="e1", condition="c", seed=1, status="exploratory", metrics={"bpb": 1.6},
                artifacts=["x.json"], extras={"note": "n"}, **kw)
    pr.register(experiment="e2", condition="d", seed=0, status="exploratory", metrics={}, registry_path=reg,
                git_sha="abc", git_dirty=True, config_hash="h2")
    assert a.timestamp.endswith("Z") and a.key() == ("e1", "c", 0, "confirmatory")
    assert [r.seed for r in pr.query(experiment="e1", registry_path=reg)] == [0, 1]
    assert len(pr.query(status="exploratory", registry_path=reg)) == 2
    s = pr.verify(reg)
    assert s == {"n_records": 3, "experiments": ["e1", "e2"], "confirmatory": 1, "exploratory": 2, "dirty_records": 1}
    with pytest.raises(ValueError):
        pr.RunRecord("e", "c", 0, "final", {}, "h")
    pr.register(experiment="e1", condition="c", seed=0, status="confirmatory", metrics={}, **kw)
    with pytest.raises(ValueError, match="duplicate"):
        pr.verify(reg)
    reg2 = tmp_path / "r2.jsonl"
    pr.register(experiment="e", condition="c", seed=0, status="confirmatory", metrics={}, config_hash="h",
                registry_path=reg2, git_sha="s", git_dirty=True)
    with pytest.raises(ValueError, match="dirty"):
        pr.verify(reg2)
    reg2.write_text("{not json\n")
    with pytest.raises(ValueError, match="invalid JSON"):
        pr.load(reg2)
    assert pr.load(tmp_path / "none.jsonl") == []
    assert pr.main(["--registry", str(reg2), "verify"]) == 1
    reg3 = tmp_path / "r3.jsonl"
    assert pr.main(["--registry", str(reg3), "register", "--experiment", "e", "--condition", "c", "--status",
                    "exploratory", "--config-hash", "h", "--seed", "3", "--metrics", '{"a": 1}']) == 0
    assert pr.main(["--registry", str(reg3), "list", "--experiment", "e"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["seed"] == 3


def test_canonical_configs(tmp_path):
    p = tmp_path / "canon.json"
    assert pr.load_canonical_configs(p) == {}
    p.write_text(json.dumps({"canonical": {"h1": {"experiment": "e", "condition": "c", "rationale": "r", "lineage": []}}}))
    assert pr.is_canonical(config_hash="h1", experiment="e", condition="c", path=p)
    assert not pr.is_canonical(config_hash="h1", experiment="e", condition="other", path=p)
    assert not pr.is_canonical(config_hash="zz", experiment="e", condition="c", path=p)
