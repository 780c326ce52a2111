"""Warm multi-run worker: idempotence, config check, error isolation (single process and two gloo ranks)."""
import json
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

from chaoscontrol_b200 import runner_persistent_ddp as rp

ROOT = Path(__file__).resolve().parents[1]


def _entries():
    return rp.build_default_matrix(world_size=1, base_lr=0.064, seeds=[0, 1], conditions=["bf16", "fp8"])


def test_matrix_builders_and_launcher_checks(tmp_path):
    e = _entries()
    assert [(x["name"], x["seed"]) for x in e] == [("bf16", 0), ("bf16", 1), ("fp8", 0), ("fp8", 1)]
    assert set(rp.REQUIRED_ENTRY_FIELDS) <= set(e[0]) and rp.config_hash(e[0]) != rp.config_hash(e[1])
    rp.validate_matrix_world_size(e, 1)
    with pytest.raises(ValueError):
        rp.validate_matrix_world_size(e, 8)
    run, skipped = rp.filter_matrix_for_fp8(e, tmp_path, probe=lambda: False)
    assert len(run) == 2 and len(skipped) == 2
    assert rp.filter_matrix_for_fp8(e, tmp_path, probe=lambda: True) == (e, [])
    rp.write_skip_markers(skipped, tmp_path)
    rp.reject_stale_skip_markers(e, tmp_path, probe=lambda: False)
    with pytest.raises(RuntimeError, match="stale skip markers"):
        rp.reject_stale_skip_markers(e, tmp_path, probe=lambda: True)
    rp.write_result_json(tmp_path / "bf16_s0.json", {"config": e[0], "train": {}, "eval": {}})
    rp.write_result_json(tmp_path / "bf16_s1.json", {"config": e[1], "error": "RuntimeError: boom"})
    ok, benign, bad = rp.check_output_integrity(tmp_path, e)
    assert (ok, benign) == (1, 2) and len(bad) == 1 and "boom" in bad[0]
    assert rp.main(["--data-path", "x", "--config-matrix", str(_write(tmp_path, e)), "--output-dir", str(tmp_path),
                    "--dry-run"]) == 0
    with pytest.raises(ValueError, match="missing required fields"):
        rp.main(["--data-path", "x", "--config-matrix", str(_write(tmp_path, [{"name": "a", "seed": 0}])),
                 "--output-dir", str(tmp_path), "--dry-run"])


def _write(d, entries):
    p = d / "matrix.json"
    p.write_text(json.dumps(entries))
    return p


def test_worker_loop_skips_isolates_and_checks_config(tmp_path):
    e = _entries()[:3]
    calls = []

    def fake(*, config, out_path, **kw):
        calls.append(config["name"] + str(config["seed"]))
        if config["seed"] == 1:
            raise RuntimeError("synthetic failure")
        rp.write_result_json(out_path, {"config": config, "train": {"steps": 1}, "eval": {}})

    c = rp.run_matrix_worker(e, output_dir=tmp_path, data_path="d", sp_model_path=None, budget_seconds=1, run_entry=fake)
    assert c == {"completed": 2, "skipped": 0, "errored": 1}
    assert "synthetic failure" in json.loads((tmp_path / "bf16_s1.json").read_text())["error"]
    c2 = rp.run_matrix_worker(e, output_dir=tmp_path, data_path="d", sp_model_path=None, budget_seconds=1, run_entry=fake)
    assert c2 == {"completed": 0, "skipped": 3, "errored": 0} and len(calls) == 3
    edited = [dict(e[0], base_lr=0.5)]
    with pytest.raises(RuntimeError, match="config mismatch"):
        rp.run_matrix_worker(edited, output_dir=tmp_path, data_path="d", sp_model_path=None, budget_seconds=1,
                             run_entry=fake)
    with pytest.raises(ValueError, match="disagree on vocab_size"):
        rp.run_matrix_worker([e[0], dict(e[1], vocab_size=5)], output_dir=tmp_path / "x", data_path="d",
                             sp_model_path=None, budget_seconds=1, run_entry=fake)


def test_warmup_and_restore_returns_model_to_snapshot():
    m = torch.nn.Linear(4, 4)
    before = {k: v.clone() for k, v in m.state_dict().items()}

    def warm():
        opt = torch.optim.SGD(m.parameters(), lr=1.0)
        m(torch.randn(2, 4)).sum().backward()
        opt.step()

    opt = rp.warmup_and_restore(model=m, warmup_call_fn=warm, build_optimizer_fn=lambda: torch.optim.SGD(m.parameters(), lr=0.1),
                                device=torch.device("cpu"), ddp_active=False)
    assert all(torch.equal(before[k], v) for k, v in m.state_dict().items())
    assert all(p.grad is None for p in m.parameters()) and not opt.state


def test_two_rank_error_on_one_rank_skips_entry_on_both(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(f"""
        import json, sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch.distributed as dist
        from pathlib import Path
        from chaoscontrol_b200 import runner_persistent_ddp as rp
        dist.init_process_group("gloo")
        rank = dist.get_rank()
        out = Path({str(tmp_path)!r}) / "out"
        entries = [dict(name="a", seed=0, vocab_size=8), dict(name="b", seed=0, vocab_size=8)]
        def run(*, config, out_path, **kw):
            if config["name"] == "a" and rank == 1:
                raise RuntimeError("rank 1 only")
            if rank == 0:
                rp.write_result_json(out_path, dict(config=config, train=dict(), eval=dict()))
            dist.barrier()
        def run_safe(**kw):
            if kw["config"]["name"] == "a" and rank == 0:
                return          # rank 0 must not wait in a barrier its failing peer never reaches
            return run(**kw)
        c = rp.run_matrix_worker(entries, output_dir=out, data_path="d", sp_model_path=None, budget_seconds=1, run_entry=run_safe)
        (Path({str(tmp_path)!r}) / f"counts{{rank}}.json").write_text(json.dumps(c))
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29631")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29631", str(script)],
                       capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    for rank in range(2):
        assert json.loads((tmp_path / f"counts{rank}.json").read_text()) == {"completed": 1, "skipped": 0, "errored": 1}
    assert json.loads((tmp_path / "out" / "a_s0.json").read_text())["error"] == "peer_rank_error"
