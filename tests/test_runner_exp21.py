"""Lean runner with the model-type switch and the constructor-kwargs checkpoint."""
import json
import sys
import types

import numpy as np
import pytest
import torch

from chaoscontrol_b200 import runner_exp21 as R
from chaoscontrol_b200.baselines_nanogpt_lean import NanoGPTLeanLM
from chaoscontrol_b200.models.model import CareStudentLM
from tests.test_runner_fast_path import _FakeSP, _shards


def _cfg(**kw):
    cfg = dict(vocab_size=64, model_dim=16, num_layers=2, ff_mult=2, seq_len=16, stride=8, batch_size=4, dtype="fp32",
               precision="fp32", device="cpu", optimizer="muon", base_lr=0.02, eval_batches=2, seed=1, chunk_size=8)
    cfg.update(kw)
    return cfg


def test_constructor_kwargs_and_build():
    kw = R.constructor_kwargs(_cfg())
    assert kw["dim"] == 16 and kw["outer_model_dim"] == 0
    assert isinstance(R.build_model(_cfg(), torch.device("cpu"), torch.float32), CareStudentLM)
    tk = R.constructor_kwargs(_cfg(model_type="transformer_nanogpt_lean", model_dim=128))
    assert tk == dict(vocab_size=64, d_model=128, n_head=2, n_layer=2, ffn_mult=2, activation_checkpoint=False)
    assert isinstance(R.build_model(_cfg(model_type="transformer_nanogpt_lean", model_dim=64), torch.device("cpu"),
                                    torch.float32), NanoGPTLeanLM)
    crct = R.constructor_kwargs(_cfg(crct_enabled=True))
    assert crct["outer_model_dim"] == 64 and crct["buffer_mode"] == "append_only" and crct["outer_max_slots"] == 4096
    for bad in (dict(outer_model_dim=0), dict(buffer_mode="legacy"), dict(outer_model_type="single")):
        with pytest.raises(ValueError):
            R.constructor_kwargs(_cfg(crct_enabled=True, **bad))
    assert R.shard_train_starts(list(range(10)), rank=1, world_size=4) == [1, 5, 9]
    with pytest.raises(RuntimeError):
        R.shard_train_starts([0], rank=1, world_size=2)
    with pytest.raises(ValueError):
        R.build_optimizer("sgd", torch.nn.Linear(2, 2), base_lr=0.1, weight_decay=0.0)


def test_run_ddp_cpu_with_embed_init_and_checkpoint(tmp_path, monkeypatch):
    _shards(tmp_path)
    fake = types.ModuleType("sentencepiece")

    class _Proc(_FakeSP):
        def Load(self, path):
            return True
    fake.SentencePieceProcessor = _Proc
    monkeypatch.setitem(sys.modules, "sentencepiece", fake)
    table = torch.randn(64, 16)
    torch.save(table, tmp_path / "embed.pt")
    out_json, out_ckpt = tmp_path / "o" / "r.json", tmp_path / "o" / "r.pt"
    res = R.run_ddp(_cfg(embed_init_path=str(tmp_path / "embed.pt")), data_path=str(tmp_path), sp_model_path="x",
                    budget_seconds=30.0, output_json=str(out_json), world_size_override=None, output_ckpt=str(out_ckpt),
                    max_steps=3)
    assert res["train"]["steps"] == 3 and np.isfinite(res["train"]["final_loss"]) and 0 < res["eval"]["bpb"] < 20
    assert json.loads(out_json.read_text())["params"] == res["params"]
    ck = torch.load(out_ckpt, weights_only=False)
    model = CareStudentLM(**ck["config"])
    model.load_state_dict(ck["model"], strict=True)
    assert all(v.device.type == "cpu" for v in ck["model"].values())
    with pytest.raises(ValueError):
        R.run_ddp(_cfg(optimizer=""), data_path=str(tmp_path), sp_model_path="x", budget_seconds=1.0, output_json=None,
                  world_size_override=None, max_steps=1)
    with pytest.raises(ValueError):
        R.run_ddp(_cfg(embed_init_path=str(tmp_path / "embed.pt"), model_dim=32), data_path=str(tmp_path),
                  sp_model_path="x", budget_seconds=1.0, output_json=None, world_size_override=None, max_steps=1)


def test_finite_gate_and_ckpt_payloads(tmp_path):
    res = {"train": {"final_loss": float("nan")}, "eval": {"bpb": 1.0}}
    with pytest.raises(RuntimeError, match="poisoned"):
        R._finite_gate(res, {})
    R._finite_gate(res, {"allow_nonfinite": True})
    assert res["nonfinite"]["flag"]
    m = CareStudentLM(vocab_size=8, dim=8, num_layers=1)

    class Cache:
        def to_dict(self):
            return {"capacity": 2}
    R.save_output_ckpt(str(tmp_path / "c.pt"), m, _cfg(vocab_size=8, model_dim=8, num_layers=1), episodic_cache=Cache(),
                       online_eval_state={"k": 1})
    ck = torch.load(tmp_path / "c.pt", weights_only=False)
    assert ck["episodic_cache"] == {"capacity": 2} and ck["online_eval_state"] == {"k": 1}
    with pytest.raises(TypeError):
        R.save_output_ckpt(str(tmp_path / "d.pt"), m, _cfg(vocab_size=8, model_dim=8, num_layers=1), episodic_cache=3)
