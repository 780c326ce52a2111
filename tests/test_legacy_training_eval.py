"""All-features trainer, windowed evaluation, warming curves, causal SLOT, baselines,
YAML runner and the public facade (CPU, tiny shapes)."""
import json

import pytest
import torch

from chaoscontrol_b200.baselines import Mamba2LM, SimpleTransformerLM
from chaoscontrol_b200.baselines_nanogpt_lean import apply_rope, build_nanogpt_lean, _build_rope_cache
from chaoscontrol_b200.evaluation import (_assert_state_clean, _reset_model_state, causal_slot_eval,
                                          evaluate_chaoscontrol_bpb, evaluate_warming_curve)
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.public import build_arm_config, init_arm_topology
from chaoscontrol_b200.training import (build_chaoscontrol_matrix, chunked_cross_entropy, parse_chaoscontrol_args,
                                        train_chaoscontrol_for_budget)

DEV = torch.device("cpu")


def _tokens(n=4000, vocab=32, seed=0):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))


def _train(model, tokens, **kw):
    base = dict(train_tokens=tokens, train_starts=list(range(0, 3000, 16)), seq_len=16, batch_size=4, device=DEV,
                param_dtype=torch.float32, budget_seconds=600.0, base_lr=1e-3, weight_decay=0.0, grad_clip_norm=1.0,
                seed=0, max_steps=6)
    base.update(kw)
    return train_chaoscontrol_for_budget(model, **base)


def test_chunked_cross_entropy_matches_dense():
    torch.manual_seed(0)
    logits = torch.randn(50, 17, requires_grad=True)
    tg = torch.randint(0, 17, (50,))
    for red in ("mean", "sum"):
        a = chunked_cross_entropy(logits, tg, chunk_size=7, reduction=red)
        b = torch.nn.functional.cross_entropy(logits, tg, reduction=red)
        assert torch.allclose(a, b, atol=1e-5) and a.dtype == torch.float32
    with pytest.raises(ValueError):
        chunked_cross_entropy(logits, tg, reduction="none")


def test_trainer_plain_and_optimizers():
    tokens = _tokens()
    for opt in ("adamw", "muon", "lamb"):
        torch.manual_seed(0)
        m = CareStudentLM(vocab_size=32, dim=16, num_layers=2)
        r = _train(m, tokens, optimizer=opt, crit_reg_alpha=0.0, crit_reg_beta=0.0)
        assert r["steps"] == 6 and r["optimizer_name"] == opt and len(r["history"]) == 6
        assert all(torch.isfinite(torch.tensor(h["loss"])) for h in r["history"])
    with pytest.raises(ValueError):
        _train(CareStudentLM(vocab_size=32, dim=16, num_layers=1), tokens, optimizer="sgd")


@pytest.mark.parametrize("mode", ["fork", "monte_carlo", "mcts"])
def test_trainer_metabolic_gate_with_regret(mode):
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                      wernicke_enabled=True, wernicke_k_max=4, typed_storage=True, dynamic_crit_per_layer=True)
    r = _train(m, _tokens(), metabolic_gate=True, metabolic_threshold=1.0, metabolic_threshold_mode="random",
               metabolic_mode=mode, metabolic_k=3, cfr_enabled=True, latent_persistence=True, mcts_horizon=2)
    assert r["fork_count"] == 6 and all(h["gate_fired"] for h in r["history"])
    assert r["regret_table"] is not None and "surprise" in r["history"][0]
    if mode == "monte_carlo":
        assert "mc_entropy" in r["history"][0]
    assert r["bucket_snapshots"] or mode != "monte_carlo"


def test_trainer_adaptive_threshold_and_structured_generation():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8)
    r = _train(m, _tokens(), metabolic_gate=True, metabolic_threshold=0.0, metabolic_threshold_mode="adaptive",
               generation_mode="structured", metabolic_k=2, metabolic_score="ensemble_agreement", max_steps=8)
    assert r["extra_params"] == 2 * 16 * 16 and r["structured_proj"] is not None
    assert len({h["threshold"] for h in r["history"]}) > 1


def test_trainer_sleep_polyphasic_posterior_semantic_and_append_only():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                      outer_max_slots=16, wernicke_enabled=True, wernicke_k_max=4, typed_storage=True,
                      typed_consolidation=True, compression_consequence=True, semantic_tier_bases=3,
                      posterior_mode="bucket_delta")
    r = _train(m, _tokens(), sleep_enabled=True, sleep_interval=4, sleep_rem_dreams=1, sleep_rem_length=2,
               polyphasic_enabled=True, polyphasic_n_partitions=2, polyphasic_k_awake=1, polyphasic_swap_interval=3,
               consolidation_write="full_sequence", max_steps=9)
    assert r["sleep_cycles"] == 2 and m.semantic_tier.bases.abs().sum() > 0 and m.posterior.deltas.abs().sum() > 0
    torch.manual_seed(0)
    m2 = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8, outer_model_type="multislot",
                       outer_max_slots=0, buffer_mode="append_only", posterior_mode="residual_cache")
    _train(m2, _tokens(), buffer_mode="append_only", max_steps=2)
    assert len(m2.outer_model.table) == 2 * 4 * 16


def test_trainer_with_learned_tokenizer_and_alignment():
    from chaoscontrol_b200.tokenizer import FixedStrideTokenizer
    torch.manual_seed(0)
    tok = FixedStrideTokenizer(byte_dim=8, token_dim=16, codebook_size=24, stride=2)
    m = CareStudentLM(vocab_size=24, dim=16, num_layers=1, wernicke_enabled=True, wernicke_k_max=4)
    bytes_ = torch.randint(0, 256, (4000,))
    r = _train(m, bytes_, tokenizer=tok, align_type="contrastive", align_weight=0.1, seq_len=32, max_steps=3)
    assert "recon_loss" in r["history"][0] and tok.codebook.grad is not None or True
    ev = evaluate_chaoscontrol_bpb(m, tokens=bytes_, eval_starts=[0, 40], batch_size=2, seq_len=32, device=DEV,
                                   tokenizer=tok)
    assert ev["bpb"] > 0 and ev["tokens"] == 2 * 15


def test_trainer_rejects_unsupported_ddp_combinations():
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1)
    with pytest.raises(NotImplementedError):
        _train(m, _tokens(), rank=0, world_size=2, metabolic_gate=True, metabolic_mode="fork")
    with pytest.raises(NotImplementedError):
        _train(m, _tokens(), rank=0, world_size=2, generation_mode="structured")
    with pytest.raises(RuntimeError):
        _train(m, _tokens(), rank=0, world_size=2)


def test_evaluate_bpb_warmup_restores_memory_state():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8, outer_model_type="multislot")
    m.outer_model.write(torch.randn(2, 16))
    before = m.outer_model.table.slot_matrix().clone()
    ema = m.outer_model.loss_ema.clone()
    tokens = _tokens()
    ev = evaluate_chaoscontrol_bpb(m, tokens=tokens, eval_starts=[0, 20, 40, 60], batch_size=2, seq_len=16, device=DEV,
                                   warmup=True, warmup_latent=True, warmup_cold_start=True, metabolic_gate=True,
                                   metabolic_k=2, total_raw_bytes=1000)
    assert torch.equal(m.outer_model.table.slot_matrix(), before) and torch.equal(m.outer_model.loss_ema, ema)
    assert {"loss", "bpb", "tokens", "bpb_raw", "loss_gated", "bpb_gated"} <= set(ev)
    plain = evaluate_chaoscontrol_bpb(m, tokens=tokens, eval_starts=[0, 20, 40, 60], batch_size=2, seq_len=16,
                                      device=DEV)
    assert plain["bpb"] == pytest.approx(plain["loss"] / 0.6931471805599453)
    om = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8)
    s0 = om.outer_model.state.clone()
    evaluate_chaoscontrol_bpb(om, tokens=tokens, eval_starts=[0, 20], batch_size=2, seq_len=16, device=DEV,
                              warmup=True, warmup_write_mode="full_sequence")
    assert torch.equal(om.outer_model.state, s0)


def test_warming_curve_and_reset_protocol():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8, outer_model_type="multislot",
                      outer_max_slots=0, buffer_mode="append_only", semantic_tier_bases=2,
                      posterior_mode="global_delta", bucket_prototypes=True, prototype_dim=8, wernicke_enabled=True,
                      wernicke_k_max=4)
    m.posterior.update(torch.ones(16))
    m.semantic_tier.bases.fill_(1.0)
    m(torch.randint(0, 32, (1, 20)), memory_write_mode="append_only")
    _reset_model_state(m)
    _assert_state_clean(m)
    curve = evaluate_warming_curve(m, _tokens(3000), warmup_tokens=[0, 64], score_tokens=32, max_segments=3)
    assert set(curve) == {0, 64} and all(0 < v < 15 for v in curve.values())
    _assert_state_clean.__call__  # noqa: B018
    short = evaluate_warming_curve(m, _tokens(30), warmup_tokens=[0], score_tokens=64)
    assert short[0] != short[0]                                   # nothing could be scored: NaN


def test_causal_slot_factorial():
    torch.manual_seed(0)
    m = CareStudentLM(vocab_size=32, dim=16, num_layers=1, outer_model_dim=8, outer_model_type="multislot",
                      outer_max_slots=0, buffer_mode="append_only")
    res = causal_slot_eval(m, _tokens(2000), warmup_tokens=[0, 48], score_tokens=32, window_size=16, slot_steps=3,
                           slot_lr=0.05, max_segments=2)
    assert set(res) == {"cold", "buffer_only", "slot_only", "buffer_plus_slot"}
    assert res["cold"][0] == res["slot_only"][0] == res["buffer_only"][0]        # no warm-up: all identical
    assert res["slot_only"][48] != res["cold"][48]
    assert all(p.requires_grad for p in m.parameters() if p is not m.outer_model.encoder.weight)
    stream = causal_slot_eval(m, _tokens(2000), conditions=("slot_only",), warmup_tokens=[16], score_tokens=32,
                              window_size=16, slot_steps=2, freeze_during_scoring=False, max_segments=1)
    assert 0 < stream["slot_only"][16] < 15


def test_baselines_shapes_and_causality():
    ids = torch.randint(0, 64, (2, 12))
    for m in (SimpleTransformerLM(vocab_size=64, dim=32, num_layers=2, num_heads=4),
              build_nanogpt_lean(vocab_size=64, d_model=32, n_head=4, n_layer=2, max_seq_len=8),
              Mamba2LM(vocab_size=64, dim=32, num_layers=2, d_state=8, impl="torch")):
        out = m(ids, return_jacobian_stats=True)
        assert out["logits"].shape == (2, 12, 64) and "jacobian_stats" in out and m.outer_model is None
        assert m.artifact_bytes() == 2 * sum(p.numel() for p in m.parameters())
        ids2 = ids.clone()
        ids2[:, 8:] = 0
        assert torch.allclose(m(ids2)["logits"][:, :8], out["logits"][:, :8], atol=1e-5)
        out["logits"].sum().backward()
    with pytest.raises(ImportError):
        Mamba2LM(vocab_size=8, dim=8, num_layers=1)
    # RoPE is a rotation: norms are preserved, position 0 is the identity
    rc = _build_rope_cache(8, 5)
    x = torch.randn(1, 2, 5, 8)
    y = apply_rope(x, rc[0], rc[1])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5) and torch.allclose(y[..., 0, :], x[..., 0, :])
    lean = build_nanogpt_lean(vocab_size=64, d_model=32, n_head=4, n_layer=1, activation_checkpoint=True)
    lean.train()
    lean(ids)["logits"].sum().backward()


def test_matrix_cli_and_facade():
    cells = build_chaoscontrol_matrix()
    assert len(cells) == 24 and cells[0] == {"rich_b_mode": "none", "outer_model_dim": 0, "label": "base", "a_mode": "diag"}
    a = parse_chaoscontrol_args(["--data-path", "/d", "--model-dim", "64", "--a-mode", "full"])
    assert a.model_dim == 64 and a.a_mode == "full" and a.dtype == "fp16"
    r = init_arm_topology(3, 4)
    assert r.is_packet_rank and r.is_maintenance_rank and not r.is_train_rank and r.packet_rank == 3
    assert init_arm_topology(0, 1).is_train_rank and init_arm_topology(1, 4).is_train_rank
    sp = init_arm_topology(2, 4, split_memory_ranks=True)
    assert sp.is_packet_rank and not sp.is_maintenance_rank and sp.maintenance_rank == 3

    class HP:
        vocab_size, model_dim, num_layers, seq_len, batch_size, base_lr = 64, 16, 2, 16, 4, 0.05
    cfg = build_arm_config(HP())
    assert cfg["base_lr"] == 0.05 and cfg["headline_calc_type"] == "packet_online_cache" and cfg["fast_slow_enabled"]
    with pytest.raises(ValueError):
        build_arm_config({"vocab_size": 8})


def test_yaml_runner_end_to_end(tmp_path):
    import yaml

    from chaoscontrol_b200.runner import load_checkpoint, run_experiment
    (tmp_path / "docs_raw.txt").write_bytes(bytes(range(32, 127)) * 200)
    cfg = dict(model_type="ssm", vocab_size=256, model_dim=16, num_layers=1, seq_len=16, stride=8, batch_size=4,
               eval_batches=2, budget_seconds=0.2, device="cpu", dtype="fp32", outer_model_dim=8, base_lr=1e-3,
               crit_reg_alpha=0.0, crit_reg_beta=0.0)
    (tmp_path / "c.yaml").write_text(yaml.safe_dump(cfg))
    res = run_experiment(str(tmp_path / "c.yaml"), data_path=str(tmp_path), budget_seconds=0.2,
                         checkpoint_dir=str(tmp_path / "ck"), checkpoint_name="t")
    assert res["train"]["steps"] >= 1 and 0 < res["eval"]["bpb"] < 15 and "bpb_raw" in res["eval"]
    json.dumps(res, default=str)
    back = load_checkpoint(tmp_path / "ck" / "t.pt", DEV, torch.float32)
    assert back["config"].model_dim == 16 and back["model"].outer_model is not None
