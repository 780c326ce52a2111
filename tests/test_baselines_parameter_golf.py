"""The contest harness on this package's parts: environment contract, shard format, model wiring,
parameter split, schedules, int8 export round trip, and a tiny end-to-end run on CPU."""
import math

import numpy as np
import pytest
import torch

from chaoscontrol_b200 import baselines_parameter_golf as G


def _tiny(**over):
    kw = dict(vocab_size=64, num_layers=4, model_dim=32, num_heads=4, num_kv_heads=2, mlp_mult=2, train_seq_len=16,
              train_batch_tokens=8 * 2 * 16, val_batch_size=4 * 16, iterations=3, warmup_steps=1, warmdown_iters=2,
              max_wallclock_seconds=0.0, val_loss_every=0, train_log_every=1)
    kw.update(over)
    return G.GolfConfig(**kw)


def test_config_reads_the_environment(monkeypatch):
    monkeypatch.setenv("NUM_LAYERS", "11")
    monkeypatch.setenv("TIE_EMBEDDINGS", "0")
    monkeypatch.setenv("MATRIX_LR", "0.02")
    monkeypatch.setenv("RUN_ID", "abc")
    c = G.GolfConfig.from_env()
    assert (c.num_layers, c.tie_embeddings, c.matrix_lr, c.run_id) == (11, False, 0.02, "abc")
    assert c.model_dim == 512 and c.train_batch_tokens == 524_288 and c.logit_softcap == 30.0
    assert c.train_files.endswith("fineweb_train_*.bin")


def test_shard_round_trip_and_header_checks(tmp_path):
    tok = np.arange(1000, dtype=np.uint16)
    G.write_data_shard(tmp_path / "fineweb_train_000.bin", tok)
    assert torch.equal(G.load_data_shard(tmp_path / "fineweb_train_000.bin"), torch.from_numpy(tok))
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"\0" * 2048)
    with pytest.raises(ValueError, match="header"):
        G.load_data_shard(bad)
    raw = bytearray((tmp_path / "fineweb_train_000.bin").read_bytes())
    (tmp_path / "short.bin").write_bytes(bytes(raw[:-10]))
    with pytest.raises(ValueError, match="size mismatch"):
        G.load_data_shard(tmp_path / "short.bin")


def test_stream_wraps_and_ranks_get_disjoint_spans(tmp_path):
    G.write_data_shard(tmp_path / "fineweb_train_000.bin", np.arange(0, 100, dtype=np.uint16))
    G.write_data_shard(tmp_path / "fineweb_train_001.bin", np.arange(100, 150, dtype=np.uint16))
    s = G.TokenStream(str(tmp_path / "fineweb_train_*.bin"))
    assert s.take(120).tolist() == list(range(120))
    assert s.take(40).tolist() == list(range(120, 150)) + list(range(10))          # wrapped to the first shard
    dev = torch.device("cpu")
    l0 = G.DistributedTokenLoader(str(tmp_path / "fineweb_train_*.bin"), 0, 2, dev)
    l1 = G.DistributedTokenLoader(str(tmp_path / "fineweb_train_*.bin"), 1, 2, dev)
    x0, y0 = l0.next_batch(32, 8, 1)
    x1, y1 = l1.next_batch(32, 8, 1)
    assert x0.shape == (2, 8) and torch.equal(y0.reshape(-1)[:-1], x0.reshape(-1)[1:])
    assert x0.reshape(-1).tolist() == list(range(16)) and x1.reshape(-1).tolist() == list(range(17, 33))


def test_model_wiring_and_parameter_split():
    torch.manual_seed(0)
    cfg = _tiny()
    m = G.GPT(cfg)
    names = dict(m.named_parameters())
    assert "blocks.0.attn.c_q.weight" in names and "blocks.3.resid_mix" in names and "skip_weights" in names
    assert m.lm_head is None and names["skip_weights"].shape == (2, 32)
    assert float(names["blocks.1.mlp.proj.weight"].detach().abs().sum()) == 0.0
    assert float(names["blocks.1.attn.proj.weight"].detach().abs().sum()) == 0.0
    x = torch.randint(0, 64, (2, 16))
    lg = m.logits(x)
    assert lg.shape == (2, 16, 64) and float(lg.detach().abs().max()) <= cfg.logit_softcap
    y = torch.randint(0, 64, (2, 16))
    assert float(m(x, y).detach()) == pytest.approx(math.log(64), abs=0.1)             # zero-init projections: near uniform
    # causal: changing a late token does not move earlier logits
    x2 = x.clone()
    x2[:, 10] = (x2[:, 10] + 1) % 64
    assert torch.allclose(m.logits(x2)[:, :10], lg[:, :10], atol=1e-6)
    g = G.split_parameters(m)
    assert len(g["matrix"]) == 4 * 6 and all(p.ndim == 2 for p in g["matrix"])
    assert len(g["scalar"]) == 4 * 4 + 1 and g["head"] == [] and g["embed"][0] is m.tok_emb.weight
    total = sum(len(v) for v in g.values())
    assert total == len(list(m.parameters()))
    untied = G.GPT(_tiny(tie_embeddings=False))
    assert len(G.split_parameters(untied)["head"]) == 1 and len(G.build_optimizers(untied, untied.cfg)) == 4


def test_schedules():
    c = _tiny(iterations=100, warmdown_iters=20, max_wallclock_seconds=0.0)
    assert G.lr_multiplier(c, 50, 0.0) == 1.0 and G.lr_multiplier(c, 90, 0.0) == pytest.approx(0.5)
    assert G.lr_multiplier(c, 100, 0.0) == 1.0                                   # past the end: the loop has stopped
    w = _tiny(warmdown_iters=10, max_wallclock_seconds=1.0)
    assert G.lr_multiplier(w, 100, 500.0) == 1.0                                 # 5 ms steps: 50 ms window, 500 ms left
    assert G.lr_multiplier(w, 190, 975.0) == pytest.approx(25.0 / (10 * 975.0 / 190))
    assert G.lr_multiplier(_tiny(warmdown_iters=0), 5, 1.0) == 1.0
    m = _tiny(muon_momentum_warmup_steps=100)
    assert G.muon_momentum_at(m, 0) == pytest.approx(0.85) and G.muon_momentum_at(m, 50) == pytest.approx(0.90)
    assert G.muon_momentum_at(m, 500) == pytest.approx(0.95)


def test_int8_export_round_trip():
    torch.manual_seed(1)
    cfg = _tiny(model_dim=256, num_heads=4, num_kv_heads=2, num_layers=2, vocab_size=512)
    m = G.GPT(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.ndim == 2:
                p.normal_(0, 0.05)
    obj, stats = G.quantize_state_dict_int8(m.state_dict())
    assert obj["__quant_format__"] == "int8_clean_per_row_v1"
    assert "blocks.0.mlp.fc.weight" in obj["quantized"] and obj["quantized"]["blocks.0.mlp.fc.weight"].dtype == torch.int8
    assert obj["scales"]["blocks.0.mlp.fc.weight"].shape == (512,)
    assert "blocks.0.attn_scale" in obj["passthrough"] and obj["passthrough"]["blocks.0.attn_scale"].dtype == torch.float32
    assert stats["int8_payload_bytes"] < 0.4 * stats["baseline_tensor_bytes"]
    blob, st = G.export_int8_zlib(m)
    before = {k: v.clone() for k, v in m.state_dict().items()}
    G.load_int8_zlib(m, blob)
    for k, v in m.state_dict().items():
        err = (v.float() - before[k].float()).abs().max().item()
        # per-row scales are floored at 1 / 127: half a step is the largest rounding error of a matrix entry
        assert err <= (0.5 / 127 + 1e-4 if v.ndim == 2 and v.numel() > G.INT8_KEEP_FLOAT_MAX_NUMEL else 2e-3), k
    assert len(blob) < st["raw_torch_bytes"]


def test_end_to_end_on_cpu(tmp_path):
    rng = np.random.default_rng(0)
    d = tmp_path / "data"
    d.mkdir()
    G.write_data_shard(d / "fineweb_train_000.bin", rng.integers(0, 64, 20000).astype(np.uint16))
    G.write_data_shard(d / "fineweb_val_000.bin", rng.integers(0, 64, 16 * 12 + 1).astype(np.uint16))
    cfg = _tiny(data_path=str(d), iterations=4, warmup_steps=2, val_loss_every=2)
    luts = (torch.full((64,), 2, dtype=torch.int16), torch.zeros(64, dtype=torch.bool), torch.zeros(64, dtype=torch.bool))
    lines = []
    out = G.train(cfg, device=torch.device("cpu"), log=lines.append, luts=luts, out_dir=tmp_path / "out")
    assert out["steps"] == 4 and math.isfinite(out["val_loss"]) and out["val_bpb"] == pytest.approx(out["val_loss"] / math.log(2) / 2)
    assert abs(out["roundtrip_val_loss"] - out["val_loss"]) < 0.05
    assert (tmp_path / "out" / "final_model.int8.ptz").exists() and (tmp_path / "out" / "final_model.pt").exists()
    assert sum(l.startswith("warmup_step:") for l in lines) == 2
    assert any(l.startswith("step:0/4 val_loss:") for l in lines) and any("final_int8_zlib_roundtrip_exact" in l for l in lines)
    # a wall-clock cap stops the run early and says so
    lines2 = []
    G.train(_tiny(data_path=str(d), iterations=10_000, warmup_steps=0, max_wallclock_seconds=0.2), device=torch.device("cpu"),
            log=lines2.append, luts=luts)
    assert any(l.startswith("stopping_early: wallclock_cap") for l in lines2)
