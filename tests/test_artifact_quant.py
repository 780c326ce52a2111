"""Artifact packer (int8 -> int6 ladder, size budget, round trip) and GPTQ int6."""
import torch
import pytest

from chaoscontrol_b200.artifact import eval_artifact, load_artifact, serialize_artifact
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.quantization import (GPTQQuantizer, ar_self_generated_calibration, pack_int6_lzma,
                                            quantize_int6_gptq, quantize_int6_percentile, unpack_int6_lzma)


def _model():
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=128, dim=32, num_layers=2)


def test_artifact_roundtrip_and_ladder(tmp_path):
    m = _model()
    cfg = {"vocab_size": 128, "model_dim": 32, "num_layers": 2, "ff_mult": 2}
    info = serialize_artifact(m, None, cfg, tmp_path / "a.bin")
    assert info["quantization"] == "int8" and info["size_bytes"] <= 16_000_000
    m2, tok, cfg2 = load_artifact(tmp_path / "a.bin")
    assert tok is None and cfg2["vocab_size"] == 128
    for (n, p), (_, q) in zip(m.named_parameters(), m2.named_parameters()):
        tol = p.abs().max().item() / 127 + 1e-3
        assert (p - q).abs().max().item() <= tol, n
    # a budget int8 cannot meet escalates to int6; an impossible one raises
    small = serialize_artifact(m, None, cfg, tmp_path / "b.bin", target_bytes=info["size_bytes"] - 2000)
    assert small["quantization"] == "int6"
    with pytest.raises(ValueError):
        serialize_artifact(m, None, cfg, tmp_path / "c.bin", target_bytes=1000)
    forced = serialize_artifact(m, None, cfg, tmp_path / "d.bin", force_quantization="int6",
                                online_eval_state={"k": torch.ones(2)})
    assert forced["quantization"] == "int6" and forced["online_eval_state"] == ["k"]
    rep = eval_artifact(tmp_path / "a.bin", torch.randint(0, 128, (4000,)), eval_batches=2, batch_size=2,
                        seq_len=32)
    assert rep["tokens"] == 128 and rep["mean_ce"] > 0
    assert m.artifact_bytes() == 2 * sum(p.numel() for p in m.parameters())


def test_gptq_beats_round_to_nearest_on_hessian_weighted_error():
    torch.manual_seed(1)
    W = torch.randn(64, 96)
    X = torch.randn(512, 96) * torch.linspace(0.1, 3.0, 96)      # anisotropic inputs
    H = X.T @ X / 512
    q_rtn, s_rtn = quantize_int6_percentile(W)
    q_g, s_g = quantize_int6_gptq(W, hessian=H, block_size=32)
    assert q_g.dtype == torch.int8 and q_g.abs().max() <= 31 and s_g.dtype == torch.float16

    def out_err(q, s):
        return ((X @ (W - q.float() * s.float()[:, None]).T) ** 2).mean().item()
    assert out_err(q_g, s_g) < out_err(q_rtn, s_rtn)
    q1, s1 = quantize_int6_gptq(torch.randn(50), hessian=None)
    assert q1.shape == (50,) and s1.ndim == 0


def test_gptq_quantizer_state_dict_roundtrip():
    m = _model()
    seqs = ar_self_generated_calibration(m, num_seqs=2, seq_len=12)
    assert seqs[0].shape == (1, 12)
    qz = GPTQQuantizer(block_size=16)
    H = qz.calibrate(m, seqs)
    assert "lm_head.weight" in H and H["lm_head.weight"].shape == (32, 32)
    res, meta = qz.quantize_state_dict(m.state_dict(), min_numel=1000)
    assert meta["embed.weight"]["type"] == "int6" and meta["final_norm.weight"]["type"] == "passthrough_fp16"
    blob = pack_int6_lzma(res, meta)
    r2, m2 = unpack_int6_lzma(blob)
    sd = GPTQQuantizer.dequantize_state_dict(r2, m2)
    ref = m.state_dict()
    for k in ref:
        assert sd[k].shape == ref[k].shape
        # scale floor 1/31 plus GPTQ error compensation under a tiny calibration set
        assert (sd[k].float() - ref[k].float()).abs().mean() <= 0.03
    with pytest.raises(ValueError):
        unpack_int6_lzma(__import__("lzma").compress(__import__("pickle").dumps({"x": 1})))
