"""Side-by-side checks against the unmodified reference package.

Skipped when the reference is not installed under ``baseline/_ref``.  Everything
runs on CPU in fp32: the byte-level configuration (vocab 256, dim 64, 2 layers,
seq 128, batch 8, Zipf(1.1) tokens from seed 0, 20 Muon steps at lr 0.064 with
momentum 0.95 and 5 Newton-Schulz iterations, AdamW on the non-matrix
parameters).  Both implementations are built from the same seed, exchange
state dicts strictly in both directions, and must agree on logits, gradients
and the 20-step loss curve.  ``tie_embeddings`` and ``log_a_init="log_uniform"``
are options of this package only; they are compared against a reference model
tied / initialised by hand.
"""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "chaoscontrol").exists(), reason="reference not installed under baseline/_ref")

V, D, L, T, B = 256, 64, 2, 128, 8


def _ref_mod():
    if str(REF) not in sys.path:
        sys.path.append(str(REF))
    import chaoscontrol.model as rmodel
    import chaoscontrol.optim.muon as rmuon
    import chaoscontrol.train_ssm as rtrain
    return rmodel, rmuon, rtrain


def _zipf_batches(n_steps):
    ranks = np.arange(1, V + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** -1.1)
    cdf /= cdf[-1]
    rng = np.random.default_rng(0)
    out = []
    for _ in range(n_steps):
        ids = np.searchsorted(cdf, rng.random(B * (T + 1)), side="left").clip(0, V - 1)
        out.append(torch.from_numpy(ids.astype(np.int64)).view(B, T + 1))
    return out


def _pair(**ours_kw):
    from chaoscontrol_b200.models.model import CareStudentLM
    rmodel, _, _ = _ref_mod()
    torch.manual_seed(0)
    ref = rmodel.CareStudentLM(vocab_size=V, dim=D, num_layers=L)
    torch.manual_seed(0)
    ours = CareStudentLM(vocab_size=V, dim=D, num_layers=L, **ours_kw)
    return ref, ours


def test_state_dict_keys_and_strict_load_both_ways():
    ref, ours = _pair()
    assert list(ref.state_dict().keys()) == list(ours.state_dict().keys())
    for k, v in ref.state_dict().items():
        assert ours.state_dict()[k].shape == v.shape, k
        assert torch.equal(ours.state_dict()[k], v), f"same seed, different init: {k}"
    # strict load in both directions, with perturbed values so the copy is observable
    sd = {k: v + 0.01 for k, v in ref.state_dict().items()}
    assert not ours.load_state_dict(sd, strict=True).missing_keys
    sd2 = {k: v - 0.02 for k, v in ours.state_dict().items()}
    assert not ref.load_state_dict(sd2, strict=True).missing_keys
    for k in sd2:
        assert torch.equal(ref.state_dict()[k], sd2[k])


def test_logits_and_gradients_match():
    ref, ours = _pair()
    blk = _zipf_batches(1)[0]
    inp, tgt = blk[:, :-1], blk[:, 1:]
    out_r = ref(inp)
    out_o = ours(inp)
    lr_, lo_ = out_r["logits"] if isinstance(out_r, dict) else out_r, out_o["logits"]
    assert (lr_ - lo_).abs().max().item() < 1e-5
    F.cross_entropy(lr_.reshape(-1, V), tgt.reshape(-1)).backward()
    F.cross_entropy(lo_.reshape(-1, V), tgt.reshape(-1)).backward()
    gr = dict(ref.named_parameters())
    for n, p in ours.named_parameters():
        assert (p.grad - gr[n].grad).abs().max().item() < 1e-6, n


def _run20(model, muon_cls, step_fn, batches, *, fused):
    opt = muon_cls(model.parameters(), lr=0.064, momentum=0.95, ns_steps=5, weight_decay=0.01, adamw_lr=0.064,
                   adamw_weight_decay=0.01, fused=fused)
    opt.bind_param_names(list(model.named_parameters()))
    losses = []
    model.train()
    for blk in batches:
        opt.zero_grad(set_to_none=True)
        loss = step_fn(model, blk[:, :-1], blk[:, 1:], 32, precision="fp32", lm_head_backward_mode="chunked")
        opt.step()
        losses.append(float(loss))
    return losses


@pytest.mark.parametrize("fused", [False, True])
def test_twenty_muon_steps_give_the_same_loss_curve(fused):
    from chaoscontrol_b200.optim.muon import Muon
    from chaoscontrol_b200.train_ssm import train_ssm_step
    _, rmuon, rtrain = _ref_mod()
    ref, ours = _pair()
    batches = _zipf_batches(20)
    lr = _run20(ref, rmuon.Muon, rtrain.train_ssm_step, batches, fused=fused)
    lo = _run20(ours, Muon, train_ssm_step, batches, fused=fused)
    assert max(abs(a - b) for a, b in zip(lr, lo)) < 2e-4, list(zip(lr, lo))
    assert lo[-1] < lo[0] - 0.3                     # and it learns
    drift = max((p - dict(ref.named_parameters())[n]).abs().max().item() for n, p in ours.named_parameters())
    assert drift < 2e-3, drift


def test_tied_embeddings_and_log_uniform_decay_against_a_hand_built_reference():
    from chaoscontrol_b200.optim.muon import Muon
    from chaoscontrol_b200.train_ssm import train_ssm_step
    _, rmuon, rtrain = _ref_mod()
    ref, ours = _pair(tie_embeddings=True, log_a_init="log_uniform")
    assert ours.lm_head.weight is ours.embed.weight
    # the reference has neither option: tie and initialise it by hand from this package's draw
    ref.lm_head.weight = ref.embed.weight
    with torch.no_grad():
        for rb, ob in zip(ref.layers, ours.layers):
            assert float(ob.core.log_a.min()) >= -4.0 and float(ob.core.log_a.max()) <= 0.0
            assert float(ob.core.log_a.std()) > 0.5      # spread over the interval, not a constant
            rb.core.log_a.copy_(ob.core.log_a)
        ours.embed.weight.copy_(ref.embed.weight)
    batches = _zipf_batches(8)
    lr = _run20(ref, rmuon.Muon, rtrain.train_ssm_step, batches, fused=False)
    lo = _run20(ours, Muon, train_ssm_step, batches, fused=False)
    assert max(abs(a - b) for a, b in zip(lr, lo)) < 2e-4, list(zip(lr, lo))
