"""Behaviour-cloning pretrain of the simplex policy: torch twin == native forward, convergence,
export/import."""
import numpy as np
import torch

from chaoscontrol_b200.episodic import pretrain as P
from chaoscontrol_b200.episodic.controller import load_simplex_policy


def test_torch_twin_matches_native_forward():
    cfg = P.PretrainConfig(temperature=0.7, seed=3)
    torch.manual_seed(3)
    model = P.SimplexPolicyModule(cfg)
    with torch.no_grad():
        model.W_sb.normal_(0, 0.3)
        model.alpha.fill_(0.4)
        model.b_lh.fill_(-0.2)
        model.b_vp.normal_(0, 0.1)
    V, E, feats, _ = P.synthetic_batch(5, cfg, torch.Generator().manual_seed(1))
    want = torch.softmax(model(V, E, feats), dim=-1).detach().numpy()
    pol = P.to_native(model)
    for b in range(5):
        p, _ = pol.forward(V[b].numpy(), E[b].numpy(), feats[b].numpy())
        np.testing.assert_allclose(p, want[b], atol=2e-5)


def test_pretrain_learns_the_heuristic_and_round_trips(tmp_path, capsys):
    res = P.train(P.PretrainConfig(n_batches=300, seed=7))
    assert res["final_policy_acc"] > 0.8 and res["final_loss"] < 1.0     # chance is 1/16
    assert res["mean_max_p"] > 0.3                                        # well away from uniform 0.0625
    out = tmp_path / "pol" / "simplex.pt"
    assert P.main(["--n-batches", "50", "--seed", "7", "--out", str(out)]) == 0
    assert "final_policy_acc=" in capsys.readouterr().out
    pol = load_simplex_policy(out)
    assert (pol.N, pol.K_v, pol.K_s, pol.H) == (16, 16, 4, 32) and np.isfinite(pol.flat).all()
    cswg = tmp_path / "simplex.cswg"
    assert P.main(["--n-batches", "5", "--out", str(cswg)]) == 0
    assert load_simplex_policy(cswg).flat.shape == pol.flat.shape
