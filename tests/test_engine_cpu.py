"""The no-autograd training engine on CPU tensors (op stand-ins) against plain
autograd through the module: loss and every parameter gradient."""
import torch
import torch.nn.functional as F

from chaoscontrol_b200.engine import TrainEngine
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.utils.arena import ParamArena


def _model(seed=0, vocab=64, dim=16, layers=2):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=vocab, dim=dim, num_layers=layers)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("norm.weight"):
                p.uniform_(0.7, 1.3)
            if n.endswith("log_a"):
                p.normal_()
    return m


def test_engine_step_matches_autograd():
    m = _model()
    tok = torch.randint(0, 64, (3, 10))
    tgt = torch.randint(0, 64, (3, 10))
    out = m(tok)
    loss_ref = F.cross_entropy(out["logits"].reshape(-1, 64), tgt.reshape(-1))
    loss_ref.backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    arena = ParamArena.install(m)
    eng = TrainEngine(m, arena)
    loss = eng.step(tok, tgt)
    assert torch.allclose(loss, loss_ref, atol=1e-5)
    for n in ref:
        assert torch.allclose(arena.grad_view(n), ref[n], atol=3e-5), n
    arena.materialize_grads()
    for n, p in m.named_parameters():
        assert p.grad is not None and torch.allclose(p.grad, ref[n], atol=3e-5)


def test_arena_preserves_state_dict_and_views():
    m = _model(1)
    sd = {k: v.clone() for k, v in m.state_dict().items()}
    arena = ParamArena.install(m)
    assert arena.still_valid()
    for k, v in m.state_dict().items():
        assert torch.equal(v, sd[k])
    # packed projections are adjacent: select, in, gate, delta
    c = m.layers[0].core
    step = c.select_proj.weight.numel() * 4
    base = c.select_proj.weight.data_ptr()
    assert c.in_proj.weight.data_ptr() == base + step
    assert c.gate_proj.weight.data_ptr() == base + 2 * step
    assert c.delta_proj.weight.data_ptr() == base + 3 * step
    m.to(torch.float64)
    assert not arena.still_valid()


def test_muon_on_arena_model_cpu_matches_plain():
    """Arena-backed params through the generic fused path == plain per-param path."""
    m1, m2 = _model(2), _model(2)
    ParamArena.install(m2)
    tok = torch.randint(0, 64, (2, 8))
    tgt = torch.randint(0, 64, (2, 8))
    o1 = Muon(m1.parameters(), lr=0.05)
    o1.bind_param_names(m1.named_parameters())
    o2 = Muon(m2.parameters(), lr=0.05, fused=True)
    o2.bind_param_names(m2.named_parameters())
    for _ in range(3):
        for m, o in ((m1, o1), (m2, o2)):
            o.zero_grad()
            F.cross_entropy(m(tok)["logits"].reshape(-1, 64), tgt.reshape(-1)).backward()
            o.step()
    for (n, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(p1, p2, atol=1e-5), n
