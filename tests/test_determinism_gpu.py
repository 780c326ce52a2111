"""Bit-reproducibility of the training step on the GPU.

The reference's lean loop is deterministic (its DDP test asserts identical
parameters across ranks under a fake clock, tests/test_train_ssm_ddp.py:60-72).
Here every reduction on the step has a fixed summation order -- the sorted
embedding backward, the split-K second stages, the clip norm and Muon's
Frobenius norms -- so the same seed gives the same parameter bits in two
fresh processes, and two replicas that hold the same gradient take the same
optimizer step.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.ops import trunk as T

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _zipf_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
    p = ranks ** -1.1
    return torch.multinomial(p / p.sum(), n, replacement=True, generator=g)


@pytest.mark.parametrize("R,V,D", [(33, 7, 256), (4096, 50, 256), (20000, 16384, 256), (5000, 300, 512),
                                   (3001, 64, 1024)])
def test_embed_backward_matches_index_add_and_repeats_bitwise(R, V, D):
    tok = _zipf_tokens(R, V, seed=R).cuda()
    dx = torch.randn(R, D, device="cuda").bfloat16()
    a = T.embed_bwd(tok, dx, V)
    b = T.embed_bwd(tok, dx, V)
    _lib.assert_ok()
    assert torch.equal(a, b)
    ref = torch.zeros(V, D, device="cuda", dtype=torch.float64).index_add_(0, tok, dx.double())
    scale = ref.abs().max().item()
    assert (a.double() - ref).abs().max().item() <= 1e-5 * scale + 1e-6
    # one token everywhere: every chunk is a boundary chunk
    tok1 = torch.full((R,), V - 1, device="cuda", dtype=torch.long)
    c = T.embed_bwd(tok1, dx, V)
    assert torch.allclose(c[V - 1].double(), dx.double().sum(0), rtol=1e-5, atol=1e-3)
    assert c[: V - 1].abs().max().item() == 0.0


def test_clip_and_muon_norms_repeat_bitwise():
    from chaoscontrol_b200.parallel.distributed import clip_arena_grad_norm

    class _A:
        pass
    torch.manual_seed(0)
    g0 = torch.randn(10_800_000, device="cuda")
    norms = []
    for _ in range(3):
        a = _A()
        a.flat_grad = g0.clone()
        n = clip_arena_grad_norm(a, 1.0)
        norms.append((float(n), a.flat_grad.clone()))
    _lib.assert_ok()
    assert norms[0][0] == norms[1][0] == norms[2][0]
    assert torch.equal(norms[0][1], norms[1][1]) and torch.equal(norms[0][1], norms[2][1])
    assert abs(norms[0][0] - float(g0.double().norm())) <= 1e-4 * norms[0][0]


_CHILD = r"""
import json, sys, hashlib
import torch
sys.path.insert(0, {root!r})
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.parallel.distributed import clip_arena_grad_norm
from chaoscontrol_b200.train_ssm import _engine_for
from chaoscontrol_b200.utils.arena import ParamArena
from chaoscontrol_b200.ops import _lib
torch.manual_seed(0)
m = CareStudentLM(vocab_size=2048, dim=256, num_layers=2, ff_mult=2).cuda().to(torch.bfloat16)
arena = ParamArena.install(m)
m.train()
opt = Muon(m.parameters(), lr=0.064, weight_decay=0.01, adamw_lr=0.064, adamw_weight_decay=0.01, fused=True)
opt.bind_arena(arena)
eng = _engine_for(m)
g = torch.Generator().manual_seed(1)
ranks = torch.arange(1, 2049, dtype=torch.float64) ** -1.1
losses = []
for step in range(10):
    tok = torch.multinomial(ranks / ranks.sum(), 16 * 257, replacement=True, generator=g).view(16, 257).cuda()
    loss = eng.step(tok[:, :-1].to(torch.int32).contiguous(), tok[:, 1:].contiguous())
    clip_arena_grad_norm(arena, 1.0)
    opt.step()
    losses.append(float(loss))
_lib.assert_ok()
h = hashlib.sha256(arena.flat_param.view(torch.int16).cpu().numpy().tobytes()).hexdigest()
print(json.dumps({{"hash": h, "losses": losses}}))
"""


def test_ten_engine_steps_repeat_bitwise_in_fresh_processes():
    outs = []
    for _ in range(2):
        res = subprocess.run([sys.executable, "-c", _CHILD.format(root=str(ROOT))], capture_output=True,
                             text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        outs.append(json.loads(res.stdout.strip().splitlines()[-1]))
    assert outs[0]["losses"] == outs[1]["losses"], (outs[0]["losses"], outs[1]["losses"])
    assert outs[0]["hash"] == outs[1]["hash"]
    assert outs[0]["losses"][-1] < outs[0]["losses"][0]
