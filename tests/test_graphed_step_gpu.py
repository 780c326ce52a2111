"""``GraphedTrainStep``: a replayed step is the eager step, bit for bit, on one GPU (the two-GPU
case, with the overlapped peer-memory exchange inside the graph, lives in test_peer_comm_gpu.py)."""
import copy

import pytest
import torch

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.ops import _lib
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.parallel.distributed import clip_arena_grad_norm
from chaoscontrol_b200.train_ssm import GraphedTrainStep, train_ssm_step
from chaoscontrol_b200.utils.arena import ParamArena, get_arena

pytestmark = pytest.mark.gpu


def _setup(seed=0):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=2048, dim=256, num_layers=2, ff_mult=2).cuda().to(torch.bfloat16)
    arena = ParamArena.install(m)
    m.train()
    opt = Muon(m.parameters(), lr=0.02, weight_decay=0.01, adamw_lr=0.02, adamw_weight_decay=0.01, fused=True)
    opt.bind_arena(arena)
    return m, arena, opt


def test_graph_replay_equals_eager_steps_bitwise():
    g = torch.Generator().manual_seed(3)
    batches = [torch.randint(0, 2048, (16, 257), generator=g).cuda() for _ in range(6)]
    m1, a1, o1 = _setup()
    losses1 = []
    for b in batches:
        loss = train_ssm_step(m1, b[:, :-1], b[:, 1:], 64, precision="bf16",
                              lm_head_backward_mode="fused_streaming_cached")
        clip_arena_grad_norm(a1, 1.0)
        o1.step()
        losses1.append(float(loss))
    m2, a2, o2 = _setup()
    step = GraphedTrainStep(m2, grad_clip_norm=1.0, eager_steps=2)
    losses2 = []
    for b in batches:
        loss = step(b[:, :-1], b[:, 1:])
        o2.step()
        losses2.append(float(loss))
    _lib.assert_ok()
    assert step.graph is not None and step.replays == 4 and step.launches_per_replay > 50
    assert losses1 == losses2
    assert torch.equal(a1.flat_param, a2.flat_param)
    with pytest.raises(ValueError):
        step(batches[0][:8, :-1], batches[0][:8, 1:])
