"""The ScOpt training step: pressure, split-step rare gradients and channel pressures, the commit-after-clip
contract, and cross-rank agreement of everything it synchronises (gloo ranks)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim import scopt_step as S
from chaoscontrol_b200.optim.scopt import (FrequencyBucketBaseline, ScarcityAwareOptimizer, scarcity_pressure_from_ce,
                                           scopt_optimizer_config)


def _setup(seed=0, vocab=64, dim=32):
    torch.manual_seed(seed)
    m = CareStudentLM(vocab_size=vocab, dim=dim, num_layers=2, ff_mult=2)
    opt = ScarcityAwareOptimizer(m.parameters(), lr=0.02, warmup_steps=0, **scopt_optimizer_config(m, 0))
    opt.bind_param_names(list(m.named_parameters()))
    freq = torch.arange(1, vocab + 1, dtype=torch.float32).flip(0)
    return m, opt, freq


def test_split_step_matches_a_direct_autograd_statement():
    m, opt, freq = _setup()
    tok = torch.randint(0, 64, (3, 17))
    x, y = tok[:, :-1], tok[:, 1:]
    loss, pending = S.run_scopt_train_step(model=m, optimizer=opt, inputs=x, targets=y, step=0, split_interval=4,
                                           token_frequencies=freq, precision="fp32", lm_head_backward_mode="single")
    assert pending is not None and set(pending.rare_map) == {n for n, p in m.named_parameters() if p.grad is not None}
    # direct statement
    out = m(x)
    logits = out["logits"] if isinstance(out, dict) else out
    ce = F.cross_entropy(logits.reshape(-1, 64).float(), y.reshape(-1), reduction="none").reshape_as(y)
    assert float(loss) == pytest.approx(float(ce.mean()), rel=1e-5)
    pr = scarcity_pressure_from_ce(ce.detach(), y, token_frequencies=freq, baseline=0.0)
    rare = (ce * pr).sum() / pr.sum().clamp_min(1.0)
    g_common = torch.autograd.grad(ce.mean(), list(m.parameters()), retain_graph=True, allow_unused=True)
    g_rare = torch.autograd.grad(rare, list(m.parameters()), allow_unused=True)
    for (n, p), gc, gr in zip(m.named_parameters(), g_common, g_rare):
        if gc is None:
            assert p.grad is None
            continue
        assert torch.allclose(p.grad, gc, rtol=1e-4, atol=1e-6), n
        assert torch.allclose(pending.rare_map[n], gr, rtol=1e-4, atol=1e-6), n
    keys = [k for k, _ in pending.channel_pressure_items]
    assert keys == sorted(keys) and set(keys) <= S.activation_keys(opt) and len(keys) >= 6
    for _, v in pending.channel_pressure_items:
        assert v.shape == (32,) and bool((v >= 0).all())
    assert pending.row_pressure.shape == (64,) and pending.pressure_stats["max"] >= pending.pressure_stats["mean"] >= 0


def test_non_split_steps_stage_nothing_and_hooks_are_removed():
    m, opt, freq = _setup()
    tok = torch.randint(0, 64, (2, 9))
    _, pending = S.run_scopt_train_step(model=m, optimizer=opt, inputs=tok[:, :-1], targets=tok[:, 1:], step=1,
                                        split_interval=4, token_frequencies=freq, precision="fp32",
                                        lm_head_backward_mode="single")
    assert pending is None and all(p.grad is not None for n, p in m.named_parameters() if "lm_head" in n)
    assert all(not mod._forward_hooks and not mod._forward_pre_hooks for mod in m.modules())
    assert S.should_run_split_step(opt, step=8, split_interval=4) and not S.should_run_split_step(opt, step=9, split_interval=4)


def test_commit_after_clip_contract():
    m, opt, freq = _setup()
    tok = torch.randint(0, 64, (2, 9))
    base = FrequencyBucketBaseline(freq, num_buckets=4)
    _, pending = S.run_scopt_train_step(model=m, optimizer=opt, inputs=tok[:, :-1], targets=tok[:, 1:], step=0,
                                        split_interval=1, token_frequencies=freq, precision="fp32", baseline=base,
                                        lm_head_backward_mode="single")
    S.apply_pending(opt, pending, skip=True)                   # clipped: row pressure only
    assert opt._row_pressure_ema is not None and not opt._channel_pressure
    assert all("rare_grad_ema" not in opt.state[p] for p in m.parameters())
    S.apply_pending(opt, pending, skip=False)
    assert opt._channel_pressure and any("rare_grad_ema" in opt.state[p] for p in m.parameters())
    S.apply_pending(opt, None, skip=False)                     # nothing staged: no-op
    opt.step()                                                 # the optimizer consumes what was committed
    assert all(torch.isfinite(p).all() for p in m.parameters())


def _rank(rank, ws, port, outdir):
    torch.set_num_threads(1)      # several ranks share this machine's cores: no intra-op thread pools
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        m, opt, freq = _setup()
        g = torch.Generator().manual_seed(100 + rank)                       # different data per rank
        tok = torch.randint(0, 64, (2, 13), generator=g)
        _, pending = S.run_scopt_train_step(model=m, optimizer=opt, inputs=tok[:, :-1], targets=tok[:, 1:], step=0,
                                            split_interval=1, token_frequencies=freq, ddp_active=True, world_size=ws,
                                            precision="fp32", lm_head_backward_mode="single")
        parts = [m.lm_head.weight.grad.reshape(-1), pending.rare_map["layers.0.core.in_proj.weight"].reshape(-1),
                 pending.channel_pressure_items[0][1], pending.row_pressure]
        torch.save([p.clone() for p in parts], os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ranks_agree_on_everything_that_is_synchronised():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank, args=(2, port, d), nprocs=2, join=True)
        a, b = torch.load(os.path.join(d, "r0.pt")), torch.load(os.path.join(d, "r1.pt"))
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # and the synchronised values are averages, not one rank's own
    m, opt, freq = _setup()
    g = torch.Generator().manual_seed(100)
    tok = torch.randint(0, 64, (2, 13), generator=g)
    S.run_scopt_train_step(model=m, optimizer=opt, inputs=tok[:, :-1], targets=tok[:, 1:], step=0, split_interval=1,
                           token_frequencies=freq, precision="fp32", lm_head_backward_mode="single")
    assert not torch.allclose(m.lm_head.weight.grad.reshape(-1), a[0])
