"""Gradient exchange modes of the training step: one reduce after backward, or per-parameter reduces that
overlap backward.  Two gloo ranks on CPU; both modes must give the same parameters (CPU)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.parallel.distributed import AsyncGradAllReducer
from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
from chaoscontrol_b200.train_ssm import train_ssm_step


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, ws, port, outdir):
    torch.set_num_threads(1)      # several ranks share this machine's cores: no intra-op thread pools
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        out = {}
        tokens = torch.randint(0, 64, (3000,), dtype=torch.int16, generator=torch.Generator().manual_seed(0))
        for mode in ("bulk", "async_param"):
            torch.manual_seed(7)                                        # same init on both ranks and in both modes
            model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
            optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-2, weight_decay=0.0), model)
            res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=3000, stride=8, seq_len=16,
                                        batch_size=4, device=torch.device("cpu"), optimizer=optim, budget_seconds=600.0,
                                        precision="fp32", stop_check_interval=1, max_steps=3, rank=rank, world_size=ws,
                                        lm_head_backward_mode="fused", prefetch_batches=False, seed=3,
                                        grad_allreduce_mode=mode)
            out[mode] = {"sd": {k: v.clone() for k, v in model.state_dict().items()}, "loss": res["loss_history"],
                         "mode": res["grad_allreduce_mode"],
                         "hooks": sum(len(p._post_accumulate_grad_hooks or {}) for p in model.parameters())}
        # the reducer by itself: gradients become the rank mean, hooks go away on close
        lin = torch.nn.Linear(3, 2)
        with torch.no_grad():
            lin.weight.fill_(1.0)
            lin.bias.fill_(0.0)
        red = AsyncGradAllReducer(lin, ws)
        lin(torch.full((1, 3), float(rank + 1))).sum().backward()
        red.wait()
        out["reducer_grad"] = lin.weight.grad.clone()
        red.close()
        lin.zero_grad()
        lin(torch.full((1, 3), float(rank + 1))).sum().backward()
        out["after_close_grad"] = lin.weight.grad.clone()
        torch.save(out, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_async_param_matches_bulk_on_two_ranks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank, args=(2, _port(), d), nprocs=2, join=True)
        r0, r1 = (torch.load(os.path.join(d, f"r{i}.pt")) for i in range(2))
    for mode in ("bulk", "async_param"):
        assert r0[mode]["mode"] == mode and r0[mode]["hooks"] == 0        # the loop removed its hooks
        for k in r0[mode]["sd"]:
            assert torch.equal(r0[mode]["sd"][k], r1[mode]["sd"][k]), (mode, k)
    for k in r0["bulk"]["sd"]:
        assert torch.allclose(r0["bulk"]["sd"][k], r0["async_param"]["sd"][k], atol=1e-6), k
    assert r0["bulk"]["loss"] == pytest.approx(r0["async_param"]["loss"], abs=1e-6)
    assert r0["bulk"]["loss"] != r1["bulk"]["loss"]                       # the ranks did see different batches
    assert torch.allclose(r0["reducer_grad"], torch.full((2, 3), 1.5)) and torch.equal(r0["reducer_grad"], r1["reducer_grad"])
    assert torch.allclose(r0["after_close_grad"], torch.full((2, 3), 1.0)) and torch.allclose(r1["after_close_grad"], torch.full((2, 3), 2.0))


def _loop(**kw):
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    optim = _build_optimizer(dict(optimizer=kw.pop("opt", "adamw"), base_lr=1e-3), model)
    tokens = torch.randint(0, 64, (600,), dtype=torch.int16)
    return train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=600, stride=8, seq_len=16, batch_size=4,
                                 device=torch.device("cpu"), optimizer=optim, budget_seconds=60.0, precision="fp32",
                                 max_steps=1, prefetch_batches=False, lm_head_backward_mode="fused", **kw)


def test_mode_is_validated_and_recorded():
    assert _loop(grad_allreduce_mode="async_param")["grad_allreduce_mode"] == "async_param"   # one rank: nothing to do
    assert _loop()["grad_allreduce_mode"] == "bulk"
    with pytest.raises(ValueError, match="grad_allreduce_mode"):
        _loop(grad_allreduce_mode="ring")


@pytest.mark.parametrize("kw,name", [(dict(crct_enabled=True), "crct_enabled"), (dict(dreamworld_enabled=True), "dreamworld_enabled"),
                                     (dict(distributed_muon=True), "distributed_muon"),
                                     (dict(predictive_aux_weight=0.1, predictive_aux_horizon=2), "predictive_aux_weight")])
def test_async_param_refuses_steps_with_more_than_one_gradient_source(kw, name):
    with pytest.raises(ValueError, match=name):
        _loop(grad_allreduce_mode="async_param", **kw)


def test_scopt_requires_bulk():
    with pytest.raises(ValueError, match="requires grad_allreduce_mode='bulk'"):
        _loop(opt="scopt", grad_allreduce_mode="async_param")


def test_step_function_checks_its_arguments():
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=1)
    x = torch.randint(0, 64, (2, 8))
    with pytest.raises(ValueError, match="grad_allreduce_mode"):
        train_ssm_step(model, x, x, 4, precision="fp32", grad_allreduce_mode="tree")
    with pytest.raises(ValueError, match="single backward pass"):
        train_ssm_step(model, x, x, 4, precision="fp32", lm_head_backward_mode="chunked", grad_allreduce_mode="async_param")
    with pytest.raises(ValueError, match="AsyncGradAllReducer instance"):
        train_ssm_step(model, x, x, 4, precision="fp32", lm_head_backward_mode="single", ddp_active=True, world_size=2,
                       grad_allreduce_mode="async_param")
    loss = train_ssm_step(model, x, x, 4, precision="fp32", lm_head_backward_mode="single", grad_allreduce_mode="async_param")
    assert torch.isfinite(loss)                                           # not distributed: the mode is inert
