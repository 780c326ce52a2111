"""Distributed Muon: ownership plan, gloo (CPU) equivalence with the replicated
optimizer, and the peer-memory path on 2 GPUs."""
import os
import socket
import tempfile

import pytest
import torch

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.parallel.dist_muon import DistributedMuon, plan_ownership
from chaoscontrol_b200.utils.arena import ParamArena


def _model(dtype=torch.float32, device="cpu", dim=32, vocab=64, layers=2):
    torch.manual_seed(0)
    return CareStudentLM(vocab_size=vocab, dim=dim, num_layers=layers).to(device=device, dtype=dtype)


def test_plan_covers_every_matrix_once_and_balances():
    arena = ParamArena.install(_model())
    for ws in (1, 2, 3, 8):
        plan = plan_ownership(arena, ws)
        for gi, g in enumerate(arena.muon_groups):
            seen = []
            for r in range(ws):
                a, b = plan.shards[r][gi]
                seen += list(range(a, b))
            assert sorted(seen) == list(range(g.count))
        owned = [(o, n) for o, n, w in plan.ranges if w >= 0]
        assert sum(n for _, n in owned) == sum(g.numel for g in arena.muon_groups)
        assert all(o % 8 == 0 and n % 8 == 0 for o, n, _ in plan.ranges)
        rep = [(o, n) for o, n, w in plan.ranges if w < 0]
        for a0, a1 in arena.adamw_ranges:
            assert any(o <= a0 and a1 <= o + n for o, n in rep)
    plan = plan_ownership(arena, 2)
    cost = [0.0, 0.0]
    for r in range(2):
        for gi, g in enumerate(arena.muon_groups):
            a, b = plan.shards[r][gi]
            cost[r] += (b - a) * g.shape[0] * g.shape[1] * min(g.shape)
    assert max(cost) / sum(cost) < 0.7


def _fake_grads(model, seed):
    g = torch.Generator().manual_seed(seed)
    for p in model.parameters():
        p.grad = torch.randn(p.shape, generator=g).to(p.dtype)


def _gloo_worker(rank, ws, port, outdir):
    torch.set_num_threads(1)      # several ranks share this machine's cores: no intra-op thread pools
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        model = _model()
        arena = ParamArena.install(model)
        opt = Muon(model.parameters(), lr=0.05, weight_decay=0.01)
        opt.bind_param_names(model.named_parameters())
        dm = DistributedMuon(opt, arena, grad_clip_norm=1.0)
        norms = []
        for step in range(3):
            _fake_grads(model, 1000 * step + rank)
            arena.grads_fresh = False
            norms.append(float(dm.step()))
        torch.save({"params": arena.flat_param.clone(), "norms": norms, "ns_calls": opt.ns_calls},
                   os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_match_replicated_muon():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_gloo_worker, args=(2, port, d), nprocs=2, join=True)
        outs = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    assert torch.equal(outs[0]["params"], outs[1]["params"])
    # reference: one process, averaged gradients, same clip, plain Muon
    model = _model()
    arena = ParamArena.install(model)
    opt = Muon(model.parameters(), lr=0.05, weight_decay=0.01)
    opt.bind_param_names(model.named_parameters())
    twin = _model()
    for step in range(3):
        _fake_grads(model, 1000 * step + 0)
        _fake_grads(twin, 1000 * step + 1)
        for p, q in zip(model.parameters(), twin.parameters()):
            p.grad = (p.grad + q.grad) / 2
        norm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in model.parameters()))
        assert float(norm) == pytest.approx(outs[0]["norms"][step], rel=1e-4)
        scale = min(1.0, 1.0 / (float(norm) + 1e-6))
        for p in model.parameters():
            p.grad.mul_(scale)
        opt.step()
    assert torch.allclose(outs[0]["params"], arena.flat_param, atol=2e-5)
    assert outs[0]["ns_calls"] < opt.ns_calls or outs[0]["ns_calls"] <= opt.ns_calls


def _gpu_worker(rank, ws, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device("cuda", rank))
    ok, msg = True, ""
    try:
        from chaoscontrol_b200.ops import _lib
        from chaoscontrol_b200.parallel.peer import PeerComm
        model = _model(torch.bfloat16, "cuda", dim=256, vocab=1024, layers=2)
        ref = _model(torch.bfloat16, "cuda", dim=256, vocab=1024, layers=2)
        arena = ParamArena.install(model)
        arena_ref = ParamArena.install(ref)
        comm = PeerComm.create(arena.flat_grad.numel())
        opt = Muon(model.parameters(), lr=0.02, weight_decay=0.01)
        opt.bind_param_names(model.named_parameters())
        dm = DistributedMuon(opt, arena, comm=comm, grad_clip_norm=1.0)
        assert dm._use_peer
        opt_ref = Muon(ref.parameters(), lr=0.02, weight_decay=0.01)
        opt_ref.bind_param_names(ref.named_parameters())
        opt_ref.bind_arena(arena_ref)
        for step in range(4):
            g = torch.Generator(device="cuda").manual_seed(17 * step + rank)
            grads = torch.randn(arena.flat_grad.numel(), device="cuda", generator=g) * 0.01
            arena.flat_grad.copy_(grads)
            arena.grads_fresh = True
            norm = dm.step()
            # replicated reference: bf16-staged mean (what the pack kernel sends), NCCL sum, same clip
            gr = grads.bfloat16().float() / ws
            # the pack kernel scales before rounding
            gr = (grads / ws).bfloat16().float()
            dist.all_reduce(gr)
            n_ref = gr.norm()
            gr.mul_((1.0 / (n_ref + 1e-6)).clamp(max=1.0))
            arena_ref.flat_grad.copy_(gr)
            arena_ref.grads_fresh = True
            opt_ref.step()
            torch.cuda.synchronize()
            if abs(float(norm) - float(n_ref)) > 1e-3 * float(n_ref):
                ok, msg = False, f"step {step}: norm {float(norm)} vs {float(n_ref)}"
            # summation order differs from NCCL's: allow two bf16 ulps
            a, b = arena.flat_param.float(), arena_ref.flat_param.float()
            bad = ((a - b).abs() > 1e-3 + 2.0 ** -6 * b.abs()).sum().item()
            if bad:
                ok, msg = False, f"step {step}: {bad} parameters differ, max {(a - b).abs().max().item()}"
        chk = arena.flat_param.float().double().sum().reshape(1)
        gathered = [torch.zeros_like(chk) for _ in range(ws)]
        dist.all_gather(gathered, chk)
        if any(float(t) != float(gathered[0]) for t in gathered):
            ok, msg = False, "ranks hold different parameters"
        if _lib.read_status() != 0:
            ok, msg = False, f"status {_lib.read_status()}"
        # plain all-reduce still works after the sharded path (shared flags / epochs)
        y = torch.ones(arena.flat_grad.numel(), device="cuda")
        comm.all_reduce_(y, average=False)
        torch.cuda.synchronize()
        if float(y.min()) != ws or float(y.max()) != ws:
            ok, msg = False, "all-reduce after sharded sync is wrong"
        dist.barrier()
        comm.close()
    except Exception as exc:  # pragma: no cover
        import traceback
        ok, msg = False, f"{type(exc).__name__}: {exc} {traceback.format_exc()[-400:]}"
    finally:
        with open(os.path.join(outdir, f"r{rank}.txt"), "w") as f:
            f.write("OK" if ok else "FAIL " + msg)
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_distributed_muon_peer_path_two_gpus():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_gpu_worker, args=(2, port, d), nprocs=2, join=True)
        outs = [open(os.path.join(d, f"r{r}.txt")).read() for r in range(2)]
    assert all(o == "OK" for o in outs), outs
