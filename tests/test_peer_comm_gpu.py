"""NVLink peer-memory all-reduce (csrc/comm.cu).

* single GPU: the bounded flag wait runs out on a flag nothing sets and reports
  through the status word; the context stays usable (no fault, no hang);
* two GPUs (child processes, NVLS off): one-shot and two-shot kernels against
  an NCCL all-reduce, several rounds in a row to exercise the epoch flags.
"""
import os
import socket
import tempfile

import pytest
import torch

from chaoscontrol_b200.ops import _lib

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_reports():
    from chaoscontrol_b200.parallel import peer  # registers signatures
    L = _lib.lib()
    _lib.read_status(reset=True)
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _lib.check(L.ccb_comm_wait_probe(flag.data_ptr(), 5, 50, res.data_ptr(), _lib.stream_ptr()), "probe")
    torch.cuda.synchronize()
    assert int(res.item()) == 0
    assert _lib.read_status(reset=True) == 3          # CCB_ERR_PEER_TIMEOUT
    # a satisfied flag passes, and the context is still healthy
    flag.fill_(7)
    _lib.check(L.ccb_comm_wait_probe(flag.data_ptr(), 5, 50, res.data_ptr(), _lib.stream_ptr()), "probe")
    torch.cuda.synchronize()
    assert int(res.item()) == 1 and _lib.read_status() == 0
    assert torch.ones(8, device="cuda").sum().item() == 8


def _worker(rank, ws, port, outdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import traceback
    import torch.distributed as dist
    ok = True
    msg = ""
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device("cuda", rank))
        from chaoscontrol_b200.parallel.peer import PeerComm
        n = 1 << 20
        comm = PeerComm.create(n)
        assert comm is not None
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        for rnd in range(4):
            x = torch.randn(n, device="cuda", generator=g)
            ref = x.bfloat16().float() / ws          # what the kernel packs
            dist.all_reduce(ref)
            for mode in (0, 1):
                y = x.clone()
                comm.all_reduce_(y, average=True, mode=mode)
                torch.cuda.synchronize()
                err = (y - ref).abs().max().item()
                if err > 2e-2:
                    ok, msg = False, f"round {rnd} mode {mode} err {err}"
        # identical bits on every rank
        y = torch.randn(n, device="cuda", generator=g)
        comm.all_reduce_(y)
        chk = y.double().sum().reshape(1)
        gathered = [torch.zeros_like(chk) for _ in range(ws)]
        dist.all_gather(gathered, chk)
        if any(float(t) != float(gathered[0]) for t in gathered):
            ok, msg = False, "ranks disagree bitwise"
        st = _lib.read_status()
        if st != 0:
            ok, msg = False, f"status {st}"
        # --- bucketed exchange on a side stream: disjoint ranges, one epoch each -------------
        x = torch.randn(n, device="cuda", generator=g)
        ref = x.bfloat16().float() / ws
        dist.all_reduce(ref)
        table = comm.make_ranges([(0, 4096, -1), (8192, 65536, -1), (4096, 4096, -1), (73728, n - 73728, -1)])
        side = torch.cuda.Stream()
        y = x.clone()
        ev = torch.cuda.Event()
        ev.record()
        side.wait_event(ev)
        for r0, r1, blocks in ((0, 1, 4), (1, 3, 8), (3, 4, 0)):
            comm.all_reduce_ranges_(y, table, r0, r1, blocks=blocks, stream=side.cuda_stream)
        done = torch.cuda.Event()
        done.record(side)
        torch.cuda.current_stream().wait_event(done)
        torch.cuda.synchronize()
        err = (y - ref).abs().max().item()
        if err > 2e-2:
            ok, msg = False, f"bucketed exchange err {err}"
        # --- broadcast through the root's buffer ------------------------------------------------
        p = torch.full((n,), float(rank + 1), device="cuda").bfloat16()
        comm.broadcast_(p, src=1)
        torch.cuda.synchronize()
        if not bool((p == 2).all()):
            ok, msg = False, "broadcast did not deliver rank 1's values"
        # --- stop-flag consensus through the pads -------------------------------------------
        from chaoscontrol_b200.parallel import symm
        from chaoscontrol_b200.parallel.distributed import should_stop_now
        for want in (0, 1, 0, 3, 7):
            got = comm.flag_max(want if rank == 1 else 0)
            if got != want:
                ok, msg = False, f"flag_max gave {got}, wanted {want}"
        symm.set_active_comm(comm)
        dev = torch.device("cuda", rank)
        if should_stop_now(False, dev, True) or not should_stop_now(rank == 0, dev, True):
            ok, msg = False, "should_stop_now consensus wrong"
        # --- a rank skips one collective: the other times out, nothing is touched, both resync ---
        comm.timeout_ms = 300
        z = torch.randn(n, device="cuda", generator=g)
        z0 = z.clone()
        if rank == 0:
            comm.all_reduce_(z)
            torch.cuda.synchronize()
            if not comm.timed_out():
                ok, msg = False, "missing peer did not produce a timeout status"
            if not torch.equal(z, z0):
                ok, msg = False, "a timed-out all-reduce modified the gradient"
        else:
            if comm.timed_out():
                ok, msg = False, "the rank that skipped reports a timeout"
        comm.resync()
        comm.timeout_ms = 2000
        for rnd in range(2):
            x = torch.randn(n, device="cuda", generator=g)
            ref = x.bfloat16().float() / ws
            dist.all_reduce(ref)
            comm.all_reduce_(x)
            torch.cuda.synchronize()
            err = (x - ref).abs().max().item()
            if err > 2e-2:
                ok, msg = False, f"after resync round {rnd} err {err}"
        # --- a reported timeout makes every rank raise on the same step --------------------
        from chaoscontrol_b200.parallel.peer import PeerCommError
        if rank == 0:
            _lib.check(_lib.lib().ccb_comm_wait_probe(torch.zeros(4, dtype=torch.int32, device="cuda").data_ptr(),
                                                      5, 20, torch.zeros(1, dtype=torch.int32, device="cuda").data_ptr(),
                                                      _lib.stream_ptr()), "probe")      # leaves status 3
        raised = False
        try:
            should_stop_now(False, dev, True)
        except PeerCommError:
            raised = True
        if not raised:
            ok, msg = False, "a timeout on rank 0 did not raise on this rank"
        symm.set_active_comm(None)
        comm.resync()
        if _lib.read_status() != 0:
            ok, msg = False, f"status {_lib.read_status()} after resync"
        dist.barrier()
        comm.close()
    except BaseException as exc:  # pragma: no cover
        ok, msg = False, f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"
    finally:
        with open(os.path.join(outdir, f"r{rank}.txt"), "w") as f:
            f.write("OK" if ok else "FAIL " + msg)
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # pragma: no cover
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_peer_allreduce_two_gpus():
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, port, d), nprocs=2, join=True)
        outs = [open(os.path.join(d, f"r{r}.txt")).read() for r in range(2)]
    assert all(o == "OK" for o in outs), outs


def _graph_worker(rank, ws, port, outdir, overlap):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      CCB_GRAD_OVERLAP="1" if overlap else "0")
    import torch.distributed as dist
    ok, msg = True, ""
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device("cuda", rank))
        from chaoscontrol_b200.models.model import CareStudentLM
        from chaoscontrol_b200.optim.muon import Muon
        from chaoscontrol_b200.parallel import symm_comm
        from chaoscontrol_b200.parallel.distributed import broadcast_params, clip_arena_grad_norm
        from chaoscontrol_b200.train_ssm import GraphedTrainStep, train_ssm_step
        from chaoscontrol_b200.utils.arena import ParamArena

        def build():
            torch.manual_seed(0)
            m = CareStudentLM(vocab_size=2048, dim=256, num_layers=2, ff_mult=2).cuda().to(torch.bfloat16)
            arena = ParamArena.install(m)
            m.train()
            opt = Muon(m.parameters(), lr=0.02, weight_decay=0.01, adamw_lr=0.02, adamw_weight_decay=0.01, fused=True)
            opt.bind_arena(arena)
            return m, arena, opt

        g = torch.Generator().manual_seed(10 + rank)              # every rank trains on its own batches
        batches = [torch.randint(0, 2048, (16, 257), generator=g).cuda() for _ in range(6)]
        m1, a1, o1 = build()
        symm_comm.enable(a1.flat_grad.numel())
        broadcast_params(m1)
        from chaoscontrol_b200.parallel.grad_overlap import reducer_for
        from chaoscontrol_b200.train_ssm import _engine_for
        if (reducer_for(_engine_for(m1), ws) is not None) != bool(overlap):
            ok, msg = False, "CCB_GRAD_OVERLAP did not select the exchange"
        for b in batches:                                           # eager: exchange (overlapped or not), then clip
            train_ssm_step(m1, b[:, :-1], b[:, 1:], 64, ddp_active=True, world_size=ws, precision="bf16",
                           lm_head_backward_mode="fused_streaming_cached")
            clip_arena_grad_norm(a1, 1.0)
            o1.step()
        m2, a2, o2 = build()
        broadcast_params(m2)
        step = GraphedTrainStep(m2, ddp_active=True, world_size=ws, grad_clip_norm=1.0, eager_steps=2)
        for b in batches:                                           # two eager steps, then graph replays
            step(b[:, :-1], b[:, 1:])
            o2.step()
        torch.cuda.synchronize()
        if step.graph is None or step.replays != 4:
            ok, msg = False, f"graph not used (graph {step.graph}, replays {step.replays})"
        if not torch.equal(a1.flat_param, a2.flat_param):
            d = (a1.flat_param.float() - a2.flat_param.float()).abs().max().item()
            ok, msg = False, f"graphed DDP steps differ from eager ones (max {d})"
        chk = a2.flat_param.float().double().sum().reshape(1)
        gathered = [torch.zeros_like(chk) for _ in range(ws)]
        dist.all_gather(gathered, chk)
        if any(float(t) != float(gathered[0]) for t in gathered):
            ok, msg = False, "replicas disagree after graphed DDP steps"
        if _lib.read_status() != 0:
            ok, msg = False, f"status {_lib.read_status()}"
        dist.barrier()
        symm_comm.disable()
    except BaseException as exc:  # pragma: no cover
        import traceback
        ok, msg = False, f"{type(exc).__name__}: {exc} {traceback.format_exc()[-1200:]}"
    finally:
        with open(os.path.join(outdir, f"r{rank}.txt"), "w") as f:
            f.write("OK" if ok else "FAIL " + msg)
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # pragma: no cover
            pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("overlap", [False, True], ids=["one_exchange", "overlapped_buckets"])
def test_graphed_data_parallel_step_two_gpus(overlap):
    """The whole data-parallel step (peer-memory exchange included: one exchange after backward, or the
    bucketed exchange overlapped with it) replayed from a CUDA graph gives the same parameter bits as
    the eager steps, on every rank."""
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_graph_worker, args=(2, port, d, overlap), nprocs=2, join=True)
        outs = [open(os.path.join(d, f"r{r}.txt")).read() for r in range(2)]
    assert all(o == "OK" for o in outs), outs
