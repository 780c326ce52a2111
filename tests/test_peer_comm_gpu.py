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
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=torch.device("cuda", rank))
    ok = True
    msg = ""
    try:
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
        dist.barrier()
        comm.close()
    except Exception as exc:  # pragma: no cover
        ok, msg = False, f"{type(exc).__name__}: {exc}"
    finally:
        with open(os.path.join(outdir, f"r{rank}.txt"), "w") as f:
            f.write("OK" if ok else "FAIL " + msg)
        dist.destroy_process_group()


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
