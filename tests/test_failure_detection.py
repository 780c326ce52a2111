"""Failure detection without a GPU fault: the signal-pad protocol on host threads with injected
stalls, a rank that never joins a gloo collective, stop-flag and error-flag consensus."""
import ctypes as C
import os
import subprocess
import sys
import textwrap
import threading
import time
from pathlib import Path

import numpy as np
import pytest

from chaoscontrol_b200.episodic import native

ROOT = Path(__file__).resolve().parents[1]


def _lib():
    L = native.lib()
    L.ccbc_pad_words.restype = C.c_int64
    L.ccbc_pad_wait.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_int64]
    L.ccbc_pad_signal.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_uint32]
    L.ccbc_pad_allreduce.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint32,
                                     C.c_float, C.c_int64, C.c_int]
    return L


def _world(ws, n):
    L = _lib()
    words = int(L.ccbc_pad_words())
    pads = [np.zeros(words, np.uint32) for _ in range(ws)]
    stage = [np.zeros(n, np.float32) for _ in range(ws)]
    pad_ptrs = (C.c_void_p * ws)(*[p.ctypes.data for p in pads])
    stage_ptrs = (C.c_void_p * ws)(*[s.ctypes.data for s in stage])
    return L, pads, stage, pad_ptrs, stage_ptrs


def _run_ranks(ws, fn):
    out = [None] * ws
    ths = [threading.Thread(target=lambda r=r: out.__setitem__(r, fn(r))) for r in range(ws)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(30)
    assert not any(t.is_alive() for t in ths)
    return out


def test_allreduce_protocol_on_threads_is_exact_over_epochs():
    ws, n = 4, 1000
    L, pads, stage, pp, sp = _world(ws, n)
    rng = np.random.default_rng(0)
    for epoch in range(1, 6):
        grads = [rng.standard_normal(n).astype(np.float32) for _ in range(ws)]
        want = np.zeros(n, np.float32)
        for g in grads:
            want = want + g * np.float32(0.25)
        st = _run_ranks(ws, lambda r: L.ccbc_pad_allreduce(grads[r].ctypes.data, n, sp, pp, r, ws, epoch, 0.25,
                                                           2_000_000, -1))
        assert st == [0] * ws
        for g in grads:
            assert np.array_equal(g, grads[0]) and np.allclose(g, want, atol=1e-6)


def test_stalled_rank_times_out_on_every_survivor_and_context_stays_usable():
    ws, n = 3, 16
    L, pads, stage, pp, sp = _world(ws, n)
    grads = [np.ones(n, np.float32) for _ in range(ws)]

    def rank_fn(r):
        if r == 2:
            return "absent"                      # never packs, never signals
        t0 = time.time()
        st = L.ccbc_pad_allreduce(grads[r].ctypes.data, n, sp, pp, r, ws, 1, 1.0, 200_000, -1)
        return st, time.time() - t0

    out = _run_ranks(ws, rank_fn)
    for r in (0, 1):
        st, dt = out[r]
        assert st == 3 and 0.15 < dt < 5.0        # PEER_TIMEOUT, within the limit's order of magnitude
    # a withheld "done reading" signal shows up in the NEXT epoch's first wait
    L, pads, stage, pp, sp = _world(2, n)
    st = _run_ranks(2, lambda r: L.ccbc_pad_allreduce(grads[r].ctypes.data, n, sp, pp, r, 2, 1, 1.0, 500_000,
                                                      3 if r == 1 else -1))
    assert st == [0, 0]
    st = _run_ranks(2, lambda r: L.ccbc_pad_allreduce(grads[r].ctypes.data, n, sp, pp, r, 2, 2, 1.0, 200_000, -1))
    assert st[0] == 3


def test_stale_epoch_is_reported_not_waited_for():
    L, pads, stage, pp, sp = _world(2, 4)
    L.ccbc_pad_signal(pp, 2, 0, 0, 7)
    L.ccbc_pad_signal(pp, 2, 0, 1, 7)
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 0, 2, 7, 1000) == 0
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 0, 2, 6, 1000) == 0        # one behind is a legal overlap
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 0, 2, 3, 1000) == 4        # restarted rank with a lost counter
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 0, 2, 8, 1000) == 3
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 9, 2, 1, 1000) == 2
    # wrap-around: epochs compare as signed differences
    L.ccbc_pad_signal(pp, 2, 1, 0, 2)
    L.ccbc_pad_signal(pp, 2, 1, 1, 2)
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 1, 2, 0xFFFFFFFF, 1000) == 4
    L.ccbc_pad_signal(pp, 2, 2, 0, 0)
    L.ccbc_pad_signal(pp, 2, 2, 1, 0)
    assert L.ccbc_pad_wait(pads[0].ctypes.data, 2, 2, 0xFFFFFFFF, 1000) == 0   # 0 is one past 0xFFFFFFFF


def _torchrun(script: Path, nproc: int, port: int, timeout=240):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                          capture_output=True, text=True, timeout=timeout, env=env)


def test_rank_that_never_joins_a_collective_is_detected_by_its_peers(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(f"""
        import datetime, json, sys, time
        sys.path.insert(0, {str(ROOT)!r})
        import torch, torch.distributed as dist
        from chaoscontrol_b200.parallel.distributed import should_stop_now
        from chaoscontrol_b200.runner_fast_path import _control_barrier
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
        rank = dist.get_rank()
        ctl = dist.new_group([0, 1, 2], backend="gloo", timeout=datetime.timedelta(seconds=20))
        rec = dict()
        # 1. stop-flag consensus: one rank's wall clock ran out -> everybody stops together
        rec["stop"] = bool(should_stop_now(rank == 1, torch.device("cpu"), True))
        # 2. rank 2 leaves between steps (no collective in flight) and tells nobody
        if rank == 2:
            rec["left"] = True
        else:
            t0 = time.time()
            try:
                _control_barrier(ctl, "after-step", timeout_s=2.0)
                rec["barrier"] = "passed"
            except RuntimeError as exc:
                rec["barrier"] = "timeout" if "after-step" in str(exc) else "other: " + str(exc)[:200]
            rec["waited"] = time.time() - t0
        open({str(tmp_path)!r} + f"/rec{{rank}}.json", "w").write(json.dumps(rec))
        if rank == 2:
            time.sleep(6)       # stay alive (silent) while the others time out, then exit cleanly
    """))
    import json
    r = _torchrun(script, 3, 29641)
    recs = [json.loads((tmp_path / f"rec{i}.json").read_text()) for i in range(3)]
    assert all(x["stop"] for x in recs)
    for i in (0, 1):
        assert recs[i]["barrier"] == "timeout", (recs[i], r.stderr[-1500:])
        assert 1.5 < recs[i]["waited"] < 15
    assert recs[2]["left"]
