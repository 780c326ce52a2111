#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the 4-layer x 256-d, V=16384
diagonal-SSM LM (seq 512, batch 1024 per rank, bf16, Muon lr 0.064, weight
decay 0.01, grad clip 1.0) on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

For N > 1 launch one rank per GPU with ``python -m torch.distributed.run``.
Rank 0 prints one JSON line.  ``value`` is the whole-job tokens/s with the
step's inputs already resident on the device (CUDA-event timed, max over
ranks); ``e2e`` repeats the measurement through the public training API with a
pinned-host -> device copy of every step's batch and a device -> host read of
every step's loss inside the timed region.

``--impl reference`` runs the unmodified reference package installed under
``baseline/_ref`` through its own ``train_ssm_step`` / ``Muon`` /
``clip_grad_norm_fused`` on the same model, data and schedule.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
BASELINE_TOKS_8XH100 = 25_023_217.0          # reference headline, 8 x H100 aggregate
BASELINE_TOKS_1XH100 = 3_214_781.0           # reference headline, 1 x H100

VOCAB, DIM, LAYERS, FF_MULT = 16384, 256, 4, 2
SEQ, BATCH = 512, 1024
LR, WD, CLIP = 0.064, 0.01, 1.0

# --config: the headline (default) and the two other training configurations that are benchmarked
CONFIGS = {
    "submission": dict(dim=256, layers=4, ff_mult=2, seq=512, batch=1024, dist_muon=False, fp8=False),
    # ~57.7 M parameters; gradients exchanged by the sharded reduce -> owner-side Muon -> parameter gather
    "scaled": dict(dim=512, layers=12, ff_mult=4, seq=2048, batch=128, dist_muon=True, fp8=False),
    # the submission trunk with every trunk linear in fp8: ours = block-scaled e4m3 (1x128 / 128x128 scales,
    # cast fused into the RMSNorm producer), reference = its per-tensor cuBLASLt path
    "fp8": dict(dim=256, layers=4, ff_mult=2, seq=512, batch=1024, dist_muon=False, fp8=True),
    # streaming score-only evaluation: 50,000 synthetic documents (lognormal lengths, median 700, sigma 1,
    # clipped to [32, 32768]) sharded over the ranks, 512-token chunks, state carried inside a document
    "eval": dict(dim=256, layers=4, ff_mult=2, seq=512, batch=1024, dist_muon=False, fp8=False),
    # test-time-training evaluation: every 256-token chunk is scored, then one SGD step on log_a and the delta
    # projection is taken on it from the same carried state; adapted weights are restored after each document
    "eval_ttt": dict(dim=256, layers=4, ff_mult=2, seq=512, batch=1024, dist_muon=False, fp8=False),
    # both implementations from identical initial weights on identical batches: per-step loss curves
    "parity": dict(dim=256, layers=4, ff_mult=2, seq=512, batch=1024, dist_muon=False, fp8=False),
}


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--seq", type=int, default=SEQ, help=argparse.SUPPRESS)
    ap.add_argument("--no-e2e", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--no-graph", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--scan-arith", type=int, default=-1, choices=[-1, 0, 1, 2], help=argparse.SUPPRESS)
    ap.add_argument("--gemm-pdl", type=int, default=-1, choices=[-1, 0, 1], help=argparse.SUPPRESS)
    ap.add_argument("--gemm-pres", type=int, default=-1, choices=[-1, 0, 1, 2, 3], help=argparse.SUPPRESS)
    ap.add_argument("--config", default="submission", choices=sorted(CONFIGS), help=argparse.SUPPRESS)
    a = ap.parse_args()
    cfg = CONFIGS[a.config]
    global DIM, LAYERS, FF_MULT
    DIM, LAYERS, FF_MULT = cfg["dim"], cfg["layers"], cfg["ff_mult"]
    if a.config != "submission":
        if a.batch == BATCH:
            a.batch = cfg["batch"]
        if a.seq == SEQ:
            a.seq = cfg["seq"]
    a.dist_muon = bool(cfg["dist_muon"])
    # defaults: the headline protocol (200 timed steps after 20 warm-up); the other configurations
    # have longer steps (a whole evaluation pass is one step) and get counts that end within minutes
    d_steps, d_warm = {"submission": (200, 20), "fp8": (100, 10), "scaled": (50, 10), "eval": (5, 3),
                       "eval_ttt": (5, 3), "parity": (200, 0)}[a.config]
    if a.steps is None:
        a.steps = d_steps
    if a.warmup is None:
        a.warmup = d_warm
    return a


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._th = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.rows.append([c.strip() for c in out.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._th.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._th.join(timeout=6)

    def summary(self) -> dict:
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def _make_batches(n_steps: int, batch: int, seq: int, rank: int, distinct: int = 8):
    """Pinned-host int64 Zipf(1.1) windows, one [batch, seq + 1] block per step, per-rank seed
    (``distinct`` different blocks, cycled)."""
    import numpy as np
    import torch
    ranks = np.arange(1, VOCAB + 1, dtype=np.float64)
    cdf = np.cumsum(ranks ** (-1.1))
    cdf /= cdf[-1]
    rng = np.random.default_rng(1234 + rank)
    n_distinct = min(n_steps, distinct)
    blocks = []
    for _ in range(n_distinct):
        ids = np.searchsorted(cdf, rng.random(batch * (seq + 1)), side="left").clip(0, VOCAB - 1)
        t = torch.from_numpy(ids.astype(np.int64)).view(batch, seq + 1)
        blocks.append(t.pin_memory() if torch.cuda.is_available() else t)
    return [blocks[i % n_distinct] for i in range(n_steps)]


def _train_config(args, ws: int, nparams: int, sharded_muon: bool) -> dict:
    """The workload description, printed identically by both arms (``--impl ours|reference``)."""
    return {"model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}", "params": int(nparams),
            "global_batch": ws * args.batch, "seq_len": args.seq,
            "parallelism": f"dp{ws}" + (" + Muon sharded by matrix ownership" if sharded_muon else ""),
            "optimizer": f"Muon lr {LR} wd {WD} clip {CLIP}",
            "l2": "working set per step (>10 GB of activations) exceeds the 126 MB L2"}


def _dist_setup(args):
    import torch
    import torch.distributed as dist
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if ws > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if ws != args.gpus and rank == 0:
        print(f"[bench] note: WORLD_SIZE={ws} differs from --gpus {args.gpus}; using WORLD_SIZE",
              file=sys.stderr)
    return rank, local, ws


def _max_over_ranks(ms: float, ws: int) -> float:
    if ws == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _barrier(ws: int):
    import torch
    if ws > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def _timed(fn_step, n: int, ws: int) -> float:
    """ms per step over exactly n steps, CUDA events, barrier + sync on both sides, max over ranks."""
    import torch
    _barrier(ws)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fn_step(i)
    e1.record()
    _barrier(ws)
    return _max_over_ranks(e0.elapsed_time(e1), ws) / n


class _E2EFeeder:
    """The end-to-end loop of either arm: the next batch is copied from pinned host memory on a copy
    stream while the current step computes (two device buffers), and every step's loss is copied to
    pinned host memory asynchronously and read by the host one step later, so the host never blocks
    on the step it has just launched.  ``run_step(block) -> loss tensor`` is the arm's own step."""

    FEEDING = ("batch copied from pinned host memory on a copy stream one step ahead (two device buffers); "
               "loss copied to pinned host memory every step and read by the host one step later")

    def __init__(self, host_batches, dev, run_step):
        import torch
        self.torch, self.host, self.run_step = torch, host_batches, run_step
        self.copy_stream = torch.cuda.Stream()
        self.dev_buf = [torch.empty_like(host_batches[0], device=dev) for _ in range(2)]
        self.filled = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        self.host_loss = torch.zeros(2, dtype=torch.float32).pin_memory()
        self.loss_done = [torch.cuda.Event() for _ in range(2)]
        self.read: list[float] = []
        for ev in self.consumed:
            ev.record()
        self._prefetch(0)
        self.k = 0

    def _prefetch(self, i):
        torch, j = self.torch, i % 2
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[j])
            self.dev_buf[j].copy_(self.host[i % len(self.host)], non_blocking=True)
            self.filled[j].record(self.copy_stream)

    def step(self, _i=None):
        torch, k = self.torch, self.k
        torch.cuda.current_stream().wait_event(self.filled[k % 2])
        loss = self.run_step(self.dev_buf[k % 2])
        self.consumed[k % 2].record()
        self._prefetch(k + 1)
        if k >= 1:                                   # the previous step's loss has had a whole step to arrive
            self.loss_done[(k - 1) % 2].synchronize()
            self.read.append(float(self.host_loss[(k - 1) % 2]))
        self.host_loss[k % 2: k % 2 + 1].copy_(loss.detach().float().reshape(1), non_blocking=True)
        self.loss_done[k % 2].record()
        self.k += 1


# ---------------------------------------------------------------------------
def run_ours(args):
    import torch
    sys.path.insert(0, str(ROOT))
    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.optim.muon import Muon
    from chaoscontrol_b200.parallel.distributed import (allreduce_grads, broadcast_params,
                                                        clip_arena_grad_norm)
    from chaoscontrol_b200.train_ssm import GraphedTrainStep, _engine_for, train_ssm_step
    from chaoscontrol_b200.utils.arena import ParamArena

    rank, local, ws = _dist_setup(args)
    dev = torch.device("cuda", local)
    if args.scan_arith >= 0:                  # A/B switch of the scan kernels' arithmetic (same box, same run)
        _lib.lib().ccb_scan_poly_exp(args.scan_arith)
    if args.gemm_pdl >= 0:
        _lib.lib().ccb_gemm_pdl(args.gemm_pdl)
    if args.gemm_pres >= 0:
        _lib.lib().ccb_gemm_pair_resident(args.gemm_pres)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT)
    model = model.to(dev).to(torch.bfloat16)
    arena = ParamArena.install(model)
    model.train()
    collective = "none (one GPU)"
    if ws > 1:
        # the product is the in-kernel peer-memory exchange: refuse to time a library fallback
        from chaoscontrol_b200.parallel import symm_comm
        symm_comm.enable(arena.flat_grad.numel())
        broadcast_params(model)
    opt = Muon(model.parameters(), lr=LR, weight_decay=WD, adamw_lr=LR, adamw_weight_decay=WD, fused=True)
    opt.bind_arena(arena)
    engine = _engine_for(model)
    if engine is None:
        raise RuntimeError("kernel training engine unavailable: refusing to bench a fallback path")
    reducer = None
    if ws > 1 and not args.dist_muon:
        from chaoscontrol_b200.parallel.grad_overlap import reducer_for
        reducer = reducer_for(engine, ws)
        from chaoscontrol_b200.parallel import symm
        if symm.active_comm(None) is None:
            raise RuntimeError("peer-memory gradient exchange unavailable: refusing to bench a fallback")
        from chaoscontrol_b200.parallel.peer import ONE_SHOT_MAX_BYTES
        forced = os.environ.get("CCB_ALLREDUCE_MODE")
        two = forced == "1" or (forced != "0" and arena.flat_grad.numel() * 2 > ONE_SHOT_MAX_BYTES)
        kind = "peer-twoshot (reduce-scatter + all-gather)" if two else "peer-oneshot"
        if reducer is None:
            collective = f"{kind} over CUDA-IPC symmetric buffers, one exchange after backward"
        else:
            collective = (f"peer-oneshot over CUDA-IPC symmetric buffers, {reducer.n_buckets} buckets overlapped "
                          "with backward")
    elif ws > 1:
        collective = "peer-memory reduce of owned ranges + parameter gather (distributed Muon)"
    dist_opt = None
    if args.dist_muon and ws > 1:
        from chaoscontrol_b200.parallel import symm
        from chaoscontrol_b200.parallel.dist_muon import DistributedMuon
        dist_opt = DistributedMuon(opt, arena, comm=symm.active_comm(None), grad_clip_norm=CLIP)

    n_total = args.warmup + args.steps
    host = _make_batches(n_total, args.batch, args.seq, rank)
    dev_batches = [h.to(dev) for h in host[:8]]
    dev_in = [b[:, :-1].to(torch.int32).contiguous() for b in dev_batches]
    dev_tg = [b[:, 1:].contiguous() for b in dev_batches]
    losses = []

    # the public graphed step: forward, backward, the overlapped gradient exchange and the clip are one
    # CUDA graph after two eager steps; the optimizer step stays eager (distributed Muon: all eager)
    gstep = None
    if dist_opt is None and not args.no_graph:
        gstep = GraphedTrainStep(model, chunk_size=64, ddp_active=ws > 1, world_size=ws, precision="bf16",
                                 lm_head_backward_mode="fused_streaming_cached", lm_head_tile_size=8192,
                                 grad_clip_norm=CLIP)

    def step_resident(i):
        j = i % len(dev_in)
        if gstep is not None:
            loss = gstep(dev_in[j], dev_tg[j])
            opt.step()
        else:
            loss = engine.step(dev_in[j], dev_tg[j], reducer=reducer)
            if dist_opt is not None:
                dist_opt.step()
            else:
                if ws > 1:
                    allreduce_grads(model, ws)           # no-op: the reducer ran inside the step
                clip_arena_grad_norm(arena, CLIP)
                opt.step()
        losses.append(loss.detach().clone() if gstep is not None else loss)

    for i in range(args.warmup):
        step_resident(i)
    _lib.assert_ok()
    l0 = _lib.launch_count()
    r0 = gstep.replays if gstep is not None else 0
    with ClockSampler(local) as cs:
        ms = _timed(step_resident, args.steps, ws)
    launches = _lib.launch_count() - l0
    if gstep is not None:      # kernels replayed from the graph are launches too (counted at capture)
        launches += (gstep.replays - r0) * gstep.launches_per_replay
    _lib.assert_ok()
    final_loss = float(torch.stack(losses[-args.steps:]).float().mean().item())

    # end to end through the public API: H2D of the batch and D2H of the loss every step
    e2e = None
    if not args.no_e2e:
        h2d = host[0].numel() * host[0].element_size()

        def run_block(blk):
            inputs, targets = blk[:, :-1], blk[:, 1:]
            if gstep is not None:
                loss = gstep(inputs, targets)
                opt.step()
                return loss
            opt.zero_grad(set_to_none=True)
            loss = train_ssm_step(model, inputs, targets, 64, ddp_active=ws > 1 and dist_opt is None,
                                  world_size=ws, precision="bf16",
                                  lm_head_backward_mode="fused_streaming_cached", lm_head_tile_size=8192)
            if dist_opt is not None:
                dist_opt.step()
            else:
                clip_arena_grad_norm(arena, CLIP)
                opt.step()
            return loss

        feeder = _E2EFeeder(host, dev, run_block)
        step_e2e = feeder.step
        for i in range(max(3, args.warmup // 2)):
            step_e2e(i)
        ms_e = _timed(step_e2e, args.steps, ws)
        e2e = {"value": ws * args.batch * args.seq / (ms_e / 1e3), "unit": "tokens/s",
               "ms_per_step": ms_e, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "api": ("chaoscontrol_b200.train_ssm.GraphedTrainStep + Muon.step" if gstep is not None else
                       "chaoscontrol_b200.train_ssm.train_ssm_step + Muon.step"),
               "feeding": _E2EFeeder.FEEDING, "losses_read_on_host": len(feeder.read)}

    toks = ws * args.batch * args.seq / (ms / 1e3)
    headline = args.config == "submission"
    base = BASELINE_TOKS_8XH100 * ws / 8.0
    nparams = sum(p.numel() for p in model.parameters())
    out = {"metric": ("train tokens/sec, 4Lx256d V16384 SSM (seq 512, bs 1024/rank, bf16, Muon)" if headline else
                      f"train tokens/sec, {LAYERS}Lx{DIM}d V16384 SSM (seq {args.seq}, bs {args.batch}/rank, bf16, "
                      f"{'distributed ' if dist_opt is not None else ''}Muon)"),
           "value": toks, "unit": "tokens/s", "n_gpus": ws, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": toks / base if headline else None, "dtype": "bf16",
           "data": "synthetic Zipf(1.1) tokens, random-init weights",
           "impl": "ours", "final_loss": final_loss, "gpu_launches": launches,
           "clocks": cs.summary(), "e2e": e2e,
           "config": _train_config(args, ws, nparams, dist_opt is not None),
           "impl_detail": {"lm_head": ("fused tcgen05 linear+CE, logits recomputed in backward" if DIM == 256 else
                                       "tcgen05 GEMM-epilogue linear+CE (lse partials; chunked softmax-gradient tiles)"),
                           "collective": collective,
                           "cuda_graph": (f"forward + backward + exchange + clip replayed from one graph "
                                          f"({gstep.launches_per_replay} kernels); optimizer eager"
                                          if gstep is not None and gstep.graph is not None else "none"),
                           "vs_baseline_ref": "reference 8xH100 headline 25,023,217 tok/s scaled by n_gpus/8"}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if ws > 1:
        import torch.distributed as dist
        from chaoscontrol_b200.parallel import symm_comm
        symm_comm.disable()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
def run_eval(args):
    """Score-only streaming evaluation throughput (tokens scored per second, whole job).  One step =
    one pass of this rank's document shard through the chunked carried-state scorer."""
    import numpy as np
    import torch
    if args.impl == "reference":
        return run_eval_reference(args)
    sys.path.insert(0, str(ROOT))
    from chaoscontrol_b200.data import lognormal_doc_lengths, zipf_tokens
    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.scoring import assign_docs_lpt, score_docs
    rank, local, ws = _dist_setup(args)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16).eval()
    if not model.kernel_trunk_supported():
        raise RuntimeError("kernel scorer unavailable: refusing to bench a fallback path")
    n_docs, chunk = int(os.environ.get("BENCH_EVAL_DOCS", "50000")), 512
    lens_all = _eval_lengths(n_docs)
    mine = np.asarray(sorted(assign_docs_lpt(lens_all.tolist(), ws, chunk)[rank]), dtype=np.int64)
    lens = lens_all[mine]
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    host_tokens = zipf_tokens(int(lens.sum()), VOCAB, s=1.1, seed=1 + rank).to(torch.int32).pin_memory()
    dev_tokens = host_tokens.to(dev)
    total_targets = int(np.maximum(lens_all - 1, 0).sum())
    box = {}

    def step_resident(i):
        box["res"] = score_docs(model, dev_tokens, starts, lens, chunk_size=chunk, max_batch_tokens=1 << 19)

    def step_e2e(i):
        toks = host_tokens.to(dev, non_blocking=True)
        res = score_docs(model, toks, starts, lens, chunk_size=chunk, max_batch_tokens=1 << 19)
        box["e2e_ce"] = float(res.total_ce)          # per-document CE came back to the host inside score_docs

    for i in range(args.warmup):
        step_resident(i)
    _lib.assert_ok()
    l0 = _lib.launch_count()
    with ClockSampler(local) as cs:
        ms = _timed(step_resident, args.steps, ws)
    launches = _lib.launch_count() - l0
    _lib.assert_ok()
    for i in range(2):
        step_e2e(i)
    ms_e = _timed(step_e2e, args.steps, ws)
    toks = total_targets / (ms / 1e3)
    out = {"metric": f"eval tokens/sec, streaming score-only, 4Lx256d V16384 SSM ({n_docs:,} docs, 512-token chunks, carried state)",
           "value": toks, "unit": "tokens/s", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic Zipf(1.1) tokens in lognormal-length documents, random-init weights", "impl": "ours",
           "mean_ce": float(box["res"].total_ce / max(box["res"].total_tokens, 1)), "gpu_launches": launches,
           "clocks": cs.summary(),
           "e2e": {"value": total_targets / (ms_e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e,
                   "h2d_bytes_per_step": int(host_tokens.numel() * 4), "d2h_bytes_per_step": int(len(mine) * 8),
                   "api": "chaoscontrol_b200.scoring.score_docs"},
           "config": {"model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}", "docs": n_docs,
                      "tokens_scored_per_pass": total_targets, "chunk_size": chunk, "max_batch_tokens": 1 << 19,
                      "parallelism": f"documents split over {ws} rank(s) by longest-processing-time packing",
                      "l2": "each pass streams >200 MB of tokens and >10 GB of activations: larger than the 126 MB L2"}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if ws > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def _eval_lengths(n_docs: int):
    """Lognormal document lengths of the evaluation workload (median 700, sigma 1, clipped to
    [32, 32768], seed 0) -- the generator both arms use."""
    import numpy as np
    rng = np.random.default_rng(0)
    return np.clip(np.exp(rng.normal(np.log(700.0), 1.0, n_docs)), 32, 32768).astype(np.int64)


def run_eval_reference(args):
    """The reference's own streaming scorer (``scripts/run_exp20_fast_score.py``, copied unmodified
    beside the installed package under ``baseline/_ref/scripts``) on a synthetic validation cache of
    the same shape and a random-init checkpoint of the same architecture.  One step = one call of its
    ``run()``; the value uses the scoring-loop time the script itself reports (max over ranks), so its
    set-up (checkpoint load, token staging) is not counted against it."""
    import importlib.util
    import tempfile
    import numpy as np
    import torch
    ref = ROOT / "baseline" / "_ref"
    script = ref / "scripts" / "run_exp20_fast_score.py"
    if not (ref / "chaoscontrol").exists() or not script.exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref (package or scripts/run_exp20_fast_score.py) "
                          "is missing on this box"}))
        return
    sys.path.insert(0, str(ref))
    os.environ.setdefault("CHAOSCONTROL_DIAG_SCAN_BACKEND", "ssm_scan")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    try:
        spec = importlib.util.spec_from_file_location("ref_fast_score", script)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        from chaoscontrol.model import CareStudentLM as RefLM
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}))
        return
    ws = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    n_docs, chunk = int(os.environ.get("BENCH_EVAL_DOCS", "50000")), 512
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(local)
    work = Path(tempfile.mkdtemp(prefix=f"ccb_ref_eval_r{rank}_"))
    # validation cache in the reference's on-disk format (tokens.npy uint16, docs.npy records, manifest.json)
    lens = _eval_lengths(n_docs)
    ranks_ = np.arange(1, VOCAB + 1, dtype=np.float64)
    cdf = np.cumsum(ranks_ ** -1.1)
    cdf /= cdf[-1]
    toks = np.searchsorted(cdf, np.random.default_rng(1).random(int(lens.sum())), side="left").clip(0, VOCAB - 1)
    docs = np.zeros(n_docs, dtype=np.dtype([("doc_id", np.int64), ("token_start", np.int64), ("token_len", np.int64),
                                            ("raw_bytes", np.int64)]))
    docs["doc_id"] = np.arange(n_docs)
    docs["token_start"] = np.concatenate([[0], np.cumsum(lens)[:-1]])
    docs["token_len"] = lens
    docs["raw_bytes"] = np.maximum(1, lens * 3)
    cache_dir = work / "cache"
    cache_dir.mkdir(parents=True)
    np.save(cache_dir / "tokens.npy", toks.astype(np.uint16))
    np.save(cache_dir / "docs.npy", docs)
    (cache_dir / "manifest.json").write_text(json.dumps({
        "schema_version": 1, "request": {"synthetic": True}, "num_docs": n_docs, "total_tokens": int(lens.sum()),
        "total_raw_bytes": int(docs["raw_bytes"].sum()), "cache_content_sha256": "", "tokens_file": "tokens.npy",
        "docs_file": "docs.npy", "max_docs": n_docs}))
    # random-init checkpoint of the reference's own model class
    torch.manual_seed(0)
    cfg = dict(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT)
    m = RefLM(**cfg).to(torch.bfloat16)
    ckpt = work / "ckpt.pt"
    torch.save({"model": m.state_dict(), "config": cfg}, ckpt)
    del m
    argv = ["run_exp20_fast_score.py", "--cache-dir", str(cache_dir), "--checkpoint-path", str(ckpt),
            "--output-path", str(work / "out.jsonl"), "--summary-path", str(work / "summary.json"),
            "--chunk-size", str(chunk), "--doc-batch-size", "4096", "--max-forward-tokens", str(1 << 19),
            "--budget-seconds", "3600", "--device", "cuda" if on_gpu else "cpu"]
    total_targets = int(np.maximum(lens - 1, 0).sum())
    # the script scores the 50 000-document cache in about ten minutes on one B200 (it batches only chunks
    # of equal true length, so every ragged tail is a forward of its own): one pass is the measurement and
    # no warm-up pass is spent; smaller caches (BENCH_EVAL_DOCS) get up to three passes after one warm-up
    big = n_docs > 5000
    n_steps = 1 if big else max(1, min(args.steps, 3))
    n_warm = 0 if big else max(0, min(args.warmup, 1))
    results, wall = [], []
    try:
        for i in range(n_warm + n_steps):
            old = sys.argv
            sys.argv = argv
            try:
                a = mod.parse_args()
            finally:
                sys.argv = old
            if on_gpu:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            summ = mod.run(a)
            if on_gpu:
                torch.cuda.synchronize()
            wall.append(time.perf_counter() - t0)
            results.append(summ)
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference scorer failed: {type(exc).__name__}: {exc}"[:400]}))
        return
    timed = results[-n_steps:]
    sec = sum(float(r["elapsed_seconds"]) for r in timed) / n_steps
    scored = int(timed[-1]["tokens_scored"])
    out = {"metric": f"eval tokens/sec, streaming score-only, 4Lx256d V16384 SSM ({n_docs:,} docs, 512-token chunks, carried state)",
           "value": scored / sec, "unit": "tokens/s", "n_gpus": ws, "steps": n_steps, "warmup": len(results) - n_steps,
           "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic Zipf(1.1) tokens in lognormal-length documents, random-init weights", "impl": "reference",
           "timing": "elapsed_seconds of the script's own scoring loop (max over ranks by its own all-reduce); "
                     "whole run() calls, set-up included, in whole_call_ms",
           "whole_call_ms": [w * 1e3 for w in wall[-n_steps:]], "tokens_scored": scored, "targets_in_cache": total_targets,
           "aggregate_bpb": float(timed[-1].get("aggregate_bpb", float("nan"))),
           "e2e": {"value": scored / (sum(wall[-n_steps:]) / n_steps), "unit": "tokens/s",
                   "ms_per_step": sum(wall[-n_steps:]) / n_steps * 1e3, "h2d_bytes_per_step": int(lens.sum()) * 4,
                   "d2h_bytes_per_step": n_docs * 8,
                   "api": "scripts/run_exp20_fast_score.py run() (checkpoint load and token staging inside the call)"},
           "config": {"model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}", "docs": n_docs,
                      "tokens_scored_per_pass": scored, "chunk_size": chunk, "max_batch_tokens": 1 << 19,
                      "parallelism": f"documents split over {ws} rank(s) by the script's own packing "
                                     f"({timed[-1].get('rank_assignment')})",
                      "l2": "each pass streams >200 MB of tokens and >10 GB of activations: larger than the 126 MB L2"}}
    if rank == 0:
        print(json.dumps(out), flush=True)


# ---------------------------------------------------------------------------
def run_eval_ttt(args):
    """Score-then-adapt (test-time training) evaluation throughput, whole job.  One step = one pass of
    this rank's document shard: per 256-token chunk one scoring pass and one SGD step on ``log_a`` +
    the delta projection, state and adapted weights carried inside a document and reset at its end;
    many documents advance together (``eval_stream.batched_ttt``)."""
    import numpy as np
    import torch
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference's TTT driver (scripts/run_exp20_eval.py: "
                          "run(cfg, jsonl_paths, sp_model_path)) reads JSONL text and tokenises it with a SentencePiece "
                          "model inside its loop; no tokenizer model or text corpus exists offline and synthetic token "
                          "ids cannot be fed to it"}))
        return
    sys.path.insert(0, str(ROOT))
    from chaoscontrol_b200.data import lognormal_doc_lengths, zipf_tokens
    from chaoscontrol_b200.eval_stream.types import DocRecord
    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.scoring import assign_docs_lpt, run_ttt_eval_graph
    rank, local, ws = _dist_setup(args)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16)
    n_docs, chunk = 512, 256
    lens_all = lognormal_doc_lengths(n_docs, median=700.0, sigma=1.0, lo=32, hi=8192, seed=0)
    mine = sorted(assign_docs_lpt(lens_all.tolist(), ws, chunk)[rank])
    toks = zipf_tokens(int(lens_all[mine].sum()), VOCAB, s=1.1, seed=1 + rank).tolist()
    docs, off = [], 0
    for i in mine:
        n = int(lens_all[i])
        docs.append(DocRecord(doc_id=int(i), tokens=toks[off: off + n], raw_bytes=4 * n))
        off += n
    total_targets = int(np.maximum(lens_all - 1, 0).sum())
    from chaoscontrol_b200.eval_stream.batched_ttt import BatchedTTT, pick_slots, run_ttt_eval_batched
    box = {}
    slots = pick_slots([len(d.tokens) for d in docs], chunk)
    runner = BatchedTTT(model, adapt_set="log_a+delta_proj", chunk_size=chunk, slots=slots, lr=LR)
    doc_tokens = [d.tokens for d in docs]

    def one_pass_e2e(i):
        # host token lists in, per-document CE on the host out: plan + one pinned upload + replays + read-back
        box["res"] = run_ttt_eval_batched(model, docs, chunk_size=chunk, eval_lr=LR, runner=runner)

    def one_pass_device(i):
        box["ce"] = runner.execute()

    def one_pass_graph1(i):
        box["graph1"] = run_ttt_eval_graph(model, docs, adapt_set="log_a+delta_proj", chunk_size=chunk, eval_lr=LR)

    steps, warm = max(1, min(args.steps, 5)), max(3, min(args.warmup, 5))
    for i in range(warm):
        one_pass_e2e(i)
    runner.upload(doc_tokens)
    for i in range(warm):
        one_pass_device(i)
    l0 = _lib.launch_count()
    with ClockSampler(local) as cs:
        ms = _timed(one_pass_device, steps, ws)
    launches = _lib.launch_count() - l0
    ms_e2e = _timed(one_pass_e2e, steps, ws)
    _lib.assert_ok()
    one_pass_graph1(0)
    ms_graph1 = _timed(one_pass_graph1, 1, ws)
    res = box["res"]
    # kernels per replay: count one eager step on a scratch runner of the same shape
    probe = BatchedTTT(model, adapt_set="log_a+delta_proj", chunk_size=chunk, slots=slots, lr=LR, use_graph=False)
    probe.upload(doc_tokens[:1])
    l1 = _lib.launch_count()
    probe.execute()
    per_replay = (_lib.launch_count() - l1) // max(probe._steps, 1)
    out = {"metric": "eval tokens/sec, streaming test-time training (score then 1 SGD step per 256-token chunk), "
                     "4Lx256d V16384 SSM, 512 docs",
           "value": total_targets / (ms / 1e3), "unit": "tokens/s", "n_gpus": ws, "steps": steps,
           "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic Zipf(1.1) tokens in lognormal-length documents, random-init weights", "impl": "ours",
           "mean_ce": float(res["mean_ce"]), "adapt_steps_per_pass": int(res["adapt_steps"]),
           "chunks_per_pass": int(res["chunks_scored"]), "batched_steps_per_pass": int(res["batched_steps"]),
           "slots": int(slots),
           "one_document_at_a_time": {"value": total_targets / (ms_graph1 / 1e3), "unit": "tokens/s",
                                      "ms_per_step": ms_graph1, "mean_ce": float(box["graph1"]["mean_ce"]),
                                      "api": "chaoscontrol_b200.scoring.run_ttt_eval_graph (batch 1, one graph "
                                             "replay per chunk)"},
           "gpu_launches": int(launches + steps * res["batched_steps"] * per_replay), "clocks": cs.summary(),
           "e2e": {"value": total_targets / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": int(res["h2d_bytes"]), "d2h_bytes_per_step": len(docs) * 8,
                   "api": "chaoscontrol_b200.eval_stream.batched_ttt.run_ttt_eval_batched (documents arrive as host "
                          "token lists; the pass is planned on the host, uploaded as one pinned buffer, and the "
                          "per-document CE is read back once)"},
           "config": {"model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}", "docs": n_docs,
                      "tokens_scored_per_pass": total_targets, "chunk_size": chunk, "adapt_set": "log_a+delta_proj",
                      "steps_per_chunk": 1, "optimizer": "sgd", "persistence_mode": "reset",
                      "parallelism": f"documents split over {ws} rank(s) by longest-processing-time packing; "
                                     f"{slots} documents advance per step on each rank",
                      "l2": f"{slots * chunk} rows per step: activations + per-slot weights "
                            f"({slots * LAYERS * DIM * DIM * 2 >> 20} MiB) exceed the 126 MB L2 together with the "
                            "16 MB LM-head weight sweep; gpu_launches = eager launches + replays x kernels per "
                            f"replay ({per_replay})"}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if ws > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_fp8(args):
    """fp8 trunk linears, module-by-module autograd path, either arm: same loop, same timing."""
    import torch
    ref_arm = args.impl == "reference"
    if ref_arm:
        ref = ROOT / "baseline" / "_ref"
        if not (ref / "chaoscontrol").exists():
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is missing"}))
            return
        sys.path.insert(0, str(ref))
        os.environ.setdefault("CHAOSCONTROL_DIAG_SCAN_BACKEND", "ssm_scan")
        try:
            from chaoscontrol.distributed import broadcast_params, clip_grad_norm_fused
            from chaoscontrol.kernels.fp8_linear import fused_fp8_flush_all
            from chaoscontrol.model import CareStudentLM
            from chaoscontrol.optim.muon import Muon
            from chaoscontrol.precision import maybe_promote_linears_to_fused_fp8
            from chaoscontrol.train_ssm import train_ssm_step
        except Exception as exc:  # pragma: no cover
            print(json.dumps({"impl": "reference",
                              "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}))
            return
        promote = lambda m: maybe_promote_linears_to_fused_fp8(m, True)
        precision, recipe = "fp8_fused", "per-tensor delayed scaling, cuBLASLt"
    else:
        sys.path.insert(0, str(ROOT))
        from chaoscontrol_b200.models.model import CareStudentLM
        from chaoscontrol_b200.ops import _lib
        from chaoscontrol_b200.optim.muon import Muon
        from chaoscontrol_b200.parallel.distributed import broadcast_params, clip_grad_norm_fused
        from chaoscontrol_b200.precision import maybe_promote_linears_to_fused_fp8
        from chaoscontrol_b200.train_ssm import train_ssm_step
        promote = lambda m: maybe_promote_linears_to_fused_fp8(m, True, scaling="block")
        fused_fp8_flush_all = lambda m: None
        precision, recipe = "bf16", "block-scaled e4m3 (1x128 activations, 128x128 weights), tcgen05 f8f6f4"
    rank, local, ws = _dist_setup(args)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16)
    model.train()
    try:
        n_promoted = promote(model)
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": f"fp8 promotion failed: {type(exc).__name__}: {exc}"[:300]}))
        return
    if ws > 1:
        broadcast_params(model)
    opt = Muon(model.parameters(), lr=LR, weight_decay=WD, adamw_lr=LR, adamw_weight_decay=WD, fused=True)
    opt.bind_param_names(list(model.named_parameters()))
    host = _make_batches(args.warmup + args.steps, args.batch, args.seq, rank)
    dev_batches = [h.to(dev) for h in host[:8]]
    losses = []

    def one(inputs, targets):
        opt.zero_grad(set_to_none=True)
        loss = train_ssm_step(model, inputs, targets, 64, ddp_active=ws > 1, world_size=ws, precision=precision,
                              lm_head_backward_mode="fused_streaming_cached", lm_head_tile_size=8192)
        clip_grad_norm_fused(model.parameters(), CLIP)
        opt.step()
        fused_fp8_flush_all(model)
        return loss

    def step_resident(i):
        b = dev_batches[i % len(dev_batches)]
        losses.append(one(b[:, :-1].to(torch.int32), b[:, 1:]))

    try:
        for i in range(args.warmup):
            step_resident(i)
        torch.cuda.synchronize()
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": f"fp8 step failed: {type(exc).__name__}: {exc}"[:400]}))
        return
    l0 = 0 if ref_arm else _lib.launch_count()
    with ClockSampler(local) as cs:
        ms = _timed(step_resident, args.steps, ws)
    launches = None if ref_arm else _lib.launch_count() - l0
    final_loss = float(torch.stack([l.float() for l in losses[-args.steps:]]).mean().item())
    h2d = host[0].numel() * host[0].element_size()

    feeder = _E2EFeeder(host, dev, lambda blk: one(blk[:, :-1].to(torch.int32), blk[:, 1:]))
    step_e2e = feeder.step
    for i in range(3):
        step_e2e(i)
    ms_e = _timed(step_e2e, args.steps, ws)
    toks = ws * args.batch * args.seq / (ms / 1e3)
    out = {"metric": "train tokens/sec, 4Lx256d V16384 SSM, fp8 trunk linears (seq 512, bs 1024/rank, Muon)",
           "value": toks, "unit": "tokens/s", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "fp8 (e4m3) linears, bf16 elsewhere", "data": "synthetic Zipf(1.1) tokens, random-init weights",
           "impl": args.impl, "final_loss": final_loss, "gpu_launches": launches, "clocks": cs.summary(),
           "e2e": {"value": ws * args.batch * args.seq / (ms_e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
           "config": {"model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}", "promoted_linears": n_promoted,
                      "fp8_recipe": recipe, "global_batch": ws * args.batch, "seq_len": args.seq,
                      "parallelism": f"dp{ws}", "optimizer": f"Muon lr {LR} wd {WD} clip {CLIP}",
                      "l2": "working set per step exceeds the 126 MB L2"}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if ws > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
def run_parity(args):
    """Loss curves of both implementations from the SAME initial weights on the SAME batches, one GPU.

    The reference model is built first (seed 0); its ``state_dict`` is loaded, strictly, into this
    package's model, so both arms start from identical bf16 weights.  Every arm then runs the
    headline recipe (Muon lr 0.064, wd 0.01, clip 1.0) for ``--steps`` steps on the same Zipf(1.1)
    batches and the per-step training losses are compared.  This package runs twice: with the
    one-sweep LM head (default) and with the two-sweep one.  Prints one JSON line."""
    import torch
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "chaoscontrol").exists():
        print(json.dumps({"config": "parity", "unavailable": "baseline/_ref is missing"}))
        return
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ROOT))
    os.environ.setdefault("CHAOSCONTROL_DIAG_SCAN_BACKEND", "ssm_scan")
    from chaoscontrol.distributed import clip_grad_norm_fused as ref_clip
    from chaoscontrol.model import CareStudentLM as RefLM
    from chaoscontrol.optim.muon import Muon as RefMuon
    from chaoscontrol.train_ssm import train_ssm_step as ref_step
    from chaoscontrol_b200.models.model import CareStudentLM
    from chaoscontrol_b200.ops import _lib
    from chaoscontrol_b200.ops import lm_head as LH
    from chaoscontrol_b200.optim.muon import Muon
    from chaoscontrol_b200.parallel.distributed import clip_arena_grad_norm
    from chaoscontrol_b200.train_ssm import _engine_for
    from chaoscontrol_b200.utils.arena import ParamArena

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = args.steps
    host = _make_batches(n, args.batch, args.seq, 0, distinct=n)
    torch.manual_seed(0)
    rmodel = RefLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16)
    init = {k: v.detach().clone() for k, v in rmodel.state_dict().items()}
    del rmodel

    def reference(perturb: bool):
        """The reference recipe from ``init``; ``perturb`` nudges ONE weight (embed[0, 0]) by one bf16
        ulp first: the control that shows how far this recipe's loss curve moves under the smallest
        possible change of the starting point."""
        rmodel = RefLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16)
        rmodel.load_state_dict(init, strict=True)
        if perturb:
            with torch.no_grad():
                w = rmodel.embed.weight
                w[0, 0] = (w[0, 0].view(torch.int16) + 1).view(torch.bfloat16)
        rmodel.train()
        ropt = RefMuon(rmodel.parameters(), lr=LR, weight_decay=WD, adamw_lr=LR, adamw_weight_decay=WD, fused=True)
        ropt.bind_param_names(list(rmodel.named_parameters()))
        out = []
        for i in range(n):
            blk = host[i].to(dev, non_blocking=True)
            ropt.zero_grad(set_to_none=True)
            loss = ref_step(rmodel, blk[:, :-1].to(torch.int32), blk[:, 1:], 64, ddp_active=False, world_size=1,
                            precision="bf16", lm_head_backward_mode="fused_streaming_cached", lm_head_tile_size=8192)
            ref_clip(rmodel.parameters(), CLIP)
            ropt.step()
            out.append(loss.detach().float())
        curve = torch.stack(out).cpu().tolist()
        del rmodel, ropt
        torch.cuda.empty_cache()
        return curve

    ref_curve = reference(False)
    ref_perturbed = reference(True)

    def ours(one_sweep: bool):
        LH.ONE_SWEEP = bool(one_sweep)
        model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT).to(dev).to(torch.bfloat16)
        missing = model.load_state_dict(init, strict=True)
        assert not missing.missing_keys and not missing.unexpected_keys
        arena = ParamArena.install(model)
        model.train()
        opt = Muon(model.parameters(), lr=LR, weight_decay=WD, adamw_lr=LR, adamw_weight_decay=WD, fused=True)
        opt.bind_arena(arena)
        eng = _engine_for(model)
        if eng is None:
            raise RuntimeError("kernel training engine unavailable")
        out = []
        for i in range(n):
            blk = host[i].to(dev, non_blocking=True)
            loss = eng.step(blk[:, :-1].to(torch.int32).contiguous(), blk[:, 1:].contiguous())
            clip_arena_grad_norm(arena, CLIP)
            opt.step()
            out.append(loss.detach().float())
        _lib.assert_ok()
        curve = torch.stack(out).cpu().tolist()
        del model, opt, eng, arena
        torch.cuda.empty_cache()
        return curve

    curves = {"reference": ref_curve, "reference_one_ulp_perturbed": ref_perturbed,
              "ours_one_sweep": ours(True), "ours_two_sweeps": ours(False), "ours_one_sweep_again": ours(True)}

    def cmp(a, b):
        d = [abs(x - y) for x, y in zip(a, b)]
        tail = max(1, len(d) // 10)
        sm = lambda x, i: sum(x[i:i + 10]) / len(x[i:i + 10])          # 10-step means
        ds = [abs(sm(a, i) - sm(b, i)) for i in range(0, len(a), 10)]
        half = len(ds) // 2
        return {"max_abs": max(d), "mean_abs": sum(d) / len(d), "final_abs": d[-1],
                "mean_abs_last_tenth": sum(d[-tail:]) / tail, "first_step_abs": d[0],
                "max_abs_of_10_step_means": max(ds), "max_abs_of_10_step_means_second_half": max(ds[half:] or ds)}

    out = {"config": "parity", "steps": n, "model": f"CareStudentLM {LAYERS}x{DIM} V{VOCAB} ff_mult {FF_MULT}",
           "global_batch": args.batch, "seq_len": args.seq, "optimizer": f"Muon lr {LR} wd {WD} clip {CLIP}",
           "init": "reference model, torch.manual_seed(0), state_dict loaded strictly into this package's model",
           "vs_reference": {k: cmp(v, ref_curve) for k, v in curves.items() if k != "reference"},
           "one_vs_two_sweeps": cmp(curves["ours_one_sweep"], curves["ours_two_sweeps"]),
           "rerun_identical": curves["ours_one_sweep"] == curves["ours_one_sweep_again"],
           "curves": {k: [round(x, 5) for x in v] for k, v in curves.items() if k != "ours_one_sweep_again"}}
    print(json.dumps(out), flush=True)


# ---------------------------------------------------------------------------
def run_reference(args):
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "chaoscontrol").exists():
        print(json.dumps({"impl": "reference",
                          "unavailable": "baseline/_ref is missing: the reference is not installed on this box"}))
        return
    sys.path.insert(0, str(ref))
    os.environ.setdefault("CHAOSCONTROL_DIAG_SCAN_BACKEND", "ssm_scan")
    import torch
    try:
        from chaoscontrol.distributed import (allreduce_grads, broadcast_params,  # noqa: F401
                                              clip_grad_norm_fused)
        from chaoscontrol.model import CareStudentLM
        from chaoscontrol.optim.muon import Muon
        from chaoscontrol.train_ssm import train_ssm_step
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}))
        return

    rank, local, ws = _dist_setup(args)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=VOCAB, dim=DIM, num_layers=LAYERS, ff_mult=FF_MULT)
    model = model.to(dev).to(torch.bfloat16)
    model.train()
    if ws > 1:
        broadcast_params(model)
    opt = Muon(model.parameters(), lr=LR, weight_decay=WD, adamw_lr=LR, adamw_weight_decay=WD, fused=True)
    opt.bind_param_names(list(model.named_parameters()))
    mode = os.environ.get("BENCH_REF_HEAD_MODE", "fused_streaming_cached")

    n_total = args.warmup + args.steps
    host = _make_batches(n_total, args.batch, args.seq, rank)
    dev_batches = [h.to(dev) for h in host[:8]]
    losses = []

    def one(inputs, targets):
        opt.zero_grad(set_to_none=True)
        loss = train_ssm_step(model, inputs, targets, 64, ddp_active=ws > 1, world_size=ws,
                              precision="bf16", lm_head_backward_mode=mode, lm_head_tile_size=8192)
        clip_grad_norm_fused(model.parameters(), CLIP)
        opt.step()
        return loss

    def step_resident(i):
        b = dev_batches[i % len(dev_batches)]
        losses.append(one(b[:, :-1].to(torch.int32), b[:, 1:]))

    try:
        for i in range(args.warmup):
            step_resident(i)
        torch.cuda.synchronize()
    except Exception as exc:
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": f"reference step failed: {type(exc).__name__}: {exc}"[:400]}))
        return
    with ClockSampler(local) as cs:
        ms = _timed(step_resident, args.steps, ws)
    final_loss = float(torch.stack([l.float() for l in losses[-args.steps:]]).mean().item())

    e2e = None
    if not args.no_e2e:
        h2d = host[0].numel() * host[0].element_size()

        feeder = _E2EFeeder(host, dev, lambda blk: one(blk[:, :-1].to(torch.int32), blk[:, 1:]))
        step_e2e = feeder.step
        for i in range(max(3, args.warmup // 2)):
            step_e2e(i)
        ms_e = _timed(step_e2e, args.steps, ws)
        e2e = {"value": ws * args.batch * args.seq / (ms_e / 1e3), "unit": "tokens/s",
               "ms_per_step": ms_e, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "api": "chaoscontrol.train_ssm.train_ssm_step + Muon.step",
               "feeding": _E2EFeeder.FEEDING, "losses_read_on_host": len(feeder.read)}

    toks = ws * args.batch * args.seq / (ms / 1e3)
    headline = args.config == "submission"
    out = {"metric": ("train tokens/sec, 4Lx256d V16384 SSM (seq 512, bs 1024/rank, bf16, Muon)" if headline else
                      f"train tokens/sec, {LAYERS}Lx{DIM}d V16384 SSM (seq {args.seq}, bs {args.batch}/rank, bf16, Muon)"),
           "value": toks, "unit": "tokens/s", "n_gpus": ws, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": toks / (BASELINE_TOKS_8XH100 * ws / 8.0) if headline else None, "dtype": "bf16",
           "data": "synthetic Zipf(1.1) tokens, random-init weights", "impl": "reference",
           "final_loss": final_loss, "clocks": cs.summary(), "e2e": e2e,
           "config": _train_config(args, ws, sum(p.numel() for p in model.parameters()), False),
           "impl_detail": {"lm_head": mode, "scan_backend": os.environ.get("CHAOSCONTROL_DIAG_SCAN_BACKEND"),
                           "collective": "NCCL (torch.distributed)" if ws > 1 else "none"}}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if ws > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    a = _parse()
    if a.config == "parity":
        run_parity(a)
    elif a.config == "eval":
        run_eval(a)
    elif a.config == "eval_ttt":
        run_eval_ttt(a)
    elif a.config == "fp8":
        run_fp8(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
