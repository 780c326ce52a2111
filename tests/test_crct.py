"""CRCT teacher runtime on CPU: roles, payloads, the shared-memory mailbox (request -> score ->
result, fail-open, stale drops, weight snapshots, shutdown record), the lock-step transport and the
memory-rank loop over gloo ranks."""
import os
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from chaoscontrol_b200 import crct as C
from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.wake_cache import TransactionalWakeCache


def _memory_model(seed=0, vocab=48, dim=16):
    torch.manual_seed(seed)
    return CareStudentLM(vocab_size=vocab, dim=dim, num_layers=2, outer_model_dim=8, outer_model_type="multislot",
                         outer_max_slots=0, buffer_mode="append_only")


def _batch(B=3, T=8, vocab=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (B, T + 1), generator=g)
    return ids[:, :-1].to(torch.int32), ids[:, 1:].long()


def test_topology_and_stop_predicates():
    t = C.crct_rank_topology(world_size=4)
    assert t["train_ranks"] == [0, 1, 2] and t["memory_ranks"] == [3] and t["grad_world_size"] == 3
    assert t["memory_owner"] == "packet_and_maintenance_shared"
    s = C.crct_rank_topology(world_size=8, split_memory_ranks=True)
    assert s["packet_rank"] == 6 and s["maintenance_rank"] == 7 and s["grad_world_size"] == 6
    one = C.crct_rank_topology(world_size=1)
    assert one["train_ranks"] == [0] and one["memory_ranks"] == []
    with pytest.raises(ValueError):
        C.crct_rank_topology(world_size=0)
    # a memory rank may have served nothing and must still stop on the clock
    assert C.memory_rank_should_stop(steps=0, elapsed_s=9.0, budget_seconds=10.0, stop_margin_seconds=2.0)
    assert not C.memory_rank_should_stop(steps=0, elapsed_s=7.0, budget_seconds=10.0, stop_margin_seconds=2.0)
    assert C.memory_rank_should_stop(steps=5, elapsed_s=0.0, budget_seconds=10.0, stop_margin_seconds=0.0, max_steps=5)
    kw = dict(budget_seconds=10.0, stop_margin_seconds=2.0)
    assert C.memory_rank_defer_stop(local_stop=True, elapsed_s=12.0, shutdown_requested=False, **kw)
    assert not C.memory_rank_defer_stop(local_stop=True, elapsed_s=15.1, shutdown_requested=False, **kw)
    assert not C.memory_rank_defer_stop(local_stop=True, elapsed_s=12.0, shutdown_requested=True, **kw)
    assert not C.memory_rank_defer_stop(local_stop=False, elapsed_s=12.0, shutdown_requested=False, **kw)


def test_inline_payloads_and_weighted_row_scale():
    model = _memory_model()
    cache = TransactionalWakeCache()
    x, y = _batch()
    kw = dict(model=model, cache=cache, scarcity_optimizer=C.ScarcityAwareMemoryOptimizer(), inputs=x, targets=y,
              total_steps=10, tau=0.1, strength=0.1, w_max=1.2, alpha_max=0.15, memory_write_tokens=4)
    with torch.no_grad():
        p0 = C.score_payload_inline(step=0, update_model_memory_after=True, **kw)
        p1 = C.score_payload_inline(step=5, update_model_memory_after=True, **kw)
    for p in (p0, p1):
        for k in ("target", "confidence", "loss_weight", "utility"):
            assert p[k].shape == (3, 8)
    assert int(model._last_crct_probe_step) == 5 and model._last_crct_probe_input_ids.shape == (3, 9)
    assert len(p0["memory_write_records"]) == 4
    # the second batch reads what the first wrote
    assert float(p1["utility"].abs().max()) > 0
    if "memory_residual" in p1:
        assert p1["memory_gate_alias_target"] is True and torch.equal(p1["memory_gate"], p1["target"])
    approx = C.packet_payload_inline(model=model, cache=cache, inputs=x, targets=y, step=6, memory_write_tokens=2)
    assert approx["packet_approximate"] and approx["memory_residual"].shape[0] == 3
    assert float(approx["target"].abs().sum()) == 0 and torch.equal(approx["loss_weight"], torch.ones(3, 8))
    w = torch.tensor([[0.5, 1.5], [1.0, 1.0]])
    ce = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    want = (ce * w).sum() / w.sum()
    assert torch.allclose((ce.reshape(-1) * C.weighted_row_scale(w)).mean(), want)


def _mailbox_pair(name, **kw):
    base = dict(name=name, batch_size=3, seq_len=8, hidden_dim=16, device=torch.device("cpu"), capacity=4,
                max_local_batches=4, max_payload_lag_steps=3)
    base.update(kw)
    train = C.TeacherMailbox(role="train", **base)
    mem = C.TeacherMailbox(role="memory", **base)
    return train, mem


def test_mailbox_round_trip_fail_open_and_stale_drop():
    train, mem = _mailbox_pair(f"/ccb_t_mb_{os.getpid()}", payload_dtype=torch.bfloat16)
    try:
        x, y = _batch()
        assert train.begin_step(inputs=x, targets=y, step=0) is None          # nothing scored yet: fail open
        rid, step, ids = mem.pop_request()
        assert (rid, step) == (0, 0) and torch.equal(ids.long(), C.crct_full_input_ids(x, y))
        scored = {"target": torch.rand(3, 8), "confidence": torch.rand(3, 8), "loss_weight": torch.rand(3, 8) + 0.5,
                  "utility": torch.randn(3, 8), "memory_residual": torch.randn(3, 1, 16),
                  "memory_gate_alias_target": True, "plasticity_budget": torch.rand(16)}
        scored["memory_gate"] = scored["target"]
        assert mem.push_result(request_id=rid, step=step, scored=scored, score_seconds=0.25)
        x1, y1 = _batch(seed=1)
        payload, xi, yi = train.begin_step(inputs=x1, targets=y1, step=1)
        assert torch.equal(xi, x) and torch.equal(yi, y) and payload["step_id_int"] == 0
        for k in ("target", "confidence", "loss_weight", "utility", "memory_residual"):
            assert torch.allclose(payload[k], scored[k].bfloat16().float()), k
        assert payload["memory_gate"] is payload["target"] and payload["memory_residual"].shape == (3, 1, 16)
        assert torch.allclose(payload["plasticity_budget"], scored["plasticity_budget"])
        assert abs(payload["score_seconds"] - 0.25) < 1e-6
        # a result that arrives more than max_payload_lag_steps late is dropped, the step fails open
        rid, step, _ = mem.pop_request()
        assert step == 1
        for s in range(2, 6):
            assert train.begin_step(inputs=x1, targets=y1, step=s) is None
        mem.push_result(request_id=rid, step=step, scored=scored, score_seconds=0.0)
        assert train.begin_step(inputs=x1, targets=y1, step=6) is None
        assert train.metrics.results_dropped_stale + train.metrics.results_dropped_unknown_step == 1
        # the memory side serves the newest waiting request only (step 6 found the ring full and was dropped)
        r = mem.pop_request()
        assert r is not None and r[1] == 5 and mem.metrics.requests_skipped_stale == 3
        assert train.metrics.requests_dropped_full == 1
        # shutdown record
        assert not mem.shutdown_requested
        train.request_shutdown()
        assert mem.pop_request() is None and mem.shutdown_requested
    finally:
        mem.close()
        train.close()


def test_mailbox_request_ring_full_is_a_drop_not_a_wait():
    train, mem = _mailbox_pair(f"/ccb_t_full_{os.getpid()}", capacity=2, max_local_batches=16)
    try:
        x, y = _batch()
        t0 = time.monotonic()
        for s in range(6):
            train.begin_step(inputs=x, targets=y, step=s)
        assert time.monotonic() - t0 < 1.0
        assert train.metrics.requests_submitted == 2 and train.metrics.requests_dropped_full == 4
    finally:
        mem.close()
        train.close()


def test_weight_snapshot_double_buffer():
    src, dst = _memory_model(seed=1), _memory_model(seed=2)
    nbytes = C._weight_bytes(src, "full")
    train, mem = _mailbox_pair(f"/ccb_t_w_{os.getpid()}", weight_bytes=nbytes)
    try:
        assert not mem.poll_weight_snapshot(dst)                             # nothing published
        assert train.maybe_publish_weight_snapshot(src, step=0, interval=4)
        assert not train.maybe_publish_weight_snapshot(src, step=1, interval=4)
        assert mem.poll_weight_snapshot(dst) and not mem.poll_weight_snapshot(dst)
        for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
            assert torch.equal(a, b), n
        with torch.no_grad():
            for p in src.parameters():
                p.add_(1.0)
        assert train.maybe_publish_weight_snapshot(src, step=4, interval=4)
        assert mem.poll_weight_snapshot(dst)
        assert torch.equal(src.lm_head.weight, dst.lm_head.weight)
        assert mem.metrics.weight_snapshots_applied == 2 and train.metrics.weight_snapshots_published == 2
        with pytest.raises(ValueError):
            C.TeacherMailbox(name=f"/ccb_t_w2_{os.getpid()}", role="train", batch_size=1, seq_len=1, hidden_dim=1,
                             device=torch.device("cpu"), weight_bytes=64).maybe_publish_weight_snapshot(
                                 src, step=0, interval=1)
    finally:
        mem.close()
        train.close()
        from chaoscontrol_b200.episodic import native as N
        for suffix in ("req", "res", "slab", "w"):
            N.lib().ccbc_shm_unlink(f"/ccb_t_w2_{os.getpid()}_{suffix}".encode())


# ---------------------------------------------------------------- training loop integration
def _loop_kw(**kw):
    base = dict(stride=8, seq_len=8, batch_size=3, device=torch.device("cpu"), budget_seconds=600.0, precision="fp32",
                stop_check_interval=1, lm_head_backward_mode="fused", prefetch_batches=False, vocab_size=48)
    base.update(kw)
    return base


def test_train_loop_inline_teacher_and_maintenance():
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    model = _memory_model()
    tokens = torch.randint(0, 48, (4000,), dtype=torch.int16, generator=torch.Generator().manual_seed(0))
    cfg = dict(crct_enabled=True, crct_score_interval_steps=2, crct_memory_write_tokens_per_step=4,
               replay_eviction_enabled=True, replay_eviction_min_slot_age_steps=0, model_dim=16)
    rt = C.CrctRuntime(model=model, config=cfg, rank=0, world_size=1, device=torch.device("cpu"), batch_size=3,
                       seq_len=8, total_steps=8)
    assert rt.mode == "inline" and rt.replay_loop is not None and not rt.is_memory_rank
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, max_steps=8,
                                crct=rt, replay_eviction_enabled=True, **_loop_kw())
    d = res["crct"]
    assert res["steps"] == 8 and d["teacher_requests"] == 4 and d["teacher_payloads"] == 4
    assert d["teacher_fail_open"] == 4                                   # the unscored steps train plainly
    assert d["replay_eviction"]["frames_ingested"] == 4
    assert all(map(lambda v: v == v, res["loss_history"]))
    assert model.outer_model.table.n_active > 0                          # the teacher wrote slots
    with pytest.raises(ValueError):
        train_fast_for_budget(_memory_model(), train_tokens=tokens, train_num_tokens=4000, optimizer=optim,
                              max_steps=1, **_loop_kw())                 # episodic store without CRCT
    with pytest.raises(ValueError):
        m2 = CareStudentLM(vocab_size=48, dim=16, num_layers=1)
        train_fast_for_budget(m2, train_tokens=tokens, train_num_tokens=4000, max_steps=1,
                              optimizer=_build_optimizer(dict(optimizer="adamw"), m2),
                              replay_eviction_enabled=True, **_loop_kw())


def _crct_rank(rank, world, port, mode, out_dir, split=False, cuda=False):
    torch.set_num_threads(1)      # several ranks share this machine's cores: no intra-op thread pools
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    dev = torch.device("cpu")
    if cuda:
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                            **({"device_id": dev} if cuda else {}))
    try:
        from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
        model = _memory_model(seed=rank)                                  # different inits: rank 0 must win
        if cuda:
            model = model.to(dev).to(torch.bfloat16)
        tokens = torch.randint(0, 48, (4000,), dtype=torch.int16, generator=torch.Generator().manual_seed(0))
        cfg = dict(crct_enabled=True, crct_teacher_transport_mode=mode, crct_memory_write_tokens_per_step=4,
                   crct_teacher_param_sync_interval=2, crct_mailbox_name=f"/ccb_t_run_{port}", model_dim=16,
                   crct_max_payload_lag_steps=64, crct_max_local_batches=64, crct_mailbox_capacity=64,
                   crct_split_memory_ranks=split, replay_eviction_enabled=split,
                   replay_eviction_min_slot_age_steps=0)
        rt = C.CrctRuntime(model=model, config=cfg, rank=rank, world_size=world, device=dev,
                           batch_size=3, seq_len=8, total_steps=12)
        optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
        # slow the train ranks a little so the asynchronous teacher has time to answer
        t_real = time.perf_counter

        def slow_clock():
            if mode != "sync" and not rt.is_memory_rank:
                time.sleep(0.01)
            return t_real()
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, max_steps=12,
                                    crct=rt, rank=rank, world_size=world, time_fn=slow_clock,
                                    replay_eviction_enabled=split,
                                    **_loop_kw(budget_seconds=20.0, stop_margin_seconds=0.0, device=dev,
                                               precision="bf16" if cuda else "fp32"))
        torch.save({"res": {k: v for k, v in res.items() if k != "spectral"},
                    "w": model.lm_head.weight.detach().float().cpu(),
                    "slots": int(model.outer_model.table.n_active)}, os.path.join(out_dir, f"r{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,port", [("async_rank0_memory_mailbox", 29741), ("sync", 29743)])
def test_two_train_ranks_and_a_memory_rank(tmp_path, mode, port):
    mp.spawn(_crct_rank, args=(3, port, mode, str(tmp_path)), nprocs=3, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(3)]
    assert r[0]["res"]["steps"] == 12 and r[1]["res"]["steps"] == 12
    assert torch.allclose(r[0]["w"], r[1]["w"], atol=1e-6)               # one gradient group, same weights
    mem = r[2]["res"]
    assert mem["role"] == "memory" and mem["steps"] >= 1
    d0, d1 = r[0]["res"]["crct"], r[1]["res"]["crct"]
    assert d0["topology"]["train_ranks"] == [0, 1] and d0["topology"]["memory_ranks"] == [2]
    if mode == "sync":
        assert mem["steps"] == 12 and d0["teacher_payloads"] == 12 and d1["teacher_payloads"] == 12
        assert d0["param_syncs"] >= 6 and mem["crct"]["param_syncs"] >= 6
    else:
        assert d1["teacher_bypass_steps"] == 12 and d1["teacher_payloads"] == 0
        assert d0["teacher_payloads"] >= 1 and d0["teacher_payloads"] + d0["teacher_fail_open"] == 12
        assert d0["mailbox"]["weight_snapshots_published"] >= 1
        assert mem["crct"]["mailbox"]["weight_snapshots_applied"] >= 1
        assert mem["crct"]["mailbox"]["requests_served"] == mem["steps"]


def test_slot_commit_lane_appends_maintenance_and_drops():
    from chaoscontrol_b200.slot_commit import SlotCommit, SlotCommitAction
    packet_model, maint_model = _memory_model(), _memory_model()
    kw = dict(name=f"/ccb_t_lane_{os.getpid()}", packet_rank=2, maintenance_rank=3, queue_capacity=4)
    a = C.SlotCommitPeerLane(rank=2, **kw)
    b = C.SlotCommitPeerLane(rank=3, **kw)
    idle = C.SlotCommitPeerLane(rank=0, **kw)
    try:
        assert not idle.participant and idle.pump(packet_model) == 0
        # the packet rank appends locally, then publishes the same records
        hidden = torch.randn(1, 3, 16)
        recs = packet_model.append_memory_from_hidden(hidden, max_tokens=3)
        for r in recs:
            a.submit(SlotCommit(slot_id=r["slot_id"], action=SlotCommitAction.APPEND, step=1, base_generation=None,
                                new_generation=r["generation"], bucket_id=r["bucket_id"], event_id=r["event_id"],
                                tensor=r["tensor"]))
        assert a.pump(packet_model) == 0 and a.metrics["sent"] == 3
        assert b.pump(maint_model) == 3 and maint_model.outer_model.table.n_active == 3
        sid = recs[0]["slot_id"]
        assert torch.allclose(maint_model.outer_model.table.get_tensor(sid), recs[0]["tensor"])
        # a maintenance decision travels back and lands on the packet rank's mirror
        gen = int(maint_model.outer_model.table.record(sid).write_generation)
        b.submit(SlotCommit(slot_id=sid, action=SlotCommitAction.EVICT, step=2, base_generation=gen,
                            new_generation=gen + 1, reason="test"))
        b.submit(SlotCommit(slot_id=recs[1]["slot_id"], action=SlotCommitAction.EVICT, step=2,
                            base_generation=gen + 7, new_generation=gen + 8))
        b.pump(maint_model)
        assert a.pump(packet_model) == 1
        assert a.metrics["maintenance_commits_applied"] == 1 and a.metrics["stale_generation_drops"] == 1
        assert packet_model.outer_model.table.n_active == 2
        # bounded queue and payload
        for i in range(6):
            a.submit(SlotCommit(slot_id=100 + i, action=SlotCommitAction.APPEND, step=3, base_generation=None,
                                new_generation=1, tensor=torch.zeros(1, 8)))
        assert a.metrics["queue_overwrites"] == 2
        a.submit(SlotCommit(slot_id=999, action=SlotCommitAction.APPEND, step=3, base_generation=None,
                            new_generation=1, tensor=torch.zeros(1, 2048)))
        a.pump(packet_model)
        assert a.metrics["oversize_drops"] == 1
    finally:
        b.close(maint_model)
        a.close(packet_model)


def test_split_memory_ranks_exchange_slot_commits(tmp_path):
    """2 train ranks + packet rank + maintenance rank: appends made while serving packets reach the
    maintenance replica over the peer lane."""
    mp.spawn(_crct_rank, args=(4, 29747, "async_rank0_memory_mailbox", str(tmp_path), True), nprocs=4, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(4)]
    assert torch.allclose(r[0]["w"], r[1]["w"], atol=1e-6)
    packet, maint = r[2]["res"], r[3]["res"]
    assert packet["crct"]["topology"]["split_memory_ranks"] and packet["crct"]["topology"]["train_ranks"] == [0, 1]
    pl, ml = packet["crct"]["slot_commit_lane"], maint["crct"]["slot_commit_lane"]
    assert packet["steps"] >= 1 and pl["submitted"] >= 4 and pl["sent"] >= 1
    assert ml["append_commits_applied"] >= 1 and ml["append_commits_applied"] == ml["received"] - ml["dropped"]
    assert r[3]["slots"] == ml["append_commits_applied"]                 # the replica holds what arrived
    assert pl["mode"] == "slot_commit_shm_ring"
    assert maint["crct"]["replay_eviction"]["frames_ingested"] >= 1
    assert "replay_eviction" not in packet["crct"]


@pytest.mark.gpu
def test_mailbox_on_cuda_uses_pinned_shared_memory():
    dev = torch.device("cuda:0")
    base = dict(name=f"/ccb_t_cuda_{os.getpid()}", batch_size=4, seq_len=64, hidden_dim=32, device=dev, capacity=4)
    model = CareStudentLM(vocab_size=64, dim=32, num_layers=1).to(dev).to(torch.bfloat16)
    twin = CareStudentLM(vocab_size=64, dim=32, num_layers=1).to(dev).to(torch.bfloat16)
    wb = C._weight_bytes(model, "full")
    train = C.TeacherMailbox(role="train", weight_bytes=wb, **base)
    mem = C.TeacherMailbox(role="memory", weight_bytes=wb, **base)
    try:
        assert train._pinned and mem._pinned
        ids = torch.randint(0, 64, (4, 65), device=dev)
        x, y = ids[:, :-1].to(torch.int32), ids[:, 1:]
        assert train.begin_step(inputs=x, targets=y, step=0) is None
        torch.cuda.synchronize()
        train._flush_pending()
        rid, step, got = mem.pop_request()
        assert torch.equal(got.long(), ids)
        scored = {k: torch.rand(4, 64, device=dev) for k in ("target", "confidence", "loss_weight", "utility")}
        assert mem.push_result(request_id=rid, step=step, scored=scored, score_seconds=0.0)
        payload, xi, _ = train.begin_step(inputs=x, targets=y, step=1)
        torch.cuda.synchronize()
        assert payload["loss_weight"].is_cuda and torch.equal(payload["loss_weight"], scored["loss_weight"])
        assert train.maybe_publish_weight_snapshot(model, step=0, interval=1)
        torch.cuda.synchronize()
        train._finish_weight_publish()
        assert mem.poll_weight_snapshot(twin)
        assert torch.equal(twin.lm_head.weight, model.lm_head.weight)
    finally:
        mem.close()
        train.close()


@pytest.mark.gpu
def test_inline_teacher_on_cuda_bf16():
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    model = CareStudentLM(vocab_size=256, dim=64, num_layers=2, outer_model_dim=32, outer_model_type="multislot",
                          outer_max_slots=0, buffer_mode="append_only").to(dev).to(torch.bfloat16)
    tokens = torch.randint(0, 256, (1 << 15,), dtype=torch.int16)
    cfg = dict(crct_enabled=True, crct_score_interval_steps=2, crct_memory_write_tokens_per_step=16, model_dim=64,
               replay_eviction_enabled=True, replay_eviction_min_slot_age_steps=0)
    rt = C.CrctRuntime(model=model, config=cfg, rank=0, world_size=1, device=dev, batch_size=4, seq_len=64,
                       total_steps=8)
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=tokens.numel(), optimizer=optim,
                                max_steps=8, crct=rt, replay_eviction_enabled=True,
                                **_loop_kw(device=dev, precision="bf16", seq_len=64, stride=32, batch_size=4,
                                           vocab_size=256, lm_head_backward_mode="fused_streaming_cached"))
    d = res["crct"]
    assert d["teacher_payloads"] == 4 and model.outer_model.table.n_active > 0
    assert all(v == v for v in res["loss_history"])


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode,port", [("async_rank0_memory_mailbox", 29775), ("sync", 29777)])
def test_crct_on_two_gpus(tmp_path, mode, port):
    """One train GPU and one memory GPU: pinned mailbox, side-stream copies and weight snapshots on hardware."""
    mp.spawn(_crct_rank, args=(2, port, mode, str(tmp_path), False, True), nprocs=2, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(2)]
    assert r[0]["res"]["steps"] == 12 and r[1]["res"]["role"] == "memory" and r[1]["res"]["steps"] >= 1
    d0 = r[0]["res"]["crct"]
    if mode == "sync":
        assert r[1]["res"]["steps"] == 12 and d0["teacher_payloads"] == 12
    else:
        assert d0["teacher_payloads"] + d0["teacher_fail_open"] == 12
    assert all(v == v for v in r[0]["res"]["loss_history"])


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 3, reason="needs 3 GPUs")
@pytest.mark.parametrize("mode,port", [("async_rank0_memory_mailbox", 29771), ("sync", 29773)])
def test_crct_on_three_gpus(tmp_path, mode, port):
    """Two train GPUs in an NCCL gradient subgroup, the third GPU is the memory rank."""
    mp.spawn(_crct_rank, args=(3, port, mode, str(tmp_path), False, True), nprocs=3, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(3)]
    assert r[0]["res"]["steps"] == 12 and torch.allclose(r[0]["w"], r[1]["w"], atol=1e-6)
    mem = r[2]["res"]
    assert mem["role"] == "memory" and mem["steps"] >= 1
    d0 = r[0]["res"]["crct"]
    if mode == "sync":
        assert mem["steps"] == 12 and d0["teacher_payloads"] == 12
    else:
        assert d0["teacher_payloads"] + d0["teacher_fail_open"] == 12
        assert mem["crct"]["mailbox"]["weight_snapshots_applied"] >= 1
