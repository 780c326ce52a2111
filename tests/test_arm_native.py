"""Native maintenance scheduler, fused CPU NLL, evidence engine, per-slot SSM learner."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from chaoscontrol_b200.episodic import arm_native as A
from chaoscontrol_b200.episodic import cpu_ssm_controller as csc
from chaoscontrol_b200.episodic import native


def test_scheduler_round_robin_reservations_ttl():
    s = A.ArmMaintenanceScheduler(memory_streams=4, slot_work_chunk_size=3, frame_ttl_steps=10, max_frames=2)
    assert s.next_job(1, [1, 2, 3]) is None and s.diagnostics()["skipped_no_frame"] == 1
    assert s.ingest_frame(7, 1, 9, None) and not s.ingest_frame(7, 1, 9, None)
    vis = [10, 11, 12, 13, 14]
    j1 = s.next_job(2, vis)
    assert j1["frame_id"] == 7 and j1["slot_count"] == 3 and j1["stream_id"] == 1 and j1["cache_read_cutoff"] is None
    j2 = s.next_job(2, vis)
    assert set(j1["slot_ids"]).isdisjoint(j2["slot_ids"]) and set(j1["slot_ids"]) | set(j2["slot_ids"]) == set(vis)
    assert s.next_job(2, vis) is None and s.diagnostics()["skipped_inflight"] == 1
    s.record_result({"job_id": j1["job_id"], "frame_id": 7, "step": 2, "status": 0, "slots_scored": 3,
                     "actions_confirmed": 1, "probe_seconds": 0.5})
    s.record_result({"job_id": j2["job_id"], "frame_id": 7, "step": 2, "status": 1, "slots_scored": 0})
    j3 = s.next_job(3, vis)          # the failed job's slots come back
    assert sorted(j3["slot_ids"]) == sorted(j2["slot_ids"])
    s.record_result({"job_id": j3["job_id"], "frame_id": 7, "step": 3, "status": 0, "slots_scored": 2})
    assert s.next_job(3, vis) is None
    d = s.diagnostics()
    assert d["frames_completed"] == 1 and d["result_errors"] == 1 and d["slots_scored_total"] == 5
    assert d["probe_seconds_total"] == pytest.approx(0.5) and d["jobs_emitted"] == 3
    for fid in (8, 9, 10):
        s.ingest_frame(fid, 5, 0, 77)
    assert s.diagnostics()["frames_dropped_overflow"] == 1
    assert s.next_job(100, vis) is None and s.diagnostics()["frames_dropped_stale"] == 2
    assert s.next_job(100, []) is None and s.diagnostics()["skipped_no_slots"] == 1
    s.close()


def test_fused_cpu_nll_matches_torch():
    torch.manual_seed(0)
    T, D, V = 37, 64, 700
    hidden = torch.randn(T, D).bfloat16()
    W = (torch.randn(V, D) * 0.2).bfloat16()
    nw = torch.rand(D) + 0.5
    y = torch.randint(0, V, (T,))
    head = A.PackedLmHead(nw, W)
    nll, _amx = A.rms_lmhead_nll(head, hidden, y)
    xn = (F.rms_norm(hidden.float(), (D,), eps=1e-6) * nw).bfloat16().float()
    ref = F.cross_entropy(xn @ W.float().t(), y, reduction="none")
    assert torch.allclose(nll, ref, atol=2e-3, rtol=2e-3), (nll - ref).abs().max()
    head.close()


@pytest.mark.parametrize("T,D,V", [(37, 64, 700), (16, 384, 4099), (5, 40, 33)])
def test_packed_amx_nll_agrees_with_the_generic_path_and_torch(T, D, V):
    """The VNNI-packed fused path (AMX CPUs) against the generic tile-matmul path and the fp32
    statement, with token counts / model dims / vocabularies that are not multiples of the tile."""
    torch.manual_seed(2)
    hidden = torch.randn(T, D).bfloat16()
    W = (torch.randn(V, D) * 0.2).bfloat16()
    nw = torch.rand(D) + 0.5
    y = torch.randint(0, V, (T,))
    head = A.PackedLmHead(nw, W)
    fused, used = A.rms_lmhead_nll(head, hidden, y)
    generic, _ = A.rms_lmhead_nll(head, hidden, y, packed_amx=False)
    xn = (F.rms_norm(hidden.float(), (D,), eps=1e-6) * nw).bfloat16().float()
    ref = F.cross_entropy(xn @ W.float().t(), y, reduction="none")
    assert torch.allclose(fused, generic, atol=1e-3, rtol=1e-3), (fused - generic).abs().max()
    assert torch.allclose(fused, ref, atol=3e-3, rtol=3e-3), (fused - ref).abs().max()
    if A.cpu_has_amx() if hasattr(A, "cpu_has_amx") else False:
        assert used
    head.close()


def test_evidence_engine():
    torch.manual_seed(1)
    eng = A.CpuEvidenceEngine(lanes=2, d_model=32)
    cue = torch.randn(A.CUE_TOKENS, 32).bfloat16()
    tg = torch.randint(0, 100, (A.CUE_TOKENS,), dtype=torch.int32)
    eng.ingest_frame(cue, tg, frame_id=1, step=5, stream_id=3)
    d = eng.diagnostics()
    assert d["frames_ingested"] == 1 and d["cue_nll_calls_total"] == 0 and d["lane_tile_advances_total"] == {"0": 0, "1": 1}
    W, nw = (torch.randn(100, 32) * 0.3).bfloat16(), torch.ones(32)
    eng.set_lm_head(nw, W)
    eng.ingest_frame(cue, tg, frame_id=2, step=6, stream_id=0)
    d = eng.diagnostics()
    xn = F.rms_norm(cue.float(), (32,), eps=1e-6).bfloat16().float()
    ref = F.cross_entropy(xn @ W.float().t(), tg.long(), reduction="none")
    assert d["cue_nll_calls_total"] == 1 and d["last_cue_nll_mean"] == pytest.approx(float(ref.mean()), rel=2e-3)
    assert d["last_cue_nll_max"] == pytest.approx(float(ref.max()), rel=2e-3) and d["last_cue_nll_finite_fraction"] == 1.0
    assert d["lane_work_items_emitted_total"]["0"] == 64
    with pytest.raises(ValueError):
        eng.ingest_frame(cue.float(), tg, frame_id=3, step=7, stream_id=0)
    with pytest.raises(ValueError):
        eng.set_lm_head(torch.ones(8), W)
    eng.shutdown()
    with pytest.raises(RuntimeError):
        eng.ingest_frame(cue, tg, frame_id=3, step=7, stream_id=0)
    assert not eng.diagnostics()["enabled"]
    eng.close()


def _weights(F_=4, G=5, S=3, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    return csc.CpuSsmControllerWeights(r(G, F_), r(S, F_), torch.rand(G, generator=g), torch.rand(S, generator=g),
                                       r(G), r(S), torch.tensor(0.1))


def test_native_forward_step_and_learner_moves_logit_toward_reward():
    w = _weights()
    f, g, s = torch.randn(4), torch.randn(5), torch.randn(3)
    ng, ns, logit = A.ssm_forward_step(w, f, g, s)
    ref = csc.forward_step(f, csc.CpuSsmControllerState(g, s), w, prefer_cpp=False)
    assert torch.allclose(ng, ref.global_state, atol=1e-5) and torch.allclose(ns, ref.slot_state, atol=1e-5)
    assert float(logit) == pytest.approx(float(ref.logit), abs=1e-5)
    L = A.OnlineLearningController(num_slots=8, max_entries_per_slot=2, gamma=1.0, gerber_c=0.0, learning_rate=0.002,
                                   sgd_interval=1, ema_alpha=0.5, ema_interval=2)
    ev = np.zeros((), dtype=native.REPLAY_OUTCOME)
    ev["slot_id"], ev["gpu_step"], ev["reward_shaped"] = 2, 10, 1.0
    L.on_replay_outcome(ev)
    assert L.telemetry()["backward_skipped_missing_weights"] == 1
    L.initialize_weights(w)
    for step in range(3):
        L.record_replay_selection(slot_id=2, gpu_step=step, policy_version=0, output_logit=float(logit), selected_rank=0,
                                  features=f, global_state=g, slot_state=s)
    assert L.history_size(2) == 2           # bounded per slot
    L.record_replay_selection(slot_id=99, gpu_step=0, policy_version=0, output_logit=0.0, selected_rank=0,
                              features=f, global_state=g, slot_state=s)
    for _ in range(4):
        L.on_replay_outcome(ev)
    t = L.telemetry()
    assert t["sgd_steps"] >= 4 and t["ema_blends"] >= 1 and t["invalid_slot_skips"] == 1 and t["last_credit_sum"] > 0
    fast = csc.CpuSsmControllerWeights.from_dict(L.fast_weights())
    new_logit = csc.forward_step(f, csc.CpuSsmControllerState(g, s), fast, prefer_cpp=False).logit
    assert float(new_logit) > float(logit)          # rewarded action: its logit went up
    slow = L.slow_weights()
    assert not torch.equal(slow["bias"], torch.tensor(0.1)) and not torch.equal(slow["bias"], L.fast_weights()["bias"])
    L.mark_evicted(2, 100)
    assert L.is_evicted(2)
    L.gc(120, 50)
    assert L.history_size(2) == 2
    L.gc(200, 50)
    assert L.history_size(2) == 0
    L.close()
