"""Episodic runtime in the training loop: one rank playing both parts, and two train ranks plus an
episodic rank over gloo (event rings in shared memory, replay on the episodic rank, one SUM join)."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from chaoscontrol_b200.episodic.runtime import EpisodicRuntime
from chaoscontrol_b200.models.model import CareStudentLM


def _kw(**over):
    kw = dict(stride=8, seq_len=16, batch_size=4, device=torch.device("cpu"), budget_seconds=600.0, precision="fp32",
              stop_check_interval=1, lm_head_backward_mode="fused", prefetch_batches=False, vocab_size=64, max_steps=8)
    kw.update(over)
    return kw


_CFG = dict(episodic_capacity=64, episodic_writes_per_step=4, episodic_fingerprint_window=2, model_dim=16,
            episodic_replay_max_replays_per_step=2)


def test_one_rank_produces_consumes_and_replays(tmp_path):
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    rt = EpisodicRuntime(model=model, config=dict(_CFG, episodic_replay_log_path=str(tmp_path / "replay.ndjson")),
                         rank=0, world_size=1, device=torch.device("cpu"))
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, episodic=rt,
                                    **_kw())
    finally:
        rt.close()
    e = res["episodic"]
    assert e["role"] == "solo" and e["write_events_emitted"] == e["write_events_ingested"] > 0
    assert e["query_events_emitted"] == 8 and e["queries_ingested"] == 8
    assert 1 <= e["replays"] <= 16 and e["replay_status"]["ok"] == e["replays"]
    assert e["cache_entries"] == min(e["write_events_ingested"], 64)
    rows = (tmp_path / "replay.ndjson").read_text().strip().splitlines()
    assert len(rows) == e["replays"]
    blob = rt.cache_state()
    assert blob is not None and "key_fp" in str(blob.keys())


def _rank(rank, world, port, out_dir, cuda=False):
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
        from chaoscontrol_b200.utils.arena import ParamArena
        torch.manual_seed(rank)
        dim, vocab = (256, 512) if cuda else (16, 64)
        model = CareStudentLM(vocab_size=vocab, dim=dim, num_layers=2)
        extra = {}
        if cuda:
            model = model.to(dev).to(torch.bfloat16)
            ParamArena.install(model)                                   # kernel engine on the train ranks
            extra = dict(device=dev, precision="bf16", seq_len=128, stride=64, batch_size=8, vocab_size=vocab,
                         lm_head_backward_mode="fused_streaming_cached")
        tokens = torch.randint(0, vocab, (1 << 15,), dtype=torch.int16, generator=torch.Generator().manual_seed(0))
        rt = EpisodicRuntime(model=model, config=dict(_CFG, model_dim=dim, episodic_replay_weight=0.1,
                                                      episodic_event_ring_namespace=f"/ccb_t_epi_{port}"),
                             rank=rank, world_size=world, device=dev)
        optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
        try:
            res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=tokens.numel(), optimizer=optim,
                                        episodic=rt, rank=rank, world_size=world, **_kw(max_steps=10, **extra))
        finally:
            rt.close()
        torch.save({"res": {k: v for k, v in res.items() if k != "spectral"},
                    "w": model.lm_head.weight.detach().float().cpu()}, os.path.join(out_dir, f"r{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_train_ranks_and_an_episodic_rank(tmp_path):
    mp.spawn(_rank, args=(3, 29761, str(tmp_path)), nprocs=3, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(3)]
    # every rank applied the same joined gradient, the episodic rank included
    assert torch.allclose(r[0]["w"], r[1]["w"], atol=1e-6) and torch.allclose(r[0]["w"], r[2]["w"], atol=1e-6)
    e0, e1, e2 = (x["res"]["episodic"] for x in r)
    assert e0["role"] == "train" and e2["role"] == "episodic" and e2["n_train"] == 2
    assert e2["write_events_ingested"] > 0
    assert e2["write_events_ingested"] <= e0["write_events_emitted"] + e1["write_events_emitted"]
    assert e2["queries_ingested"] >= 10 and e2["replays"] >= 1 and e2["cache_entries"] > 0
    assert e0["replays"] == 0 and "cache_entries" not in e0
    # throughput counts the train ranks only
    assert r[0]["res"]["tokens_per_step"] == 4 * 16 * 2


import pytest  # noqa: E402


@pytest.mark.gpu
def test_kernel_engine_step_feeds_the_episodic_runtime():
    """bf16 bare trunk on the kernel engine: per-token CE and the trunk output come from the engine,
    write events are packed on the device and staged through pinned memory."""
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    from chaoscontrol_b200.utils.arena import ParamArena
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    tokens = torch.randint(0, 512, (1 << 16,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=512, dim=256, num_layers=2).to(dev).to(torch.bfloat16)
    ParamArena.install(model)
    rt = EpisodicRuntime(model=model, config=dict(episodic_capacity=256, episodic_writes_per_step=8, model_dim=256,
                                                  episodic_replay_weight=0.1),
                         rank=0, world_size=1, device=dev)
    optim = _build_optimizer(dict(optimizer="muon", base_lr=0.02), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=tokens.numel(), optimizer=optim,
                                    episodic=rt, **_kw(device=dev, precision="bf16", seq_len=128, stride=64,
                                                       batch_size=8, vocab_size=512, max_steps=12,
                                                       lm_head_backward_mode="fused_streaming_cached"))
        torch.cuda.synchronize()
    finally:
        rt.close()
    e = res["episodic"]
    assert e["write_events_ingested"] > 0 and e["replays"] >= 1 and e["replay_status"]["nan"] == 0
    assert e["key_rep_dim"] == 256 and all(v == v and v < 8.0 for v in res["loss_history"])
    from chaoscontrol_b200.ops import _lib
    _lib.assert_ok()


def _assert_ranks_agree_bitwise(a: torch.Tensor, b: torch.Tensor) -> None:
    """Every rank applies the same joined gradient, clips it with a norm whose summation order is
    fixed, and runs the same elementwise optimizer: the bf16 weights must end bit-identical on the
    train rank (kernel engine) and on the episodic rank (autograd replay)."""
    diff = (a - b).abs()
    assert torch.equal(a, b), (f"ranks disagree: max |dw| {float(diff.max()):.3e}, {int((diff > 0).sum())} of "
                               f"{diff.numel()} entries differ, |w| max {float(a.abs().max()):.3e}")


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_episodic_rank_on_two_gpus(tmp_path):
    """One train GPU on the kernel engine + an episodic GPU that replays; one NCCL SUM join."""
    mp.spawn(_rank, args=(2, 29765, str(tmp_path), True), nprocs=2, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(2)]
    _assert_ranks_agree_bitwise(r[0]["w"], r[1]["w"])
    e1 = r[1]["res"]["episodic"]
    assert e1["role"] == "episodic" and e1["write_events_ingested"] > 0 and e1["replays"] >= 1
    assert all(v == v for v in r[0]["res"]["loss_history"])


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 3, reason="needs 3 GPUs")
def test_episodic_rank_on_three_gpus(tmp_path):
    """Two train GPUs on the kernel engine + an episodic GPU; one NCCL SUM join over the flat arena."""
    mp.spawn(_rank, args=(3, 29763, str(tmp_path), True), nprocs=3, join=True)
    r = [torch.load(tmp_path / f"r{i}.pt", weights_only=False) for i in range(3)]
    _assert_ranks_agree_bitwise(r[0]["w"], r[1]["w"])
    _assert_ranks_agree_bitwise(r[0]["w"], r[2]["w"])
    e2 = r[2]["res"]["episodic"]
    assert e2["role"] == "episodic" and e2["write_events_ingested"] > 0 and e2["replays"] >= 1
    assert all(v == v for v in r[0]["res"]["loss_history"])


def test_simplex_controller_learns_from_replay_outcomes():
    """The native simplex policy chooses the replays and its online learner is credited by every outcome."""
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    rt = EpisodicRuntime(model=model, config=dict(_CFG, episodic_controller_runtime="simplex",
                                                  episodic_controller_sgd_interval=2, episodic_writes_per_step=8),
                         rank=0, world_size=1, device=torch.device("cpu"))
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim, episodic=rt,
                                    **_kw(max_steps=16))
    finally:
        rt.close()
    c = res["episodic"]["controller"]
    assert c["mode"] == "simplex" and c["decisions"] >= res["episodic"]["replays"] >= 4
    assert c["replay_outcomes"] == res["episodic"]["replays"] and c["history_appends"] == c["decisions"]
    assert c["credited_actions"] >= 1


@pytest.mark.parametrize("suffix", [".pt", ".cswg"])
def test_simplex_policy_file_round_trip(tmp_path, suffix):
    from chaoscontrol_b200.episodic import native
    from chaoscontrol_b200.episodic.controller import load_simplex_policy, save_simplex_policy
    pol = native.SimplexPolicy(seed=3, temperature=0.4)
    path = tmp_path / f"policy{suffix}"
    save_simplex_policy(path, pol)
    back = load_simplex_policy(path)
    assert (back.N, back.K_v, back.K_s, back.H) == (pol.N, pol.K_v, pol.K_s, pol.H)
    assert back.temperature == pytest.approx(0.4, rel=1e-3)
    np.testing.assert_allclose(back.flat, pol.flat, atol=2e-3 if suffix == ".cswg" else 0)


def _run_simplex(tmp_path, **cfg):
    from chaoscontrol_b200.runner_fast_path import _build_optimizer, train_fast_for_budget
    torch.manual_seed(0)
    tokens = torch.randint(0, 64, (4000,), dtype=torch.int16)
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    rt = EpisodicRuntime(model=model, config=dict(_CFG, episodic_controller_sgd_interval=2,
                                                  episodic_writes_per_step=8, **cfg),
                         rank=0, world_size=1, device=torch.device("cpu"))
    optim = _build_optimizer(dict(optimizer="adamw", base_lr=1e-3), model)
    try:
        res = train_fast_for_budget(model, train_tokens=tokens, train_num_tokens=4000, optimizer=optim,
                                    episodic=rt, **_kw(max_steps=16))
        flat = rt.simplex.policy.flat.copy()
    finally:
        rt.close()
    return res["episodic"], flat


def test_pretrained_simplex_frozen_and_online(tmp_path):
    """simplex_v1 needs a weight file; frozen runs select with it and never learn; online runs
    learn, copy the learner's weights into the selection policy and trace decision/credit rows."""
    import json
    from chaoscontrol_b200.episodic import native
    from chaoscontrol_b200.episodic.controller import save_simplex_policy
    model = CareStudentLM(vocab_size=64, dim=16, num_layers=2)
    with pytest.raises(ValueError, match="episodic_controller_weights_path"):
        EpisodicRuntime(model=model, config=dict(_CFG, episodic_controller_runtime="simplex_v1"),
                        rank=0, world_size=1, device=torch.device("cpu"))
    pol = native.SimplexPolicy(seed=5)
    wpath = tmp_path / "w.pt"
    save_simplex_policy(wpath, pol)
    common = dict(episodic_controller_runtime="simplex_v1", episodic_controller_weights_path=str(wpath),
                  episodic_controller_selection_mode="sample")

    frozen, flat_frozen = _run_simplex(tmp_path, controller_train_online=False, **common)
    c = frozen["controller"]
    assert not c["train_online"] and c["decisions"] >= 4 and c["replay_outcomes"] == 0 and c["sgd_steps"] == 0
    np.testing.assert_array_equal(flat_frozen, pol.flat)

    trace = tmp_path / "traces" / "t.ndjson"
    online, flat_online = _run_simplex(tmp_path, controller_train_online=True,
                                       episodic_controller_initial_temperature=0.2,
                                       episodic_controller_entropy_beta=0.05,
                                       episodic_controller_simplex_trace_path=str(trace), **common)
    c = online["controller"]
    assert c["train_online"] and c["temperature"] == pytest.approx(0.2) and c["sgd_steps"] >= 1
    assert not np.array_equal(flat_online, pol.flat)          # selection follows the learner
    rows = [json.loads(line) for line in trace.read_text().splitlines()]
    kinds = {r["row_type"] for r in rows}
    assert {"decision", "credit", "replay_outcome"} <= kinds
    dec = next(r for r in rows if r["row_type"] == "decision")
    assert 0.0 < dec["entropy"] <= np.log(16) + 1e-4 and dec["temperature"] == pytest.approx(0.2)
    cred = next(r for r in rows if r["row_type"] == "credit")
    assert {"p_chosen", "p_current_chosen", "gerber_weight", "advantage_final"} <= set(cred)
