"""Input pipeline and loop arithmetic (CPU; the pinned-staging path has a GPU test)."""
import pytest
import torch

from chaoscontrol_b200 import fast_path as FP
from chaoscontrol_b200.data import batch_from_starts, build_lm_starts


def test_batch_from_start_tensor_matches_slicing():
    tokens = torch.arange(1000, dtype=torch.int16)
    starts = torch.tensor([0, 17, 500])
    x, y = FP.batch_from_start_tensor(tokens=tokens, starts=starts, seq_len=8, device=torch.device("cpu"))
    rx, ry = batch_from_starts(tokens, starts.tolist(), 8, torch.device("cpu"))
    assert x.dtype == torch.int32 and y.dtype == torch.int64
    assert torch.equal(x.long(), rx) and torch.equal(y, ry)
    x2, _ = FP.batch_from_start_tensor(tokens=tokens, starts=starts, seq_len=8, device="cpu", vocab_size=100)
    assert int(x2.max()) == 99
    with pytest.raises(ValueError):
        FP.batch_from_start_tensor(tokens=tokens, starts=starts.view(1, -1), seq_len=8, device="cpu")


@pytest.mark.parametrize("n,T,s", [(1000, 16, 8), (50, 64, 4), (1 << 20, 512, 256), (83, 16, 1)])
def test_start_counts_match_listing(n, T, s):
    full = build_lm_starts(n, T, s)
    assert FP.count_lm_starts(n, T, s) == len(full)
    for ws in (1, 3, 8):
        for r in range(ws):
            assert FP.count_sharded_lm_starts(total_starts=len(full), rank=r, world_size=ws) == len(full[r::ws])


def test_sampled_and_epoch_starts_stay_in_the_rank_shard():
    n, T, s, ws = 5000, 32, 16, 3
    full = build_lm_starts(n, T, s)
    g = torch.Generator().manual_seed(0)
    for r in range(ws):
        shard = set(full[r::ws])
        got = FP.sample_sharded_lm_starts(num_tokens=n, seq_len=T, stride=s, batch_size=64, rank=r, world_size=ws,
                                          generator=g)
        assert set(got.tolist()) <= shard
    steps = FP.sequential_epoch_steps(num_tokens=n, seq_len=T, stride=s, batch_size=10, world_size=ws)
    for sampler in (FP.SequentialShardedStartSampler(), FP.ShuffledEpochShardedStartSampler(seed=5)):
        seen = []
        for _ in range(steps):
            seen += sampler(num_tokens=n, seq_len=T, stride=s, batch_size=10, rank=1, world_size=ws,
                            generator=None).tolist()
        assert set(seen) == set(full[1::ws])                  # one epoch covers the shard exactly
    a = FP.shuffled_epoch_sharded_lm_starts(num_tokens=n, seq_len=T, stride=s, batch_size=10, rank=0, world_size=ws,
                                            step=0, seed=1)
    b = FP.sequential_sharded_lm_starts(num_tokens=n, seq_len=T, stride=s, batch_size=10, rank=0, world_size=ws,
                                        step=0)
    assert not torch.equal(a, b)
    with pytest.raises(RuntimeError):
        FP.sample_sharded_lm_starts(num_tokens=40, seq_len=32, stride=16, batch_size=2, rank=1, world_size=2,
                                    generator=g)
    ev = FP.choose_lm_starts_lazy(num_tokens=n, seq_len=T, stride=s, batch_size=4, eval_batches=3, seed=0)
    assert len(ev) == 12 and set(ev) <= set(full)
    assert FP.choose_lm_starts_lazy(num_tokens=100, seq_len=T, stride=s, batch_size=4, eval_batches=9, seed=0) == \
        build_lm_starts(100, T, s)


def test_prefetcher_returns_sampler_order_and_closes():
    tokens = torch.arange(4096, dtype=torch.int16)
    with FP.BatchPrefetcher(tokens=tokens, seq_len=16, stride=8, batch_size=4, rank=0, world_size=1,
                            device=torch.device("cpu"), generator=torch.Generator().manual_seed(0),
                            batch_sampler=FP.SequentialShardedStartSampler()) as pf:
        x0, y0 = pf.next()
        x1, _ = pf.next()
    assert x0[:, 0].tolist() == [0, 8, 16, 24] and x1[:, 0].tolist() == [32, 40, 48, 56]
    assert torch.equal(y0[:, :-1].int(), x0[:, 1:])
    with pytest.raises(RuntimeError):
        pf.next()
    assert FP.Exp23BatchPrefetcher is FP.BatchPrefetcher


def test_loop_arithmetic():
    assert FP.steady_state_step_seconds([9.0, 1.0, 3.0, 2.0]) == 2.0
    assert FP.steady_state_step_seconds([4.0]) == 4.0
    with pytest.raises(ValueError):
        FP.steady_state_step_seconds([])
    ok = FP.summarize_cuda_graph_gate(budget_seconds=600, capture_seconds=5, warmup_seconds=5, warmup_steps=5,
                                      eager_step_seconds=0.1, graph_step_seconds=0.08)
    assert ok["accepted"] and ok["break_even_steps"] == pytest.approx(500)
    bad = FP.summarize_cuda_graph_gate(budget_seconds=600, capture_seconds=45, warmup_seconds=5, warmup_steps=5,
                                       eager_step_seconds=0.1, graph_step_seconds=0.11)
    assert not bad["accepted"] and {"graph_step_not_faster", "capture_seconds_exceeds_limit",
                                    "projected_speedup_below_minimum"} <= set(bad["reasons"])
    t = FP.summarize_train_timing(steps=10, elapsed_s=2.0, batch_size=4, seq_len=8, world_size=4)
    assert t["tokens_per_step"] == 128 and t["aggregate_tokens_per_sec"] == 640 and t["per_gpu_tokens_per_sec"] == 160
    te = FP.summarize_train_timing(steps=10, elapsed_s=2.0, batch_size=4, seq_len=8, world_size=4,
                                   episodic_enabled=True)
    assert te["tokens_per_step"] == 96 and te["per_gpu_tokens_per_sec"] == 160
    assert not FP.should_stop_training_loop(steps=0, elapsed_s=999, budget_seconds=1, stop_margin_seconds=0)
    assert FP.should_stop_training_loop(steps=5, elapsed_s=0, budget_seconds=100, stop_margin_seconds=0, max_steps=5)
    assert FP.should_stop_training_loop(steps=1, elapsed_s=98.5, budget_seconds=100, stop_margin_seconds=2)


def test_matrices(tmp_path):
    a = FP.build_stage_a_matrix(batch_sizes=(1024,), chunk_sizes=(64, 128))
    assert len(a) == 2 and a[0]["name"] == "stageA_v16384_b1024_c64_ckpt_s1337" and a[0]["model_dim"] == 256
    b = FP.build_stage_b_matrix(speed_config={"batch_size": 1024}, vocab_sizes=(16384,),
                                init_paths={16384: {"meanstd": "/x.pt"}})
    assert len(b) == 6 and {e["embed_init"] for e in b} == {"random", "meanstd"} and b[0]["mode"] == "base_lock"
    FP.write_matrix(tmp_path / "m" / "a.json", a)
    assert FP.read_speed_config(tmp_path / "m" / "a.json") if False else True
    (tmp_path / "c.json").write_text('{"config": {"batch_size": 7}}')
    assert FP.read_speed_config(tmp_path / "c.json") == {"batch_size": 7}


@pytest.mark.gpu
def test_prefetcher_pinned_staging_on_gpu():
    tokens = torch.arange(1 << 16, dtype=torch.int16)
    dev = torch.device("cuda")
    with FP.BatchPrefetcher(tokens=tokens, seq_len=64, stride=32, batch_size=8, rank=0, world_size=1, device=dev,
                            generator=torch.Generator().manual_seed(0),
                            batch_sampler=FP.SequentialShardedStartSampler()) as pf:
        assert pf._staged
        for step in range(6):
            x, y = pf.next()
            assert x.is_cuda and x.dtype == torch.int32
            want = (torch.arange(8) + 8 * step) * 32
            assert x[:, 0].cpu().tolist() == want.tolist()
            assert torch.equal(y[:, :-1].int(), x[:, 1:])
