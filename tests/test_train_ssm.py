"""train_ssm_step / train_ssm_for_budget on CPU: head modes agree, the loop
honours budget / max_steps with a fake clock, and 2-rank gloo DDP leaves the
ranks with identical parameters."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from chaoscontrol_b200.models.model import CareStudentLM
from chaoscontrol_b200.optim.muon import Muon
from chaoscontrol_b200.train_ssm import (chunked_lm_head_backward, full_lm_head_backward,
                                         train_ssm_for_budget, train_ssm_step)


def _tiny(seed=0):
    torch.manual_seed(seed)
    return CareStudentLM(vocab_size=64, dim=16, num_layers=2)


def _grads(m):
    return {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("mode", ["single", "fused", "fused_streaming_v2", "fused_norm_streaming_v2"])
def test_head_modes_match_chunked(mode):
    tok = torch.randint(0, 64, (2, 12))
    tgt = torch.randint(0, 64, (2, 12))
    m = _tiny()
    loss_c = train_ssm_step(m, tok, tgt, 5, lm_head_backward_mode="chunked")
    ref = _grads(m)
    m.zero_grad()
    loss = train_ssm_step(m, tok, tgt, 5, lm_head_backward_mode=mode)
    assert torch.allclose(loss, loss_c, atol=1e-5)
    for n, g in _grads(m).items():
        assert torch.allclose(g, ref[n], atol=2e-5), n


@pytest.mark.parametrize("chunk", [1, 5, 12, 100])
def test_chunked_head_matches_full(chunk):
    m = _tiny(1)
    hidden = torch.randn(3, 12, 16)
    tgt = torch.randint(0, 64, (3, 12))
    h1 = hidden.clone().requires_grad_(True)
    l1 = full_lm_head_backward(h1, m.final_norm, m.lm_head, tgt)
    g1 = (h1.grad.clone(), m.lm_head.weight.grad.clone(), m.final_norm.weight.grad.clone())
    m.zero_grad()
    h2 = hidden.clone().requires_grad_(True)
    l2 = chunked_lm_head_backward(h2, m.final_norm, m.lm_head, tgt, chunk)
    assert torch.allclose(l1, l2, atol=1e-5)
    for a, b in zip(g1, (h2.grad, m.lm_head.weight.grad, m.final_norm.weight.grad)):
        assert torch.allclose(a, b, atol=1e-5)


def test_chunked_head_rejects_bad_args():
    m = _tiny()
    h = torch.randn(1, 4, 16)
    with pytest.raises(ValueError):
        chunked_lm_head_backward(h.requires_grad_(True), m.final_norm, m.lm_head,
                                 torch.zeros(1, 4, dtype=torch.long), 0)
    with pytest.raises(ValueError):
        chunked_lm_head_backward(torch.randn(1, 4, 16), m.final_norm, m.lm_head,
                                 torch.zeros(1, 4, dtype=torch.long), 2)
    with pytest.raises(ValueError):
        train_ssm_step(m, torch.zeros(1, 4, dtype=torch.long), torch.zeros(1, 4, dtype=torch.long),
                       2, lm_head_backward_mode="bogus")


class _Clock:
    def __init__(self, dt):
        self.t, self.dt = 0.0, dt

    def __call__(self):
        self.t += self.dt
        return self.t


def test_budget_loop_fake_clock_and_loss_goes_down():
    m = _tiny(2)
    tokens = torch.randint(0, 64, (4000,))
    starts = list(range(0, 3900, 7))
    opt = Muon(m.parameters(), lr=0.02)
    opt.bind_param_names(m.named_parameters())
    res = train_ssm_for_budget(m, train_tokens=tokens, train_starts=starts, seq_len=16, batch_size=8,
                               device=torch.device("cpu"), optimizer=opt, budget_seconds=1e9,
                               chunk_size=8, max_steps=12, precision="fp32")
    assert res["steps"] == 12 and len(res["history"]) == 12
    assert res["history"][-1]["loss"] < res["history"][0]["loss"]
    assert set(res) == {"history", "steps", "elapsed_s", "rank", "world_size", "peak_vram_mb"}
    res2 = train_ssm_for_budget(m, train_tokens=tokens, train_starts=starts, seq_len=16,
                                batch_size=4, device=torch.device("cpu"), optimizer=opt,
                                budget_seconds=10.0, chunk_size=8, time_fn=_Clock(1.0),
                                precision="fp32")
    assert 5 <= res2["steps"] <= 12


def _ddp_worker(rank, ws, port, outdir):
    torch.set_num_threads(1)      # several ranks share this machine's cores: no intra-op thread pools
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    try:
        m = _tiny(10 + rank)          # different init per rank: broadcast must fix it
        tokens = torch.randint(0, 64, (3000,), generator=torch.Generator().manual_seed(0))
        opt = Muon(m.parameters(), lr=0.02)
        opt.bind_param_names(m.named_parameters())
        res = train_ssm_for_budget(m, train_tokens=tokens, train_starts=list(range(0, 2900, 5)),
                                   seq_len=12, batch_size=4, device=torch.device("cpu"),
                                   optimizer=opt, budget_seconds=1e9, chunk_size=6, max_steps=4,
                                   rank=rank, world_size=ws, precision="fp32")
        torch.save({"sd": m.state_dict(), "steps": res["steps"]}, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ddp_two_ranks_gloo_identical_params():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_ddp_worker, args=(2, port, d), nprocs=2, join=True)
        a = torch.load(os.path.join(d, "r0.pt"))
        b = torch.load(os.path.join(d, "r1.pt"))
    assert a["steps"] == b["steps"] == 4
    for k in a["sd"]:
        assert torch.equal(a["sd"][k], b["sd"][k]), k


def test_reference_module_paths_and_names_resolve():
    """Import paths a user of the reference package relies on."""
    import importlib
    for mod, names in {
        "chaoscontrol_b200.local_attn": ["LocalAttention", "RollingKVCache"],
        "chaoscontrol_b200.eval.ttt_eval": ["register_calc_type", "evaluate_with_calc_types", "CalcTypeContext"],
        "chaoscontrol_b200.eval.runner_dispatch": ["dispatch_eval_for_config"],
        "chaoscontrol_b200.eval.packet_online_cache_compare": ["run_packet_online_cache_compare"],
        "chaoscontrol_b200.eval_stream.delta_mod": ["DeltaModulator"],
        "chaoscontrol_b200.eval_stream.persistence": ["StateManager", "attach_trainable_h0"],
        "chaoscontrol_b200.eval_stream.ttt_runner": ["select_adapt_params"],
        "chaoscontrol_b200.eval_stream.doc_stream": ["DocStreamer"],
        "chaoscontrol_b200.eval_stream.metrics": ["MetricsCollector"],
        "chaoscontrol_b200.eval_stream.val_cache": ["ValCache", "write_val_cache", "load_val_cache"],
        "chaoscontrol_b200.optim.momentum_warmup": ["apply_momentum_warmup"],
        "chaoscontrol_b200.optim.step_wrapper": ["wrap_optimizer_step"],
        "chaoscontrol_b200.optim.weight_ema": ["WeightEMA", "eval_with_ema"],
        "chaoscontrol_b200.models.model": ["CareSSMHybridBlock", "AttentionControlBlock"],
        "chaoscontrol_b200.models.core_fused": ["get_post_scan_backend"],
        "chaoscontrol_b200.train_ssm": ["fused_lm_head_weighted_loss_with_ce"],
    }.items():
        m = importlib.import_module(mod)
        for n in names:
            assert getattr(m, n) is not None, (mod, n)


def test_weighted_lm_head_loss_with_ce_matches_the_formula():
    import torch.nn.functional as F2
    from chaoscontrol_b200.models.core import RMSNorm
    from chaoscontrol_b200.train_ssm import fused_lm_head_weighted_loss_with_ce
    torch.manual_seed(0)
    hidden = torch.randn(2, 5, 16, requires_grad=True)
    norm, head = RMSNorm(16), torch.nn.Linear(16, 32, bias=False)
    tgt = torch.randint(0, 32, (2, 5))
    w = torch.rand(2, 5)
    loss, ce = fused_lm_head_weighted_loss_with_ce(hidden=hidden, final_norm=norm, lm_head=head, targets=tgt,
                                                   token_weight=w)
    ref_ce = F2.cross_entropy(head(norm(hidden)).reshape(-1, 32), tgt.reshape(-1), reduction="none")
    assert torch.allclose(ce.reshape(-1), ref_ce.detach(), atol=1e-5)
    assert torch.allclose(loss, (ref_ce * w.reshape(-1)).sum() / w.sum().clamp_min(1.0), atol=1e-5)
    loss.backward()
    assert hidden.grad is not None and head.weight.grad is not None
