"""C++ control plane through its C ABI: wire sizes, ring semantics (in-process
and across processes through POSIX shm), credit math, simplex forward/backward
against torch autograd, the online learner, CSWG files, CPU math, and the
controller loop draining shared-memory rings."""
import multiprocessing as mp
import os
import time

import numpy as np
import pytest
import torch

from chaoscontrol_b200.episodic import native as N


def test_wire_sizes_match_spec():
    sizes = N.check_wire_sizes()
    assert sizes == {0: 40, 1: 568, 2: 736, 3: 96, 4: 168, 5: 192, 6: 72, 7: 456, 8: 96}
    assert N.WRITE_EVENT.fields["key_rep"][1] == 32 and N.WRITE_EVENT.fields["value_tok_ids"][1] == 544
    assert N.lib().ccbc_ring_capacity(1) == 16384 and N.lib().ccbc_ring_capacity(3) == 8192


def test_ring_fifo_full_empty_and_wraparound():
    r = N.Ring(N.REPLAY_OUTCOME, 8)
    assert r.pop() is None and len(r) == 0
    for rnd in range(5):                       # wraps the index mask several times
        for i in range(8):
            ev = np.zeros((), N.REPLAY_OUTCOME)
            ev["replay_id"] = rnd * 100 + i
            assert r.push(ev)
        assert not r.push(np.zeros((), N.REPLAY_OUTCOME))      # full
        assert len(r) == 8
        for i in range(8):
            assert int(r.pop()["replay_id"]) == rnd * 100 + i
        assert r.pop() is None
    r.close()
    with pytest.raises(ValueError):
        N.Ring(N.REPLAY_OUTCOME, 6)            # capacity must be a power of two


def _producer(name, n):
    r = N.Ring(N.WRITE_EVENT, 64, shm_name=name, create=False)
    sent = 0
    while sent < n:
        ev = np.zeros((), N.WRITE_EVENT)
        ev["event_type"] = 1
        ev["candidate_id"] = sent
        ev["key_rep"][:] = sent % 65536
        if r.push(ev):
            sent += 1
    r.close()


def test_shm_ring_across_processes():
    name = f"/ccb_test_ring_{os.getpid()}"
    r = N.Ring(N.WRITE_EVENT, 64, shm_name=name, create=True)
    try:
        p = mp.get_context("spawn").Process(target=_producer, args=(name, 500))
        p.start()
        got, deadline = 0, time.time() + 60
        while got < 500 and time.time() < deadline:
            ev = r.pop()
            if ev is not None:
                assert int(ev["candidate_id"]) == got and int(ev["key_rep"][7]) == got % 65536
                got += 1
        p.join(10)
        assert got == 500 and p.exitcode == 0
    finally:
        r.close(unlink=True)
    with pytest.raises(ValueError):
        N.Ring(N.WRITE_EVENT, 64, shm_name="no_leading_slash", create=True)
    with pytest.raises(ValueError):
        N.Ring(N.WRITE_EVENT, 64, shm_name=f"/ccb_missing_{os.getpid()}", create=False)


def test_credit_helpers():
    assert N.recency_decay(2.0, 10, 10, 0.9) == pytest.approx(2.0)
    assert N.recency_decay(2.0, 13, 10, 0.9) == pytest.approx(2.0 * 0.9 ** 3, rel=1e-6)
    assert N.recency_decay(2.0, 5, 10, 0.9) == pytest.approx(2.0)      # outcome before action
    assert N.gerber_weight(1.0, 2.0, 0.5) == 1.0
    assert N.gerber_weight(1.0, -2.0, 0.5) == 0.0
    assert N.gerber_weight(0.1, 2.0, 0.5) == 0.0                        # under the threshold
    assert N.gerber_weight(0.0, 0.0, 0.5) == 1.0                        # exact agreement
    rs = N.RollingStddev(0.9)
    xs = np.random.default_rng(0).normal(3.0, 2.0, 2000)
    for x in xs:
        rs.update(float(x))
    assert abs(rs.mean() - 3.0) < 0.8 and 1.0 < rs.stddev() < 3.0


def _torch_policy_loss(flat, pol, V, E, feats, chosen, adv, beta):
    Kv, Ks, H = pol.K_v, pol.K_s, pol.H
    o = 0
    W_vp = flat[o:o + Kv * H].view(Kv, H); o += Kv * H
    b_vp = flat[o:o + H]; o += H
    W_lh = flat[o:o + H]; o += H
    b_lh = flat[o]; o += 1
    W_sb = flat[o:o + Ks]; o += Ks
    alpha = flat[o]
    vh = torch.nn.functional.gelu(V @ W_vp + b_vp)
    attn = torch.softmax(vh @ vh.T / H ** 0.5 + alpha * E, dim=-1)
    mixed = attn @ vh + vh
    logits = mixed @ W_lh + b_lh
    p = torch.softmax((logits + W_sb @ feats) / pol.temperature, dim=-1)
    ent = -(p * p.log()).sum()
    return -adv * p[chosen].log() - beta * ent, p


def test_simplex_forward_and_grad_match_autograd():
    pol = N.SimplexPolicy(N=16, K_v=16, K_s=4, H=32, temperature=0.7, seed=1)
    rng = np.random.default_rng(2)
    V = rng.standard_normal((16, 16)).astype(np.float32)
    E = rng.standard_normal((16, 16)).astype(np.float32)
    feats = rng.standard_normal(4).astype(np.float32)
    p, logits = pol.forward(V, E, feats)
    flat = torch.tensor(pol.flat, dtype=torch.float64, requires_grad=True)
    loss, p_ref = _torch_policy_loss(flat, pol, torch.tensor(V, dtype=torch.float64),
                                     torch.tensor(E, dtype=torch.float64),
                                     torch.tensor(feats, dtype=torch.float64), 5, 1.3, 0.05)
    assert np.allclose(p, p_ref.detach().numpy(), atol=1e-5) and abs(p.sum() - 1) < 1e-5
    loss.backward()
    g = pol.grad(V, E, feats, chosen=5, advantage=1.3, entropy_beta=0.05)
    assert np.allclose(g, flat.grad.numpy(), atol=2e-4, rtol=2e-3)


def test_online_learner_moves_policy_toward_rewarded_action():
    pol = N.SimplexPolicy(seed=3)
    rng = np.random.default_rng(4)
    V = rng.standard_normal((16, 16)).astype(np.float32)
    E = np.zeros((16, 16), np.float32)
    feats = np.zeros(4, np.float32)
    L = N.SimplexOnlineLearner(num_slots=8, max_entries_per_slot=4, learning_rate=0.5, sgd_interval=1,
                               ema_interval=2, ema_alpha=0.5)
    L.initialize(pol)
    p0, _ = pol.forward(V, E, feats)
    for step in range(30):
        cur = N.SimplexPolicy(seed=3)
        cur.flat = L.weights()
        p, _ = cur.forward(V, E, feats)
        L.record_decision(slot_id=2, gpu_step=step, chosen=7, p_chosen=float(p[7]), V=V, E=E, feats=feats)
        ev = np.zeros((), N.REPLAY_OUTCOME)
        ev["event_type"], ev["slot_id"], ev["gpu_step"] = 3, 2, step
        ev["reward_shaped"] = 1.0 if step % 2 == 0 else 1.5
        L.on_replay_outcome(ev)
    t = L.telemetry()
    assert t["replay_outcomes"] == 30 and t["sgd_steps"] > 0 and t["ema_blends"] > 0
    assert L.history_size(2) == 4                     # bounded per-slot history
    bad = np.zeros((), N.REPLAY_OUTCOME)
    bad["slot_id"] = 999
    bad["reward_shaped"] = 1.0
    L.on_replay_outcome(bad)
    assert L.telemetry()["invalid_slot_skips"] == 1
    assert not np.allclose(L.weights(), pol.flat)
    assert not np.allclose(L.weights(slow=True), pol.flat)
    L.close()


def test_cswg_roundtrip_and_errors(tmp_path):
    payload = np.random.default_rng(0).standard_normal(100).astype(np.float32)
    path = tmp_path / "w.cswg"
    N.write_cswg(str(path), payload, n_layers=2, d_global=8, d_slot=4, feature_dim=16)
    hdr, got = N.load_cswg(str(path))
    assert hdr == {"version": 1, "n_layers": 2, "d_global": 8, "d_slot": 4, "feature_dim": 16, "dtype": 1}
    assert np.allclose(got, payload.astype(np.float16).astype(np.float32))
    bad = tmp_path / "bad.cswg"
    bad.write_bytes(b"NOPE" + b"\0" * 24)
    with pytest.raises(ValueError, match="magic"):
        N.load_cswg(str(bad))
    for v in (0.0, 1.0, -2.5, 65504.0, 1e-7, 3.14159):
        h = N.lib().ccbc_float_to_half(v)
        assert N.lib().ccbc_half_to_float(h) == pytest.approx(float(np.float16(v)), rel=1e-3, abs=1e-7)


def test_cpu_math_vector_paths_match_scalar():
    feats = N.cpu_features()
    assert set(feats) == {"avx2", "avx512f", "amx_tile", "amx_bf16", "amx_enabled"}
    rng = np.random.default_rng(0)
    W = rng.standard_normal((37, 70)).astype(np.float32)
    x = rng.standard_normal(70).astype(np.float32)
    assert np.allclose(N.matvec(W, x), N.matvec(W, x, force_scalar=True), atol=1e-4)
    assert np.allclose(N.matvec(W, x), W @ x, atol=1e-4)
    d, u, h = (rng.random(50).astype(np.float32) for _ in range(3))
    assert np.allclose(N.diag_step(d, u, h), d * h + u, atol=1e-6)
    A = torch.randn(33, 48).bfloat16()
    B = torch.randn(48, 20).bfloat16()
    Ab = A.view(torch.int16).numpy().view(np.uint16)
    Bb = B.view(torch.int16).numpy().view(np.uint16)
    Cv, _used = N.bf16_matmul(Ab, Bb)
    Cs, _ = N.bf16_matmul(Ab, Bb, force_scalar=True)
    ref = (A.float() @ B.float()).numpy()
    assert np.allclose(Cs, ref, atol=1e-3) and np.allclose(Cv, ref, atol=1e-2)


def test_controller_loop_drains_rings_and_feeds_learner():
    pid = os.getpid()
    names = {k: f"/ccb_ctl_{k}_{pid}" for k in ("w0", "w1", "q", "r", "exit", "stats")}
    rings = {"w0": N.Ring(N.WRITE_EVENT, 16384, shm_name=names["w0"]),
             "w1": N.Ring(N.WRITE_EVENT, 16384, shm_name=names["w1"]),
             "q": N.Ring(N.QUERY_EVENT, 16384, shm_name=names["q"]),
             "r": N.Ring(N.REPLAY_OUTCOME, 8192, shm_name=names["r"])}
    exit_flag = N.ShmBytes(names["exit"], 1)
    stats = N.ShmBytes(names["stats"], 24)
    pol = N.SimplexPolicy(seed=5)
    L = N.SimplexOnlineLearner(num_slots=16, sgd_interval=1)
    L.initialize(pol)
    try:
        th, box = N.controller_thread([names["w0"], names["w1"]], names["q"], names["r"], names["exit"],
                                      names["stats"], L)
        for i in range(40):
            ev = np.zeros((), N.WRITE_EVENT)
            ev["event_type"] = 1
            assert rings["w0" if i % 2 else "w1"].push(ev)
        for i in range(7):
            assert rings["q"].push(np.zeros((), N.QUERY_EVENT))
        for i in range(5):
            ev = np.zeros((), N.REPLAY_OUTCOME)
            ev["slot_id"], ev["reward_shaped"] = 3, 1.0
            assert rings["r"].push(ev)
        deadline = time.time() + 20
        while time.time() < deadline:
            c = stats.array[:24].view(np.uint64)
            if tuple(int(v) for v in c) == (40, 7, 5):
                break
            time.sleep(0.01)
        exit_flag.array[0] = 1
        th.join(10)
        assert not th.is_alive() and "error" not in box, box
        assert box["result"] == {"total": 52, "writes": 40, "queries": 7, "replays": 5}
        assert L.telemetry()["replay_outcomes"] == 5
    finally:
        exit_flag.array[0] = 1
        for r in rings.values():
            r.close(unlink=True)
        exit_flag.close(unlink=True)
        stats.close(unlink=True)
        L.close()


# ---------------------------------------------------------------------------
# residual attention heads + bucket embedding of the simplex policy, and the pretrain trunk
# ---------------------------------------------------------------------------
def _torch_policy_v3(pol, V, E, feats):
    """Torch twin of the native forward on the same flat weights (differentiable)."""
    import torch
    N, Kv, Ke, Ks, H, nh = pol.N, pol.K_v, pol.K_e, pol.K_s, pol.H, pol.n_heads
    flat = torch.tensor(pol.flat, dtype=torch.float64, requires_grad=True)
    o = 0

    def take(*shape):
        nonlocal o
        n = int(np.prod(shape)) if shape else 1
        t = flat[o:o + n].reshape(shape) if shape else flat[o]
        o += n
        return t
    W_vp, b_vp, W_lh, b_lh, W_sb, alpha = take(Kv, H), take(H), take(H), take(), take(Ks), take()
    V, E, feats = (torch.tensor(np.asarray(a), dtype=torch.float64) for a in (V, E, feats))
    E = E.reshape(N, N, Ke)
    vh = torch.nn.functional.gelu(V @ W_vp + b_vp)
    attn = torch.softmax(vh @ vh.T / H ** 0.5 + alpha * E[..., 0], dim=-1)
    mixed = attn @ vh + vh
    logits = mixed @ W_lh + b_lh
    hxh = torch.zeros(N, dtype=torch.float64)
    if nh:
        lam = take()
        Wq, Wk, Wv, Wo, We = take(nh, H, H), take(nh, H, H), take(nh, H, H), take(nh, H), take(nh, Ke)
        for h in range(nh):
            q, k, v = vh @ Wq[h], vh @ Wk[h], vh @ Wv[h]
            a = torch.softmax(q @ k.T / H ** 0.5 + (E * We[h]).sum(-1), dim=-1)
            hxh = hxh + ((a @ v) @ Wo[h]) / nh
        logits = logits + lam * hxh
    p = torch.softmax((logits + feats @ W_sb) / pol.temperature, dim=-1)
    return flat, p, logits, hxh


@pytest.mark.parametrize("n_heads,K_e", [(0, 1), (2, 3), (1, 1)])
def test_simplex_policy_residual_heads_match_a_torch_twin(n_heads, K_e):
    import torch
    from chaoscontrol_b200.episodic.native import SimplexPolicyV3
    rng = np.random.default_rng(5)
    pol = SimplexPolicyV3(N=8, K_v=6, K_e=K_e, K_s=3, H=10, n_heads=n_heads, n_buckets=4, embed_dim=5,
                          temperature=0.7, seed=3)
    pol.flat *= 4.0
    V, E, feats = rng.standard_normal((8, 6)), rng.standard_normal((8, 8, K_e)), rng.standard_normal(3)
    p, logits, hxh = pol.forward(V, E, feats, with_branch=True)
    flat, tp, tl, th = _torch_policy_v3(pol, V, E, feats)
    assert np.allclose(p, tp.detach().numpy(), atol=2e-5) and np.allclose(logits, tl.detach().numpy(), atol=2e-4)
    assert np.allclose(hxh, th.detach().numpy(), atol=2e-4)
    if n_heads:
        assert np.abs(hxh).max() > 1e-3                       # the branch is live
    chosen, adv, beta = 3, 0.8, 0.05
    loss = -adv * torch.log(tp[chosen]) + beta * (tp * torch.log(tp)).sum()      # -adv log p - beta H(p)
    loss.backward()
    g = pol.grad(V, E, feats, chosen, adv, beta)
    ref = flat.grad.numpy()
    assert np.allclose(g, ref, atol=3e-4, rtol=2e-3), np.abs(g - ref).max()
    n_embed = 4 * 5
    assert np.all(g[-n_embed:] == 0.0)                        # the stored embedding takes no gradient
    # with no heads, one edge feature and no table the flat layout is the base policy's
    if n_heads == 0:
        from chaoscontrol_b200.episodic.native import SimplexPolicy
        base = SimplexPolicy(N=8, K_v=6, K_s=3, H=10, temperature=0.7, seed=3)
        assert base.flat.size == pol.flat.size - n_embed
        base.flat[:] = pol.flat[: base.flat.size]
        pb, lb = base.forward(V, E[..., 0], feats)
        assert np.allclose(pb, p, atol=1e-6) and np.allclose(lb, logits, atol=1e-6)


def test_forward_pretrain_model_matches_torch():
    import torch
    from chaoscontrol_b200.episodic.native import forward_pretrain_model
    g = torch.Generator().manual_seed(0)
    B, F, Dg, L, Ds = 5, 7, 12, 3, 4
    w = {"trunk.in_proj.weight": torch.randn(Dg, F, generator=g) * 0.3, "trunk.in_proj.bias": torch.randn(Dg, generator=g) * 0.1,
         "trunk.decay": torch.rand(L, Dg, generator=g), "trunk.w_in": torch.randn(L, Dg, Dg, generator=g) * 0.2,
         "trunk.w_out": torch.randn(L, Dg, Dg, generator=g) * 0.3, "trunk.bias": torch.randn(L, Dg, generator=g) * 0.1,
         "policy_head.weight": torch.randn(Ds, Dg, generator=g) * 0.3, "policy_head.bias": torch.randn(Ds, generator=g) * 0.1,
         "value_head.weight": torch.randn(1, Dg, generator=g) * 0.3, "value_head.bias": torch.randn(1, generator=g) * 0.1}
    x = torch.randn(B, F, generator=g)
    h = x @ w["trunk.in_proj.weight"].T + w["trunk.in_proj.bias"]
    for l in range(L):
        h = torch.nn.functional.gelu(h * w["trunk.decay"][l] + h @ w["trunk.w_in"][l] + w["trunk.bias"][l]) @ w["trunk.w_out"][l]
    ref_logits = h @ w["policy_head.weight"].T + w["policy_head.bias"]
    ref_value = (h @ w["value_head.weight"].T + w["value_head.bias"]).squeeze(-1)
    logits, value = forward_pretrain_model(x.numpy(), {k: v.numpy() for k, v in w.items()})
    assert np.allclose(logits, ref_logits.numpy(), atol=1e-5) and np.allclose(value, ref_value.numpy(), atol=1e-5)
    with pytest.raises(ValueError):
        forward_pretrain_model(x.numpy()[:, :3], {k: v.numpy() for k, v in w.items()})
