"""Episodic controller cycle: drain the query queue, retrieve candidates from the
cache, let a policy pick, push replay tags (behaviour of
src/chaoscontrol/episodic/controller.py:71-910).

A cycle takes everything queued so far, stacks the query residuals and scores
them against ONE snapshot of the cache in a single matmul + top-k (the reference
runs one retrieval and one re-scoring per query).  What happens to a query's
candidates depends on the runtime handed in:

* no runtime            every candidate becomes a tag, ranked by the heuristic score;
* per-slot runtime      (``score_slot[_with_snapshot]``, e.g. ``CpuSsmControllerRuntime``) adds a
                        learned logit to every tag, and an optional bounded action space reranks /
                        clamps the candidates;
* simplex runtime       (anything with ``record_simplex_decision``) builds the 16-vertex simplex
                        inputs ``V [16, 16]``, ``E [16, 16]``, 4 summary features, runs the native
                        policy forward and emits exactly one tag: the chosen vertex.

Tags are plain Python scalars and lists; no tensor is ever stored on a tag.
"""
from __future__ import annotations

import hashlib
import math
import os
import threading
import time
from typing import Any, Optional

import numpy as np
import torch

from .cache import EpisodicCache
from .learned_action_space import coerce_action_space
from .query import query_topk_batch

K_V, K_S, N_VERTICES = 16, 4, 16
AGE_NORMALIZER = 1000.0
FEATURE_MANIFEST = ("simplex_v1:V0=utility_u,V1=query_cosine,V2=age_steps/1000,V3=pressure_at_write,"
                    "V4..15=0,E0=key_rep_cosine,sf=(top1_u,mean_u,top1_cos,cos_spread)")
FEATURE_MANIFEST_HASH = hashlib.sha256(FEATURE_MANIFEST.encode("utf-8")).hexdigest()[:16]

__all__ = ["run_controller_cycle", "controller_main", "build_simplex_inputs", "choose_simplex_vertex",
           "SimplexRuntime", "load_simplex_policy", "save_simplex_policy", "FEATURE_MANIFEST", "FEATURE_MANIFEST_HASH"]


def _is_simplex_runtime(runtime: Any) -> bool:
    return runtime is not None and hasattr(runtime, "record_simplex_decision")


class SimplexRuntime:
    """Native simplex policy + online learner behind the interface the cycle expects
    (``simplex_forward``, ``fast_weights``, the three meta-knob setters and
    ``record_simplex_decision``)."""

    def __init__(self, policy=None, learner=None, **learner_kw) -> None:
        from . import native
        self.policy = policy or native.SimplexPolicy()
        self.learner = learner or native.SimplexOnlineLearner(**learner_kw)
        self.learner.initialize(self.policy)
        self.entropy_beta, self.ema_alpha = 0.0, 0.25
        self.decisions: list[dict[str, Any]] = []

    def fast_weights(self):
        return self.policy

    def sync_policy(self, seen_sgd_steps: int = -1) -> int:
        """Copies the learner's fast weights into the selection policy once the learner has
        taken a step since ``seen_sgd_steps``; returns the learner's step count."""
        steps = int(self.learner.telemetry()["sgd_steps"])
        if steps != seen_sgd_steps:
            self.policy.flat[:] = self.learner.weights(slow=False)
        return steps

    def simplex_forward(self, V, E, sf):
        return self.policy.forward(V, E, sf)

    def set_temperature(self, v: float) -> None:
        self.policy.temperature = float(v)

    def set_entropy_beta(self, v: float) -> None:
        self.entropy_beta = float(v)

    def set_ema_alpha(self, v: float) -> None:
        self.ema_alpha = float(v)

    def record_simplex_decision(self, *, chosen_slot_id: int, gpu_step: int, chosen_idx: int,
                                p_chosen_decision: float, V, E, simplex_features, **meta: Any) -> None:
        self.learner.record_decision(int(chosen_slot_id), int(gpu_step), int(chosen_idx), float(p_chosen_decision),
                                     V, E, simplex_features)
        self.decisions.append({"chosen_slot_id": int(chosen_slot_id), "gpu_step": int(gpu_step),
                               "chosen_idx": int(chosen_idx), "p_chosen": float(p_chosen_decision), **meta})


_SIMPLEX_TENSORS = ("W_vp", "b_vp", "W_lh", "b_lh", "W_sb", "alpha")


def _simplex_sizes(K_v: int, K_s: int, H: int) -> tuple[int, ...]:
    return (K_v * H, H, H, 1, K_s, 1)


def save_simplex_policy(path, policy) -> None:
    """Writes a simplex policy.  ``*.pt``: ``{"manifest": {"dims": {k_v, k_s, h, n_vertices}},
    "tensors": {W_vp, b_vp, W_lh, b_lh, W_sb, alpha, temperature}}`` (the layout the reference
    reads in experiments/23_fast_path/runner_fast_path.py:8423-8443); anything else: a CSWG file
    whose header carries ``(N, K_v, K_s, H)`` and whose payload is the flat weights followed by
    the temperature."""
    flat = np.asarray(policy.flat, np.float32)
    if str(path).endswith(".pt"):
        tensors, o = {}, 0
        for name, n in zip(_SIMPLEX_TENSORS, _simplex_sizes(policy.K_v, policy.K_s, policy.H)):
            tensors[name] = torch.from_numpy(flat[o:o + n].copy())
            o += n
        tensors["W_vp"] = tensors["W_vp"].view(policy.K_v, policy.H)
        tensors["temperature"] = torch.tensor(float(policy.temperature))
        torch.save({"manifest": {"dims": {"k_v": policy.K_v, "k_s": policy.K_s, "h": policy.H,
                                          "n_vertices": policy.N},
                                 "feature_manifest_hash": FEATURE_MANIFEST_HASH},
                    "tensors": tensors}, str(path))
        return
    if str(path).endswith((".cswg3", ".v3.cswg")) or getattr(policy, "n_heads", 0) or getattr(policy, "n_buckets", 0):
        from .cswg import policy_to_cswg                  # self-describing file: carries the optional parts too
        policy_to_cswg(policy, path)
        return
    from . import native
    native.write_cswg(str(path), np.concatenate([flat, [np.float32(policy.temperature)]]),
                      n_layers=policy.N, d_global=policy.K_v, d_slot=policy.K_s, feature_dim=policy.H)


def load_simplex_policy(path):
    """Inverse of `save_simplex_policy`; raises ``ValueError`` on a size mismatch."""
    from . import native
    if str(path).endswith(".pt"):
        art = torch.load(str(path), map_location="cpu", weights_only=False)
        dims, t = art["manifest"]["dims"], art["tensors"]
        pol = native.SimplexPolicy(N=int(dims["n_vertices"]), K_v=int(dims["k_v"]), K_s=int(dims["k_s"]),
                                   H=int(dims["h"]), temperature=float(t["temperature"]))
        flat = np.concatenate([np.asarray(t[k], np.float32).reshape(-1) for k in _SIMPLEX_TENSORS])
    else:
        from .cswg import file_version, policy_from_cswg
        if file_version(path) == 3:
            return policy_from_cswg(path)
        hdr, payload = native.load_cswg(str(path))
        pol = native.SimplexPolicy(N=hdr["n_layers"], K_v=hdr["d_global"], K_s=hdr["d_slot"],
                                   H=hdr["feature_dim"])
        if payload.size != pol.flat.size + 1:
            raise ValueError(f"{path}: payload of {payload.size} values does not fit a simplex policy "
                             f"of {pol.flat.size} weights + temperature")
        flat, pol.temperature = payload[:-1], float(payload[-1])
    if flat.size != pol.flat.size:
        raise ValueError(f"{path}: {flat.size} weights, the dims ask for {pol.flat.size}")
    pol.flat[:] = flat
    return pol


# ---------------------------------------------------------------------------
# simplex inputs
# ---------------------------------------------------------------------------
def build_simplex_inputs(*, cache_view: dict[str, torch.Tensor], slots: torch.Tensor, scores: torch.Tensor,
                         current_step: int, pad_to: int = N_VERTICES):
    """``(V [pad, 16], E [pad, pad], sf [4], padded_slot_ids)`` as fp32 numpy arrays for one query.
    ``V[:, 0..3]`` = utility, retrieval score, age / 1000 steps, pressure at write; ``E`` = pairwise cosine
    of the candidates' key representations; ``sf`` = (top-1 utility, mean utility, top-1 score, score
    spread).  Vertices beyond the retrieved count are all-zero."""
    n = int(slots.numel())
    V = np.zeros((pad_to, K_V), np.float32)
    E = np.zeros((pad_to, pad_to), np.float32)
    sf = np.zeros(K_S, np.float32)
    ids = [0] * pad_to
    if n == 0:
        return V, E, sf, ids
    sl = slots.long()
    util = cache_view["utility_u"][sl].float()
    sc = scores.float()
    V[:n, 0] = util.cpu().numpy()
    V[:n, 1] = sc.cpu().numpy()
    V[:n, 2] = ((int(current_step) - cache_view["write_step"][sl]).float() / AGE_NORMALIZER).cpu().numpy()
    V[:n, 3] = cache_view["pressure_at_write"][sl].float().cpu().numpy()
    keys = cache_view["key_rep"][sl].float()
    kn = keys / keys.norm(dim=1, keepdim=True).clamp_min(1e-12)
    E[:n, :n] = (kn @ kn.T).clamp(-1.0, 1.0).cpu().numpy()
    sf[:] = (float(util.max()), float(util.mean()), float(sc.max()), float(sc.max() - sc.min()))
    ids[:n] = [int(x) for x in sl.tolist()]
    return V, E, sf, ids


def choose_simplex_vertex(probs, n_actual: int, *, mode: str = "argmax",
                          generator: Optional[torch.Generator] = None) -> tuple[int, float]:
    """Vertex index and its (renormalised over the ``n_actual`` real vertices) probability."""
    n = int(n_actual)
    if n <= 0:
        raise ValueError("n_actual must be positive for simplex selection")
    p = torch.as_tensor(np.asarray(probs, dtype=np.float32)[:n]).clamp_min(0.0)
    tot = float(p.sum())
    p = p / tot if math.isfinite(tot) and tot > 0.0 else torch.full((n,), 1.0 / n)
    m = str(mode).strip().lower()
    if m in ("argmax", "greedy"):
        i = int(torch.argmax(p))
    elif m in ("sample", "soft_sample", "stochastic"):
        i = int(torch.multinomial(p, 1, generator=generator))
    else:
        raise ValueError("simplex_selection_mode must be one of 'argmax', 'greedy', 'sample', 'soft_sample', "
                         f"or 'stochastic'; got {mode!r}")
    return i, float(p[i])


def _query_event_id(cand: dict[str, Any]) -> int:
    """Explicit id when the producer supplied one, else ``rank << 56 | sequence``."""
    for key in ("query_event_id", "candidate_id", "event_id"):
        if key in cand:
            return int(cand[key])
    return (int(cand.get("source_rank", cand.get("rank", 0))) << 56) | int(cand.get("rank_seq", cand.get("k", 0)))


def _replay_id(query_event_id: int, rank: int) -> int:
    return ((int(query_event_id) & ((1 << 56) - 1)) << 8) | (int(rank) & 0xFF)


def _drain(queue, lock: Optional[threading.Lock]) -> list[dict[str, Any]]:
    pop = getattr(queue, "popleft", None) or (lambda: queue.pop(0))
    out: list[dict[str, Any]] = []

    def take() -> None:
        while True:
            try:
                out.append(pop())
            except IndexError:
                return

    if lock is not None:
        with lock:
            take()
    else:
        take()
    return out


def _apply_meta_actions(runtime: Any, space: Any, gpu_step: int, ctx: dict[str, Any]) -> None:
    fallbacks = (("temperature", "set_temperature", float(getattr(runtime.fast_weights(), "temperature", 1.0))),
                 ("entropy_beta", "set_entropy_beta", 0.0), ("ema_alpha", "set_ema_alpha", 0.25))
    for head, setter, fallback in fallbacks:
        if space.readiness(head) <= 0.0:
            continue
        value = space.scalar_value(head_name=head, gpu_step=int(gpu_step), fallback=fallback, reward_context=ctx)
        fn = getattr(runtime, setter, None)
        if callable(fn):
            fn(float(value))


def _simplex_forward(runtime: Any, V, E, sf):
    fwd = getattr(runtime, "simplex_forward", None)
    if callable(fwd):
        return fwd(V, E, sf)
    return runtime.fast_weights().forward(V, E, sf)


# ---------------------------------------------------------------------------
# one cycle
# ---------------------------------------------------------------------------
def run_controller_cycle(*, controller_query_queue, tagged_replay_queue: list, cache: EpisodicCache, k: int = 16,
                         score_mode: str = "cosine_utility_weighted", queue_lock: Optional[threading.Lock] = None,
                         selected_at: Optional[int] = None, policy_version: int = 0,
                         controller_runtime: Any = None, action_recorder: Any = None,
                         simplex_selection_mode: str = "argmax",
                         simplex_generator: Optional[torch.Generator] = None, action_space: Any = None) -> int:
    """Returns the number of queries drained.  Each query dict carries ``step``, ``rank``, ``k``,
    ``pressure`` and ``residual`` (fp32 ``[D]``); its residual reference is dropped once used."""
    cands = _drain(controller_query_queue, queue_lock)
    if not cands:
        return 0
    if selected_at is None:
        selected_at = int(time.monotonic_ns() // 1_000_000)
    space = coerce_action_space(action_space)
    simplex = _is_simplex_runtime(controller_runtime)
    dev = cands[0]["residual"].device
    view = cache.snapshot_to(dev)
    queries = torch.stack([c["residual"].to(dev).float() for c in cands], 0)
    all_slots, all_scores = query_topk_batch(queries, view, int(k), score_mode)
    for qi, cand in enumerate(cands):
        keep = all_slots[qi] >= 0
        slots, scores = all_slots[qi][keep], all_scores[qi][keep]
        cand["residual"] = None
        if slots.numel() == 0:
            continue
        step = int(cand.get("step", -1))
        qid = _query_event_id(cand)
        slot_list = [int(s) for s in slots.tolist()]
        score_list = [float(s) for s in scores.tolist()]
        src_ids = view["source_write_id"][slots.long()].tolist()
        if simplex:
            _emit_simplex_tag(cand, step, qid, slots, scores, slot_list, score_list, view, controller_runtime,
                              action_recorder, space, simplex_selection_mode, simplex_generator, selected_at,
                              policy_version, tagged_replay_queue)
            continue
        logits, snaps = list(score_list), [{} for _ in slot_list]
        if controller_runtime is not None:
            util = view["utility_u"][slots.long()].tolist()
            for r, (s, sc) in enumerate(zip(slot_list, score_list)):
                feats = torch.tensor([sc, float(cand.get("pressure", 0.0)), float(util[r]), float(r)])
                snap_fn = getattr(controller_runtime, "score_slot_with_snapshot", None)
                if snap_fn is None:
                    logits[r] = float(controller_runtime.score_slot(feats, slot=s))
                else:
                    d = snap_fn(feats, slot=s)
                    logits[r] = float(d.logit)
                    snaps[r] = {"controller_features": d.features.float().tolist(),
                                "controller_global_state": d.global_state.float().tolist(),
                                "controller_slot_state": d.slot_state.float().tolist()}
        if space is None:
            eff, order = score_list, list(range(len(slot_list)))
        else:
            ctx = {"query_event_id": int(qid), "source_rank": int(cand.get("source_rank", cand.get("rank", 0))),
                   "score_mode": str(score_mode)}
            eff = space.effective_scores(heuristic_scores=score_list,
                                         learned_scores=logits if controller_runtime is not None else None,
                                         gpu_step=step, reward_context=ctx)
            order = space.selected_indices(effective_scores=eff, gpu_step=step, requested_budget=len(slot_list),
                                           reward_context=ctx)
        annotate = space is not None and (space.active_selection or space.max_tags_per_query is not None)
        for out_rank, i in enumerate(order):
            tag = {"step": step, "slot": slot_list[i], "score": score_list[i], "selected_at": int(selected_at),
                   "replay_id": _replay_id(qid, out_rank), "query_event_id": int(qid),
                   "source_write_id": int(src_ids[i]), "selected_rank": out_rank, "teacher_score": score_list[i],
                   "controller_logit": float(logits[i]), "selection_step": int(selected_at),
                   "policy_version": int(policy_version), "outcome_status": "pending"}
            if annotate:
                tag.update(heuristic_rank=int(i), action_space_score=float(eff[i]),
                           action_space_readiness=float(space.selection_readiness))
            tag.update(snaps[i])
            tagged_replay_queue.append(tag)
            if action_recorder is not None and snaps[i]:
                action_recorder.record_replay_selection(
                    slot_id=tag["slot"], gpu_step=tag["selection_step"], policy_version=tag["policy_version"],
                    output_logit=tag["controller_logit"], selected_rank=tag["selected_rank"],
                    features=list(tag["controller_features"]), global_state=list(tag["controller_global_state"]),
                    slot_state=list(tag["controller_slot_state"]))
    return len(cands)


def _emit_simplex_tag(cand, step, qid, slots, scores, slot_list, score_list, view, runtime, recorder, space, mode,
                      generator, selected_at, policy_version, out_queue) -> None:
    n = len(slot_list)
    V, E, sf, padded = build_simplex_inputs(cache_view=view, slots=slots, scores=scores, current_step=step)
    if space is not None:
        _apply_meta_actions(runtime, space, step, {"query_event_id": float(qid),
                                                  "pressure": float(cand.get("pressure", 0.0)),
                                                  "score": sum(score_list) / max(1, n)})
    p, logits = _simplex_forward(runtime, V, E, sf)
    idx, p_chosen = choose_simplex_vertex(p, n, mode=mode, generator=generator)
    slot = int(padded[idx])
    mass = float(np.clip(np.asarray(p[:n], dtype=np.float64), 0.0, None).sum())
    probs = ([1.0 / n] * n if not math.isfinite(mass) or mass <= 0.0
             else [max(float(x), 0.0) / mass for x in p[:n]])
    entropy = -sum(q * math.log(max(q, 1e-30)) for q in probs)
    logit_list = [float(x) for x in logits[:n]]
    rid = _replay_id(qid, idx)
    src = int(view["source_write_id"][slot])
    bucket = int(view["write_bucket"][slot])
    teacher = score_list[idx] if idx < n else 0.0
    seed = int(generator.initial_seed()) if generator is not None else -1
    arm = str(cand.get("arm", ""))
    if recorder is not None:
        recorder.record_simplex_decision(
            chosen_slot_id=slot, gpu_step=step, policy_version=int(policy_version), chosen_idx=idx,
            p_chosen_decision=p_chosen, V=V, E=E, simplex_features=sf, n_actual=n, write_bucket=bucket,
            query_event_id=int(qid), replay_id=rid, source_write_id=src, selected_rank=idx, teacher_score=teacher,
            controller_logit=logit_list[idx], arm=arm, p_behavior=probs, candidate_slot_ids=list(slot_list),
            candidate_scores=list(score_list), logits=logit_list, feature_manifest_hash=FEATURE_MANIFEST_HASH,
            selection_mode=str(mode), selection_seed=seed)
    out_queue.append({
        "step": step, "slot": slot, "score": teacher, "selected_at": int(selected_at), "replay_id": rid,
        "query_event_id": int(qid), "source_write_id": src, "write_bucket": bucket, "selected_rank": idx,
        "teacher_score": teacher, "controller_logit": logit_list[idx], "selection_step": step,
        "policy_version": int(policy_version), "outcome_status": "pending", "arm": arm, "p_chosen": p_chosen,
        "p_behavior": probs, "entropy": entropy,
        "lambda_hxh": float(getattr(runtime.fast_weights(), "lambda_hxh", 0.0)),
        "feature_manifest_hash": FEATURE_MANIFEST_HASH, "candidate_slot_ids": list(slot_list),
        "candidate_scores": list(score_list), "logits": logit_list, "simplex_p_chosen": p_chosen,
        "simplex_chosen_idx": idx, "simplex_n_actual": n, "simplex_candidate_slot_ids": list(slot_list),
        "simplex_candidate_scores": list(score_list), "simplex_logits": logit_list,
        "simplex_probabilities": probs})
    if space is not None:
        heads = [h for h in ("temperature", "entropy_beta", "ema_alpha") if space.readiness(h) > 0.0]
        if heads:
            space.record_credit_assignment(key=rid, head_names=heads, gpu_step=step,
                                           reward_context={"query_event_id": float(qid), "slot": float(slot)})


# ---------------------------------------------------------------------------
# long-running loop
# ---------------------------------------------------------------------------
def controller_main(*, controller_query_queue, tagged_replay_queue: list, cache: EpisodicCache,
                    stop_event: threading.Event, queue_lock: Optional[threading.Lock] = None, k: int = 16,
                    score_mode: str = "cosine_utility_weighted", controller_runtime: Any = None,
                    action_recorder: Any = None, simplex_selection_mode: str = "argmax",
                    simplex_generator: Optional[torch.Generator] = None, action_space: Any = None,
                    heartbeat: Optional[list] = None) -> None:
    """Thread body: cycles until ``stop_event`` is set, yielding the CPU when a cycle found nothing.
    With a lock the whole cycle runs under it; without one the producer's ``append`` and the drain's
    ``pop`` are each atomic under the interpreter lock.  ``heartbeat[0]`` counts cycles."""
    kw = dict(controller_query_queue=controller_query_queue, tagged_replay_queue=tagged_replay_queue, cache=cache, k=k,
              score_mode=score_mode, queue_lock=None, controller_runtime=controller_runtime,
              action_recorder=action_recorder, simplex_selection_mode=simplex_selection_mode,
              simplex_generator=simplex_generator, action_space=action_space)
    yield_cpu = getattr(os, "sched_yield", None) or (lambda: time.sleep(0))
    while not stop_event.is_set():
        if queue_lock is None:
            n = run_controller_cycle(**kw)
        else:
            with queue_lock:
                n = run_controller_cycle(**kw)
        if heartbeat is not None:
            heartbeat[0] += 1
        if n == 0:
            yield_cpu()
