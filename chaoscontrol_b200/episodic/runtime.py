"""Episodic memory in the training loop: train ranks publish what surprised them,
the episodic rank keeps the cache, answers queries and replays tagged spans.

Role of the reference's producer / consumer plumbing
(experiments/23_fast_path/runner_fast_path.py:6452-6660 write-event publisher,
``:6853-7130`` emit, ``:7290-7540`` GPU payload packing, ``:7543-7780`` consumer
state, ``:8023-8215`` query / replay-outcome events, ``:9010-9140`` ring drain,
``:9249-9510`` tagged replay, ``:9694-9762`` / ``:9945-10035`` asymmetric gradient
join).

Topology.  With N > 1 ranks the last rank is the episodic rank: it runs no main
forward/backward, it drains the train ranks' event rings into its
``EpisodicCache``, lets the controller turn queries into replay tags, replays up
to ``max_replays_per_step`` tagged spans, and joins ONE ``SUM`` all-reduce in
which the train ranks contribute their gradients pre-scaled by ``1 / N_train``
and it contributes the replay gradients (zeros when nothing was replayed).  With
one rank the same object plays both parts.

Transport.  One SPSC ring per producing rank and event kind, in POSIX shared
memory (process-local with one rank): 568-byte write events, 736-byte query
events.  Records are packed on the device by the write-event kernel, copied to
pinned host memory on a side stream, and pushed to the ring only once the copy's
event has completed, so the training stream never waits for a consumer; a full
ring drops the record and counts it.
"""
from __future__ import annotations

import math
import os
import threading
from collections import deque
from typing import Any, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..utils.arena import get_arena
from . import native as N
from .cache import EpisodicCache
from .controller import run_controller_cycle
from .writer import pack_write_events, select_top_p_positions

__all__ = ["EpisodicRuntime", "REPLAY_STATUS"]

REPLAY_STATUS = {"ok": 0, "slot_missing": 1, "stale": 2, "nan": 3, "skipped": 4}
_WRITE_EVENT, _QUERY_EVENT = 1, 2


def _fp16_bits(x: torch.Tensor, width: int) -> np.ndarray:
    out = np.zeros(width, dtype=np.uint16)
    v = x.detach().reshape(-1)[:width].to(torch.float16).cpu().numpy().view(np.uint16)
    out[: v.size] = v
    return out


def _bits_fp16(bits: np.ndarray, n: int) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits[:n]).view(np.float16).astype(np.float32))


class EpisodicRuntime:
    def __init__(self, *, model: torch.nn.Module, config: dict[str, Any], rank: int, world_size: int,
                 device: torch.device) -> None:
        get = config.get
        self.rank, self.world_size, self.device = int(rank), int(world_size), device
        self.solo = world_size == 1
        self.episodic_rank = world_size - 1
        self.is_episodic_rank = (not self.solo) and rank == self.episodic_rank
        self.n_train = max(1, world_size - 1)
        self.producers = [0] if self.solo else list(range(world_size - 1))
        dim = int(getattr(model, "dim", 0) or get("model_dim", 0))
        self.key_rep_dim = min(int(get("episodic_key_rep_dim", dim)), N.KEY_REP_DIM, dim)
        self.span = min(int(get("episodic_span_length", N.SPAN_LENGTH)), N.SPAN_LENGTH)
        self.window = int(get("episodic_fingerprint_window", 8))
        self.top_p = float(get("episodic_top_p", 0.0))
        self.writes_per_step = int(get("episodic_writes_per_step", 8))
        self.replay_weight = float(get("episodic_replay_weight", 1.0))
        self.max_replays = int(get("episodic_replay_max_replays_per_step", 4))
        self.topk = int(get("episodic_controller_topk_k", 16))
        # the run matrices write ``controller_query_mode``; a disagreement between the two keys is
        # refused, since picking one silently would spoil the pressure-only control
        # (experiments/23_fast_path/runner_fast_path.py:8382-8401)
        primary, alias = get("episodic_controller_score_mode"), get("controller_query_mode")
        if primary is not None and alias is not None and str(primary) != str(alias):
            raise ValueError(f"conflicting controller score mode keys: episodic_controller_score_mode={primary!r}, "
                             f"controller_query_mode={alias!r}")
        self.score_mode = str(primary if primary is not None else alias if alias is not None
                              else "cosine_utility_weighted").strip()
        # without queries the cache still fills (writes) but nothing is ever tagged for replay
        self.query_enabled = bool(get("controller_query_enabled", True))
        self.ring_capacity = int(get("episodic_ring_capacity", 4096))
        ns = str(get("episodic_event_ring_namespace", "") or
                 f"/ccb_epi_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
        self.consumer = self.solo or self.is_episodic_rank
        self.cache: Optional[EpisodicCache] = None
        if self.consumer:
            self.cache = EpisodicCache(capacity=int(get("episodic_capacity", 4096)), span_length=self.span,
                                       key_rep_dim=self.key_rep_dim,
                                       grace_steps=int(get("episodic_grace_steps", 200)),
                                       utility_ema_decay=float(get("episodic_utility_ema_decay", 0.99)),
                                       slot_state_dim=int(get("episodic_slot_state_dim", 0)),
                                       simplex_k_max=int(get("episodic_simplex_k_max", 0)))
        # how many write events the consumer takes from one producer's ring per step (0 = all that arrived)
        self.max_drain = max(0, int(get("episodic_write_ring_max_drain_per_step", 4096)))
        # the controller's bounded action space (off unless the config enables it) and its trace
        self.action_space = self.action_trace = None
        if self.consumer and bool(get("episodic_controller_action_space_enabled", False)):
            from .learned_action_space import build_action_space_from_config
            path = str(get("episodic_controller_action_trace_path", "") or "")
            if path:
                from .diagnostics import ActionSpaceTraceLogger
                self.action_trace = ActionSpaceTraceLogger(path)
            self.action_space = build_action_space_from_config(
                config, trace_log=self.action_trace if self.action_trace is not None else [])
        # rings: the consumer creates, producers attach after a barrier
        self._write_rings: dict[int, N.Ring] = {}
        self._query_rings: dict[int, N.Ring] = {}

        def open_rings(create: bool, ranks: list[int]) -> None:
            for r in ranks:
                wn, qn = (None, None) if self.solo else (f"{ns}_w{r}", f"{ns}_q{r}")
                self._write_rings[r] = N.Ring(N.WRITE_EVENT, self.ring_capacity, shm_name=wn, create=create)
                self._query_rings[r] = N.Ring(N.QUERY_EVENT, self.ring_capacity, shm_name=qn, create=create)
        if self.solo:
            open_rings(True, [0])
        elif self.is_episodic_rank:
            open_rings(True, self.producers)
            dist.barrier()
        else:
            dist.barrier()
            open_rings(False, [rank])
        self._creator = self.consumer
        self._side = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._pending: deque = deque()
        self._candidate_seq = 0
        self._cand_dev: Optional[torch.Tensor] = None
        self._query_seq = 0
        self.query_queue: list[dict[str, Any]] = []
        self.tagged: list[dict[str, Any]] = []
        self._lock = threading.Lock()
        # "simplex": the native 16-vertex policy picks the replay among the top-k candidates and the
        # native online learner (credit, Gerber gate, REINFORCE step, slow EMA) learns from every
        # replay outcome; "heuristic": cosine x utility ranking
        self.simplex = None
        self.controller_mode = str(get("episodic_controller_runtime", "heuristic")).strip().lower()
        if self.controller_mode in ("", "python_heuristic"):
            self.controller_mode = "heuristic"
        # "simplex_v1" is the pretrained policy: it must come with a weight file, so a run cannot
        # silently score with random weights (experiments/23_fast_path/runner_fast_path.py:8509-8520)
        pretrained = self.controller_mode == "simplex_v1"
        if pretrained:
            self.controller_mode = "simplex"
        if self.controller_mode not in ("heuristic", "simplex"):
            raise ValueError("episodic_controller_runtime must be heuristic, simplex or simplex_v1; "
                             f"got {self.controller_mode!r}")
        weights_path = get("episodic_controller_weights_path")
        if pretrained and not weights_path:
            raise ValueError("episodic_controller_runtime='simplex_v1' requires episodic_controller_weights_path")
        self.train_online = bool(get("controller_train_online", True))
        self._synced_sgd_steps = 0
        if self.consumer and self.controller_mode == "simplex":
            from .controller import SimplexRuntime, load_simplex_policy
            policy = load_simplex_policy(str(weights_path)) if weights_path else None
            if policy is None:
                from . import native
                policy = native.SimplexPolicy(seed=int(get("seed", 0)))
            if get("episodic_controller_initial_temperature") is not None:
                # a sharper start than the file's temperature: near-uniform sampling gives the
                # policy-gradient step nothing to lock onto (runner_fast_path.py:8477-8489)
                policy.temperature = float(get("episodic_controller_initial_temperature"))
            self.simplex = SimplexRuntime(
                policy=policy,
                num_slots=int(get("episodic_capacity", 4096)),
                max_entries_per_slot=int(get("episodic_controller_history_entries", 64)),
                gamma=float(get("episodic_controller_credit_gamma", 0.995)),
                learning_rate=float(get("episodic_controller_learning_rate",
                                        get("episodic_controller_lr", 1e-3))),
                sgd_interval=int(get("episodic_controller_sgd_interval", 16)),
                ema_alpha=float(get("episodic_controller_ema_alpha", 0.25)),
                ema_interval=int(get("episodic_controller_ema_interval", 64)),
                entropy_beta=float(get("episodic_controller_entropy_beta", 0.0)),
                gerber_c=float(get("episodic_controller_gerber_c", 0.5)))
            trace = str(get("episodic_controller_simplex_trace_path", "") or "")
            if trace:
                os.makedirs(os.path.dirname(trace) or ".", exist_ok=True)
                self.simplex.learner.set_trace_path(trace)
            self._sel_gen = torch.Generator().manual_seed(int(get("episodic_controller_selection_seed", get("seed", 0))))
            self.selection_mode = str(get("episodic_controller_selection_mode",
                                          get("episodic_simplex_selection_mode", "sample")))
            if self.selection_mode not in ("argmax", "sample"):
                raise ValueError("episodic_controller_selection_mode must be argmax or sample; "
                                 f"got {self.selection_mode!r}")
        self._closed_learner = False
        self.logger = None
        if self.consumer and get("episodic_replay_log_path"):
            from .diagnostics import DiagnosticsLogger
            self.logger = DiagnosticsLogger(str(get("episodic_replay_log_path")))
        self.stats = {"write_events_emitted": 0, "write_events_dropped": 0, "query_events_emitted": 0,
                      "query_events_dropped": 0, "write_events_ingested": 0, "queries_ingested": 0,
                      "replays": 0, "replay_status": {k: 0 for k in REPLAY_STATUS}, "replay_loss_sum": 0.0}

    # ------------------------------------------------------------------ producer
    def _flush(self) -> None:
        while self._pending:
            ev, host, kind, n = self._pending[0]
            if ev is not None and not ev.query():
                return
            self._pending.popleft()
            if kind == "write":
                recs = host.numpy().view(N.WRITE_EVENT).reshape(-1)[:n]
                ring = self._write_rings[self.rank]
                for rec in recs:
                    if int(rec["event_type"]) != _WRITE_EVENT:
                        continue                              # edge-trimmed candidate
                    if ring.push(rec):
                        self.stats["write_events_emitted"] += 1
                    else:
                        self.stats["write_events_dropped"] += 1
            else:
                if self._query_rings[self.rank].push(self._query_record(host, n)):
                    self.stats["query_events_emitted"] += 1
                else:
                    self.stats["query_events_dropped"] += 1

    def emit(self, *, inputs: torch.Tensor, targets: torch.Tensor, per_token_ce: torch.Tensor,
             hidden: torch.Tensor, step: int) -> None:
        """Producer side, once per step after the forward: the most surprising
        positions become write events, the single most surprising one also
        becomes the step's query."""
        if self.is_episodic_rank:
            return
        self._flush()
        B, T = inputs.shape
        ce = per_token_ce.detach().reshape(B, T).float()
        top_p = self.top_p if self.top_p > 0 else min(1.0, self.writes_per_step / float(B * T))
        pos = select_top_p_positions(ce, top_p)
        key_rep = hidden.detach()[..., : self.key_rep_dim]
        if self._cand_dev is None:
            self._cand_dev = torch.zeros(1, dtype=torch.int64, device=inputs.device)
        base = self._cand_dev.clone()
        self._cand_dev.add_(int(pos.shape[0]))               # device-side sequence: no host copy per step
        recs = pack_write_events(input_ids=inputs, target_ids=targets, key_rep_per_position=key_rep,
                                 per_token_ce=ce, positions=pos, candidate_base=base, pressure=ce,
                                 gpu_step=int(step), source_rank=self.rank, fingerprint_window=self.window,
                                 span_length=self.span, key_rep_dim=self.key_rep_dim)
        self._candidate_seq += int(pos.shape[0])
        b0, t0 = pos[0, 0], pos[0, 1]
        q_vec, q_ce = key_rep[b0, t0].float(), ce[b0, t0]
        pin = inputs.is_cuda
        host_w = torch.empty(recs.shape, dtype=torch.uint8, pin_memory=pin)
        host_q = torch.empty(self.key_rep_dim + 1, dtype=torch.float32, pin_memory=pin)
        ev = None
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._side):
                host_w.copy_(recs, non_blocking=True)
                host_q.copy_(torch.cat([q_vec, q_ce.reshape(1)]), non_blocking=True)
                recs.record_stream(self._side)
                ev = torch.cuda.Event()
                ev.record(self._side)
        else:
            host_w.copy_(recs)
            host_q.copy_(torch.cat([q_vec, q_ce.reshape(1)]))
        self._pending.append((ev, host_w, "write", int(pos.shape[0])))
        if self.query_enabled:
            self._pending.append((ev, host_q, "query", int(step)))    # built once its host values have landed
        self._flush()

    def _query_record(self, host_q: torch.Tensor, step: int) -> np.ndarray:
        rec = np.zeros((), dtype=N.QUERY_EVENT)
        rec["event_type"], rec["source_rank"] = _QUERY_EVENT, self.rank
        rec["query_id"] = (self.rank << 56) | self._query_seq
        self._query_seq += 1
        rec["gpu_step"] = int(step)
        rec["query_rep"] = _fp16_bits(host_q[: self.key_rep_dim], N.KEY_REP_DIM)
        ce = float(host_q[self.key_rep_dim])
        rec["pressure"], rec["pre_query_ce"] = ce, ce
        rec["candidate_slot_ids"] = np.full(N.SIMPLEX_CANDIDATES, np.iinfo(np.uint64).max, dtype=np.uint64)
        return rec

    # ------------------------------------------------------------------ consumer
    def _drain_rings(self, step: int) -> None:
        cache = self.cache
        for r in self.producers:
            ring = self._write_rings[r]
            taken = 0
            while self.max_drain <= 0 or taken < self.max_drain:
                rec = ring.pop()
                if rec is None:
                    break
                taken += 1
                cache.append(key_fp=int(rec["key_fp"]), key_rep=_bits_fp16(rec["key_rep"], self.key_rep_dim),
                             value_tok_ids=torch.from_numpy(rec["value_tok_ids"][: self.span].astype(np.int64)),
                             value_anchor_id=int(rec["value_anchor_id"]), current_step=int(rec["gpu_step"]),
                             embedding_version=0, pressure_at_write=float(rec["pressure_at_write"]),
                             source_write_id=int(rec["candidate_id"]) & 0x7FFFFFFFFFFFFFFF,
                             write_bucket=int(rec["write_bucket"]))
                self.stats["write_events_ingested"] += 1
            qring = self._query_rings[r]
            while True:
                rec = qring.pop()
                if rec is None:
                    break
                self.query_queue.append({"step": int(rec["gpu_step"]), "rank": int(rec["source_rank"]),
                                         "k": self.topk, "pressure": float(rec["pressure"]),
                                         "query_id": int(rec["query_id"]),
                                         "residual": _bits_fp16(rec["query_rep"], self.key_rep_dim)})
                self.stats["queries_ingested"] += 1

    def consume(self, model: torch.nn.Module, *, step: int, lm_head_backward_mode: str = "single",
                lm_head_tile_size: int = 1024) -> int:
        """Consumer side, once per step before the gradient join: ingest events,
        let the controller tag replay candidates, replay up to the per-step cap.
        Replay gradients ADD to ``p.grad``.  Returns the number replayed."""
        if not self.consumer:
            return 0
        from ..dreamworld import dreamworld_replay_from_cache_entry
        if self.solo:
            self._flush()
        self._drain_rings(step)
        if len(self.cache) > 0 and self.query_queue:
            extra = {}
            if self.simplex is not None:
                extra = dict(controller_runtime=self.simplex, action_recorder=self.simplex,
                             simplex_selection_mode=self.selection_mode, simplex_generator=self._sel_gen)
            run_controller_cycle(controller_query_queue=self.query_queue, tagged_replay_queue=self.tagged,
                                 cache=self.cache, k=self.topk, score_mode=self.score_mode, queue_lock=self._lock,
                                 action_space=self.action_space, **extra)
        else:
            self.query_queue.clear()
        done = 0
        while self.tagged and (self.max_replays <= 0 or done < self.max_replays):
            tag = self.tagged.pop(0)
            slot = int(tag.get("slot", -1))
            if not (0 <= slot < int(self.cache.capacity)) or not bool(self.cache.occupied[slot]):
                self.stats["replay_status"]["slot_missing"] += 1
                continue
            utility_pre = float(self.cache.utility_u[slot])
            written = {"key_fp": int(self.cache.key_fp[slot]), "write_step": int(self.cache.write_step[slot]),
                       "write_pressure": float(self.cache.pressure_at_write[slot]),
                       "write_bucket": int(self.cache.write_bucket[slot])}
            res = dreamworld_replay_from_cache_entry(model=model, cache=self.cache, slot=slot, current_step=int(step),
                                                     weight=self.replay_weight,
                                                     lm_head_backward_mode=lm_head_backward_mode,
                                                     lm_head_tile_size=int(lm_head_tile_size))
            if res is None:
                self.stats["replay_status"]["skipped"] += 1
                continue
            raw = float(res["utility_signal_raw"])
            if not math.isnan(raw):                          # no live signal: leave the utility EMA alone
                self.cache.update_utility(slot, ce_delta=float(res["utility_signal_transformed"]))
            self.cache.mark_fired(slot, int(step))
            loss = float(res["replay_loss"])
            ok = math.isfinite(loss)
            self.stats["replay_status"]["ok" if ok else "nan"] += 1
            self.stats["replay_loss_sum"] += loss if ok else 0.0
            done += 1
            if self.simplex is not None and ok:
                # reward: how much this replay's loss beats the running replay-loss baseline
                base = self.stats["replay_loss_sum"] / max(self.stats["replay_status"]["ok"], 1)
                out = np.zeros((), dtype=N.REPLAY_OUTCOME)
                out["event_type"], out["selected_rank"] = 3, int(tag.get("selected_rank", 0)) & 0xFF
                out["replay_id"] = int(tag.get("replay_id", 0)) & 0xFFFFFFFFFFFFFFFF
                out["gpu_step"], out["selection_step"] = int(step), int(tag.get("selection_step", step))
                out["query_event_id"] = int(tag.get("query_event_id", 0)) & 0xFFFFFFFFFFFFFFFF
                out["source_write_id"] = int(tag.get("source_write_id", 0)) & 0xFFFFFFFFFFFFFFFF
                out["slot_id"], out["policy_version"] = slot, int(tag.get("policy_version", 0))
                out["teacher_score"] = float(tag.get("teacher_score", 0.0))
                out["controller_logit"] = float(tag.get("controller_logit", 0.0))
                out["ce_before_replay"], out["bucket_baseline"] = loss, base
                out["ce_delta_raw"] = out["reward_shaped"] = base - loss
                if self.train_online:                      # frozen: select with the loaded weights, never learn
                    self.simplex.learner.on_replay_outcome(out)
            if self.logger is not None:
                from .diagnostics import REPLAY_LOG_SCHEMA
                nan = float("nan")
                row: dict[str, Any] = {c: tag.get(c) for c in REPLAY_LOG_SCHEMA}
                row.update({
                    "step": int(step), "slot": slot, "key_fp": written["key_fp"],
                    "write_step": written["write_step"], "write_pressure": written["write_pressure"],
                    "write_bucket": written["write_bucket"], "query_cosine": float(tag.get("score", 0.0)),
                    "utility_pre": utility_pre, "utility_post": float(self.cache.utility_u[slot]),
                    "replay_loss": loss, "replay_grad_norm": float(res["replay_grad_norm"]),
                    "replay_grad_cos_common": res["replay_grad_cos_common"],
                    "replay_grad_cos_rare": res["replay_grad_cos_rare"],
                    "replay_grad_cos_total": res["replay_grad_cos_total"], "utility_signal_raw": raw,
                    "utility_signal_transformed": float(res["utility_signal_transformed"]),
                    "ce_before_replay": loss, "ce_after_replay": nan, "ce_delta_raw": nan,
                    "outcome_status": REPLAY_STATUS["ok" if ok else "nan"], "flags": 0})
                self.logger.write_row(row)
        self.stats["replays"] += done
        if self.simplex is not None and self.train_online and done:
            self._synced_sgd_steps = self.simplex.sync_policy(self._synced_sgd_steps)
        return done

    # ------------------------------------------------------------------ gradient join
    def join_gradients(self, model: torch.nn.Module) -> None:
        """ONE ``SUM`` all-reduce over every rank: train ranks bring their gradients
        scaled by ``1 / N_train``, the episodic rank brings its replay gradients
        (zeros where it has none).  Every rank leaves with the same gradients."""
        if self.solo:
            return
        arena = get_arena(model)
        if arena is not None:
            if self.is_episodic_rank or not arena.grads_fresh:
                arena.pull_grads()
                arena.grads_fresh = True
            if not self.is_episodic_rank:
                arena.flat_grad.mul_(1.0 / self.n_train)
            dist.all_reduce(arena.flat_grad, op=dist.ReduceOp.SUM)
            arena.materialize_grads()
            return
        grads = []
        for p in model.parameters():
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            grads.append(p.grad)
        flat = torch._utils._flatten_dense_tensors(grads)
        if not self.is_episodic_rank:
            flat.mul_(1.0 / self.n_train)
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        for g, s in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
            g.copy_(s)

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self._side is not None:
            self._side.synchronize()
        self._flush()
        if self.logger is not None:
            self.logger.close()
        if self.action_trace is not None:
            self.action_trace.close()
            self.action_trace = None
        if self.simplex is not None and not self._closed_learner:
            self._final_controller = self.simplex.learner.telemetry()
            self._closed_learner = True
        for ring in list(self._write_rings.values()) + list(self._query_rings.values()):
            ring.close(unlink=self._creator and not self.solo)
        self._write_rings.clear()
        self._query_rings.clear()

    def diagnostics(self) -> dict[str, Any]:
        d = {"enabled": True, "role": "episodic" if self.is_episodic_rank else ("solo" if self.solo else "train"),
             "n_train": self.n_train, "key_rep_dim": self.key_rep_dim, "span_length": self.span, **self.stats}
        if self.simplex is not None:
            d["controller"] = {"mode": "simplex", "decisions": len(self.simplex.decisions),
                               "train_online": self.train_online, "selection_mode": self.selection_mode,
                               "temperature": float(self.simplex.policy.temperature),
                               **self.simplex.learner.telemetry()}
        if self.action_space is not None:
            sp = self.action_space
            d["action_space"] = {"trace_only": bool(sp.trace_only), "selection_readiness": float(sp.selection_readiness),
                                 "selection_max_delta": float(sp.selection_max_delta),
                                 "max_tags_per_query": sp.max_tags_per_query,
                                 "shared_event_ssm": sp.event_ssm is not None,
                                 "online_learning_rate": float(sp.online_learning_rate)}
        if self.cache is not None:
            d["cache_entries"] = len(self.cache)
            d["cache_capacity"] = int(self.cache.capacity)
        return d

    def cache_state(self) -> Optional[dict[str, Any]]:
        """What a checkpoint stores under ``episodic_cache``."""
        return None if self.cache is None else self.cache.to_dict()
