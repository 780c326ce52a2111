"""Long-term memory modules that sit beside the recurrence.

``OuterModel``           single lossy slot with surprise-gated consolidation
                         (reference src/chaoscontrol/memory.py:20-193)
``MultiSlotOuterModel``  many slots, cue-dependent retrieval, survival scores,
                         typed compression, latent traces, bucket affinity
                         (reference memory.py:196-1163)
``BucketPrototypes``     one EMA prototype per routing bucket (memory.py:1166-1224)
``SemanticTier``         always-on slow basis bias (memory.py:1227-1261)

Parameter / buffer names match the reference so checkpoints interchange.  The
multi-slot store is a dense device matrix (see ``slot_table.SlotTable``): every
retrieval mode below is a masked softmax / mean over rows of that matrix, done
by ONE shared mixing routine instead of a copy of the arithmetic per mode.
"""
from __future__ import annotations

import random as _random
from collections import defaultdict
from typing import Any

import torch
import torch.nn as nn

from ..slot_table import SlotTable

__all__ = ["OuterModel", "MultiSlotOuterModel", "BucketPrototypes", "SemanticTier"]


def _surprise(mode: str, current_loss: float, running_avg: float, learned_w: torch.Tensor | None) -> float:
    pain = max(current_loss - running_avg, 0.0)
    reward = max(running_avg - current_loss, 0.0)
    if mode == "symmetric":
        return abs(current_loss - running_avg)
    if mode == "pain_biased":
        return pain + 0.5 * reward
    if mode == "learned":
        w = torch.sigmoid(learned_w).item()
        return w * pain + (1.0 - w) * reward
    raise ValueError(f"unsupported consolidation_mode: {mode}")


class _Consolidating(nn.Module):
    """Trigger logic shared by the single- and multi-slot memories.

    ``immediate`` writes on surprise; ``resolution`` writes when the loss has
    settled back to its pre-spike level; ``windowed`` writes ``trigger_window``
    steps after the spike.  In ``learned`` mode a scalar is nudged, without
    gradients, toward whichever kind of event (pain / reward) preceded an
    improvement the last time a write happened.
    """

    def _init_consolidation(self, consolidation_mode: str, ema_decay: float, trigger: str, trigger_window: int):
        self.consolidation_mode = consolidation_mode
        self.ema_decay = ema_decay
        self.trigger = trigger
        self.trigger_window = trigger_window
        self._spike_seen = False
        self._steps_since_spike = 0
        self._pre_spike_loss = 0.0

    def _register_consolidation_buffers(self) -> None:
        if self.consolidation_mode == "learned":
            self.register_buffer("consolidation_w", torch.tensor(0.0))
            self.register_buffer("_last_signal_was_pain", torch.tensor(False))
            self.register_buffer("_last_loss", torch.tensor(0.0))
            self.register_buffer("_last_wrote", torch.tensor(False))

    def compute_consolidation_signal(self, current_loss: float, running_avg: float) -> float:
        return _surprise(self.consolidation_mode, current_loss, running_avg,
                         getattr(self, "consolidation_w", None))

    def _should_write(self, surprised: bool, current_loss: float, running_avg: float) -> bool:
        if self.trigger == "immediate":
            return surprised
        if self.trigger == "resolution":
            if surprised and not self._spike_seen:
                self._spike_seen = True
                self._pre_spike_loss = running_avg
            if self._spike_seen and current_loss <= self._pre_spike_loss:
                self._spike_seen = False
                return True
            return False
        if self.trigger == "windowed":
            if surprised and not self._spike_seen:
                self._spike_seen = True
                self._steps_since_spike = 0
            if self._spike_seen:
                self._steps_since_spike += 1
                if self._steps_since_spike >= self.trigger_window:
                    self._spike_seen = False
                    return True
            return False
        return False

    def _before_write_decision(self, current_loss: float) -> None:
        """Hook between the learned-weight update and the trigger decision."""

    def consolidation_step(self, h: torch.Tensor, current_loss: float,
                           per_sample_weights: torch.Tensor | None = None,
                           bucket_id: int | None = None) -> float:
        running_avg = self.loss_ema.item()
        signal = self.compute_consolidation_signal(current_loss, running_avg)
        is_pain = current_loss > running_avg
        if self.consolidation_mode == "learned" and self._last_wrote.item():
            if current_loss < self._last_loss.item():
                step = 0.01 if self._last_signal_was_pain.item() else -0.01
                self.consolidation_w = self.consolidation_w + step
        self._before_write_decision(current_loss)
        surprised = running_avg > 0 and signal / running_avg > 0.01
        wrote = self._should_write(surprised, current_loss, running_avg)
        if wrote:
            self._consolidate_write(h, per_sample_weights, bucket_id)
        if self.consolidation_mode == "learned":
            dev = self.loss_ema.device
            self._last_signal_was_pain = torch.tensor(is_pain, device=dev)
            self._last_loss = torch.tensor(current_loss, device=dev)
            self._last_wrote = torch.tensor(wrote, device=dev)
        self.loss_ema = self.ema_decay * self.loss_ema + (1 - self.ema_decay) * current_loss
        return signal

    def _encode_pool(self, h: torch.Tensor, per_sample_weights: torch.Tensor | None) -> torch.Tensor:
        enc = torch.tanh(self.encoder(h.detach().to(dtype=self.encoder.weight.dtype)))
        if per_sample_weights is None:
            return enc.mean(dim=0, keepdim=True)
        w = per_sample_weights.detach()
        w = w / w.sum().clamp_min(1e-8)
        return (w.unsqueeze(-1) * enc).sum(dim=0, keepdim=True)


class OuterModel(_Consolidating):
    """One persistent outer-space state; encode and decode are different maps,
    so a round trip is lossy by construction."""

    def __init__(self, model_dim: int, outer_dim: int = 64, consolidation_mode: str = "symmetric",
                 ema_decay: float = 0.99, trigger: str = "immediate", trigger_window: int = 8) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.outer_dim = outer_dim
        self._init_consolidation(consolidation_mode, ema_decay, trigger, trigger_window)
        self.encoder = nn.Linear(model_dim, outer_dim, bias=False)     # structural, never trained
        self.encoder.weight.requires_grad_(False)
        self.decoder = nn.Linear(outer_dim, model_dim, bias=False)     # on the forward path
        self.log_inertia = nn.Parameter(torch.tensor(2.0, dtype=torch.float32), requires_grad=False)
        self._register_consolidation_buffers()
        self.register_buffer("state", torch.zeros(1, outer_dim))
        self.register_buffer("loss_ema", torch.tensor([2.0]))

    def read(self, batch_size: int) -> torch.Tensor:
        return self.decoder(self.state.expand(batch_size, -1).to(dtype=self.decoder.weight.dtype))

    def write(self, h: torch.Tensor, *, per_sample_weights: torch.Tensor | None = None) -> None:
        pooled = self._encode_pool(h, per_sample_weights)
        inertia = torch.sigmoid(self.log_inertia)
        self.state = (inertia * self.state.detach() + (1 - inertia) * pooled).detach()

    def _consolidate_write(self, h, per_sample_weights, bucket_id) -> None:
        self.write(h, per_sample_weights=per_sample_weights)


class MultiSlotOuterModel(_Consolidating):
    """Multi-slot episodic store.  Each consolidation appends a slot; past
    ``max_slots`` the oldest low-survival slots of a bucket are merged (lossy
    compression is the forgetting mechanism) and leave a latent trace that a
    later surprise can reactivate."""

    def __init__(self, model_dim: int, outer_dim: int = 64, consolidation_mode: str = "symmetric",
                 ema_decay: float = 0.99, trigger: str = "immediate", trigger_window: int = 8,
                 max_slots: int = 64, compress_ratio: int = 2, compression_selection: str = "survival") -> None:
        super().__init__()
        self.model_dim = model_dim
        self.outer_dim = outer_dim
        self._init_consolidation(consolidation_mode, ema_decay, trigger, trigger_window)
        self.max_slots = max_slots
        self.compress_ratio = max(2, compress_ratio)
        self.compression_selection = compression_selection
        self._compress_rng = _random.Random(42)
        self.encoder = nn.Linear(model_dim, outer_dim, bias=False)
        self.encoder.weight.requires_grad_(False)
        self.decoder = nn.Linear(outer_dim, model_dim, bias=False)
        self.cue_proj = nn.Linear(model_dim, outer_dim, bias=False)
        self._register_consolidation_buffers()
        self.register_buffer("loss_ema", torch.tensor([2.0]))
        self.table = SlotTable()
        self._retrieval_weights: torch.Tensor | None = None
        self._retrieval_indices: list[int] | None = None
        self._compression_consequences: list[tuple[int, float]] = []
        self._latent_traces: list[dict] = []
        self._bucket_affinity: torch.Tensor | None = None

    # ---- list-style access kept for callers that predate the table ----------
    @property
    def _slots(self):
        return self.table._slots

    @_slots.setter
    def _slots(self, value) -> None:
        self.table._slots = list(value)
        self._rebuild_table_identity()

    @property
    def _survival(self) -> list[float]:
        return self.table._survival

    @_survival.setter
    def _survival(self, value) -> None:
        self.table._survival = list(value)

    @property
    def _slot_buckets(self) -> list[int]:
        return self.table._slot_buckets

    @_slot_buckets.setter
    def _slot_buckets(self, value) -> None:
        self.table._slot_buckets = list(value)

    @property
    def _slot_event_ids(self) -> list[int]:
        return self.table._slot_event_ids

    @_slot_event_ids.setter
    def _slot_event_ids(self, value) -> None:
        self.table._slot_event_ids = list(value)

    def _rebuild_table_identity(self) -> None:
        t = self.table
        n = len(t)
        t._records.clear()
        t._next_id = n
        t._priority = [1.0] * n
        t._id_to_physical = {i: i for i in range(n)}
        t._physical_to_id = {i: i for i in range(n)}
        for name, fill in (("_survival", 0.0), ("_slot_buckets", -1), ("_slot_event_ids", 0)):
            cur = getattr(t, name)
            setattr(t, name, (list(cur) + [fill] * n)[:n])

    def _ensure_slot_event_ids(self) -> None:
        t = self.table
        t._slot_event_ids = (list(t._slot_event_ids) + [0] * len(t))[: len(t)]

    def _visible_slot_indices(self, *, read_cutoff: int | None = None, bucket_id: int | None = None) -> list[int]:
        return self.table.visible_indices(read_cutoff=read_cutoff, bucket_id=bucket_id)

    # ---- appends ---------------------------------------------------------------
    def _maintenance_owns_capacity(self) -> bool:
        return str(self.compression_selection).lower() in {"maintenance", "learned", "none"}

    def append_kv_batch(self, encoded_batch: torch.Tensor, bucket_ids: torch.Tensor) -> list[int]:
        """Appends ``[N, outer_dim]`` pre-encoded rows with one device copy and
        one host transfer of the bucket ids."""
        return self._append_kv_batch_committed(encoded_batch, bucket_ids, event_ids=None)

    def _append_kv_batch_committed(self, encoded_batch: torch.Tensor, bucket_ids: torch.Tensor,
                                   event_ids: torch.Tensor | None = None) -> list[int]:
        """Append with explicit multi-version event ids.  Id 0 is visible to every
        reader; a transaction passes newer ids so its own writes stay invisible
        to reads taken at an older cutoff."""
        n = int(encoded_batch.shape[0])
        if n == 0:
            return []
        owns = self._maintenance_owns_capacity()
        if owns and self.max_slots > 0:
            free = int(self.max_slots) - len(self.table)
            if free <= 0:
                return []
            n = min(n, free)
        bids = [int(b) for b in bucket_ids.detach().reshape(-1).tolist()]
        eids = [0] * len(bids) if event_ids is None else [int(e) for e in event_ids.detach().reshape(-1).tolist()]
        if owns:
            bids, eids = bids[:n], eids[:n]
        if len(bids) != n:
            raise ValueError(f"bucket_ids length {len(bids)} does not match encoded batch {n}")
        if len(eids) != n:
            raise ValueError(f"event_ids length {len(eids)} does not match encoded batch {n}")
        out = self.table.append_rows(encoded_batch[:n], bids, eids, survival=1.0)
        if not owns and self.max_slots > 0 and len(self.table) > self.max_slots:
            self._compress()
        return out

    def append_kv(self, encoded: torch.Tensor, bucket_id: int | None = None) -> None:
        """Unconditional append of a pre-encoded vector (``max_slots == 0`` means unlimited)."""
        self.table.append(encoded.detach(), bucket_id=-1 if bucket_id is None else bucket_id, survival=1.0)
        if self.max_slots > 0 and len(self.table) > self.max_slots:
            self._compress()

    # ---- persistence -----------------------------------------------------------
    def get_extra_state(self) -> dict:
        ts = self.table.state_dict()
        state = {
            "slots": ts["slots"],
            "survival": ts["survival"],
            "slot_buckets": ts["slot_buckets"],
            "slot_event_ids": ts["slot_event_ids"],
            "table_state": ts,
            "latent_traces": [{"bucket_id": t["bucket_id"], "centroid_contrib": t["centroid_contrib"].cpu()}
                              for t in self._latent_traces],
        }
        if self._bucket_affinity is not None:
            state["bucket_affinity"] = self._bucket_affinity.cpu()
        return state

    def set_extra_state(self, state: dict) -> None:
        device = self.decoder.weight.device
        if "table_state" in state:
            self.table.load_state_dict(state["table_state"], device=device)
        else:
            self.table._slots = [s.to(device) for s in state["slots"]]
            n = len(self.table)
            self.table._survival = list(state["survival"])
            self.table._slot_buckets = list(state.get("slot_buckets", [-1] * n))
            self.table._slot_event_ids = list(state.get("slot_event_ids", [0] * n))
            self._rebuild_table_identity()
        self._latent_traces = [{"bucket_id": t["bucket_id"], "centroid_contrib": t["centroid_contrib"].to(device)}
                               for t in state.get("latent_traces", [])]
        if "bucket_affinity" in state:
            self._bucket_affinity = state["bucket_affinity"].to(device)

    # ---- retrieval -------------------------------------------------------------
    def _slot_override_for_matrix(self, *, slot_matrix: torch.Tensor, indices: list[int], batch_size: int,
                                  slot_override_index: int | None,
                                  slot_override_values: torch.Tensor | None):
        """Counterfactual read: pretend slot ``slot_override_index`` held
        ``slot_override_values`` without touching the table."""
        if slot_override_index is None or slot_override_values is None:
            return None, None
        try:
            pos = indices.index(int(slot_override_index))
        except ValueError:
            return None, None
        v = slot_override_values.detach().to(device=slot_matrix.device, dtype=slot_matrix.dtype)
        if v.dim() == 3 and v.shape[1] == 1:
            v = v.squeeze(1)
        if v.dim() == 1:
            v = v.unsqueeze(0)
        if v.dim() != 2 or v.shape[-1] != slot_matrix.shape[-1]:
            raise ValueError("slot_override_values must have shape (outer_dim,), "
                             "(batch, outer_dim), or (batch, 1, outer_dim)")
        if v.shape[0] == 1 and batch_size != 1:
            v = v.expand(batch_size, -1)
        elif v.shape[0] != batch_size:
            raise ValueError(f"slot_override_values batch {v.shape[0]} does not match read batch {batch_size}")
        return pos, v

    @staticmethod
    def _apply_retrieval_override(retrieved, weights, slot_matrix, *, override_pos, override_values):
        if override_pos is None or override_values is None:
            return retrieved
        return retrieved + weights[:, override_pos:override_pos + 1] * (
            override_values - slot_matrix[override_pos].unsqueeze(0))

    def _mix(self, M: torch.Tensor, batch_size: int, *, q: torch.Tensor | None, mask: torch.Tensor | None,
             pos: int | None, ov: torch.Tensor | None, topk: int | None = None):
        """One mixing rule for every retrieval mode.

        ``q`` given: softmax over ``q @ M^T`` (masked entries excluded; restricted
        to each row's top-k scores when ``topk`` is set; an all-masked row mixes
        nothing).  No ``q``: uniform mean over the masked-in rows.  Returns
        ``(mixed [B or 1, dim], weights or None)``.
        """
        n = M.shape[0]
        if q is not None:
            s = q @ M.T
            if pos is not None:
                s[:, pos] = (q * ov).sum(dim=-1)
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            if topk is not None and topk < n:
                kept = torch.zeros_like(s, dtype=torch.bool).scatter_(1, s.topk(topk, dim=-1).indices, True)
                s = s.masked_fill(~kept, float("-inf"))
            dead = torch.isinf(s).all(dim=-1, keepdim=True)
            w = torch.where(dead.expand_as(s), torch.zeros_like(s), torch.softmax(s, dim=-1))
            w = torch.nan_to_num(w, nan=0.0)
            out = self._apply_retrieval_override(w @ M, w, M, override_pos=pos, override_values=ov)
            return out, w
        if mask is not None:
            w = mask.to(dtype=M.dtype)
            w = w / w.sum(dim=-1, keepdim=True).clamp(min=1.0)
            return self._apply_retrieval_override(w @ M, w, M, override_pos=pos, override_values=ov), None
        out = M.mean(dim=0, keepdim=True).expand(batch_size, -1)
        if pos is not None:
            out = out + (ov - M[pos].unsqueeze(0)) / max(1, n)
        return out, None

    def _zeros(self, batch_size: int) -> torch.Tensor:
        return torch.zeros(batch_size, self.model_dim, device=self.decoder.weight.device)

    def _decode(self, retrieved: torch.Tensor, batch_size: int) -> torch.Tensor:
        out = self.decoder(retrieved.to(dtype=self.decoder.weight.dtype))
        return out.expand(batch_size, -1) if out.shape[0] == 1 and batch_size != 1 else out

    def read(self, batch_size: int, *, cue: torch.Tensor | None = None, read_cutoff: int | None = None,
             slot_mask: torch.Tensor | None = None, slot_override_index: int | None = None,
             slot_override_values: torch.Tensor | None = None) -> torch.Tensor:
        """Cue-dependent retrieval over all visible slots, decoded to ``model_dim``.
        Slot priority is control-plane telemetry only and never rescales a read."""
        self._retrieval_weights = None
        self._retrieval_indices = None
        indices = self.table.visible_indices(read_cutoff=read_cutoff) if len(self.table) else []
        if not indices:
            return self._zeros(batch_size)
        M = self.table.slot_matrix(indices)
        mask = None if slot_mask is None else slot_mask.to(device=M.device, dtype=torch.bool)[:, indices]
        pos, ov = self._slot_override_for_matrix(slot_matrix=M, indices=indices, batch_size=batch_size,
                                                 slot_override_index=slot_override_index,
                                                 slot_override_values=slot_override_values)
        q = None
        if cue is not None:
            q = self.cue_proj(cue.to(dtype=self.cue_proj.weight.dtype)).to(dtype=M.dtype)
        out, w = self._mix(M, batch_size, q=q, mask=mask, pos=pos, ov=ov)
        if w is not None:
            self._retrieval_weights = w.detach()
            self._retrieval_indices = indices
        return self._decode(out, batch_size)

    def read_bucket(self, batch_size: int, bucket_id: int, mode: str = "bucket_mean", k: int = 8,
                    cue: torch.Tensor | None = None, read_cutoff: int | None = None,
                    slot_mask: torch.Tensor | None = None, slot_override_index: int | None = None,
                    slot_override_values: torch.Tensor | None = None) -> torch.Tensor:
        """Bucket-scoped retrieval; ``cue`` is already in outer space here.

        ``bucket_mean`` mean of the bucket; ``bucket_recent`` mean of its last
        ``k``; ``bucket_topk`` softmax over the ``k`` best cue matches;
        ``softmax_all`` softmax (or mean without a cue) over every slot.
        """
        if mode not in ("bucket_mean", "bucket_recent", "bucket_topk", "softmax_all"):
            raise ValueError(f"Unknown retrieval mode: {mode}")
        if len(self.table) == 0:
            return self._zeros(batch_size)
        dtype = self.decoder.weight.dtype
        indices = self.table.visible_indices(read_cutoff=read_cutoff,
                                             bucket_id=None if mode == "softmax_all" else bucket_id)
        if not indices:
            return self._zeros(batch_size)
        if mode == "bucket_recent":
            indices_all = indices
            indices = indices[max(0, len(indices) - k):]
            if slot_override_index is not None and int(slot_override_index) not in indices:
                slot_override_index = None
            del indices_all
        M = self.table.slot_matrix(indices).to(dtype=dtype)
        mask = None if slot_mask is None else slot_mask.to(device=M.device, dtype=torch.bool)[:, indices]
        pos, ov = self._slot_override_for_matrix(slot_matrix=M, indices=indices, batch_size=batch_size,
                                                 slot_override_index=slot_override_index,
                                                 slot_override_values=slot_override_values)
        q = None
        topk = None
        if mode == "bucket_topk":
            if cue is None:
                raise ValueError("bucket_topk requires a cue tensor")
            q, topk = cue.to(dtype=dtype), k
        elif mode == "softmax_all" and cue is not None:
            q = cue.to(dtype=dtype)
        out, _ = self._mix(M, batch_size, q=q, mask=mask, pos=pos, ov=ov, topk=topk)
        return self._decode(out, batch_size)

    # ---- writes ----------------------------------------------------------------
    def write(self, h: torch.Tensor, *, per_sample_weights: torch.Tensor | None = None,
              bucket_id: int | None = None) -> None:
        """Encodes, pools over the batch and appends one slot (typed by
        ``bucket_id`` when given; typed slots only merge with their own type)."""
        slot = self._encode_pool(h, per_sample_weights)
        self.table.append(slot.detach(), bucket_id=-1 if bucket_id is None else bucket_id)
        if len(self.table) > self.max_slots:
            self._compress()

    def write_sequence(self, h_seq: torch.Tensor, *, per_sample_weights: torch.Tensor | None = None,
                       bucket_id: int | None = None) -> None:
        """Pools ``[B, T, D]`` over time with exponential recency weights
        (last position weight 1 before normalisation), then ``write``."""
        T = h_seq.shape[1]
        pos = torch.arange(T, dtype=torch.float32, device=h_seq.device)
        w = torch.softmax(pos, dim=0)          # == exp(pos - pos[-1]) normalised
        self.write(torch.einsum("btd,t->bd", h_seq.float(), w).to(h_seq.dtype),
                   per_sample_weights=per_sample_weights, bucket_id=bucket_id)

    def _consolidate_write(self, h, per_sample_weights, bucket_id) -> None:
        self.write(h, per_sample_weights=per_sample_weights, bucket_id=bucket_id)

    def _before_write_decision(self, current_loss: float) -> None:
        self.update_survival(current_loss)

    def update_survival(self, current_loss: float) -> None:
        """Credits the slots of the last cued read with ``(ema - loss) * weight``."""
        if self._retrieval_weights is None or len(self.table) == 0:
            return
        impact = self.loss_ema.item() - current_loss
        mean_w = self._retrieval_weights.mean(dim=0).tolist()
        idx = self._retrieval_indices or list(range(len(mean_w)))
        surv = self.table._survival
        for p, slot_idx in enumerate(idx[: len(mean_w)]):
            if 0 <= slot_idx < len(surv):
                surv[slot_idx] += impact * mean_w[p]

    # ---- compression / reactivation -------------------------------------------------
    def _compress(self) -> None:
        """Merges, inside the older half, the ``compress_ratio`` lowest-survival
        slots (or random ones) of each bucket that has enough of them into one
        survival-weighted average; merged slots leave latent traces."""
        t = self.table
        n = len(t)
        n_old = n // 2
        if n <= self.compress_ratio or n_old < self.compress_ratio:
            return
        old_sids = sorted(t.active_slot_ids())[:n_old]
        phys = [t.slot_id_to_physical(s) for s in old_sids]
        vecs = [t._store[p:p + 1].clone() for p in phys]       # copies: rows move on retirement
        surv = [t._survival[p] for p in phys]
        buckets = [t._slot_buckets[p] for p in phys]
        eids = [t._slot_event_ids[p] for p in phys]
        typed = any(b != -1 for b in buckets)
        groups: dict[int, list[int]] = defaultdict(list)
        for i, b in enumerate(buckets):
            groups[b if typed else -1].append(i)
        retire: list[int] = []
        merged: list[tuple[torch.Tensor, float, int, int]] = []
        for b, members in groups.items():
            if len(members) < self.compress_ratio:
                continue
            order = list(members)
            if self.compression_selection == "random":
                self._compress_rng.shuffle(order)
            else:
                order.sort(key=lambda i: surv[i])
            pick = order[: self.compress_ratio]
            w = torch.tensor([max(surv[i], 0.01) for i in pick])
            w = (w / w.sum()).tolist()
            stack = torch.cat([vecs[i] for i in pick], dim=0)
            slot = (stack * torch.tensor(w, device=stack.device, dtype=stack.dtype).unsqueeze(-1)).sum(0, keepdim=True)
            if typed:
                self._compression_consequences.append(
                    (b, -float((slot - stack.mean(0, keepdim=True)).norm())))
            for i in pick:
                self._latent_traces.append({"bucket_id": buckets[i], "centroid_contrib": vecs[i]})
                retire.append(old_sids[i])
            merged.append((slot, sum(surv[i] for i in pick) / len(pick), b if typed else -1,
                           max(eids[i] for i in pick)))
        if retire:
            t.retire_many(retire, reason="compressed")
        for slot, s, b, e in merged:
            t.append(slot, bucket_id=b, event_id=e, survival=s)
        del self._latent_traces[: max(0, len(self._latent_traces) - self.max_slots)]

    def try_reactivate(self, bucket_id: int | None, surprise: float, reactivation_threshold: float = 1.0) -> bool:
        """On enough surprise, rebuilds (with noise: recall is reconstructive) the
        first latent trace of ``bucket_id`` (any trace when ``None``) as a slot."""
        if surprise < reactivation_threshold:
            return False
        for i, tr in enumerate(self._latent_traces):
            if bucket_id is None or tr["bucket_id"] == bucket_id:
                v = tr["centroid_contrib"]
                self.table.append(v + 0.1 * torch.randn_like(v), bucket_id=tr["bucket_id"])
                self._latent_traces.pop(i)
                if len(self.table) > self.max_slots:
                    self._compress()
                return True
        return False

    # ---- partitions ------------------------------------------------------------------
    def get_partition_slot_indices(self, partition: Any) -> list[int]:
        return [i for i, b in enumerate(self._slot_buckets) if partition.owns_bucket(b)]

    def partition_slot_count(self, partition: Any) -> int:
        return len(self.get_partition_slot_indices(partition))

    def is_write_allowed(self, bucket_id: int, partitions: list[Any]) -> bool:
        return any(p.owns_bucket(bucket_id) and p.is_awake for p in partitions)

    # ---- bucket affinity ---------------------------------------------------------------
    def _ensure_affinity(self, n_buckets: int) -> torch.Tensor:
        a = self._bucket_affinity
        if a is None or a.shape[0] < n_buckets:
            new = torch.eye(n_buckets)
            if a is not None:
                new[: a.shape[0], : a.shape[1]] = a
            self._bucket_affinity = new
        return self._bucket_affinity

    def bucket_affinity(self, a: int, b: int) -> float:
        m = self._bucket_affinity
        if m is None or a >= m.shape[0] or b >= m.shape[0]:
            return 1.0 if a == b else 0.0
        return float(m[a, b].item())

    def update_affinity(self, a: int, b: int, delta: float, lr: float = 0.05) -> None:
        """Symmetric, clamped to [0, 1]; the diagonal stays 1."""
        if a == b:
            return
        m = self._ensure_affinity(max(a, b) + 1)
        m[a, b] = m[b, a] = max(0.0, min(1.0, float(m[a, b]) + lr * delta))

    def affinity_clusters(self, threshold: float = 0.3) -> list[set[int]]:
        """Connected components of the graph ``affinity > threshold``."""
        m = self._bucket_affinity
        if m is None:
            return []
        adj = (m > threshold).tolist()
        n = len(adj)
        seen: set[int] = set()
        out: list[set[int]] = []
        for root in range(n):
            if root in seen:
                continue
            comp, stack = set(), [root]
            while stack:
                u = stack.pop()
                if u in seen:
                    continue
                seen.add(u)
                comp.add(u)
                stack.extend(v for v in range(n) if adj[u][v] and v not in seen)
            out.append(comp)
        return out


class BucketPrototypes(nn.Module):
    """One EMA prototype per routing bucket in ``prototype_dim``, decoded to
    ``model_dim`` on read; ships in the artifact as a cold-start prior."""

    def __init__(self, k_max: int, prototype_dim: int, model_dim: int, update_rate: float = 0.1) -> None:
        super().__init__()
        self.k_max = k_max
        self.prototype_dim = prototype_dim
        self.model_dim = model_dim
        self.update_rate = update_rate
        self.register_buffer("prototypes", torch.zeros(k_max, prototype_dim))
        self.decoder = nn.Linear(prototype_dim, model_dim, bias=False)

    def read(self, batch_size: int, bucket_id: int) -> torch.Tensor:
        p = self.prototypes[bucket_id].unsqueeze(0).to(dtype=self.decoder.weight.dtype)
        return self.decoder(p).expand(batch_size, -1)

    def update(self, bucket_id: int, value: torch.Tensor) -> None:
        v = value.detach().mean(dim=0)
        self.prototypes[bucket_id].lerp_(v.to(self.prototypes.dtype), self.update_rate)

    def update_batch(self, bucket_ids: torch.Tensor, values: torch.Tensor) -> None:
        """Per-bucket mean of ``values`` then one EMA step per touched bucket,
        entirely on the device (segment sums by ``index_add_``; no host sync)."""
        ids = bucket_ids.reshape(-1).to(device=self.prototypes.device, dtype=torch.long)
        vals = values.detach().to(device=self.prototypes.device, dtype=self.prototypes.dtype)
        sums = torch.zeros_like(self.prototypes).index_add_(0, ids, vals)
        cnt = torch.zeros(self.k_max, device=ids.device, dtype=self.prototypes.dtype).index_add_(
            0, ids, torch.ones_like(ids, dtype=self.prototypes.dtype))
        touched = (cnt > 0).unsqueeze(-1)
        mean = sums / cnt.clamp(min=1.0).unsqueeze(-1)
        self.prototypes.copy_(torch.where(touched, torch.lerp(self.prototypes, mean, self.update_rate),
                                          self.prototypes))


class SemanticTier(nn.Module):
    """Slow, always-on bias: a few basis activations distilled from episodic
    slots, decoded and added at every step (gist, not episodes)."""

    def __init__(self, model_dim: int, num_bases: int = 8, update_rate: float = 0.01) -> None:
        super().__init__()
        self.model_dim = model_dim
        self.num_bases = num_bases
        self.update_rate = update_rate
        self.decoder = nn.Linear(num_bases, model_dim, bias=False)
        self.encoder = nn.Linear(model_dim, num_bases, bias=False)
        self.encoder.weight.requires_grad_(False)
        self.register_buffer("bases", torch.zeros(1, num_bases))

    def read(self, batch_size: int) -> torch.Tensor:
        return self.decoder(self.bases.expand(batch_size, -1))

    def consolidate_from_episodes(self, episode_vectors: torch.Tensor) -> None:
        enc = self.encoder(episode_vectors.detach().to(dtype=self.encoder.weight.dtype)).mean(dim=0, keepdim=True)
        self.bases = torch.lerp(self.bases.detach(), enc, self.update_rate).detach()
