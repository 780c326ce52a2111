"""Score-before-update enforcement for test-time training
(cf. src/chaoscontrol/eval_stream/legality.py:14-275).

``score_chunk`` is forward-only under the current weights; ``adapt_on_chunk``
takes gradient steps on a chunk that has already been scored, seeded with the
same recurrent state.  With ``leak_detection`` a chunk that is scored *after*
having been adapted on raises ``LeakDetectedError``.  On a CUDA bare-SSM model
the score path runs the kernel trunk and the fused LM head (no logits tensor).
"""
from __future__ import annotations

import hashlib
from typing import Callable, Optional

import torch
import torch.nn as nn


class LeakDetectedError(RuntimeError):
    pass


def summed_ce(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Default loss: mean CE over all positions."""
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(),
                                             targets.reshape(-1))


class LegalityController:
    def __init__(self, model: nn.Module, *, loss_fn: Callable = summed_ce, leak_detection: bool = False,
                 cache=None, fingerprint_window: int = 4, last_token_is_target_only: bool = False) -> None:
        """``last_token_is_target_only``: the caller's chunks overlap by one token (chunk ``k`` ends
        with the token chunk ``k + 1`` starts with, so that every position of a document is a target
        exactly once).  The model then reads all but the last token, and the returned final state has
        seen every token once; without the flag a chunk is self-contained, as in the reference."""
        self.model = model
        self.last_token_is_target_only = bool(last_token_is_target_only)
        self.loss_fn = loss_fn
        self.leak_detection = leak_detection
        self.cache = cache
        self.fingerprint_window = int(fingerprint_window)
        self._adapted: set[bytes] = set()
        self._pending_cache_hits: list = []

    @staticmethod
    def _chunk_hash(chunk: torch.Tensor) -> bytes:
        return hashlib.blake2b(chunk.detach().cpu().numpy().tobytes(), digest_size=8).digest()

    def _query_cache(self, chunk: torch.Tensor) -> list:
        if self.cache is None or self.fingerprint_window <= 0:
            return []
        if chunk.dim() != 2 or chunk.size(1) < self.fingerprint_window:
            return []
        from ..episodic.cache import fingerprint_tokens
        entry = self.cache.query(int(fingerprint_tokens(chunk[0, -self.fingerprint_window:])))
        return [entry] if entry is not None else []

    def _forward_loss(self, chunk: torch.Tensor, initial_states):
        kw = {"initial_states": initial_states} if initial_states else {}
        if self.last_token_is_target_only:
            out = self.model(chunk[:, :-1], **kw)
            logits = out["logits"] if isinstance(out, dict) else out
            loss = self.loss_fn(logits, chunk[:, 1:])
        else:
            out = self.model(chunk, **kw)
            logits = out["logits"] if isinstance(out, dict) else out
            loss = self.loss_fn(logits[:, :-1], chunk[:, 1:])
        finals = list(out["final_states"]) if isinstance(out, dict) and "final_states" in out else []
        return loss, finals

    def score_chunk(self, chunk: torch.Tensor, *, initial_states: Optional[list] = None):
        """``(loss, final_states)`` under the current weights; no mutation."""
        if chunk.size(1) < 2:
            raise ValueError("score_chunk needs chunk length >= 2 for teacher-forcing CE; "
                             f"got shape {tuple(chunk.shape)}.")
        if self.leak_detection and self._chunk_hash(chunk) in self._adapted:
            raise LeakDetectedError("chunk was adapt_on_chunk'd before score_chunk: "
                                    "score-before-update violation.")
        self.model.eval()
        with torch.no_grad():
            loss, finals = self._forward_loss(chunk, initial_states)
        if self.cache is not None:
            self._pending_cache_hits = self._query_cache(chunk)
        return float(loss.item()), finals

    def adapt_on_chunk(self, chunk: torch.Tensor, *, optimizer, steps: int = 1,
                       initial_states: Optional[list] = None, cache_replay_steps: int = 1):
        """``steps`` optimizer updates on ``chunk`` (plus cache replays); returns the last loss."""
        if steps <= 0 and not self._pending_cache_hits:
            return None
        if self.leak_detection:
            self._adapted.add(self._chunk_hash(chunk))
        self.model.train()
        last = None
        for _ in range(steps):
            optimizer.zero_grad(set_to_none=True)
            loss, _ = self._forward_loss(chunk, initial_states)
            loss.backward()
            optimizer.step()
            last = loss.detach()
        if self.cache is not None and self._pending_cache_hits:
            for hit in self._pending_cache_hits[:max(0, int(cache_replay_steps))]:
                self._replay(hit, optimizer)
            self._pending_cache_hits = []
        return None if last is None else float(last.item())

    def _replay(self, entry, optimizer):
        span = torch.as_tensor(entry.value_tok_ids, dtype=torch.long,
                               device=next(self.model.parameters()).device).view(1, -1)
        if span.size(1) < 2:
            return None
        optimizer.zero_grad(set_to_none=True)
        loss, _ = self._forward_loss(span, None)
        loss.backward()
        optimizer.step()
        if hasattr(self.cache, "mark_fired"):
            self.cache.mark_fired(entry.slot, current_step=-1)
        return loss.detach()

    def mark_new_epoch(self) -> None:
        """Document boundary: chunk-reuse tracking and pending cache hits are per document."""
        self._adapted.clear()
        self._pending_cache_hits = []
