"""SentencePiece byte accounting and the windowed bits-per-byte evaluator
(functions of experiments/17_local_attn_sidecar/runner_exp17.py:142-296).

Bytes of a target token = its piece's UTF-8 length (1 for byte tokens, 0 for
control / unknown / unused), plus one for a leading-space marker unless the
previous token is a boundary token.  The evaluator scores through the fused
linear+CE head (no ``[B*T, V]`` logits) when the model supports it.
"""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

from .data import batch_from_starts, load_fineweb_tokens, maybe_autocast
from .scoring import compute_bpb

__all__ = ["build_sentencepiece_luts", "load_sp_data", "evaluate_bpb_sp", "token_byte_counts"]


def build_sentencepiece_luts(sp, vocab_size: int, device) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(base_bytes int16, has_leading_space bool, is_boundary_token bool)`` tables
    of size ``max(sp.vocab_size(), vocab_size)``."""
    n_sp = int(sp.vocab_size())
    size = max(n_sp, int(vocab_size))
    base = np.zeros(size, dtype=np.int16)
    lead = np.zeros(size, dtype=np.bool_)
    boundary = np.ones(size, dtype=np.bool_)
    for t in range(n_sp):
        if sp.is_control(t) or sp.is_unknown(t) or sp.is_unused(t):
            continue
        boundary[t] = False
        if sp.is_byte(t):
            base[t] = 1
            continue
        piece = sp.id_to_piece(t)
        if piece.startswith("▁"):
            lead[t] = True
            piece = piece[1:]
        base[t] = len(piece.encode("utf-8"))
    return (torch.tensor(base, dtype=torch.int16, device=device), torch.tensor(lead, dtype=torch.bool, device=device),
            torch.tensor(boundary, dtype=torch.bool, device=device))


def token_byte_counts(prev_ids: torch.Tensor, tgt_ids: torch.Tensor, base_bytes_lut, has_leading_space_lut,
                      is_boundary_token_lut) -> torch.Tensor:
    """Scored bytes per target token (int64), same shape as ``tgt_ids``."""
    t, p = tgt_ids.long(), prev_ids.long()
    return base_bytes_lut[t].long() + (has_leading_space_lut[t] & ~is_boundary_token_lut[p]).long()


def load_sp_data(data_dir: str, vocab_size: int = 8192):
    """Pre-tokenised shards with out-of-range ids clamped (a few header words decode
    as stray ids); more than 0.1 % out of range means the shards and the tokenizer
    do not belong together, which is an error."""
    train, val = load_fineweb_tokens(data_dir)

    def _oor(t: torch.Tensor) -> int:
        return int(((t < 0) | (t >= vocab_size)).sum())

    n_tr, n_va = _oor(train), _oor(val)
    f_tr, f_va = n_tr / max(train.numel(), 1), n_va / max(val.numel(), 1)
    if f_tr > 0.001 or f_va > 0.001:
        raise ValueError(f"load_sp_data: tokenizer/data mismatch at {data_dir}. More than 0.1% of tokens are outside "
                         f"[0, {vocab_size}). train oor={n_tr}/{train.numel()} ({f_tr:.4%}), val oor={n_va}/"
                         f"{val.numel()} ({f_va:.4%}). Check that --data-path matches --sp-model-path.")
    train, val = train.clamp(0, vocab_size - 1), val.clamp(0, vocab_size - 1)
    return train, val, train[:0]


def evaluate_bpb_sp(model: Any, *, tokens: torch.Tensor, eval_starts: list[int], batch_size: int, seq_len: int,
                    device: torch.device, base_bytes_lut, has_leading_space_lut, is_boundary_token_lut) -> dict[str, float]:
    """Windowed evaluation: ``{"loss", "bpb", "tokens", "total_ce_nats", "total_scored_bytes"}``."""
    from .scoring import _chunk_loss_rows
    was_training = model.training
    model.eval()
    ce = torch.zeros((), dtype=torch.float64, device=device)
    nbytes = torch.zeros((), dtype=torch.int64, device=device)
    ntok = 0
    with torch.no_grad():
        for i in range(0, len(eval_starts), batch_size):
            inputs, targets = batch_from_starts(tokens, eval_starts[i:i + batch_size], seq_len, device)
            dt = next(model.parameters()).dtype if device.type == "cuda" else torch.float32
            with maybe_autocast(device, dt):
                rows, _ = _chunk_loss_rows(model, inputs, targets, None)       # per-token CE, fused head
            ce += rows.double().sum()
            ntok += int(targets.numel())
            nbytes += token_byte_counts(inputs.reshape(-1), targets.reshape(-1), base_bytes_lut,
                                        has_leading_space_lut, is_boundary_token_lut).sum()
    if was_training:
        model.train()
    total_ce, total_bytes = float(ce), int(nbytes)
    return {"loss": total_ce / max(ntok, 1), "bpb": compute_bpb(total_ce, total_bytes), "tokens": float(ntok),
            "total_ce_nats": total_ce, "total_scored_bytes": total_bytes}
