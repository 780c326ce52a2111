"""Write-trigger logic of the episodic cache: which positions of a training
batch deserve a write, and their payloads (public surface of
src/chaoscontrol/optim/episodic_writer.py:38-434).

Selection: ``write_signal = pressure * per_token_ce``; the top ``top_p``
fraction of positions is kept, highest first.  A candidate without a full
fingerprint window before it or a full value span after it is dropped.

Two paths produce the same records.  ``select_writes`` returns Python
``WritePayload`` objects (and optionally pushes dict events / writes the
admission trace).  ``pack_write_events`` builds the 568-byte wire records for
all selected positions in ONE device kernel, so a publisher thread only has to
copy a contiguous buffer to pinned memory and push bytes into the ring.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, MutableSequence, Optional, Sequence

import torch

from ..ops import _lib
from .cache import FINGERPRINT_BASE, FINGERPRINT_MODULUS, fingerprint_tokens, fingerprint_tokens_batch

__all__ = ["WritePayload", "select_writes", "select_top_p_positions", "build_write_payload",
           "build_write_event_dict", "tensor_fp16_to_u16_wire", "token_ids_to_u16_wire", "fingerprint_tokens",
           "fingerprint_tokens_batch", "fingerprints_match", "pack_write_events", "pack_write_events_reference",
           "KEY_REP_WIRE_DIM", "VALUE_TOK_WIRE_LEN", "WRITE_EVENT_BYTES"]

_FINGERPRINT_MODULUS = FINGERPRINT_MODULUS
_FINGERPRINT_BASE = FINGERPRINT_BASE
KEY_REP_WIRE_DIM = 256
VALUE_TOK_WIRE_LEN = 4
WRITE_EVENT_BYTES = 568

# rank-local sequence behind candidate ids: (source_rank << 56) | sequence
_admission_trace_seq = 0


def _reset_admission_trace_seq() -> None:
    global _admission_trace_seq
    _admission_trace_seq = 0


def _reserve_admission_trace_seq(count: int) -> int:
    """Reserves ``count`` ids and returns the first."""
    global _admission_trace_seq
    first = _admission_trace_seq
    _admission_trace_seq += max(0, int(count))
    return first


def _next_admission_trace_seq() -> int:
    return _reserve_admission_trace_seq(1)


def tensor_fp16_to_u16_wire(values: torch.Tensor, *, width: int = KEY_REP_WIRE_DIM) -> list[int]:
    flat = values.detach().flatten().cpu().to(torch.float16)
    if flat.numel() > width:
        raise ValueError(f"wire key_rep width is {width}, got {int(flat.numel())}")
    return [int(x) for x in flat.view(torch.uint16).tolist()] + [0] * (width - flat.numel())


def token_ids_to_u16_wire(values: torch.Tensor, *, width: int = VALUE_TOK_WIRE_LEN) -> list[int]:
    flat = values.detach().flatten().cpu().to(torch.int64)
    if flat.numel() > width:
        raise ValueError(f"wire value_tok_ids width is {width}, got {int(flat.numel())}")
    return [int(x) for x in flat.tolist()] + [0] * (width - flat.numel())


@dataclass(frozen=True)
class WritePayload:
    batch_index: int
    position: int
    key_fp: int
    key_rep: torch.Tensor
    value_tok_ids: torch.Tensor
    value_anchor_id: int


def build_write_event_dict(*, candidate_id: int, gpu_step: int, source_rank: int, key_fp: int, key_rep: torch.Tensor,
                           value_tok_ids: torch.Tensor, value_anchor_id: int, pressure_at_write: float,
                           pre_write_ce: float, write_bucket: int) -> dict:
    """A WRITE_EVENT in wire field order."""
    return {"event_type": 1, "source_rank": int(source_rank), "write_bucket": int(write_bucket),
            "candidate_id": int(candidate_id), "gpu_step": int(gpu_step), "key_fp": int(key_fp),
            "key_rep": tensor_fp16_to_u16_wire(key_rep), "value_tok_ids": token_ids_to_u16_wire(value_tok_ids),
            "value_anchor_id": int(value_anchor_id), "pressure_at_write": float(pressure_at_write),
            "pre_write_ce": float(pre_write_ce)}


def select_top_p_positions(write_signal: torch.Tensor, top_p: float) -> torch.Tensor:
    """``[K, 2]`` (batch, position) pairs, ``K = max(1, round(B*T*top_p))``, descending signal."""
    if write_signal.dim() != 2:
        raise ValueError(f"write_signal must be 2-D [B, T]; got shape {tuple(write_signal.shape)}")
    if not 0.0 < top_p <= 1.0:
        raise ValueError(f"top_p must be in (0, 1]; got {top_p}")
    B, T = write_signal.shape
    k = max(1, int(round(B * T * float(top_p))))
    idx = torch.topk(write_signal.reshape(-1), k=k, largest=True).indices
    return torch.stack([(idx // T).long(), (idx % T).long()], dim=1)


def build_write_payload(*, batch_index: int, position: int, input_ids: torch.Tensor, target_ids: torch.Tensor,
                        key_rep_per_position: torch.Tensor, fingerprint_window: int,
                        span_length: int) -> WritePayload | None:
    B, T = input_ids.shape
    if not 0 <= batch_index < B:
        raise IndexError(f"batch_index {batch_index} out of range for B={B}")
    if not 0 <= position < T:
        raise IndexError(f"position {position} out of range for T={T}")
    if position < fingerprint_window or position + span_length > T:
        return None
    return WritePayload(
        batch_index=int(batch_index), position=int(position),
        key_fp=fingerprint_tokens(input_ids[batch_index, position - fingerprint_window:position]),
        key_rep=key_rep_per_position[batch_index, position].clone(),
        value_tok_ids=target_ids[batch_index, position:position + span_length].clone().to(torch.int64),
        value_anchor_id=int(target_ids[batch_index, position]))


def _check_shapes(input_ids, target_ids, pressure, per_token_ce, key_rep, source_rank) -> None:
    if pressure.shape != per_token_ce.shape:
        raise ValueError(f"pressure {tuple(pressure.shape)} and per_token_ce {tuple(per_token_ce.shape)} must match")
    if pressure.shape != input_ids.shape:
        raise ValueError(f"pressure {tuple(pressure.shape)} must match input_ids {tuple(input_ids.shape)}")
    if target_ids.shape != input_ids.shape:
        raise ValueError(f"target_ids {tuple(target_ids.shape)} must match input_ids {tuple(input_ids.shape)}")
    if key_rep.dim() != 3:
        raise ValueError(f"key_rep_per_position must be 3-D [B, T, D]; got shape {tuple(key_rep.shape)}")
    if key_rep.shape[:2] != input_ids.shape:
        raise ValueError(f"key_rep_per_position [B, T] {tuple(key_rep.shape[:2])} must match input_ids "
                         f"{tuple(input_ids.shape)}")
    if not 0 <= int(source_rank) < 256:
        raise ValueError(f"source_rank must fit in u8; got {source_rank}")


def select_writes(*, input_ids: torch.Tensor, target_ids: torch.Tensor, pressure: torch.Tensor,
                  per_token_ce: torch.Tensor, key_rep_per_position: torch.Tensor, top_p: float,
                  fingerprint_window: int, span_length: int, source_rank: int = 0, gpu_step: int = 0,
                  write_bucket: int = 0, admission_trace_path: str | None = None, write_ring: Any | None = None,
                  write_ring_drops: MutableSequence[int] | None = None) -> list[WritePayload]:
    """Payloads for one training step, most surprising first.

    With ``write_ring`` each admitted payload is also pushed as a dict event
    (failed pushes bump ``write_ring_drops[0]``).  With ``admission_trace_path``
    every top-K candidate, admitted or edge-rejected (``key_fp`` 0), is appended
    as one NDJSON row.  Neither changes the returned list.  All host transfers
    happen once for the whole selection, and the fingerprints are hashed as one
    batch.
    """
    _check_shapes(input_ids, target_ids, pressure, per_token_ce, key_rep_per_position, source_rank)
    T = input_ids.shape[1]
    signal = pressure.detach().float() * per_token_ce.detach().float()
    pos = select_top_p_positions(signal, top_p).cpu()
    bs, ts = pos[:, 0], pos[:, 1]
    ok = (ts >= fingerprint_window) & (ts + span_length <= T)
    need_ids = admission_trace_path is not None or write_ring is not None
    first_seq = _reserve_admission_trace_seq(pos.shape[0]) if need_ids else 0
    ids_c, tgt_c = input_ids.detach().cpu(), target_ids.detach().cpu()
    pr_c, ce_c = pressure.detach().float().cpu(), per_token_ce.detach().float().cpu()
    keep = ok.nonzero(as_tuple=True)[0]
    fps: list[int] = []
    if keep.numel():
        win = ts[keep].unsqueeze(1) - fingerprint_window + torch.arange(fingerprint_window).unsqueeze(0)
        fps = fingerprint_tokens_batch(ids_c[bs[keep].unsqueeze(1), win]) if fingerprint_window > 0 else [0] * keep.numel()
    reps = key_rep_per_position.detach()[bs.to(key_rep_per_position.device), ts.to(key_rep_per_position.device)].cpu()
    fp_of = dict(zip(keep.tolist(), fps))
    payloads: list[WritePayload] = []
    rows: list[dict] = []
    for i in range(pos.shape[0]):
        b, t = int(bs[i]), int(ts[i])
        cand = ((int(source_rank) << 56) | ((first_seq + i) & ((1 << 56) - 1))) if need_ids else None
        payload = None
        if i in fp_of:
            payload = WritePayload(batch_index=b, position=t, key_fp=fp_of[i], key_rep=reps[i].clone(),
                                   value_tok_ids=tgt_c[b, t:t + span_length].clone().to(torch.int64),
                                   value_anchor_id=int(tgt_c[b, t]))
            payloads.append(payload)
            if write_ring is not None:
                ev = build_write_event_dict(candidate_id=cand, gpu_step=int(gpu_step), source_rank=int(source_rank),
                                            key_fp=payload.key_fp, key_rep=payload.key_rep,
                                            value_tok_ids=payload.value_tok_ids,
                                            value_anchor_id=payload.value_anchor_id,
                                            pressure_at_write=float(pr_c[b, t]), pre_write_ce=float(ce_c[b, t]),
                                            write_bucket=int(write_bucket))
                if not bool(write_ring.push(ev)) and write_ring_drops is not None:
                    write_ring_drops[0] = int(write_ring_drops[0]) + 1
        if admission_trace_path is not None:
            rows.append({"candidate_id": cand, "decision": 1 if payload is not None else 0, "gpu_step": int(gpu_step),
                         "source_rank": int(source_rank), "key_fp": payload.key_fp if payload else 0,
                         "key_rep_l2": float(torch.linalg.vector_norm(reps[i].float())),
                         "value_anchor_id": int(tgt_c[b, t]), "pressure_at_write": float(pr_c[b, t]),
                         "pre_write_ce": float(ce_c[b, t]), "write_bucket": int(write_bucket)})
    if rows:
        with open(admission_trace_path, "a") as fh:
            fh.writelines(json.dumps(r, separators=(",", ":")) + "\n" for r in rows)
    return payloads


def fingerprints_match(a: Sequence[int], b: Sequence[int]) -> bool:
    return list(a) == list(b)


# ---------------------------------------------------------------------------
# Device-side packing into wire records
# ---------------------------------------------------------------------------
_REP_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def pack_write_events(*, input_ids: torch.Tensor, target_ids: torch.Tensor, key_rep_per_position: torch.Tensor,
                      per_token_ce: torch.Tensor, positions: torch.Tensor, candidate_base: torch.Tensor,
                      pressure: Optional[torch.Tensor] = None, gpu_step: int = 0, source_rank: int = 0,
                      write_bucket: int = 0, fingerprint_window: int = 8, span_length: int = VALUE_TOK_WIRE_LEN,
                      key_rep_dim: Optional[int] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[M, 568]`` uint8 WriteEvent records for ``positions`` ``[M, 2]``.

    Edge-trimmed candidates come back as all-zero records (``event_type`` 0).
    ``candidate_base`` is a one-element int64 tensor on the same device (the
    rank-local sequence number of record 0), read by the kernel.  On a CPU tensor
    this runs :func:`pack_write_events_reference`.
    """
    M = int(positions.shape[0])
    D = int(key_rep_per_position.shape[-1])
    rd = D if key_rep_dim is None else int(key_rep_dim)
    if not input_ids.is_cuda:
        res = pack_write_events_reference(
            input_ids=input_ids, target_ids=target_ids, key_rep_per_position=key_rep_per_position,
            per_token_ce=per_token_ce, positions=positions, candidate_base=int(candidate_base), pressure=pressure,
            gpu_step=gpu_step, source_rank=source_rank, write_bucket=write_bucket,
            fingerprint_window=fingerprint_window, span_length=span_length, key_rep_dim=rd)
        return res if out is None else out.copy_(res)
    if out is None:
        out = torch.empty((M, WRITE_EVENT_BYTES), dtype=torch.uint8, device=input_ids.device)
    rep = key_rep_per_position
    if rep.dtype not in _REP_DTYPE or not rep.is_contiguous():
        rep = rep.float().contiguous() if rep.dtype not in _REP_DTYPE else rep.contiguous()
    B, T = input_ids.shape
    _lib.check(_lib.lib().ccb_pack_write_events(
        out.data_ptr(), input_ids.long().contiguous().data_ptr(), target_ids.long().contiguous().data_ptr(),
        rep.data_ptr(), _REP_DTYPE[rep.dtype], _lib.ptr(None if pressure is None else pressure.float().contiguous()),
        per_token_ce.float().contiguous().data_ptr(), positions.long().contiguous().data_ptr(),
        candidate_base.data_ptr(), M, B, T, D, int(gpu_step), int(source_rank), int(write_bucket),
        int(fingerprint_window), int(span_length), rd, _lib.stream_ptr()), "pack_write_events")
    return out


def pack_write_events_reference(*, input_ids, target_ids, key_rep_per_position, per_token_ce, positions,
                                candidate_base: int, pressure=None, gpu_step: int = 0, source_rank: int = 0,
                                write_bucket: int = 0, fingerprint_window: int = 8,
                                span_length: int = VALUE_TOK_WIRE_LEN, key_rep_dim: Optional[int] = None):
    """Host construction of the same records through the numpy wire dtype."""
    import numpy as np

    from .native import WRITE_EVENT as WRITE_EVENT_DTYPE
    B, T = input_ids.shape
    D = key_rep_per_position.shape[-1]
    rd = D if key_rep_dim is None else int(key_rep_dim)
    M = int(positions.shape[0])
    rec = np.zeros(M, dtype=WRITE_EVENT_DTYPE)
    ids, tgt = input_ids.detach().cpu().long(), target_ids.detach().cpu().long()
    for m in range(M):
        b, t = int(positions[m, 0]), int(positions[m, 1])
        if not (0 <= b < B and t >= fingerprint_window and t + span_length <= T and 0 < rd <= KEY_REP_WIRE_DIM
                and 0 < span_length <= VALUE_TOK_WIRE_LEN and D >= rd):
            continue
        r = rec[m]
        r["event_type"], r["source_rank"], r["write_bucket"] = 1, source_rank, write_bucket
        r["candidate_id"] = (int(source_rank) << 56) | ((int(candidate_base) + m) & ((1 << 56) - 1))
        r["gpu_step"] = gpu_step
        r["key_fp"] = fingerprint_tokens(ids[b, t - fingerprint_window:t])
        r["key_rep"][:rd] = key_rep_per_position[b, t, :rd].detach().cpu().to(torch.float16).view(torch.uint16).numpy()
        r["value_tok_ids"][:span_length] = (tgt[b, t:t + span_length] & 0xFFFF).numpy().astype(np.uint16)
        r["value_anchor_id"] = int(tgt[b, t]) & 0xFFFFFFFF
        r["pressure_at_write"] = 1.0 if pressure is None else float(pressure[b, t])
        r["pre_write_ce"] = float(per_token_ce[b, t])
    return torch.from_numpy(rec.view(np.uint8).reshape(M, WRITE_EVENT_BYTES).copy())
