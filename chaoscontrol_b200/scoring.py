"""Streaming per-document scorer (score-only) and per-chunk test-time training.

Documents are scored in fixed-size chunks with the recurrent state carried
across chunks inside a document and reset between documents.  The batched
scorer sorts documents by length, runs ``[docs, chunk]`` blocks through the
kernel trunk with a native ``h0 -> hT`` carry and scores them with the fused
LM head, so neither a per-token loop nor a ``[docs, chunk, vocab]`` logits
tensor ever exists (the reference materialises logits and drops to a Python
per-token loop for carried state: scripts/run_exp20_fast_score.py:787-1020,
src/chaoscontrol/core.py:689-728).

Ranks split the documents by longest-processing-time bin packing over padded
token counts and combine ``(sum CE, tokens, bytes)`` with one all-reduce.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch
import torch.nn as nn

from .eval_stream.budget import BudgetTracker
from .eval_stream.legality import LegalityController
from .eval_stream.state import DeltaModulator, StateManager, select_adapt_params
from .ops import lm_head as LH
from .ops.trunk import fold_colscale


def compute_bpb(total_ce_nats: float, total_raw_bytes: float) -> float:
    """bits per byte = nats / ln 2 / bytes."""
    if total_raw_bytes <= 0:
        return float("nan")
    return float(total_ce_nats) / math.log(2.0) / float(total_raw_bytes)


def assign_docs_lpt(lengths: Sequence[int], world_size: int, chunk_size: int) -> list[list[int]]:
    """Longest-processing-time assignment of documents to ranks; work = tokens
    padded to whole chunks.  Returns per-rank lists of document indices."""
    work = [max(1, math.ceil(max(int(n) - 1, 1) / chunk_size)) * chunk_size for n in lengths]
    order = sorted(range(len(lengths)), key=lambda i: -work[i])
    loads = [0] * world_size
    out: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: loads[k])
        out[r].append(i)
        loads[r] += work[i]
    return out


@dataclass
class ScoreResult:
    doc_ce: np.ndarray            # fp64 summed CE per document (nats)
    doc_tokens: np.ndarray        # scored targets per document
    total_ce: float = 0.0
    total_tokens: int = 0
    total_bytes: int = 0
    bpb: float = float("nan")
    elapsed_s: float = 0.0
    tokens_per_s: float = 0.0
    extra: dict = field(default_factory=dict)


def _chunk_loss_rows(model: nn.Module, inputs: torch.Tensor, targets: torch.Tensor, states):
    """Per-position CE ``[B, T]`` and final states for one block of chunks."""
    if getattr(model, "kernel_trunk_supported", lambda: False)() and LH.kernel_supported(
            model.embed.weight.new_empty(1, model.dim), model.lm_head.weight):
        hidden, ss, finals = model.encode_with_stats(inputs, initial_states=states)
        W_f = fold_colscale(model.lm_head.weight, model.final_norm.weight)
        B, T, D = hidden.shape
        rows, _ = LH.lm_head_lse(hidden.reshape(B * T, D), ss, W_f, targets.reshape(-1),
                                 eps=model.final_norm.eps)
        return rows.view(B, T), finals
    out = model(inputs, initial_states=states)
    logits = out["logits"].float()
    rows = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1),
                                             reduction="none").view(targets.shape)
    return rows, list(out["final_states"])


@torch.no_grad()
def score_docs(model: nn.Module, tokens: torch.Tensor, doc_starts: Sequence[int],
               doc_lens: Sequence[int], *, chunk_size: int = 512, max_batch_tokens: int = 1 << 19,
               raw_bytes: Optional[Sequence[int]] = None, deadline_s: Optional[float] = None) -> ScoreResult:
    """Score documents stored back to back in ``tokens`` (device tensor).

    Every document contributes ``len - 1`` targets (the first token has no
    context; chunk-boundary targets are included).  State is carried across the
    chunks of a document and starts from zero for each document.
    """
    t0 = time.perf_counter()
    device = tokens.device
    n_docs = len(doc_lens)
    lens = np.asarray(doc_lens, dtype=np.int64)
    starts = np.asarray(doc_starts, dtype=np.int64)
    doc_ce = np.zeros(n_docs, dtype=np.float64)
    doc_tok = np.maximum(lens - 1, 0)
    order = np.argsort(-lens, kind="stable")
    L = len(model.layers)
    batch_docs = max(1, max_batch_tokens // chunk_size)
    model.eval()
    tokens_l = tokens.long()
    timed_out = False
    for b0 in range(0, n_docs, batch_docs):
        idx = order[b0: b0 + batch_docs]
        idx = idx[lens[idx] >= 2]
        if idx.size == 0:
            continue
        nb = idx.size
        st = torch.as_tensor(starts[idx], device=device)
        ln = torch.as_tensor(lens[idx], device=device)
        states = None
        ce_acc = torch.zeros(nb, dtype=torch.float64, device=device)
        max_targets = int(lens[idx[0]]) - 1
        for c0 in range(0, max_targets, chunk_size):
            # documents are sorted by length: the active ones form a prefix
            active = int((lens[idx] - 1 > c0).sum())          # host-side count: no device sync per chunk
            if active == 0:
                break
            pos = c0 + torch.arange(chunk_size + 1, device=device)[None, :]          # [1, C+1]
            valid = pos < ln[:active, None]                                         # token exists
            gather = (st[:active, None] + pos).clamp_max(tokens_l.numel() - 1)
            blk = torch.where(valid, tokens_l[gather], torch.zeros_like(gather))
            inputs, targets = blk[:, :-1].contiguous(), blk[:, 1:].contiguous()
            tmask = valid[:, 1:]
            cur = None if states is None else [s[:active].contiguous() for s in states]
            rows, finals = _chunk_loss_rows(model, inputs, targets, cur)
            ce_acc[:active] += (rows.double() * tmask).sum(dim=1)
            states = [f.float() for f in finals]
            if deadline_s is not None and time.perf_counter() - t0 > deadline_s:
                timed_out = True
                break
        doc_ce[idx] = ce_acc.cpu().numpy()
        if timed_out:
            break
    if device.type == "cuda":
        torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    res = ScoreResult(doc_ce=doc_ce, doc_tokens=doc_tok)
    res.total_ce = float(doc_ce.sum())
    res.total_tokens = int(doc_tok.sum())
    res.total_bytes = int(np.sum(raw_bytes)) if raw_bytes is not None else 0
    res.bpb = compute_bpb(res.total_ce, res.total_bytes) if res.total_bytes else float("nan")
    res.elapsed_s = elapsed
    res.tokens_per_s = res.total_tokens / elapsed if elapsed > 0 else 0.0
    res.extra = {"timed_out": timed_out, "num_layers": L}
    return res


def score_val_cache(model: nn.Module, cache, *, chunk_size: int = 512, rank: int = 0, world_size: int = 1,
                    max_docs: Optional[int] = None, max_batch_tokens: int = 1 << 19,
                    device: Optional[torch.device] = None) -> dict:
    """Score a :class:`~chaoscontrol_b200.eval_stream.io.ValCache` with documents
    sharded across ranks; returns the aggregated summary on every rank."""
    device = device or next(model.parameters()).device
    docs = cache.docs if max_docs is None else cache.docs[:max_docs]
    lens = np.asarray(docs["token_len"])
    shards = assign_docs_lpt(lens.tolist(), world_size, chunk_size)
    mine = np.asarray(sorted(shards[rank]), dtype=np.int64)
    tokens = torch.as_tensor(np.asarray(cache.tokens).astype(np.int32), device=device)
    res = score_docs(model, tokens, np.asarray(docs["token_start"])[mine], lens[mine], chunk_size=chunk_size,
                     raw_bytes=np.asarray(docs["raw_bytes"])[mine], max_batch_tokens=max_batch_tokens)
    agg = torch.tensor([res.total_ce, float(res.total_tokens), float(res.total_bytes), float(len(mine))],
                       dtype=torch.float64, device=device)
    mx = torch.tensor([res.elapsed_s], dtype=torch.float64, device=device)
    if world_size > 1:
        import torch.distributed as dist
        dist.all_reduce(agg, op=dist.ReduceOp.SUM)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    ce, ntok, nbytes, ndocs = (float(v) for v in agg.cpu())
    elapsed = float(mx.item())
    return {"docs_scored": int(ndocs), "tokens_scored": int(ntok), "total_ce_nats": ce,
            "total_raw_bytes": int(nbytes), "bpb": compute_bpb(ce, nbytes), "mean_ce": ce / max(ntok, 1),
            "elapsed_s": elapsed, "tokens_per_s": ntok / elapsed if elapsed > 0 else 0.0,
            "rank_docs": int(len(mine)), "world_size": world_size, "chunk_size": chunk_size}


# ---------------------------------------------------------------------------
# per-chunk test-time training (score, then adapt, never the other way round)
# ---------------------------------------------------------------------------
def run_ttt_eval(model: nn.Module, docs, *, adapt_set: str = "log_a+delta_proj",
                 persistence_mode: str = "reset", chunk_size: int = 256, steps_per_chunk: int = 1,
                 eval_lr: float = 0.064, optimizer: str = "sgd", budget_seconds: float = 600.0,
                 score_floor_seconds: float = 0.0, safety_margin_seconds: float = 0.0,
                 delta_scale: float = 1.0, log_a_shift: float = 0.0, restore_weights_per_doc: bool = True,
                 metrics=None, max_docs: Optional[int] = None) -> dict:
    """Score-then-adapt evaluation over an iterable of ``DocRecord``s.

    For every chunk: ``score_chunk`` under the current weights, then (while
    budget slack remains) ``steps_per_chunk`` optimizer steps on that chunk seeded
    with the same recurrent state.  With ``restore_weights_per_doc`` the adapted
    parameters are snapshotted at the start of a document and restored at its
    end (``carry_weights`` / ``carry_both`` persistence keep them instead).
    """
    device = next(model.parameters()).device
    params = select_adapt_params(model, adapt_set=adapt_set)
    if optimizer == "muon":
        from .optim.muon import Muon
        opt = Muon(params, lr=eval_lr, fused=True) if params else None
        if opt is not None:
            opt.bind_param_names([(n, p) for n, p in model.named_parameters()])
    else:
        opt = torch.optim.SGD(params, lr=eval_lr) if params else None
    keep_weights = persistence_mode in ("carry_weights", "carry_both") or not restore_weights_per_doc
    ctl = LegalityController(model, loss_fn=lambda lg, tg: torch.nn.functional.cross_entropy(
        lg.reshape(-1, lg.shape[-1]).float(), tg.reshape(-1), reduction="sum"), last_token_is_target_only=True)
    sm = StateManager(model, persistence_mode=persistence_mode)
    budget = BudgetTracker(total_budget_seconds=budget_seconds, score_floor_seconds=score_floor_seconds,
                           safety_margin_seconds=safety_margin_seconds)
    t_start = time.perf_counter()
    tot_ce = 0.0
    tot_tok = tot_bytes = n_docs = n_chunks = n_steps = 0
    timed_out = False
    with DeltaModulator(model, delta_scale=delta_scale, log_a_shift=log_a_shift, adapt_set_hint=adapt_set):
        for rec in docs:
            if max_docs is not None and n_docs >= max_docs:
                break
            if len(rec.tokens) < 2:
                continue
            snap = [p.detach().clone() for p in params] if (params and not keep_weights) else None
            sm.start_doc(doc_id=rec.doc_id, batch_size=1)
            ctl.mark_new_epoch()
            toks = torch.as_tensor(rec.tokens, dtype=torch.long, device=device).view(1, -1)
            C = toks.size(1) if chunk_size <= 0 else chunk_size
            doc_ce, loss_after, t_doc = 0.0, None, time.perf_counter()
            for s in range(0, toks.size(1) - 1, C):
                chunk = toks[:, s: s + C + 1]
                if chunk.size(1) < 2:
                    break
                state = sm.get_state()
                t0 = time.perf_counter()
                loss, finals = ctl.score_chunk(chunk, initial_states=state if state else None)
                budget.add_score_time(time.perf_counter() - t0)
                doc_ce += loss
                n_chunks += 1
                if opt is not None and steps_per_chunk > 0 and budget.can_adapt():
                    t0 = time.perf_counter()
                    loss_after = ctl.adapt_on_chunk(chunk, optimizer=opt, steps=steps_per_chunk,
                                                    initial_states=state if state else None)
                    budget.add_adapt_time(time.perf_counter() - t0)
                    n_steps += steps_per_chunk
                if finals:
                    sm.set_state([f.detach() for f in finals])
                if time.perf_counter() - t_start > budget_seconds:
                    timed_out = True
                    break
            if snap is not None:
                with torch.no_grad():
                    for p, s_ in zip(params, snap):
                        p.copy_(s_)
            ntok = toks.size(1) - 1
            tot_ce += doc_ce
            tot_tok += ntok
            tot_bytes += rec.raw_bytes
            n_docs += 1
            if metrics is not None:
                metrics.record_doc(doc_id=rec.doc_id, bpb=compute_bpb(doc_ce, rec.raw_bytes), tokens=ntok,
                                   loss_before=doc_ce / max(ntok, 1), loss_after=loss_after,
                                   step_count=n_steps, wall_ms=(time.perf_counter() - t_doc) * 1e3,
                                   grad_norm=0.0, state_norm=float(sum(float(f.float().norm()) for f in
                                                                       sm.get_state())))
                if metrics.collapsed:
                    break
            if timed_out:
                break
    elapsed = time.perf_counter() - t_start
    summary = budget.summary(docs_scored=n_docs, chunks_scored=n_chunks, tokens_scored=tot_tok,
                             adapt_steps=n_steps, timed_out=timed_out,
                             collapsed=bool(metrics is not None and metrics.collapsed),
                             score_only_mode=opt is None, elapsed_seconds=elapsed, chunk_size=chunk_size,
                             max_docs=max_docs,
                             gpu_name=torch.cuda.get_device_name(0) if torch.cuda.is_available() else None,
                             torch_version=torch.__version__, cuda_version=torch.version.cuda)
    summary.update(total_ce_nats=tot_ce, total_raw_bytes=tot_bytes, bpb=compute_bpb(tot_ce, tot_bytes),
                   mean_ce=tot_ce / max(tot_tok, 1), tokens_per_s=tot_tok / elapsed if elapsed > 0 else 0.0,
                   adapt_set=adapt_set, persistence_mode=persistence_mode)
    return summary


# ---------------------------------------------------------------------------
# test-time training with the per-chunk work captured in a CUDA graph
# ---------------------------------------------------------------------------
class GraphTTTRunner:
    """Score a fixed-length chunk, then take one SGD step on it, as ONE CUDA graph.

    Per-document TTT runs at batch 1, so a chunk is a few hundred small launches
    and the Python/driver launch path, not the GPU, sets the pace.  The body
    (kernel-trunk scoring pass with the carried state, fused-head per-row CE
    accumulated on the device, autograd forward + backward of the summed CE from
    the SAME state, ``p -= lr * grad`` on the adapt set, carried state := the
    scoring pass's final state) is captured once for ``chunk_size`` tokens and
    replayed per chunk; only the ragged tail of a document runs eagerly.
    Nothing is read back inside a document."""

    def __init__(self, model: nn.Module, params: list, *, chunk_size: int, lr: float) -> None:
        if not getattr(model, "kernel_trunk_supported", lambda: False)():
            raise ValueError("GraphTTTRunner needs the bf16 kernel trunk")
        self.model, self.params, self.C, self.lr = model, list(params), int(chunk_size), float(lr)
        dev = model.embed.weight.device
        self.device = dev
        self.tok = torch.zeros(1, self.C + 1, dtype=torch.long, device=dev)
        self.state = [torch.zeros(1, model.dim, device=dev, dtype=model.embed.weight.dtype) for _ in model.layers]
        self.ce_acc = torch.zeros((), dtype=torch.float32, device=dev)
        self.n_valid = torch.full((), self.C, dtype=torch.long, device=dev)     # targets that count in this chunk
        self._pos = torch.arange(self.C, device=dev).view(1, -1)
        self._one = torch.ones((), dtype=torch.float32, device=dev)
        self._frozen = [p for p in model.parameters() if p.requires_grad and all(p is not q for q in self.params)]
        for p in self._frozen:
            p.requires_grad_(False)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.replays = self.padded_chunks = 0
        # warm up off the capture stream (allocator, kernel attributes), then capture
        snap = [p.detach().clone() for p in self.params]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._body(self.tok)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        for p in self.params:
            p.grad = None
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self._body(self.tok)
        self.graph = g
        with torch.no_grad():
            for p, s in zip(self.params, snap):
                p.copy_(s)
        self.start_doc()

    def _body(self, tok: torch.Tensor) -> None:
        from .kernels.lm_head_loss import fused_linear_cross_entropy_weighted, fused_rms_norm
        m = self.model
        inp, tgt = tok[:, :-1].to(torch.int32), tok[:, 1:]
        mask = (self._pos < self.n_valid).float()             # a document's ragged tail is padded, not re-traced
        with torch.no_grad():
            rows, finals = _chunk_loss_rows(m, inp, tgt, self.state)
            self.ce_acc += (rows.float() * mask).sum()
        if self.params:
            hidden = m.encode(inp, initial_states=self.state)
            loss, _ = fused_linear_cross_entropy_weighted(
                fused_rms_norm(hidden, m.final_norm.weight, eps=m.final_norm.eps), m.lm_head.weight, tgt,
                mask.reshape(-1), normalizer=self._one)
            loss.backward()
            with torch.no_grad():
                torch._foreach_add_(self.params, [p.grad for p in self.params], alpha=-self.lr)
        with torch.no_grad():
            for s, f in zip(self.state, finals):
                s.copy_(f)

    def start_doc(self) -> None:
        torch._foreach_zero_(self.state + [self.ce_acc])

    def run_doc(self, doc_tokens: torch.Tensor) -> tuple[torch.Tensor, int]:
        """``doc_tokens``: ``[n]`` long on the device.  Returns ``(summed CE as a
        device scalar, chunks)``; state and accumulator are reset first.  The last,
        shorter chunk is zero-padded to the captured length and masked out of both
        the score and the adaptation loss (its state is never used again)."""
        self.start_doc()
        n, C, chunks = int(doc_tokens.numel()), self.C, 0
        for s in range(0, n - 1, C):
            piece = doc_tokens[s: s + C + 1]
            k = int(piece.numel())
            if k < 2:
                break
            if k == C + 1:
                self.tok.copy_(piece.view(1, -1))
            else:
                self.tok.zero_()
                self.tok[0, :k].copy_(piece)
                self.n_valid.fill_(k - 1)
                self.padded_chunks += 1
            self.graph.replay()
            if k != C + 1:
                self.n_valid.fill_(C)
            self.replays += 1
            chunks += 1
        return self.ce_acc.clone(), chunks

    def close(self) -> None:
        for p in self._frozen:
            p.requires_grad_(True)
        self.graph = None


def run_ttt_eval_graph(model: nn.Module, docs, *, adapt_set: str = "log_a+delta_proj", chunk_size: int = 256,
                       eval_lr: float = 0.064, max_docs: Optional[int] = None, metrics=None) -> dict:
    """``run_ttt_eval`` for its most common setting -- SGD, one step per chunk,
    ``reset`` persistence, adapted weights restored after every document -- with
    the per-chunk work replayed from a CUDA graph and per-document CE read back
    once at the end (per document when ``metrics`` wants rows)."""
    device = next(model.parameters()).device
    params = select_adapt_params(model, adapt_set=adapt_set)
    was_training = model.training
    model.eval()
    runner = GraphTTTRunner(model, params, chunk_size=chunk_size, lr=eval_lr)
    snap = [p.detach().clone() for p in params]
    t0 = time.perf_counter()
    ces, toks, byts, n_chunks, ids = [], [], [], 0, []

    def groups(it, n_tokens=1 << 20):
        """Documents in groups of about a million tokens: one pinned upload per group."""
        batch, count = [], 0
        for rec in it:
            if max_docs is not None and len(ces) + len(batch) >= max_docs:
                break
            if len(rec.tokens) < 2:
                continue
            batch.append(rec)
            count += len(rec.tokens)
            if count >= n_tokens:
                yield batch
                batch, count = [], 0
        if batch:
            yield batch
    try:
        for batch in groups(docs):
            flat = torch.as_tensor(np.concatenate([np.asarray(r.tokens, dtype=np.int64) for r in batch]))
            flat = (flat.pin_memory() if device.type == "cuda" else flat).to(device, non_blocking=True)
            off = 0
            for rec in batch:
                dev_toks = flat[off: off + len(rec.tokens)]
                off += len(rec.tokens)
                ce, ch = runner.run_doc(dev_toks)
                if params:
                    with torch.no_grad():
                        torch._foreach_copy_(params, snap)
                ces.append(ce)
                toks.append(len(rec.tokens) - 1)
                byts.append(rec.raw_bytes)
                ids.append(rec.doc_id)
                n_chunks += ch
                if metrics is not None:
                    doc_ce = float(ce)
                    metrics.record_doc(doc_id=rec.doc_id, bpb=compute_bpb(doc_ce, rec.raw_bytes), tokens=toks[-1],
                                       loss_before=doc_ce / max(toks[-1], 1), loss_after=None, step_count=n_chunks,
                                       wall_ms=0.0, grad_norm=0.0, state_norm=0.0)
        ce_all = torch.stack(ces).double().cpu() if ces else torch.zeros(0, dtype=torch.float64)
    finally:
        replays, eager = runner.replays, runner.padded_chunks
        runner.close()
        model.train(was_training)
    elapsed = time.perf_counter() - t0
    tot_ce, tot_tok, tot_bytes = float(ce_all.sum()), int(sum(toks)), int(sum(byts))
    return {"docs_scored": len(ces), "chunks_scored": n_chunks, "tokens_scored": tot_tok,
            "adapt_steps": n_chunks if params else 0, "elapsed_seconds": elapsed, "chunk_size": chunk_size,
            "total_ce_nats": tot_ce, "total_raw_bytes": tot_bytes, "bpb": compute_bpb(tot_ce, tot_bytes),
            "mean_ce": tot_ce / max(tot_tok, 1), "tokens_per_s": tot_tok / elapsed if elapsed > 0 else 0.0,
            "adapt_set": adapt_set, "persistence_mode": "reset", "graph_replays": replays, "padded_chunks": eager,
            "per_doc_ce": {int(i): float(c) for i, c in zip(ids, ce_all.tolist())}}
