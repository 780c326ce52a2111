"""Built-in calc types (cf. src/chaoscontrol/eval/calc_types/*.py):

``score_only_reset``    every document from a zero state, no adaptation;
``carry_state``         the recurrent state flows from one document into the
                        next (optionally decayed);
``adaptive_carry``      online mixture over several carry decays, weights
                        updated multiplicatively from each document's loss;
``dreamworld_eval``     per document: snapshot -> K dream roll-outs from the
                        document's prefix state -> CE backward on the dreams ->
                        SGD step -> score the document -> restore;
``packet_online_cache`` score-first online episodic cache: after a document is
                        scored its hidden states are written to the model's
                        memory, which later documents may read.

``score_only_reset`` and ``carry_state`` run through the batched / chunked
kernel scorer; the others are per-document loops by construction.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from ..scoring import compute_bpb, score_docs
from .registry import CalcTypeContext, CalcTypeResult, register_calc_type


def _doc_tensor(ctx: CalcTypeContext, doc) -> torch.Tensor:
    return torch.as_tensor(np.asarray(ctx.val_cache.tokens_for_doc(doc)).astype(np.int64),
                           device=ctx.device).unsqueeze(0)


def _score(model, ids, states):
    out = model(ids, initial_states=states)
    ce = F.cross_entropy(out["logits"][0, :-1].float(), ids[0, 1:], reduction="sum")
    return ce, out["final_states"]


def _result(ce, ntok, nbytes, ndocs, hyper, extra=None) -> CalcTypeResult:
    return CalcTypeResult(bpb=compute_bpb(ce, nbytes) if nbytes > 0 else 0.0, loss=ce / max(ntok, 1),
                          docs_scored=ndocs, tokens_scored=ntok, raw_bytes=nbytes, hyperparams=hyper,
                          extra=extra or {})


@register_calc_type("score_only_reset", description="zero state per document, no adaptation")
def score_only_reset(ctx: CalcTypeContext) -> CalcTypeResult:
    vc = ctx.val_cache
    max_docs = ctx.config.get("max_docs")
    docs = vc.docs if max_docs is None else vc.docs[: int(max_docs)]
    chunk = int(ctx.config.get("chunk_size", 512))
    tokens = torch.as_tensor(np.asarray(vc.tokens).astype(np.int32), device=ctx.device)
    was_training = ctx.model.training
    try:
        res = score_docs(ctx.model, tokens, np.asarray(docs["token_start"]), np.asarray(docs["token_len"]),
                         chunk_size=chunk, raw_bytes=np.asarray(docs["raw_bytes"]),
                         max_batch_tokens=int(ctx.config.get("max_forward_tokens", 1 << 19)))
    finally:
        ctx.model.train(was_training)
    keep = np.asarray(docs["token_len"]) >= 2
    return _result(res.total_ce, res.total_tokens, int(np.asarray(docs["raw_bytes"])[keep].sum()),
                   int(keep.sum()), {"chunk_size": chunk},
                   {"elapsed_s": res.elapsed_s, "tokens_per_s": res.tokens_per_s})


@register_calc_type("carry_state", requires_source_order=True,
                    description="recurrent state carried across documents")
def carry_state(ctx: CalcTypeContext) -> CalcTypeResult:
    decay = float(ctx.config.get("decay", 1.0))
    model, was_training = ctx.model, ctx.model.training
    model.eval()
    ce = 0.0
    ntok = nbytes = ndocs = 0
    prev = None
    try:
        with torch.no_grad():
            for doc in ctx.val_cache.iter_docs():
                if doc.token_len < 2:
                    continue
                ids = _doc_tensor(ctx, doc)
                c, finals = _score(model, ids, prev)
                ce += float(c)
                ntok += ids.size(1) - 1
                nbytes += doc.raw_bytes
                ndocs += 1
                prev = [s.detach() * decay for s in finals] if decay != 1.0 else [s.detach() for s in finals]
    finally:
        model.train(was_training)
    return _result(ce, ntok, nbytes, ndocs, {"decay": decay})


@register_calc_type("adaptive_carry", requires_source_order=True,
                    description="online mixture over carry decays")
def adaptive_carry(ctx: CalcTypeContext) -> CalcTypeResult:
    decays = tuple(float(d) for d in ctx.config.get("decays", (0.0, 0.5, 1.0)))
    eta = float(ctx.config.get("eta", 1.0))
    if not decays:
        raise ValueError("adaptive_carry needs at least one decay")
    model, was_training = ctx.model, ctx.model.training
    model.eval()
    logw = torch.zeros(len(decays), dtype=torch.float64)
    prev = [None] * len(decays)
    ce = 0.0
    ntok = nbytes = ndocs = 0
    try:
        with torch.no_grad():
            for doc in ctx.val_cache.iter_docs():
                if doc.token_len < 2:
                    continue
                ids = _doc_tensor(ctx, doc)
                tgt = ids[0, 1:]
                logps, finals_all = [], []
                for k in range(len(decays)):
                    out = model(ids, initial_states=prev[k])
                    lp = F.log_softmax(out["logits"][0, :-1].float(), dim=-1).gather(1, tgt[:, None])[:, 0]
                    logps.append(lp.double().cpu())
                    finals_all.append(out["final_states"])
                w = torch.softmax(logw, 0)
                mix = torch.logsumexp(torch.stack(logps, 0) + torch.log(w)[:, None], dim=0)
                ce += float(-mix.sum())
                # multiplicative-weights update from per-expert mean log-likelihood (score first, then update)
                logw = logw + eta * torch.stack([lp.mean() for lp in logps])
                logw = logw - logw.max()
                for k, d in enumerate(decays):
                    prev[k] = None if d == 0.0 else [s.detach() * d for s in finals_all[k]]
                ntok += ids.size(1) - 1
                nbytes += doc.raw_bytes
                ndocs += 1
    finally:
        model.train(was_training)
    return _result(ce, ntok, nbytes, ndocs, {"decays": list(decays), "eta": eta},
                   {"final_weights": [float(x) for x in torch.softmax(logw, 0)]})


def _snapshot(model):
    return {n: p.detach().clone() for n, p in model.named_parameters() if p.requires_grad}


def _restore(model, snap):
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n in snap:
                p.copy_(snap[n])


@register_calc_type("dreamworld_eval", requires_source_order=False, requires_grad=True,
                    description="per-document dream roll-outs, one SGD step, score, restore")
def dreamworld_eval(ctx: CalcTypeContext) -> CalcTypeResult:
    cfg = ctx.config
    K = int(cfg.get("K", cfg.get("num_dreams", 4)))
    L = int(cfg.get("L", cfg.get("dream_length", 16)))
    lr = float(cfg.get("lr", 1e-3))
    steps = int(cfg.get("steps", 1))
    prefix_tokens = int(cfg.get("prefix_tokens", 16))
    temperature = float(cfg.get("dream_temperature", 1.0))
    if not bool(cfg.get("per_doc_reset", True)):
        raise ValueError("per_doc_reset=False is not supported for dreamworld_eval; "
                         "weights are restored after every document")
    gen = torch.Generator().manual_seed(int(cfg.get("seed", 0)))
    model, was_training = ctx.model, ctx.model.training
    ce = 0.0
    ntok = nbytes = ndocs = 0
    try:
        for doc in ctx.val_cache.iter_docs():
            if doc.token_len < 2:
                continue
            ids = _doc_tensor(ctx, doc)
            snap = _snapshot(model)
            try:
                for _ in range(steps):
                    # roll K dreams out of the state reached after the document's first tokens
                    model.eval()
                    with torch.no_grad():
                        pre = ids[:, : max(1, min(prefix_tokens, ids.size(1) - 1))]
                        st = [s.repeat(K, 1) for s in model(pre)["final_states"]]
                        tok = pre[:, -1:].repeat(K, 1)
                        dream = [tok]
                        for _t in range(L):
                            logits, _, st = model.step(tok, st)
                            probs = torch.softmax(logits.float() / max(temperature, 1e-6), -1)
                            tok = torch.multinomial(probs.cpu(), 1, generator=gen).to(ctx.device)
                            dream.append(tok)
                        dream = torch.cat(dream, dim=1)
                    model.train()
                    model.zero_grad(set_to_none=True)
                    out = model(dream)
                    loss = F.cross_entropy(out["logits"][:, :-1].reshape(-1, out["logits"].shape[-1]).float(),
                                           dream[:, 1:].reshape(-1))
                    loss.backward()
                    with torch.no_grad():
                        for p in model.parameters():
                            if p.grad is not None:
                                p.add_(p.grad, alpha=-lr)
                model.eval()
                with torch.no_grad():
                    c, _ = _score(model, ids, None)
                ce += float(c)
            finally:
                _restore(model, snap)
                model.zero_grad(set_to_none=True)
            ntok += ids.size(1) - 1
            nbytes += doc.raw_bytes
            ndocs += 1
    finally:
        model.train(was_training)
    return _result(ce, ntok, nbytes, ndocs, {"K": K, "L": L, "lr": lr, "steps": steps,
                                              "prefix_tokens": prefix_tokens,
                                              "dream_temperature": temperature})


@register_calc_type("packet_online_cache", requires_source_order=True,
                    description="score-first online episodic cache")
def packet_online_cache(ctx: CalcTypeContext) -> CalcTypeResult:
    """Each document is scored with whatever the memory holds from *earlier*
    documents (read through the packet lane), and only afterwards written to
    memory.  Without an outer memory on the model the pass equals
    ``score_only_reset``."""
    model, was_training = ctx.model, ctx.model.training
    write = bool(ctx.config.get("write_after_score", True))
    gate_value = float(ctx.config.get("gate", 1.0))
    model.eval()
    ce = 0.0
    ntok = nbytes = ndocs = writes = 0
    om = getattr(model, "outer_model", None)
    try:
        with torch.no_grad():
            for doc in ctx.val_cache.iter_docs():
                if doc.token_len < 2:
                    continue
                ids = _doc_tensor(ctx, doc)
                if om is not None and hasattr(om, "read") and getattr(om, "num_slots", lambda: 0)() > 0:
                    bias = om.read(1).to(model.embed.weight.dtype)
                    residual = bias.unsqueeze(1).expand(1, ids.size(1), -1)
                    gate = torch.full((1, ids.size(1)), gate_value, device=ctx.device, dtype=residual.dtype)
                    hidden = model.encode(ids, memory_mode="packet", episodic_residual=residual,
                                          episodic_gate=gate)
                else:
                    hidden = model.encode(ids)
                logits = model.lm_head(model.final_norm(hidden))
                ce += float(F.cross_entropy(logits[0, :-1].float(), ids[0, 1:], reduction="sum"))
                if write and om is not None and hasattr(om, "write"):
                    om.write(hidden.detach().mean(dim=1))
                    writes += 1
                ntok += ids.size(1) - 1
                nbytes += doc.raw_bytes
                ndocs += 1
    finally:
        model.train(was_training)
    return _result(ce, ntok, nbytes, ndocs, {"write_after_score": write, "gate": gate_value},
                   {"cache_writes": writes})
