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


def _docs(ctx: CalcTypeContext):
    """The cache's documents in source order, cut to the first ``max_docs`` when the pass's
    config sets it (calibration probes and smoke runs)."""
    import itertools
    limit = int(ctx.config.get("max_docs", 0) or 0)
    it = ctx.val_cache.iter_docs()
    return itertools.islice(it, limit) if limit > 0 else it


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
            for doc in _docs(ctx):
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


def _float_tuple(value, name: str) -> tuple[float, ...]:
    if isinstance(value, str):
        value = [p for p in (q.strip() for q in value.split(",")) if p]
    elif not isinstance(value, (list, tuple)):
        value = [value]
    if len(value) == 0:
        raise ValueError(f"{name} must not be empty")
    return tuple(float(v) for v in value)


def _online_mix(nll: torch.Tensor, log_w0: torch.Tensor, eta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """Token-causal exponential-weights mixture of H experts from their target NLLs
    ``[H, T]`` (fp64).  The weights that score token t have seen tokens < t only:
    ``log w_t = log_softmax(log w_0 - eta * sum_{s<t} nll[:, s])`` is one exclusive
    prefix sum, so the whole chunk is three vector ops instead of a per-token loop.
    Returns the mixture's per-token NLL ``[T]`` and the weights after the chunk.  Only
    the experts' target log-probabilities are needed: each expert is a normalised
    distribution and the weights sum to one, so the mixture is normalised too."""
    csum = torch.cumsum(nll, dim=1)
    log_w = torch.log_softmax(log_w0[:, None] - eta * (csum - nll), dim=0)
    mixed = -torch.logsumexp(log_w - nll, dim=0)
    return mixed, torch.log_softmax(log_w0 - eta * csum[:, -1], dim=0)


@register_calc_type("adaptive_carry", requires_source_order=True,
                    description="carried state + token-causal online mixture over recurrent horizon shifts")
def adaptive_carry(ctx: CalcTypeContext) -> CalcTypeResult:
    """Gradient-free test-time adaptation (src/chaoscontrol/eval/calc_types/adaptive_carry.py:299-546):
    the trunk is frozen, each head runs it with ``log_a`` shifted by its ``horizon_shifts``
    entry and carries its own recurrent state across chunks and documents (times ``decay``),
    and an exponential-weights mixer with rate ``online_eta`` combines the heads token by
    token, its weights surviving from one document to the next.  Every head reads the
    episodic store through the packet lane with its own prefix-only cue; after a chunk is
    scored the base head's hidden states with the highest mixed NLL are committed
    (``online_episodic_chunk_tokens`` 256, ``online_episodic_write_tokens_per_chunk`` 16,
    ``online_episodic_gate`` 1.0), and the document's last token enters state and store
    once its score is fixed."""
    from ..eval_stream.state import DeltaModulator
    cfg = ctx.config
    shifts = _float_tuple(cfg.get("horizon_shifts", (-0.5, 0.0, 0.5)), "horizon_shifts")
    eta = float(cfg.get("online_eta", 1.0))
    decay = float(cfg.get("decay", 1.0))
    chunk_tokens = int(cfg.get("online_episodic_chunk_tokens", 256))
    write_k = int(cfg.get("online_episodic_write_tokens_per_chunk", 16))
    gate_value = float(cfg.get("online_episodic_gate", 1.0))
    init_w = cfg.get("online_initial_weights")
    init_w = None if init_w is None else _float_tuple(init_w, "online_initial_weights")
    for ok, msg in ((eta >= 0.0, f"online_eta must be non-negative, got {eta}"),
                    (chunk_tokens >= 1, "online_episodic_chunk_tokens must be >= 1"),
                    (write_k >= 0, "online_episodic_write_tokens_per_chunk must be >= 0"),
                    (gate_value >= 0.0, "online_episodic_gate must be non-negative"),
                    (init_w is None or len(init_w) == len(shifts),
                     "online_initial_weights length does not match horizon_shifts length"),
                    (init_w is None or all(w > 0 for w in init_w),
                     "all initial online weights must be positive")):
        if not ok:
            raise ValueError(msg)
    model, dev = ctx.model, ctx.device
    H = len(shifts)
    base = shifts.index(0.0) if 0.0 in shifts else 0
    w0 = torch.tensor(init_w if init_w is not None else [1.0] * H, dtype=torch.float64, device=dev)
    log_w = (w0 / w0.sum()).log()
    states: list = [None] * H
    no_ctrl = {"enabled": False, "k": 0, "mode": "cosine_survival"}
    can_write = write_k > 0 and callable(getattr(model, "append_memory_from_hidden", None)) and \
        getattr(model, "outer_model", None) is not None
    ce = torch.zeros((), dtype=torch.float64, device=dev)
    head_ce = torch.zeros(H, dtype=torch.float64, device=dev)
    wins = torch.zeros(H, dtype=torch.long, device=dev)
    ntok = nbytes = ndocs = reads = writes = chunks = 0

    def run_heads(x):
        nonlocal reads
        hiddens, finals = [], []
        for h, shift in enumerate(shifts):
            residual, gate, hit, _ = _packet_from_prefix(model, states=states[h], batch_size=int(x.shape[0]),
                                                        gate_value=gate_value, controller=no_ctrl)
            reads += int(hit)
            with DeltaModulator(model, log_a_shift=shift):
                hid, fin = _packet_encode(model, x, states[h], residual, gate)
            hiddens.append(hid)
            finals.append([f * decay for f in fin] if decay != 1.0 else fin)
        return hiddens, finals

    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            for doc in _docs(ctx):
                if doc.token_len < 2:
                    continue
                ids = _doc_tensor(ctx, doc)
                n, pos, last_base = int(ids.shape[1]), 1, None
                while pos < n:
                    end = min(n, pos + chunk_tokens)
                    x, y = ids[:, pos - 1: end - 1], ids[:, pos: end]
                    hiddens, finals = run_heads(x)
                    nll = torch.stack([_token_nll(model, hid, y)[0].double() for hid in hiddens], 0)   # [H, T]
                    mixed, log_w = _online_mix(nll, log_w, eta) if H > 1 else (nll[0], log_w)
                    ce += mixed.sum()
                    head_ce += nll.sum(1)
                    wins += torch.bincount(nll.argmin(0), minlength=H)
                    ntok += int(y.numel())
                    states = finals
                    if can_write:
                        writes += int(bool(model.append_memory_from_hidden(
                            hiddens[base].detach(), score=mixed.float().unsqueeze(0), max_tokens=write_k)))
                    last_base = hiddens[base]
                    chunks += 1
                    pos = end
                hiddens, states = run_heads(ids[:, -1:])
                last_base = hiddens[base]
                if can_write and last_base is not None:
                    writes += int(bool(model.append_memory_from_hidden(last_base.detach(), max_tokens=1)))
                nbytes += int(doc.raw_bytes)
                ndocs += 1
    finally:
        model.train(was_training)
    hyper = {"horizon_shifts": list(shifts), "online_eta": eta, "decay": decay,
             "online_episodic_chunk_tokens": chunk_tokens, "online_episodic_write_tokens_per_chunk": write_k,
             "online_episodic_gate": gate_value,
             "online_initial_weights": None if init_w is None else list(init_w)}
    extra = {"final_online_weights": [float(v) for v in log_w.exp().cpu()] if H > 1 else None,
             "winner_counts": {str(s_): int(c) for s_, c in zip(shifts, wins.cpu())},
             "per_head_loss": {str(s_): float(c) / max(ntok, 1) for s_, c in zip(shifts, head_ce.cpu())},
             "episodic_reads": reads, "episodic_writes": writes, "episodic_chunks": chunks,
             "slot_count_final": _slot_count(model)}
    return _result(float(ce), ntok, nbytes, ndocs, hyper, extra)


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
    """Per-document self-distillation (src/chaoscontrol/eval/calc_types/dreamworld_eval.py:1-444):
    snapshot the weights, roll ``K`` dreams of ``L`` tokens out of the state reached after the
    document's first ``prefix_len`` tokens (``dream_target_mode`` argmax, or softmax sampling at
    ``dream_temperature``), take ``steps`` SGD steps of rate ``lr`` on the teacher-forced CE of the
    dreams, score the document, restore (``per_doc_reset``, default; without it the adaptation
    accumulates over the stream and is undone once at the end)."""
    cfg = ctx.config
    K = int(cfg.get("K", cfg.get("num_dreams", 8)))
    L = int(cfg.get("L", cfg.get("dream_length", 64)))
    lr = float(cfg.get("lr", 1e-3))
    steps = int(cfg.get("steps", 1))
    prefix_tokens = int(cfg.get("prefix_len", cfg.get("prefix_tokens", 16)))
    temperature = float(cfg.get("dream_temperature", 1.0))
    target_mode = str(cfg.get("dream_target_mode", "argmax")).strip().lower()
    if target_mode not in ("argmax", "softmax"):
        raise ValueError(f"dream_target_mode must be 'argmax' or 'softmax', got {target_mode!r}")
    # per_doc_reset=False is the continual mode: adapted weights carry over to later documents
    # (order-sensitive) and are restored once, at the end of the pass
    per_doc_reset = bool(cfg.get("per_doc_reset", True))
    pass_snapshot = None if per_doc_reset else _snapshot(ctx.model)
    gen = torch.Generator().manual_seed(int(cfg.get("seed", 0)))
    model, was_training = ctx.model, ctx.model.training
    ce = 0.0
    ntok = nbytes = ndocs = 0
    try:
        for doc in _docs(ctx):
            if doc.token_len < 2:
                continue
            ids = _doc_tensor(ctx, doc)
            snap = _snapshot(model) if per_doc_reset else None
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
                            if target_mode == "argmax":
                                tok = logits.float().argmax(dim=-1, keepdim=True)
                            else:
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
                if snap is not None:
                    _restore(model, snap)
                model.zero_grad(set_to_none=True)
            ntok += ids.size(1) - 1
            nbytes += doc.raw_bytes
            ndocs += 1
    finally:
        if pass_snapshot is not None:
            _restore(model, pass_snapshot)
        model.train(was_training)
    return _result(ce, ntok, nbytes, ndocs, {"K": K, "L": L, "lr": lr, "steps": steps, "prefix_len": prefix_tokens,
                                              "per_doc_reset": per_doc_reset, "dream_target_mode": target_mode,
                                              "dream_temperature": temperature})


# ---------------------------------------------------------------------------
# packet_online_cache: the submission-facing evaluation
# ---------------------------------------------------------------------------
_CONTROLLER_MODES = ("cosine", "cosine_survival", "cosine_utility_weighted", "dot", "dot_survival")


def _slot_count(model) -> int:
    table = getattr(getattr(model, "outer_model", None), "table", None)
    return 0 if table is None else int(len(table))


def _clear_outer_cache(model) -> None:
    """Retire every active slot (the unseeded variant starts from an empty store)."""
    table = getattr(getattr(model, "outer_model", None), "table", None)
    if table is not None:
        ids = list(table.active_slot_ids())
        if ids:
            table.retire_many(ids, reason="eval_reset")


def _controller_slot_mask(model, *, cue, batch_size: int, topk: int, mode: str):
    """``[B, max physical index + 1]`` mask of the ``topk`` slots a strict-prefix cue
    ranks highest (by cosine or dot product, optionally times slot survival), and how
    many were selected.  The packet read still forms the residual; this only narrows
    which slots may take part (packet_online_cache.py:167-252)."""
    outer = getattr(model, "outer_model", None)
    table = getattr(outer, "table", None)
    if table is None or topk <= 0:
        return None, 0
    idx = [int(i) for i in table.visible_indices()]
    if not idx:
        return None, 0
    M = table.slot_matrix(idx)
    surv = torch.tensor([float(table._survival[i]) if 0 <= i < len(table._survival) else 1.0 for i in idx],
                        device=M.device, dtype=M.dtype)
    if cue is None:
        scores = surv.unsqueeze(0).expand(batch_size, -1)
    else:
        c = cue.detach().reshape(cue.shape[0], -1)
        if c.shape[0] != batch_size:
            c = c[:1].expand(batch_size, -1)
        q = outer.cue_proj(c.to(device=M.device, dtype=outer.cue_proj.weight.dtype)).to(M.dtype)
        if mode.startswith("cosine"):
            scores = F.normalize(q, dim=-1, eps=1e-8) @ F.normalize(M, dim=-1, eps=1e-8).T
        else:
            scores = q @ M.T
        if mode in ("cosine_survival", "dot_survival", "cosine_utility_weighted"):
            scores = scores * surv.unsqueeze(0)
    top = torch.topk(scores, k=min(int(topk), len(idx)), dim=-1, sorted=False).indices
    phys = torch.tensor(idx, device=M.device, dtype=torch.long)[top]
    mask = torch.zeros(batch_size, max(idx) + 1, dtype=torch.bool, device=M.device)
    mask.scatter_(1, phys, True)
    return mask, int(phys.numel())


def _packet_from_prefix(model, *, states, batch_size: int, gate_value: float, controller: dict):
    """Residual + gate read from memory that was committed BEFORE the tokens about to be
    scored; the cue is the last layer's recurrent state at the chunk boundary."""
    outer = getattr(model, "outer_model", None)
    if gate_value <= 0.0 or _slot_count(model) <= 0 or not callable(getattr(outer, "read", None)):
        return None, None, False, 0
    cue = states[-1].detach().reshape(states[-1].shape[0], -1) if states else None
    mask, selected = (None, 0)
    if controller["enabled"]:
        mask, selected = _controller_slot_mask(model, cue=cue, batch_size=batch_size, topk=controller["k"],
                                               mode=controller["mode"])
    kw = {"cue": cue}
    if mask is not None:
        kw["slot_mask"] = mask
    residual = outer.read(int(batch_size), **kw)
    gate = torch.full((int(batch_size),), float(gate_value), device=residual.device, dtype=residual.dtype)
    return residual.detach(), gate, True, selected


def _packet_encode(model, ids, states, residual, gate):
    kw = {"initial_states": states, "return_final_states": True}
    if residual is not None and gate is not None:
        kw.update(episodic_residual=residual, episodic_gate=gate)
    hidden, finals = model.encode(ids.to(torch.int32), memory_mode="packet", **kw)
    return hidden, [f.detach() for f in finals]


def _token_nll(model, hidden, targets):
    from ..cache_utility import chunked_nll_from_hidden
    return chunked_nll_from_hidden(model, hidden, targets)      # fused head on a GPU: no logits tensor


@register_calc_type("packet_online_cache", requires_source_order=True,
                    description="prefix-safe cue + packet-lane score + post-score cache write")
def packet_online_cache(ctx: CalcTypeContext) -> CalcTypeResult:
    """Episodic memory as part of the model, evaluated online
    (src/chaoscontrol/eval/calc_types/packet_online_cache.py:506-778).  Per chunk:
    read a residual with a cue that only knows the strict prefix, score the chunk
    through ``encode(memory_mode="packet")``, and only then commit the chunk's
    highest-NLL hidden states to the store.  Recurrent state is carried across
    chunks AND documents (times ``decay`` at each boundary); the store grows
    monotonically over the source-ordered stream and is never reset per document.

    ``chunk_tokens`` 256, ``write_tokens_per_chunk`` 16, ``gate_value`` 1.0,
    ``decay`` 1.0, ``seeded`` True (False clears the store first), ``max_docs``,
    ``batch_docs`` / ``batch_token_budget`` (score a source-ordered microbatch of
    whole documents before committing its evidence), ``controller_read_enabled`` +
    ``controller_topk_k`` + ``controller_score_mode`` (top-k slot mask before the read).
    A store that grows between the cue read and the score is a hard error."""
    cfg = ctx.config
    chunk_tokens = int(cfg.get("chunk_tokens", 256))
    write_k = int(cfg.get("write_tokens_per_chunk", 16))
    gate_value = float(cfg.get("gate_value", cfg.get("gate", 1.0)))
    decay = float(cfg.get("decay", 1.0))
    seeded = bool(cfg.get("seeded", True))
    max_docs = int(cfg.get("max_docs", 0) or 0)
    batch_docs = int(cfg.get("batch_docs", 1))
    token_budget = int(cfg.get("batch_token_budget", 0) or 0)
    controller = {"enabled": bool(cfg.get("controller_read_enabled", False)),
                  "k": int(cfg.get("controller_topk_k", 16)),
                  "mode": str(cfg.get("controller_score_mode", "cosine_survival")).strip().lower()}
    for ok, msg in ((chunk_tokens >= 1, "chunk_tokens must be >= 1"),
                    (write_k >= 0, "write_tokens_per_chunk must be >= 0"),
                    (gate_value >= 0.0, "gate_value must be non-negative"),
                    (batch_docs >= 1, "batch_docs must be >= 1"),
                    (token_budget >= 0, "batch_token_budget must be >= 0"),
                    (controller["k"] >= 1, "controller_topk_k must be >= 1"),
                    (not controller["enabled"] or controller["mode"] in _CONTROLLER_MODES,
                     f"controller_score_mode must be one of {sorted(_CONTROLLER_MODES)}, "
                     f"got {controller['mode']!r}")):
        if not ok:
            raise ValueError(msg)
    model, vc, dev = ctx.model, ctx.val_cache, ctx.device
    can_write = write_k > 0 and callable(getattr(model, "append_memory_from_hidden", None)) and \
        getattr(model, "outer_model", None) is not None
    if not seeded:
        _clear_outer_cache(model)
    slots0 = _slot_count(model)
    stats = {"episodic_reads": 0, "episodic_writes": 0, "chunks_scored": 0, "controller_reads": 0,
             "controller_selected_slots": 0}
    ce = torch.zeros((), dtype=torch.float64, device=dev)
    ntok = nbytes = ndocs = 0

    def read_packet(states, B):
        residual, gate, hit, sel = _packet_from_prefix(model, states=states, batch_size=B, gate_value=gate_value,
                                                       controller=controller)
        stats["episodic_reads"] += int(hit)
        if sel > 0:
            stats["controller_reads"] += 1
            stats["controller_selected_slots"] += sel
        return residual, gate

    def commit(hidden, score, limit):
        if can_write and limit > 0:
            stats["episodic_writes"] += int(bool(model.append_memory_from_hidden(
                hidden.detach(), score=score.detach(), max_tokens=int(limit))))

    def docs_in_order():
        n = 0
        for doc in vc.iter_docs():
            if max_docs > 0 and n >= max_docs:
                break
            if doc.token_len >= 2:
                n += 1
                yield doc

    was_training = model.training
    model.eval()
    try:
        with torch.no_grad():
            if batch_docs > 1 or token_budget > 0:
                group: list = []
                longest = 0

                def flush(group):
                    nonlocal ce, ntok, nbytes, ndocs
                    arrs = [np.asarray(vc.tokens_for_doc(d)).astype(np.int64) for d in group]
                    lens = [a.shape[0] - 1 for a in arrs]
                    B, L = len(group), max(lens)
                    ids = torch.zeros(B, L, dtype=torch.long, device=dev)
                    tgt = torch.zeros(B, L, dtype=torch.long, device=dev)
                    mask = torch.zeros(B, L, dtype=torch.bool, device=dev)
                    for i, a in enumerate(arrs):
                        t = torch.as_tensor(a, device=dev)
                        ids[i, : lens[i]], tgt[i, : lens[i]], mask[i, : lens[i]] = t[:-1], t[1:], True
                    before = _slot_count(model)
                    residual, gate = read_packet(None, B)
                    hidden, _ = _packet_encode(model, ids, None, residual, gate)
                    nll = _token_nll(model, hidden, tgt)
                    if _slot_count(model) != before:
                        raise RuntimeError("score-before-write violated: the store grew between the batched cue "
                                           "read and the score")
                    ce += (nll.double() * mask).sum()
                    n = int(sum(lens))
                    ntok += n
                    nbytes += int(sum(int(d.raw_bytes) for d in group))
                    ndocs += B
                    stats["chunks_scored"] += 1
                    commit(hidden, nll.masked_fill(~mask, float("-inf")), min(write_k * B, n))

                for doc in docs_in_order():
                    n_in = int(doc.token_len) - 1
                    if group and ((batch_docs > 0 and len(group) + 1 > batch_docs) or
                                  (token_budget > 0 and (len(group) + 1) * max(longest, n_in) > token_budget)):
                        flush(group)
                        group, longest = [], 0
                    group.append(doc)
                    longest = max(longest, n_in)
                if group:
                    flush(group)
            else:
                states = None
                for doc in docs_in_order():
                    ids = _doc_tensor(ctx, doc)
                    n = int(ids.shape[1])
                    pos = 1
                    while pos < n:
                        end = min(n, pos + chunk_tokens)
                        x, y = ids[:, pos - 1: end - 1], ids[:, pos: end]
                        before = _slot_count(model)
                        residual, gate = read_packet(states, 1)
                        hidden, finals = _packet_encode(model, x, states, residual, gate)
                        nll = _token_nll(model, hidden, y)
                        if _slot_count(model) != before:
                            raise RuntimeError("score-before-write violated: the store grew between the cue read "
                                               "and the score")
                        ce += nll.double().sum()
                        ntok += int(y.numel())
                        states = [f * decay for f in finals] if decay != 1.0 else finals
                        commit(hidden, nll, write_k)
                        stats["chunks_scored"] += 1
                        pos = end
                    # the document's last token enters the carried state without being scored again
                    residual, gate = read_packet(states, 1)
                    _, finals = _packet_encode(model, ids[:, -1:], states, residual, gate)
                    states = [f * decay for f in finals] if decay != 1.0 else finals
                    nbytes += int(doc.raw_bytes)
                    ndocs += 1
    finally:
        model.train(was_training)
    hyper = {"chunk_tokens": chunk_tokens, "write_tokens_per_chunk": write_k, "gate_value": gate_value,
             "decay": decay, "seeded": seeded, "max_docs": max_docs, "batch_docs": batch_docs,
             "batch_token_budget": token_budget, "controller_read_enabled": controller["enabled"],
             "controller_topk_k": controller["k"], "controller_score_mode": controller["mode"]}
    stats.update(slot_count_initial=slots0, slot_count_final=_slot_count(model))
    return _result(float(ce), ntok, nbytes, ndocs, hyper, stats)
