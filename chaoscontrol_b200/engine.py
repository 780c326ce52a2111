"""Training engine for the bare-SSM model on one B200: embedding, trunk, fused
LM head, backward and gradient placement with no autograd graph.

``TrainEngine.step(inputs, targets)`` leaves the averaged-loss gradient of every
parameter in the arena's flat fp32 buffer and returns the detached loss.  It is
what ``train_ssm_step`` runs when the model qualifies
(:meth:`TrainEngine.supported`); all other configurations go through autograd.

Kernel schedule of one step (L layers)::

    embed gather (+row ss)                                   1 launch
    per layer fwd: 2 weight folds, 4 GEMMs, 1 scan           7 launches
    LM head: fold, lse+dX kernel, dW kernel, split-K reduce  5 launches
    per layer bwd: 4 dX GEMMs, 4 dW GEMMs + reduces, 1 scan  ~16 launches
    embedding backward (sort + scatter-add)                  3 launches
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .ops import lm_head as LH
from .ops import trunk as T
from .utils.arena import ParamArena, get_arena


class TrainEngine:
    def __init__(self, model: nn.Module, arena: Optional[ParamArena] = None) -> None:
        self.model = model
        self.arena = arena or get_arena(model) or ParamArena.install(model)
        self._names = []
        for i, _ in enumerate(model.layers):
            pre = f"layers.{i}."
            self._names.append({
                "sel": pre + "core.select_proj.weight", "in": pre + "core.in_proj.weight",
                "gate": pre + "core.gate_proj.weight", "delta": pre + "core.delta_proj.weight",
                "out": pre + "core.out_proj.weight", "fc": pre + "ff.fc.weight",
                "proj": pre + "ff.proj.weight", "wn1": pre + "input_norm.weight",
                "wn2": pre + "ff_norm.weight", "log_a": pre + "core.log_a"})
        self.last_loss_rows: Optional[torch.Tensor] = None
        self.last_hidden: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------
    @staticmethod
    def supported(model: nn.Module) -> bool:
        """Bare-SSM model with bf16 CUDA parameters and shapes the kernels take."""
        fn = getattr(model, "kernel_trunk_supported", None)
        if fn is None or not fn():
            return False
        if getattr(model, "tie_embeddings", False):
            return False
        w = model.lm_head.weight
        return LH.kernel_supported(w.new_empty(1, w.shape[1]), w)

    def _packed(self, i: int):
        a, n = self.arena, self._names[i]
        sel = a.param_view(n["sel"])
        D = sel.shape[0]
        off = a.slots[n["sel"]][0]
        Wp = a.flat_param[off: off + 4 * D * D].view(4 * D, D)
        gWp = a.flat_grad[off: off + 4 * D * D].view(4 * D, D)
        return Wp, gWp

    def _layer_weights(self, i: int) -> T.LayerWeights:
        a, n = self.arena, self._names[i]
        Wp, _ = self._packed(i)
        return T.LayerWeights(Wp=Wp, Wo=a.param_view(n["out"]), Wfc=a.param_view(n["fc"]),
                              Wproj=a.param_view(n["proj"]), wn1=a.param_view(n["wn1"]),
                              wn2=a.param_view(n["wn2"]), log_a=a.param_view(n["log_a"])).prepare()

    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self, inputs: torch.Tensor, targets: torch.Tensor, *, loss_weight: float = 1.0,
             row_weight: Optional[torch.Tensor] = None, reducer=None) -> torch.Tensor:
        """``reducer`` (an :class:`~chaoscontrol_b200.parallel.grad_overlap.OverlappedGradReducer`)
        averages the gradients over the data-parallel ranks bucket by bucket while the rest of
        backward runs; the step then returns with reduced gradients and ``arena.grads_reduced`` set."""
        model, a = self.model, self.arena
        B, Tn = inputs.shape
        R = B * Tn
        V = model.lm_head.weight.shape[0]
        flat_in = inputs.reshape(-1)
        # token sort for the embedding backward: depends on the inputs only
        sort_cache = torch.sort(flat_in.long(), stable=True)
        x, ss = T.embed_fwd(inputs, a.param_view("embed.weight"))
        ws, ctxs = [], []
        for i in range(len(model.layers)):
            w = self._layer_weights(i)
            x, ss, _hT, c = T.layer_forward(x, ss, w, B, Tn, None, save=True)
            ws.append(w)
            ctxs.append(c)
        # LM head
        wnF = a.param_view("final_norm.weight")
        Wlm = a.param_view("lm_head.weight")
        W_f = T.fold_colscale(Wlm, wnF)
        gscale = float(loss_weight) / R
        loss_rows, _lse, dx, part = LH.lm_head_train(x, ss, W_f, targets, gscale=gscale,
                                                     rowweight=row_weight)
        T.splitk_reduce(part, colscale=wnF, W=Wlm, out=a.grad_view("lm_head.weight"),
                        dcol_out=a.grad_view("final_norm.weight"))
        if reducer is not None:
            reducer.bucket_ready(reducer.head_bucket)
        self.last_loss_rows = loss_rows
        self.last_hidden = x                    # [B*T, D] trunk output (pre final norm), for event producers
        if row_weight is None:
            loss = loss_rows.mean()
        else:
            loss = (loss_rows * row_weight).sum() / R
        # trunk backward
        for i in reversed(range(len(model.layers))):
            n = self._names[i]
            _, gWp = self._packed(i)
            outs = {"dWp": gWp, "dWo": a.grad_view(n["out"]), "dWfc": a.grad_view(n["fc"]),
                    "dWproj": a.grad_view(n["proj"]), "dwn1": a.grad_view(n["wn1"]),
                    "dwn2": a.grad_view(n["wn2"]), "dlog_a": a.grad_view(n["log_a"])}
            dx, _ = T.layer_backward(dx, ctxs[i], ws[i], B, Tn, None, outs=outs)
            ctxs[i] = None
            if reducer is not None:
                reducer.bucket_ready(reducer.layer_bucket(i, len(model.layers)))
        T.embed_bwd(inputs, dx, V, sort_cache=sort_cache, out=a.grad_view("embed.weight"))
        a.grads_fresh = True
        if reducer is not None:
            reducer.bucket_ready(reducer.last_bucket)
            reducer.finish()
        return loss
