"""``CareStudentLM``: embedding -> N x (RMSNorm, diagonal-SSM core, residual,
RMSNorm, SiLU feed-forward, residual) -> final RMSNorm -> LM head.

Public surface and state-dict keys match the reference
(src/chaoscontrol/model.py:27-140 for the block, model.py:573-2035 for the LM),
so ``CareStudentLM(**cfg).load_state_dict(ckpt["model"], strict=True)`` works
on reference checkpoints.  On a CUDA device with bf16 parameters the bare-SSM
configuration runs the hand-scheduled kernel trunk (:mod:`..ops.trunk`) behind
one autograd node; every other configuration (CPU, fp32, research add-ons)
runs the plain PyTorch statement of the same math, which is also the oracle
the kernels are tested against.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from ..ops import trunk as T
from .core import CareSSMCore, FeedForward, RMSNorm

__all__ = ["CareSSMBlock", "CareStudentLM", "RMSNorm", "FeedForward", "CareSSMCore", "CareSSMHybridBlock",
           "AttentionControlBlock"]


def __getattr__(name: str):
    # the hybrid / attention blocks live in .attention (which imports this module's blocks): resolve lazily
    if name in ("CareSSMHybridBlock", "AttentionControlBlock"):
        from . import attention
        return getattr(attention, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


class CareSSMBlock(nn.Module):
    """input_norm -> core -> residual -> ff_norm -> FeedForward -> residual."""

    def __init__(self, dim: int, ff_mult: int = 2, *, a_mode: str = "diag", a_full_rank: int = 8,
                 a_full_gamma: float = 0.05, ssm_delta_rank: int = 0, rich_b_mode: str = "none",
                 rich_b_bottleneck: int = 32, rich_b_num_subnets: int = 4,
                 rich_b_settling_steps: int = 2) -> None:
        super().__init__()
        self.input_norm = RMSNorm(dim)
        self.ff_norm = RMSNorm(dim)
        self.ff = FeedForward(dim, ff_mult)
        self.core = CareSSMCore(dim, a_mode=a_mode, a_full_rank=a_full_rank,
                                a_full_gamma=a_full_gamma, delta_rank=ssm_delta_rank)
        if rich_b_mode == "none":
            self.rich_b: Optional[nn.Module] = None
        elif rich_b_mode == "nn":
            from .routing import RichBNN
            self.rich_b = RichBNN(dim, bottleneck=rich_b_bottleneck)
        elif rich_b_mode in ("hub", "assembly", "hybrid"):
            from .routing import DistributedB
            self.rich_b = DistributedB(dim, num_subnets=rich_b_num_subnets,
                                       bottleneck=rich_b_bottleneck, topology=rich_b_mode,
                                       settling_steps=rich_b_settling_steps)
        else:
            raise ValueError(f"unsupported rich_b_mode: {rich_b_mode}")

    def step(self, x: torch.Tensor, state: torch.Tensor):
        y, new_state = self.core.step(self.input_norm(x), state, rich_b=self.rich_b)
        x = x + y
        x = x + self.ff(self.ff_norm(x))
        return x, new_state

    def forward(self, x: torch.Tensor, *, return_jacobian_stats: bool = False,
                initial_state: Optional[torch.Tensor] = None, return_final_state: bool = False):
        result = self.core(self.input_norm(x), rich_b=self.rich_b,
                           return_jacobian_stats=return_jacobian_stats,
                           initial_state=initial_state, return_final_state=return_final_state)
        stats = final_state = None
        if return_jacobian_stats and return_final_state:
            y, stats, final_state = result
        elif return_jacobian_stats:
            y, stats = result
        elif return_final_state:
            y, final_state = result
        else:
            y = result
        x = x + y
        x = x + self.ff(self.ff_norm(x))
        if return_jacobian_stats and return_final_state:
            return x, stats, final_state
        if return_jacobian_stats:
            return x, stats
        if return_final_state:
            return x, final_state
        return x


# ---------------------------------------------------------------------------
# kernel trunk behind one autograd node
# ---------------------------------------------------------------------------
_PER_LAYER = 10  # select, in, gate, delta, out, fc, proj, input_norm, ff_norm, log_a


def _layer_weights(params: tuple, i: int) -> T.LayerWeights:
    sel, inp, gate, delta, out, fc, proj, wn1, wn2, log_a = params[i * _PER_LAYER:(i + 1) * _PER_LAYER]
    # The four [D, D] projections are consumed as one packed [4D, D] weight.
    base = sel.data_ptr()
    step = sel.numel() * sel.element_size()
    packed = (inp.data_ptr() == base + step and gate.data_ptr() == base + 2 * step and
              delta.data_ptr() == base + 3 * step and sel.is_contiguous())
    if packed:
        Wp = torch.as_strided(sel, (4 * sel.shape[0], sel.shape[1]), (sel.shape[1], 1))
    else:
        Wp = torch.cat((sel, inp, gate, delta), dim=0)
    return T.LayerWeights(Wp=Wp, Wo=out, Wfc=fc, Wproj=proj, wn1=wn1, wn2=wn2, log_a=log_a).prepare()


class _TrunkFn(torch.autograd.Function):
    """tokens -> (hidden, final row sums of squares, final states) through the
    kernel trunk; backward replays the layers in reverse with saved activations."""

    @staticmethod
    def forward(ctx, tokens, h0_stack, want_grad, embed_w, *params):
        B, Tn = tokens.shape
        L = len(params) // _PER_LAYER
        x, ss = T.embed_fwd(tokens, embed_w)
        ws, ctxs, hTs = [], [], []
        for i in range(L):
            w = _layer_weights(params, i)
            h0 = h0_stack[i].float().contiguous() if h0_stack is not None else None
            x, ss, hT, c = T.layer_forward(x, ss, w, B, Tn, h0, save=want_grad)
            ws.append(w)
            ctxs.append(c)
            hTs.append(hT)
        ctx.ws, ctxs_, ctx.tokens = ws, ctxs, tokens
        ctx.ctxs = ctxs_
        ctx.shape = (B, Tn, embed_w.shape[0])
        ctx.has_h0 = h0_stack is not None
        ctx.mark_non_differentiable(ss)
        # unused outputs arrive in backward as None instead of zero tensors: no value has to be read
        # back to find out whether the final states carry a gradient
        ctx.set_materialize_grads(False)
        return x.view(B, Tn, -1), ss, torch.stack(hTs, dim=0)

    @staticmethod
    def backward(ctx, dhidden, _dss, dhT_stack):
        B, Tn, V = ctx.shape
        if dhidden is None:
            w0 = ctx.ws[0].Wo
            dhidden = torch.zeros(B * Tn, w0.shape[0], dtype=w0.dtype, device=w0.device)
        dx = dhidden.reshape(B * Tn, -1).contiguous()
        grads: list = []
        L = len(ctx.ws)
        dh0s = []
        use_dhT = dhT_stack is not None
        for i in reversed(range(L)):
            w, c = ctx.ws[i], ctx.ctxs[i]
            dhT = dhT_stack[i].float().contiguous() if use_dhT else None
            dx, g = T.layer_backward(dx, c, w, B, Tn, dhT, want_dh0=ctx.has_h0)
            D = w.Wo.shape[0]
            pd = w.Wo.dtype
            dsel, dinp, dgate, ddelta = (t.to(pd) for t in g.dWp.split(D, dim=0))
            grads = [dsel, dinp, dgate, ddelta, g.dWo.to(pd), g.dWfc.to(pd), g.dWproj.to(pd),
                     g.dwn1.to(w.wn1.dtype), g.dwn2.to(w.wn2.dtype),
                     g.dlog_a.to(w.log_a.dtype)] + grads
            dh0s.append(g.dh0)
            ctx.ctxs[i] = None
        dE = T.embed_bwd(ctx.tokens, dx, V).to(ctx.ws[0].Wo.dtype)
        dh0 = torch.stack(list(reversed(dh0s)), 0) if ctx.has_h0 else None
        return (None, dh0, None, dE, *grads)


class CareStudentLM(nn.Module):
    """Diagonal-SSM language model.  See the module docstring for the layout."""

    def __init__(self, *, vocab_size: int, dim: int, num_layers: int, ff_mult: int = 2,
                 block_type: str = "ssm", attention_num_heads: int = 8,
                 attention_dropout: float = 0.0, a_mode: str = "diag", a_full_rank: int = 8,
                 a_full_gamma: float = 0.05, ssm_delta_rank: int = 0, rich_b_mode: str = "none",
                 rich_b_bottleneck: int = 32, rich_b_num_subnets: int = 4,
                 rich_b_settling_steps: int = 2, outer_model_dim: int = 0,
                 consolidation_mode: str = "symmetric", consolidation_ema_decay: float = 0.99,
                 consolidation_trigger: str = "immediate", consolidation_window: int = 8,
                 outer_model_type: str = "single", outer_max_slots: int = 64,
                 outer_compress_ratio: int = 2, wernicke_enabled: bool = False,
                 wernicke_k_max: int = 16, wernicke_window: int = 8, wernicke_router: str = "vq",
                 wernicke_balance_weight: float = 0.01, wernicke_expert_dim: int = 0,
                 wernicke_layers: int = 1, wernicke_k_max_fine: int = 16,
                 buffer_mode: str = "legacy", retrieval_mode: str = "softmax_all",
                 retrieval_k: int = 8, bucket_prototypes: bool = False, prototype_dim: int = 64,
                 prototype_update_rate: float = 0.1, semantic_tier_bases: int = 0,
                 semantic_tier_update_rate: float = 0.01, typed_storage: bool = False,
                 typed_consolidation: bool = False, compression_consequence: bool = False,
                 cue_projection: bool = True, dynamic_crit_per_layer: bool = False,
                 compression_selection: str = "survival", posterior_mode: str = "none",
                 posterior_lr: float = 0.01, residual_cache_k: int = 4, local_attn_window: int = 0,
                 local_attn_heads: int = 1, local_attn_dim: int = 64, local_attn_topk: int = 0,
                 local_attn_topk_random: bool = False,
                 depth_recurrence_shared_layers: Optional[list[int]] = None,
                 depth_recurrence_count: int = 1, activation_checkpoint: bool = False,
                 tie_embeddings: bool = False, log_a_init: str = "zeros") -> None:
        super().__init__()
        self.vocab_size = vocab_size
        self.dim = dim
        self.activation_checkpoint = bool(activation_checkpoint)
        self.local_attn_window = local_attn_window
        self.embed = nn.Embedding(vocab_size, dim)
        self.buffer_mode = buffer_mode
        self.retrieval_mode = retrieval_mode
        self.retrieval_k = retrieval_k
        self.block_type = block_type
        self.wernicke_balance_weight = wernicke_balance_weight

        self.wernicke: Optional[nn.Module] = None
        if wernicke_enabled:
            from .wernicke import HierarchicalWernicke, WernickeLayer
            expert = wernicke_expert_dim if wernicke_expert_dim > 0 else None
            if wernicke_layers >= 2:
                self.wernicke = HierarchicalWernicke(
                    dim=dim, k_coarse=wernicke_k_max, k_fine=wernicke_k_max_fine,
                    window=wernicke_window, router_type=wernicke_router,
                    balance_weight=wernicke_balance_weight, expert_dim=expert)
            else:
                self.wernicke = WernickeLayer(
                    dim, k_max=wernicke_k_max, window=wernicke_window, router_type=wernicke_router,
                    balance_weight=wernicke_balance_weight, expert_dim=expert)

        if block_type == "attention":
            from .attention import AttentionControlBlock
            self.layers = nn.ModuleList([
                AttentionControlBlock(dim, ff_mult, num_heads=attention_num_heads,
                                      attn_dropout=attention_dropout)
                for _ in range(num_layers)])
        elif block_type == "ssm":
            kw = dict(a_mode=a_mode, a_full_rank=a_full_rank, a_full_gamma=a_full_gamma,
                      ssm_delta_rank=ssm_delta_rank, rich_b_mode=rich_b_mode,
                      rich_b_bottleneck=rich_b_bottleneck, rich_b_num_subnets=rich_b_num_subnets,
                      rich_b_settling_steps=rich_b_settling_steps)
            if local_attn_window > 0:
                from .attention import CareSSMHybridBlock
                blocks: list[nn.Module] = [CareSSMBlock(dim, ff_mult, **kw)
                                           for _ in range(num_layers - 1)]
                blocks.append(CareSSMHybridBlock(
                    dim, ff_mult, a_mode=a_mode, a_full_rank=a_full_rank, a_full_gamma=a_full_gamma,
                    ssm_delta_rank=ssm_delta_rank, local_attn_window=local_attn_window,
                    local_attn_heads=local_attn_heads, local_attn_dim=local_attn_dim,
                    local_attn_topk=local_attn_topk, local_attn_topk_random=local_attn_topk_random))
                self.layers = nn.ModuleList(blocks)
            else:
                self.layers = nn.ModuleList([CareSSMBlock(dim, ff_mult, **kw)
                                             for _ in range(num_layers)])
        else:
            raise ValueError(
                f"unsupported block_type: {block_type!r} (expected 'ssm' or 'attention')")

        shared = list(depth_recurrence_shared_layers or [])
        self.depth_recurrence_shared_layers: list[int] = shared
        self.depth_recurrence_count = int(depth_recurrence_count)
        if self.depth_recurrence_count < 1:
            raise ValueError(f"depth_recurrence_count must be >= 1, got {self.depth_recurrence_count}")
        if shared:
            if any(not (0 <= i < len(self.layers)) for i in shared):
                raise ValueError(f"depth_recurrence_shared_layers indices out of range "
                                 f"[0, {len(self.layers)}): {shared}")
            if sorted(shared) != shared:
                raise ValueError(f"depth_recurrence_shared_layers must be sorted ascending: {shared}")
            if any(shared[i] + 1 != shared[i + 1] for i in range(len(shared) - 1)):
                raise ValueError(f"depth_recurrence_shared_layers must be contiguous: {shared}")
            a, b = shared[0], shared[-1]
            self._virtual_layer_indices = (list(range(0, a)) + shared * self.depth_recurrence_count +
                                           list(range(b + 1, len(self.layers))))
        else:
            self._virtual_layer_indices = list(range(len(self.layers)))

        self.final_norm = RMSNorm(dim)
        self.lm_head = nn.Linear(dim, vocab_size, bias=False)
        self.tie_embeddings = bool(tie_embeddings)
        if self.tie_embeddings:
            self.lm_head.weight = self.embed.weight
        if log_a_init == "log_uniform":
            # option asked for by some configs: diag A spread uniformly in log space over [-4, 0]
            for blk in self.layers:
                core = getattr(blk, "core", None)
                if core is not None and hasattr(core, "log_a"):
                    with torch.no_grad():
                        core.log_a.uniform_(-4.0, 0.0)
        elif log_a_init != "zeros":
            raise ValueError(f"log_a_init must be 'zeros' or 'log_uniform', got {log_a_init!r}")

        self.outer_model_type = outer_model_type
        self.outer_model: Optional[nn.Module] = None
        if outer_model_dim > 0:
            from .memory import MultiSlotOuterModel, OuterModel
            common = dict(consolidation_mode=consolidation_mode, ema_decay=consolidation_ema_decay,
                          trigger=consolidation_trigger, trigger_window=consolidation_window)
            if outer_model_type == "multislot":
                self.outer_model = MultiSlotOuterModel(
                    dim, outer_dim=outer_model_dim, max_slots=outer_max_slots,
                    compress_ratio=outer_compress_ratio,
                    compression_selection=compression_selection, **common)
            else:
                self.outer_model = OuterModel(dim, outer_dim=outer_model_dim, **common)
        self.semantic_tier: Optional[nn.Module] = None
        if semantic_tier_bases > 0:
            from .memory import SemanticTier
            self.semantic_tier = SemanticTier(dim, num_bases=semantic_tier_bases,
                                              update_rate=semantic_tier_update_rate)
        self.bucket_prototypes_module: Optional[nn.Module] = None
        if bucket_prototypes and outer_model_dim > 0:
            from .memory import BucketPrototypes
            total_k = wernicke_k_max * wernicke_k_max_fine if wernicke_layers >= 2 else wernicke_k_max
            self.bucket_prototypes_module = BucketPrototypes(
                k_max=total_k, prototype_dim=prototype_dim, model_dim=dim,
                update_rate=prototype_update_rate)
        self.posterior: Optional[nn.Module] = None
        self.posterior_mode = posterior_mode
        if posterior_mode != "none":
            from .posterior import BucketDelta, GlobalDelta, ResidualCache
            total_buckets = (self.wernicke.total_buckets if hasattr(self.wernicke, "total_buckets")
                             else (self.wernicke.k_max if self.wernicke is not None else wernicke_k_max))
            if posterior_mode == "global_delta":
                self.posterior = GlobalDelta(dim, lr=posterior_lr)
            elif posterior_mode == "bucket_delta":
                self.posterior = BucketDelta(k_max=total_buckets, model_dim=dim, lr=posterior_lr)
            elif posterior_mode == "residual_cache":
                self.posterior = ResidualCache(model_dim=dim, k=residual_cache_k)
        self.typed_storage = typed_storage
        self.typed_consolidation = typed_consolidation
        self.compression_consequence = compression_consequence
        self.cue_projection = cue_projection
        self.dynamic_crit_per_layer = dynamic_crit_per_layer

    # -- state -----------------------------------------------------------
    def init_state(self, batch_size: int) -> list[torch.Tensor]:
        w = self.embed.weight
        return [torch.zeros(batch_size, self.dim, device=w.device, dtype=w.dtype)
                for _ in range(len(self.layers))]

    def init_kv_caches(self):
        return [layer._init_kv_cache() if hasattr(layer, "_init_kv_cache") else None
                for layer in self.layers]

    def artifact_bytes(self) -> int:
        return sum(p.numel() for p in self.parameters()) * 2

    # -- fast-path gate --------------------------------------------------
    def _is_bare_ssm(self) -> bool:
        return (self.block_type == "ssm" and self.wernicke is None and self.outer_model is None and
                self.semantic_tier is None and self.posterior is None and
                self.local_attn_window == 0 and
                all(isinstance(b, CareSSMBlock) and b.rich_b is None and b.core.a_mode == "diag" and
                    b.core.delta_rank == 0 for b in self.layers))

    def kernel_trunk_supported(self) -> bool:
        """True when ``encode`` runs the hand-scheduled sm_100a trunk."""
        w = self.embed.weight
        if not (w.is_cuda and w.dtype == torch.bfloat16 and self._is_bare_ssm()):
            return False
        if self._virtual_layer_indices != list(range(len(self.layers))):
            return False
        if self.dim % 64 != 0 or self.dim > 512:   # the RMSNorm-backward GEMM tile spans <= 512 columns
            return False
        if any(p.dtype != torch.bfloat16 for p in self.parameters()):
            return False
        # training hooks (ScOpt / TTT instrumentation) need the module-by-module path
        for blk in self.layers:
            for m in (blk.core.in_proj, blk.core.select_proj, blk.core.gate_proj, blk.core.delta_proj,
                      blk.core.out_proj, blk.ff.fc, blk.ff.proj):
                if type(m) is not nn.Linear:      # promoted (fp8) linears run module by module
                    return False
                if m._forward_hooks or m._forward_pre_hooks or m._backward_hooks:
                    return False
            if blk.core._capture_states_enabled:
                return False
        return True

    def _trunk_params(self) -> list[torch.Tensor]:
        ps: list[torch.Tensor] = []
        for blk in self.layers:
            c = blk.core
            ps += [c.select_proj.weight, c.in_proj.weight, c.gate_proj.weight, c.delta_proj.weight,
                   c.out_proj.weight, blk.ff.fc.weight, blk.ff.proj.weight, blk.input_norm.weight,
                   blk.ff_norm.weight, c.log_a]
        return ps

    def encode_with_stats(self, input_ids: torch.Tensor, *,
                          initial_states: Optional[list[torch.Tensor]] = None):
        """Kernel trunk only: ``(hidden, row_ss, final_states)`` where ``row_ss``
        is the per-token sum of squares of ``hidden`` that the fused LM head
        turns into the final RMSNorm scale without re-reading ``hidden``."""
        h0 = None
        if initial_states is not None:
            h0 = torch.stack([s.float() for s in initial_states], 0)
        want_grad = torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters())
        hidden, ss, hT = _TrunkFn.apply(input_ids, h0, want_grad, self.embed.weight,
                                        *self._trunk_params())
        return hidden, ss, [hT[i] for i in range(hT.shape[0])]

    # -- encoder ---------------------------------------------------------
    def encode(self, input_ids: torch.Tensor, *, memory_mode: str = "packet",
               cache_read_cutoff: Optional[int] = None,
               episodic_residual: Optional[torch.Tensor] = None,
               episodic_gate: Optional[torch.Tensor] = None,
               memory_slot_mask: Optional[torch.Tensor] = None,
               memory_slot_override_index: Optional[int] = None,
               memory_slot_override_values: Optional[torch.Tensor] = None,
               return_memory_meta: bool = False,
               initial_states: Optional[list[torch.Tensor]] = None,
               return_final_states: bool = False):
        """Everything before the LM head; returns ``hidden`` ``(batch, seq, dim)``
        (and the per-layer final states when asked)."""
        if memory_mode not in {"off", "force_on", "packet"}:
            raise ValueError("memory_mode must be one of 'off', 'force_on', or 'packet', "
                             f"got {memory_mode!r}")
        if memory_mode != "packet" and (episodic_residual is not None or episodic_gate is not None):
            raise ValueError("episodic_residual/episodic_gate are only valid with memory_mode='packet'")
        if memory_mode == "packet" and ((episodic_residual is None) != (episodic_gate is None)):
            raise ValueError("memory_mode='packet' requires both episodic_residual and "
                             "episodic_gate, or neither for a zero-residual no-op")
        if initial_states is not None and len(initial_states) != len(self.layers):
            raise ValueError(f"initial_states length {len(initial_states)} does not match "
                             f"num_layers {len(self.layers)}")

        plain = episodic_residual is None and not return_memory_meta
        if plain and self.kernel_trunk_supported() and not self.activation_checkpoint:
            hidden, _ss, finals = self.encode_with_stats(input_ids, initial_states=initial_states)
            return (hidden, finals) if return_final_states else hidden

        x = self.embed(input_ids)
        bucket_ids = None
        if self.wernicke is not None:
            x, bucket_ids, _balance = self.wernicke(x)
        gate: Optional[torch.Tensor] = None
        residual: Optional[torch.Tensor] = None
        if memory_mode == "packet" and episodic_residual is not None:
            gate = self._packet_gate(episodic_gate, x)
            residual = self._packet_residual(episodic_residual, x)
            x = torch.addcmul(x, residual, gate.unsqueeze(-1))
        reads_memory = memory_mode == "force_on"
        self._stash_outer_cue(x, reads_memory)
        if reads_memory:
            for bias in self._pre_recurrence_biases(
                    x, bucket_ids, cache_read_cutoff=cache_read_cutoff, slot_mask=memory_slot_mask,
                    override_index=memory_slot_override_index,
                    override_values=memory_slot_override_values):
                x = x + bias
                residual = bias if residual is None else residual + bias
        x, finals, _ = self._run_layers(x, initial_states, want_stats=False)
        if reads_memory:
            bias = self._posterior_bias(x, bucket_ids)
            if bias is not None:
                x = x + bias
                residual = bias if residual is None else residual + bias
        if reads_memory and residual is not None and gate is None:
            gate = torch.ones(x.shape[:2], device=x.device, dtype=x.dtype)
        if return_memory_meta:
            out: dict[str, Any] = {"hidden": x, "memory_meta": {
                "memory_mode": memory_mode, "cache_read_cutoff": cache_read_cutoff,
                "memory_gate": gate, "memory_residual": residual}}
            if return_final_states:
                out["final_states"] = finals
            return out
        return (x, finals) if return_final_states else x

    # -- memory injection ------------------------------------------------
    @staticmethod
    def _packet_gate(gate: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
        """Packet gate ``(B,)``, ``(B, 1)`` or ``(B, T)`` broadcast to ``(B, T)``."""
        g = gate.to(device=ref.device, dtype=ref.dtype)
        B, T = ref.shape[:2]
        bad = ValueError(f"episodic_gate shape {tuple(g.shape)} cannot gate hidden shape {(B, T)}")
        if g.dim() == 1:
            if g.shape[0] != B:
                raise bad
            return g[:, None].expand(B, T)
        if g.dim() == 2:
            if g.shape[0] != B or g.shape[1] not in (1, T):
                raise bad
            return g.expand(B, T)
        raise ValueError("episodic_gate must have shape (B,), (B, 1), or (B, T)")

    @staticmethod
    def _packet_residual(residual: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
        """Compact packet residual ``(B, D)`` or ``(B, 1, D)`` as ``(B, 1, D)``."""
        r = residual.to(device=ref.device, dtype=ref.dtype)
        B, _T, D = ref.shape
        if r.dim() == 2 and r.shape == (B, D):
            return r.unsqueeze(1)
        if r.dim() == 3 and r.shape[0] == B and r.shape[2] == D:
            if r.shape[1] != 1:
                raise ValueError("episodic_residual packets must be compact with shape "
                                 f"(B, D) or (B, 1, D); got {tuple(r.shape)}")
            return r
        if r.dim() in (2, 3):
            raise ValueError(f"episodic_residual shape {tuple(r.shape)} cannot feed hidden shape "
                             f"{tuple(ref.shape)}")
        raise ValueError("episodic_residual must have compact shape (B, D) or (B, 1, D)")

    def _stash_outer_cue(self, x: torch.Tensor, reads_memory: bool) -> None:
        """Maintenance probes compare a cheap saliency map against the full
        read, so the cue that read used is kept (detached) on the module."""
        from .memory import MultiSlotOuterModel
        keep = reads_memory and isinstance(self.outer_model, MultiSlotOuterModel) and self.cue_projection
        self._last_outer_cue = x.detach().mean(dim=1) if keep else None

    def _per_bucket(self, x: torch.Tensor, per_sample: torch.Tensor, read_fn) -> torch.Tensor:
        """``(B, 1, D)`` bias assembled from one read per distinct dominant bucket."""
        out = torch.zeros(x.size(0), 1, x.size(2), device=x.device, dtype=x.dtype)
        for b_id in per_sample.unique().tolist():
            rows = per_sample == b_id
            out[rows] = read_fn(int(b_id), rows).unsqueeze(1).to(dtype=x.dtype)
        return out

    def _pre_recurrence_biases(self, x: torch.Tensor, bucket_ids: Optional[torch.Tensor], *,
                               cache_read_cutoff: Optional[int] = None,
                               slot_mask: Optional[torch.Tensor] = None,
                               override_index: Optional[int] = None,
                               override_values: Optional[torch.Tensor] = None) -> list[torch.Tensor]:
        """Full-strength memory reads added before the recurrence, each ``(B, 1, D)``:
        the episodic store (per dominant bucket in ``append_only`` mode, whole-store
        otherwise), bucket prototypes, then the semantic tier
        (reference src/chaoscontrol/model.py:1661-1722)."""
        from .memory import MultiSlotOuterModel
        B = x.size(0)
        om = self.outer_model
        biases: list[torch.Tensor] = []
        if om is not None and self.buffer_mode == "append_only":
            per_sample = (bucket_ids.mode(dim=1).values if bucket_ids is not None
                          else torch.zeros(B, dtype=torch.long, device=x.device))
            if isinstance(om, MultiSlotOuterModel) and len(om.table):
                want_cue = self.retrieval_mode in ("bucket_topk", "softmax_all")

                def _read(b_id: int, rows: torch.Tensor) -> torch.Tensor:
                    cue = None
                    if want_cue:
                        cue = om.cue_proj(x[rows].detach().mean(dim=1).to(dtype=om.cue_proj.weight.dtype))
                    return om.read_bucket(
                        int(rows.sum()), bucket_id=b_id, mode=self.retrieval_mode, k=self.retrieval_k,
                        cue=cue, read_cutoff=cache_read_cutoff,
                        slot_mask=None if slot_mask is None else slot_mask[rows],
                        slot_override_index=override_index,
                        slot_override_values=None if override_values is None else override_values[rows])
                biases.append(self._per_bucket(x, per_sample, _read))
            if self.bucket_prototypes_module is not None and bucket_ids is not None:
                biases.append(self._per_bucket(
                    x, per_sample,
                    lambda b_id, rows: self.bucket_prototypes_module.read(int(rows.sum()), b_id)))
        elif om is not None:
            if isinstance(om, MultiSlotOuterModel):
                cue = x.detach().mean(dim=1) if self.cue_projection else None
                read = om.read(B, cue=cue, read_cutoff=cache_read_cutoff, slot_mask=slot_mask,
                               slot_override_index=override_index, slot_override_values=override_values)
            else:
                read = om.read(B)
            biases.append(read.unsqueeze(1).to(dtype=x.dtype))
        if self.semantic_tier is not None:
            biases.append(self.semantic_tier.read(B).unsqueeze(1).to(dtype=x.dtype))
        return biases

    def _posterior_bias(self, x: torch.Tensor, bucket_ids: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Error-driven correction added after the recurrence, ``(B, 1, D)`` or ``None``."""
        if self.posterior is None:
            return None
        from .posterior import BucketDelta, GlobalDelta, ResidualCache
        if isinstance(self.posterior, GlobalDelta):
            return self.posterior.read(x.size(0)).unsqueeze(1).to(x.dtype)
        if isinstance(self.posterior, BucketDelta) and bucket_ids is not None:
            per = bucket_ids.mode(dim=1).values.tolist()
            bias = torch.cat([self.posterior.read(bucket_id=int(b), batch_size=1) for b in per], dim=0)
            return bias.unsqueeze(1).to(x.dtype)
        if isinstance(self.posterior, ResidualCache):
            return self.posterior.read(x.detach().mean(dim=1)).unsqueeze(1).to(x.dtype)
        return None

    _PACKET_FORWARD_MODULE_ATTRS: tuple[str, ...] = (
        "embed", "wernicke", "outer_model", "semantic_tier", "bucket_prototypes_module")

    def packet_forward_state_keys(self) -> set[str]:
        """Tensor state-dict keys that ``build_episodic_packet`` reads: what a
        packet-serving rank needs from a trunk snapshot (no SSM layers, no head)."""
        keys: set[str] = set()
        for attr in self._PACKET_FORWARD_MODULE_ATTRS:
            mod = getattr(self, attr, None)
            if isinstance(mod, nn.Module):
                keys.update(f"{attr}.{k}" for k, v in mod.state_dict().items() if torch.is_tensor(v))
        return keys

    @torch.no_grad()
    def build_episodic_packet(self, input_ids: torch.Tensor, *,
                              cache_read_cutoff: Optional[int] = None) -> dict[str, Any]:
        """The pre-recurrence memory bias that ``memory_mode='force_on'`` would
        inject, as a compact packet, without running the recurrence or the head
        (reference model.py:1166-1301).  A serving proposal, not an oracle label."""
        x = self.embed(input_ids)
        bucket_ids = None
        if self.wernicke is not None:
            x, bucket_ids, _ = self.wernicke(x)
        self._stash_outer_cue(x, True)
        biases = self._pre_recurrence_biases(x, bucket_ids, cache_read_cutoff=cache_read_cutoff)
        B, T, D = x.shape
        residual = torch.zeros(B, 1, D, device=x.device, dtype=x.dtype)
        for bias in biases:
            residual.add_(bias)
        gate = torch.ones(B, T, device=x.device, dtype=x.dtype) if biases else \
            torch.zeros(B, T, device=x.device, dtype=x.dtype)
        return {
            "memory_residual": residual.contiguous(),
            "memory_gate": gate,
            "packet_source_hidden": x.detach(),
            "packet_source_bucket_ids": None if bucket_ids is None else bucket_ids.detach(),
            "packet_write_score": x.detach().float().square().mean(dim=-1),
            "packet_source_count": len(biases),
        }

    def encode_paired_for_score(self, input_ids: torch.Tensor, *,
                                cache_read_cutoff: Optional[int] = None):
        """``(h_off, h_mem, memory_meta)``: memory-off and force-on streams of the
        same batch, stacked through the recurrence in ONE pass over the layers
        (reference model.py:1303-1455)."""
        x_base = self.embed(input_ids)
        bucket_ids = None
        if self.wernicke is not None:
            x_base, bucket_ids, _ = self.wernicke(x_base)
        self._stash_outer_cue(x_base, True)
        residual: Optional[torch.Tensor] = None
        x_mem = x_base
        for bias in self._pre_recurrence_biases(x_base, bucket_ids, cache_read_cutoff=cache_read_cutoff):
            x_mem = x_mem + bias
            residual = bias if residual is None else residual + bias
        pair, _f, _s = self._run_layers(torch.cat([x_base, x_mem], dim=0), None, want_stats=False)
        h_off, h_mem = pair.chunk(2, dim=0)
        bias = self._posterior_bias(h_mem, bucket_ids)
        if bias is not None:
            h_mem = h_mem + bias
            residual = bias if residual is None else residual + bias
        gate = None if residual is None else torch.ones(h_mem.shape[:2], device=h_mem.device, dtype=h_mem.dtype)
        return h_off, h_mem, {"memory_mode": "force_on", "cache_read_cutoff": cache_read_cutoff,
                              "memory_gate": gate, "memory_residual": residual}

    def _run_layers(self, x, initial_states, want_stats: bool):
        finals: list[Optional[torch.Tensor]] = [None] * len(self.layers)
        cur = list(initial_states) if initial_states is not None else [None] * len(self.layers)
        all_stats = []
        for idx in self._virtual_layer_indices:
            layer = self.layers[idx]
            kw = dict(initial_state=cur[idx], return_final_state=True)
            if want_stats:
                kw["return_jacobian_stats"] = True
            if self.activation_checkpoint and self.training and torch.is_grad_enabled():
                res = _checkpoint(lambda t, _l=layer, _kw=kw: _l(t, **_kw), x, use_reentrant=False)
            else:
                res = layer(x, **kw)
            if want_stats:
                x, stats, fs = res
                all_stats.append(stats)
            else:
                x, fs = res
            finals[idx] = fs
            cur[idx] = fs
        return x, finals, all_stats

    # -- full forward ----------------------------------------------------
    def forward(self, input_ids: torch.Tensor, *, return_jacobian_stats: bool = False,
                memory_write_mode: str = "none",
                initial_states: Optional[list[torch.Tensor]] = None) -> dict[str, Any]:
        """Returns ``{"logits", "hidden", "final_states"[, "balance_loss", "bucket_ids",
        "jacobian_stats"]}``."""
        if initial_states is not None and len(initial_states) != len(self.layers):
            raise ValueError(f"initial_states length {len(initial_states)} does not match "
                             f"num_layers {len(self.layers)}")
        out: dict[str, Any] = {}
        if (not return_jacobian_stats and memory_write_mode == "none" and
                self.kernel_trunk_supported() and not self.activation_checkpoint):
            hidden, _ss, finals = self.encode_with_stats(input_ids, initial_states=initial_states)
        else:
            x = self.embed(input_ids)
            bucket_ids = None
            if self.wernicke is not None:
                x, bucket_ids, balance = self.wernicke(x)
                out["balance_loss"] = balance
                out["bucket_ids"] = bucket_ids
            for bias in self._pre_recurrence_biases(x, bucket_ids):
                x = x + bias
            x, finals, all_stats = self._run_layers(x, initial_states, want_stats=return_jacobian_stats)
            bias = self._posterior_bias(x, bucket_ids)
            if bias is not None:
                x = x + bias
            hidden = x
            if return_jacobian_stats and all_stats:
                out["jacobian_stats"] = {k: torch.stack([s[k] for s in all_stats]).mean()
                                         for k in all_stats[0]}
                if self.dynamic_crit_per_layer:
                    out["per_layer_jacobian_stats"] = all_stats
        out["hidden"] = hidden
        out["logits"] = self.lm_head(self.final_norm(hidden))
        out["final_states"] = finals
        if (memory_write_mode == "append_only" and self.buffer_mode == "append_only" and
                self.outer_model is not None and hasattr(self.outer_model, "append_kv_batch")):
            bids = out.get("bucket_ids")
            records = self.append_memory_from_hidden(hidden, bucket_ids=bids)
            if records and self.bucket_prototypes_module is not None and bids is not None:
                om = self.outer_model
                enc = torch.tanh(om.encoder(hidden.detach().reshape(-1, hidden.shape[-1])
                                            .to(dtype=om.encoder.weight.dtype)))
                if enc.shape[-1] != self.bucket_prototypes_module.prototype_dim:
                    raise ValueError(f"outer_dim ({enc.shape[-1]}) != prototype_dim "
                                     f"({self.bucket_prototypes_module.prototype_dim})")
                self.bucket_prototypes_module.update_batch(bids.detach().reshape(-1), enc)
        return out

    @torch.no_grad()
    def append_memory_from_hidden(self, hidden: torch.Tensor, *, bucket_ids: Optional[torch.Tensor] = None,
                                  score: Optional[torch.Tensor] = None, max_tokens: Optional[int] = None,
                                  event_ids: Optional[torch.Tensor] = None) -> list[dict[str, object]]:
        """Encodes per-token hidden states and appends them to the append-only
        multi-slot store (reference model.py:1043-1163).  With ``max_tokens`` the
        highest-``score`` tokens (or an even stride without scores) are kept.
        Returns one generation-stamped record per slot actually appended."""
        from .memory import MultiSlotOuterModel
        om = self.outer_model
        if self.buffer_mode != "append_only" or not isinstance(om, MultiSlotOuterModel):
            raise ValueError("append_memory_from_hidden requires append-only MultiSlotOuterModel")
        B, T, D = hidden.shape
        flat = hidden.detach().reshape(-1, D)
        dev = hidden.device
        sel = None
        cap = 0 if max_tokens is None else int(max_tokens)
        if cap > 0 and flat.shape[0] > cap:
            if score is not None:
                sel = torch.topk(score.detach().reshape(-1).to(device=dev, dtype=torch.float32), k=cap,
                                 largest=True, sorted=False).indices
            else:
                sel = torch.linspace(0, flat.shape[0] - 1, steps=cap, device=dev).long()
            flat = flat.index_select(0, sel)
        ev = None
        if event_ids is not None:
            ev = event_ids.detach().reshape(-1).to(device=dev, dtype=torch.long)
            if ev.numel() == B * T:
                ev = ev if sel is None else ev.index_select(0, sel)
            elif ev.numel() != flat.shape[0]:
                raise ValueError("event_ids must either cover the full hidden shape "
                                 f"({B * T}) or the selected write count ({flat.shape[0]}), got {ev.numel()}")
        enc = torch.tanh(om.encoder(flat.to(dtype=om.encoder.weight.dtype)))
        if bucket_ids is None:
            bids = torch.zeros(flat.shape[0], dtype=torch.long, device=dev)
        else:
            bids = bucket_ids.detach().reshape(-1).to(device=dev, dtype=torch.long)
            if sel is not None:
                bids = bids.index_select(0, sel)
        ids = (om.append_kv_batch(enc, bids) if ev is None
               else om._append_kv_batch_committed(enc, bids, event_ids=ev))
        bid_list = bids[: len(ids)].tolist()
        ev_list = None if ev is None else ev[: len(ids)].tolist()
        records: list[dict[str, object]] = []
        for i, sid in enumerate(ids):
            rec = om.table.record(int(sid))
            records.append({
                "slot_id": int(sid), "tensor": enc[i].detach().reshape(1, -1), "bucket_id": int(bid_list[i]),
                "event_id": int(ev_list[i]) if ev_list is not None else int(rec.event_id if rec else 0),
                "generation": int(rec.write_generation if rec else 0)})
        return records

    # -- single token ----------------------------------------------------
    def step(self, token_ids: torch.Tensor, states: list[torch.Tensor], kv_caches=None):
        """One token through the recurrence only: ``(logits, hidden, new_states)``."""
        if self.depth_recurrence_count > 1:
            raise NotImplementedError(
                "CareStudentLM.step() does not implement depth recurrence; use forward() for "
                f"depth_recurrence_count={self.depth_recurrence_count}")
        x = self.embed(token_ids).squeeze(1)
        if kv_caches is None:
            kv_caches = [None] * len(self.layers)
        new_states = []
        for i, layer in enumerate(self.layers):
            if hasattr(layer, "_init_kv_cache"):
                if kv_caches[i] is None:
                    raise RuntimeError(f"Layer {i} is a hybrid block but no KV cache provided. "
                                       "Call init_kv_caches() and pass the result to step().")
                x, s = layer.step(x, states[i], kv_cache=kv_caches[i])
            else:
                x, s = layer.step(x, states[i])
            new_states.append(s)
        hidden = x
        logits = self.lm_head(self.final_norm(x.unsqueeze(1)).squeeze(1))
        return logits, hidden, new_states

    def dream_step(self, token_ids: torch.Tensor, states: list[torch.Tensor], kv_caches=None):
        """Single-token step through ALL tiers (Wernicke, memory read with the
        token itself as cue, semantic tier, then the recurrence): what REM dream
        generation uses, where ``step()`` deliberately runs the recurrence alone
        (reference src/chaoscontrol/model.py:922-1000).
        Returns ``(logits (batch, vocab), hidden (batch, dim), new_states)``."""
        if self.depth_recurrence_count > 1:
            raise NotImplementedError(
                "CareStudentLM.dream_step() does not implement depth recurrence; use forward() for "
                f"depth_recurrence_count={self.depth_recurrence_count}")
        x = self.embed(token_ids).squeeze(1)
        if self.wernicke is not None:
            x = self.wernicke(x.unsqueeze(1))[0].squeeze(1)
        if self.outer_model is not None:
            om = self.outer_model
            read = om.read(x.size(0), cue=x) if hasattr(om, "table") else om.read(x.size(0))
            x = x + read.to(x.dtype)
        if self.semantic_tier is not None:
            x = x + self.semantic_tier.read(x.size(0)).to(x.dtype)
        if kv_caches is None:
            kv_caches = [None] * len(self.layers)
        new_states = []
        for i, layer in enumerate(self.layers):
            if hasattr(layer, "_init_kv_cache"):
                if kv_caches[i] is None:
                    raise RuntimeError(f"Layer {i} is a hybrid block but no KV cache provided. "
                                       "Call init_kv_caches() and pass the result to dream_step().")
                x, s = layer.step(x, states[i], kv_cache=kv_caches[i])
            else:
                x, s = layer.step(x, states[i])
            new_states.append(s)
        logits = self.lm_head(self.final_norm(x.unsqueeze(1)).squeeze(1))
        return logits, x, new_states
