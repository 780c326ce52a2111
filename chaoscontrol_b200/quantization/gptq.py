"""Hessian-aware int6 quantisation (GPTQ) for the <= 16 MB artifact.

Container format and selection rules follow the reference
(src/chaoscontrol/quantization/gptq.py:26-341, packaging.py:25-67): per-row fp16
scales, codes in [-31, 31] stored as int8, a five-point clipping-percentile
search keeping the lowest reconstruction error, tensors under ``min_numel``
kept as fp16, ``{"w": quantized, "m": meta}`` + LZMA preset 9 on disk.

The column sweep runs on whatever device the weight lives on, so calibrating
and quantising a model on the GPU is a few seconds.
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch
import torch.nn as nn

INT6_CLIP_RANGE = 31
DEFAULT_BLOCK_SIZE = 128
PERCENTILE_GRID = (0.9990, 0.9995, 0.9999, 0.99999, 1.0)


@torch.no_grad()
def ar_self_generated_calibration(model: nn.Module, *, num_seqs: int = 16, seq_len: int = 128,
                                  vocab_size: Optional[int] = None, temperature: float = 1.0,
                                  seed: int = 0, device="cpu") -> list[torch.Tensor]:
    """Calibration text sampled from the model itself (no dataset needed)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    V = vocab_size or model.vocab_size
    model = model.to(device).eval()
    seqs = []
    for _ in range(num_seqs):
        tok = torch.randint(0, V, (1, 1), generator=g).to(device)
        states = model.init_state(1)
        out = [tok]
        for _ in range(seq_len - 1):
            logits, _, states = model.step(tok, states)
            probs = torch.softmax(logits.float() / max(temperature, 1e-6), dim=-1)
            tok = torch.multinomial(probs.cpu(), 1, generator=g).to(device)
            out.append(tok)
        seqs.append(torch.cat(out, dim=1))
    return seqs


def collect_hessians(model: nn.Module, token_seqs: Iterable[torch.Tensor], *, device="cpu",
                     forward_fn: Optional[Callable[[nn.Module, torch.Tensor], torch.Tensor]] = None
                     ) -> dict[str, torch.Tensor]:
    """``H = mean_x x x^T`` of every ``nn.Linear`` input, keyed by ``<module>.weight``."""
    model = model.to(device).eval()
    H: dict[str, torch.Tensor] = {}
    counts: dict[str, int] = {}
    hooks = []
    for mname, mod in model.named_modules():
        if isinstance(mod, nn.Linear):
            key = f"{mname}.weight"

            def hook(_m, inputs, _o, key=key):
                x = inputs[0].detach().reshape(-1, inputs[0].shape[-1]).float()
                H[key] = H.get(key, 0) + x.T @ x
                counts[key] = counts.get(key, 0) + x.shape[0]
            hooks.append(mod.register_forward_hook(hook))
    try:
        with torch.no_grad():
            for seq in token_seqs:
                seq = seq.to(device)
                if forward_fn is not None:
                    forward_fn(model, seq)
                else:
                    model(seq)
    finally:
        for h in hooks:
            h.remove()
    return {k: (v / max(counts[k], 1)).cpu() for k, v in H.items()}


def _row_scales(t32: torch.Tensor, pct: float, clip_range: int) -> torch.Tensor:
    clip = torch.quantile(t32.abs(), pct, dim=1) if pct < 1.0 else t32.abs().amax(dim=1)
    return (clip / clip_range).clamp_min(1.0 / clip_range).to(torch.float16)


def quantize_int6_percentile(tensor: torch.Tensor, clip_range: int = INT6_CLIP_RANGE):
    """Round-to-nearest int6 with the best clipping percentile (2-D: per-row scale)."""
    t32 = tensor.float()
    if t32.ndim != 2:
        amax = float(t32.abs().max())
        scale = torch.tensor(amax / clip_range if amax > 0 else 1.0, dtype=torch.float16)
        return torch.clamp(torch.round(t32 / scale.float()), -clip_range, clip_range).to(torch.int8), scale
    best = None
    for pct in PERCENTILE_GRID:
        s = _row_scales(t32, pct, clip_range)
        q = torch.clamp(torch.round(t32 / s.float()[:, None]), -clip_range, clip_range).to(torch.int8)
        err = float((t32 - q.float() * s.float()[:, None]).pow(2).mean())
        if best is None or err < best[0]:
            best = (err, q, s)
    return best[1], best[2]


def quantize_int6_gptq(weight: torch.Tensor, hessian: Optional[torch.Tensor] = None,
                       clip_range: int = INT6_CLIP_RANGE, block_size: int = DEFAULT_BLOCK_SIZE):
    """GPTQ: quantise columns in order of decreasing Hessian diagonal, pushing each
    column's rounding error onto the not-yet-quantised columns through the upper
    Cholesky factor of ``H^-1``.  Falls back to the percentile search without a
    Hessian or for non-matrices.  Returns ``(int8 codes, fp16 per-row scales)``."""
    t32 = weight.float()
    if t32.ndim != 2 or hessian is None:
        return quantize_int6_percentile(t32, clip_range)
    dev = t32.device
    rows, cols = t32.shape
    H = hessian.to(dev).float().clone()
    diag = torch.diagonal(H)
    dead = diag == 0
    diag[dead] = 1.0
    diag += 0.01 * diag.mean()
    perm = torch.argsort(torch.diagonal(H), descending=True)
    inv_perm = torch.argsort(perm)
    W0 = t32[:, perm].clone()
    W0[:, dead[perm]] = 0
    Hp = H[perm][:, perm]
    U = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(Hp)), upper=True)
    best = None
    for pct in PERCENTILE_GRID:
        s = _row_scales(t32, pct, clip_range)
        sf = s.float()
        W = W0.clone()
        Q = torch.empty_like(W, dtype=torch.int8)
        for b0 in range(0, cols, block_size):
            b1 = min(b0 + block_size, cols)
            blk = W[:, b0:b1].clone()
            errs = torch.empty_like(blk)
            Ub = U[b0:b1, b0:b1]
            for j in range(b1 - b0):
                col = blk[:, j]
                q = torch.clamp(torch.round(col / sf), -clip_range, clip_range)
                Q[:, b0 + j] = q.to(torch.int8)
                e = (col - q * sf) / Ub[j, j]
                blk[:, j:] -= e[:, None] * Ub[j, j:][None, :]
                errs[:, j] = e
            if b1 < cols:
                W[:, b1:] -= errs @ U[b0:b1, b1:]
        mse = float((W0 - Q.float() * sf[:, None]).pow(2).mean())
        if best is None or mse < best[0]:
            best = (mse, Q, s)
    return best[1][:, inv_perm].contiguous(), best[2]


def dequantize_state_dict(result: dict[str, torch.Tensor], meta: dict[str, dict]) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}
    for name, m in meta.items():
        kind = m["type"]
        if kind == "int6":
            q, s = result[name + ".q"].float(), result[name + ".scale"].float()
            w = q * (s[:, None] if q.ndim == 2 and s.ndim == 1 else s)
            out[name] = w.reshape(m["shape"])
        elif kind == "passthrough_fp16":
            out[name] = result[name].float()
        else:
            out[name] = result[name]
    return out


class GPTQQuantizer:
    def __init__(self, clip_range: int = INT6_CLIP_RANGE, block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        self.clip_range = clip_range
        self.block_size = block_size
        self.hessians: dict[str, torch.Tensor] = {}

    def calibrate(self, model: nn.Module, token_seqs: Iterable[torch.Tensor], *, device="cpu",
                  forward_fn=None) -> dict[str, torch.Tensor]:
        self.hessians = collect_hessians(model, token_seqs, device=device, forward_fn=forward_fn)
        return self.hessians

    def quantize_state_dict(self, state_dict: dict[str, torch.Tensor], *,
                            int6_param_names: Optional[set[str]] = None, min_numel: int = 65536):
        result: dict[str, torch.Tensor] = {}
        meta: dict[str, dict] = {}
        for name, tensor in state_dict.items():
            t = tensor.detach().contiguous()
            if not t.is_floating_point():
                result[name] = t.cpu()
                meta[name] = {"type": "passthrough", "dtype": str(t.dtype)}
                continue
            if not (t.numel() > min_numel and (int6_param_names is None or name in int6_param_names)):
                result[name] = t.cpu().to(torch.float16)
                meta[name] = {"type": "passthrough_fp16", "dtype": str(tensor.dtype)}
                continue
            H = self.hessians.get(name)
            if H is not None and t.ndim == 2:
                q, s = quantize_int6_gptq(t, hessian=H, clip_range=self.clip_range,
                                          block_size=self.block_size)
            else:
                q, s = quantize_int6_percentile(t, clip_range=self.clip_range)
            result[name + ".q"], result[name + ".scale"] = q.cpu(), s.cpu()
            meta[name] = {"type": "int6", "dtype": str(tensor.dtype), "shape": list(t.shape)}
        return result, meta

    dequantize_state_dict = staticmethod(dequantize_state_dict)
