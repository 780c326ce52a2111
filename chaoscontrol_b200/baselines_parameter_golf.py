"""The contest's transformer baseline harness, rebuilt on this package's parts.

The reference vendors the contest's own NanoGPT-style trainer
(baselines/parameter_golf/train_gpt.py:39-1126; record variant under sota/) as the
yard-stick every SSM result is quoted against: 9 blocks x 512, 8 query / 4 key-value
heads with rotary embeddings and q/k RMS normalisation, squared-ReLU MLP, a U-shaped
stack (the first half of the blocks leaves skip tensors that the second half adds
back through learned per-channel weights), every block mixing the residual stream
with the embedding output, tanh soft-capped logits, tied embeddings; Muon for the
block matrices and Adam for embeddings / scalars / head; warm-up steps whose effect
is rolled back; a warm-down keyed to the wall-clock cap; int8 (per-row) + zlib export
and a round-trip evaluation; bits per byte from SentencePiece byte tables.

What is shared with the contest files is the contract: the environment-variable
names and defaults, the shard format (256 int32 header, magic 20240520, version 1,
uint16 tokens), parameter names of the model (so a contest checkpoint loads), the
log line keys, and the export format.  The code is this package's: ``optim.muon.Muon``
for the matrices, ``sp_eval`` byte tables, no tracing compiler and no DDP wrapper
(gradients are averaged with one flat all-reduce).
"""
from __future__ import annotations

import glob
import io
import math
import os
import time
import uuid
import zlib
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Callable, Iterator, Optional

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

SHARD_MAGIC, SHARD_VERSION, SHARD_HEADER_INTS = 20240520, 1, 256
CONTROL_PATTERNS = ("attn_scale", "mlp_scale", "resid_mix", "q_gain", "skip_weight")
INT8_CLIP_Q = 0.9999984
INT8_KEEP_FLOAT_MAX_NUMEL = 65_536


def _env(name: str, default, cast=None):
    raw = os.environ.get(name)
    if raw is None:
        return default
    cast = cast or type(default)
    return bool(int(raw)) if cast is bool else cast(raw)


@dataclass
class GolfConfig:
    """Defaults of the contest's simple baseline; every field is read from the environment
    variable of the same name in upper case."""
    data_path: str = "./data/datasets/fineweb10B_sp1024"
    tokenizer_path: str = "./data/tokenizers/fineweb_1024_bpe.model"
    run_id: str = field(default_factory=lambda: str(uuid.uuid4()))
    seed: int = 1337
    val_batch_size: int = 524_288
    val_loss_every: int = 1000
    train_log_every: int = 200
    iterations: int = 20000
    warmdown_iters: int = 1200
    warmup_steps: int = 20
    train_batch_tokens: int = 524_288
    train_seq_len: int = 1024
    max_wallclock_seconds: float = 600.0
    qk_gain_init: float = 1.5
    vocab_size: int = 1024
    num_layers: int = 9
    num_kv_heads: int = 4
    model_dim: int = 512
    num_heads: int = 8
    mlp_mult: int = 2
    tie_embeddings: bool = True
    rope_base: float = 10000.0
    logit_softcap: float = 30.0
    embed_lr: float = 0.6
    head_lr: float = 0.008
    tied_embed_lr: float = 0.05
    tied_embed_init_std: float = 0.005
    matrix_lr: float = 0.04
    scalar_lr: float = 0.04
    muon_momentum: float = 0.95
    muon_backend_steps: int = 5
    muon_momentum_warmup_start: float = 0.85
    muon_momentum_warmup_steps: int = 500
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    grad_clip_norm: float = 0.0

    @classmethod
    def from_env(cls, **over) -> "GolfConfig":
        kw = {}
        for f in fields(cls):
            default = f.default if f.default is not field else None
            if f.name == "run_id":
                kw[f.name] = os.environ.get("RUN_ID", str(uuid.uuid4()))
            else:
                kw[f.name] = _env(f.name.upper(), default, type(default))
        kw.update(over)
        return cls(**kw)

    @property
    def train_files(self) -> str:
        return os.path.join(self.data_path, "fineweb_train_*.bin")

    @property
    def val_files(self) -> str:
        return os.path.join(self.data_path, "fineweb_val_*.bin")


# ---------------------------------------------------------------------------
# data
# ---------------------------------------------------------------------------
def write_data_shard(path: Path, tokens: np.ndarray) -> None:
    """Inverse of :func:`load_data_shard` (tests and synthetic runs)."""
    header = np.zeros(SHARD_HEADER_INTS, dtype="<i4")
    header[:3] = (SHARD_MAGIC, SHARD_VERSION, int(tokens.size))
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(np.asarray(tokens, dtype="<u2").tobytes())


def load_data_shard(path: Path) -> torch.Tensor:
    header = np.fromfile(path, dtype="<i4", count=SHARD_HEADER_INTS)
    if header.size != SHARD_HEADER_INTS or int(header[0]) != SHARD_MAGIC or int(header[1]) != SHARD_VERSION:
        raise ValueError(f"Unexpected shard header for {path}")
    n = int(header[2])
    want = SHARD_HEADER_INTS * 4 + 2 * n
    if Path(path).stat().st_size != want:
        raise ValueError(f"Shard size mismatch for {path}: expected {want} bytes")
    tok = np.fromfile(path, dtype="<u2", count=n, offset=SHARD_HEADER_INTS * 4)
    return torch.from_numpy(tok.astype(np.uint16, copy=False))


class TokenStream:
    """Shards in name order, read front to back, wrapping around forever."""

    def __init__(self, pattern: str) -> None:
        self.files = [Path(p) for p in sorted(glob.glob(pattern))]
        if not self.files:
            raise FileNotFoundError(f"No files found for pattern: {pattern}")
        self._i, self._pos = 0, 0
        self._tok = load_data_shard(self.files[0])

    def take(self, n: int) -> torch.Tensor:
        parts = []
        while n > 0:
            left = self._tok.numel() - self._pos
            if left <= 0:
                self._i = (self._i + 1) % len(self.files)
                self._tok, self._pos = load_data_shard(self.files[self._i]), 0
                continue
            k = min(n, left)
            parts.append(self._tok[self._pos: self._pos + k])
            self._pos += k
            n -= k
        return parts[0] if len(parts) == 1 else torch.cat(parts)


class DistributedTokenLoader:
    """Every call takes one contiguous span for all ranks and keeps this rank's slice (+1 token for the shift)."""

    def __init__(self, pattern: str, rank: int, world_size: int, device: torch.device) -> None:
        self.rank, self.world_size, self.device = rank, world_size, device
        self.stream = TokenStream(pattern)

    def next_batch(self, global_tokens: int, seq_len: int, grad_accum_steps: int):
        local = global_tokens // (self.world_size * grad_accum_steps)
        span = local + 1
        chunk = self.stream.take(span * self.world_size)
        mine = chunk[self.rank * span: (self.rank + 1) * span].to(torch.int64)
        x, y = mine[:-1].reshape(-1, seq_len), mine[1:].reshape(-1, seq_len)
        return x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)


def load_validation_tokens(pattern: str, seq_len: int) -> torch.Tensor:
    files = sorted(glob.glob(pattern))
    if not files:
        raise FileNotFoundError(f"No files found for pattern: {pattern}")
    tok = torch.cat([load_data_shard(Path(f)) for f in files])
    usable = ((tok.numel() - 1) // seq_len) * seq_len
    if usable <= 0:
        raise ValueError(f"Validation split is too short for TRAIN_SEQ_LEN={seq_len}")
    return tok[: usable + 1]


# ---------------------------------------------------------------------------
# model (parameter names follow the contest file so its checkpoints load)
# ---------------------------------------------------------------------------
class RMSNorm(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.size(-1),))


class CastedLinear(nn.Linear):
    """fp32 master weight, cast to the activation dtype at use."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


def _rope_tables(head_dim: int, seq_len: int, base: float, device, dtype):
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos()[None, None].to(dtype), ang.sin()[None, None].to(dtype)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    h = x.size(-1) // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat((a * cos + b * sin, b * cos - a * sin), dim=-1)


class CausalSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, num_kv_heads: int, rope_base: float, qk_gain_init: float) -> None:
        super().__init__()
        if dim % num_heads or num_heads % num_kv_heads or (dim // num_heads) % 2:
            raise ValueError("model_dim / heads / kv heads do not divide, or head_dim is odd")
        self.num_heads, self.num_kv_heads, self.head_dim, self.rope_base = num_heads, num_kv_heads, dim // num_heads, rope_base
        kv = num_kv_heads * self.head_dim
        self.c_q, self.c_k, self.c_v = (CastedLinear(dim, dim, bias=False), CastedLinear(dim, kv, bias=False),
                                        CastedLinear(dim, kv, bias=False))
        self.proj = CastedLinear(dim, dim, bias=False)
        self.proj._zero_init = True
        self.q_gain = nn.Parameter(torch.full((num_heads,), qk_gain_init, dtype=torch.float32))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, D = x.shape
        split = lambda t, h: t.reshape(B, T, h, self.head_dim).transpose(1, 2)      # noqa: E731
        q, k, v = split(self.c_q(x), self.num_heads), split(self.c_k(x), self.num_kv_heads), split(self.c_v(x), self.num_kv_heads)
        q, k = F.rms_norm(q, (self.head_dim,)), F.rms_norm(k, (self.head_dim,))
        cos, sin = _rope_tables(self.head_dim, T, self.rope_base, x.device, q.dtype)
        q, k = apply_rotary_emb(q, cos, sin), apply_rotary_emb(k, cos, sin)
        q = q * self.q_gain.to(q.dtype)[None, :, None, None]
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.num_kv_heads != self.num_heads)
        return self.proj(y.transpose(1, 2).reshape(B, T, D))


class MLP(nn.Module):
    def __init__(self, dim: int, mult: int) -> None:
        super().__init__()
        self.fc, self.proj = CastedLinear(dim, mult * dim, bias=False), CastedLinear(mult * dim, dim, bias=False)
        self.proj._zero_init = True

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(torch.relu(self.fc(x)).square())


class Block(nn.Module):
    def __init__(self, cfg: GolfConfig) -> None:
        super().__init__()
        d = cfg.model_dim
        self.attn_norm, self.mlp_norm = RMSNorm(), RMSNorm()
        self.attn = CausalSelfAttention(d, cfg.num_heads, cfg.num_kv_heads, cfg.rope_base, cfg.qk_gain_init)
        self.mlp = MLP(d, cfg.mlp_mult)
        self.attn_scale = nn.Parameter(torch.ones(d))
        self.mlp_scale = nn.Parameter(torch.ones(d))
        self.resid_mix = nn.Parameter(torch.stack((torch.ones(d), torch.zeros(d))))

    def forward(self, x: torch.Tensor, x0: torch.Tensor) -> torch.Tensor:
        mix = self.resid_mix.to(x.dtype)
        x = mix[0] * x + mix[1] * x0
        x = x + self.attn_scale.to(x.dtype) * self.attn(self.attn_norm(x))
        return x + self.mlp_scale.to(x.dtype) * self.mlp(self.mlp_norm(x))


class GPT(nn.Module):
    def __init__(self, cfg: GolfConfig) -> None:
        super().__init__()
        if cfg.logit_softcap <= 0:
            raise ValueError(f"logit_softcap must be positive, got {cfg.logit_softcap}")
        self.cfg = cfg
        self.tie_embeddings, self.logit_softcap = cfg.tie_embeddings, cfg.logit_softcap
        self.tok_emb = nn.Embedding(cfg.vocab_size, cfg.model_dim)
        self.num_encoder_layers = cfg.num_layers // 2
        self.num_decoder_layers = cfg.num_layers - self.num_encoder_layers
        self.skip_weights = nn.Parameter(torch.ones(min(self.num_encoder_layers, self.num_decoder_layers), cfg.model_dim))
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.num_layers))
        self.final_norm = RMSNorm()
        self.lm_head = None if cfg.tie_embeddings else CastedLinear(cfg.model_dim, cfg.vocab_size, bias=False)
        if self.lm_head is not None:
            self.lm_head._zero_init = True
        if cfg.tie_embeddings:
            nn.init.normal_(self.tok_emb.weight, mean=0.0, std=cfg.tied_embed_init_std)
        for m in self.modules():
            if isinstance(m, nn.Linear) and getattr(m, "_zero_init", False):
                nn.init.zeros_(m.weight)

    def hidden(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = F.rms_norm(self.tok_emb(input_ids), (self.cfg.model_dim,))
        x0, skips = x, []
        for i in range(self.num_encoder_layers):
            x = self.blocks[i](x, x0)
            skips.append(x)
        for i in range(self.num_decoder_layers):
            if skips:
                x = x + self.skip_weights[i].to(x.dtype) * skips.pop()
            x = self.blocks[self.num_encoder_layers + i](x, x0)
        return self.final_norm(x)

    def logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        h = self.hidden(input_ids)
        raw = F.linear(h, self.tok_emb.weight.to(h.dtype)) if self.tie_embeddings else self.lm_head(h)
        return self.logit_softcap * torch.tanh(raw / self.logit_softcap)

    def forward(self, input_ids: torch.Tensor, target_ids: torch.Tensor) -> torch.Tensor:
        lg = self.logits(input_ids)
        return F.cross_entropy(lg.reshape(-1, lg.size(-1)).float(), target_ids.reshape(-1), reduction="mean")


def split_parameters(model: GPT) -> dict[str, list[nn.Parameter]]:
    """Block matrices -> Muon; block vectors / gains / mixing / skip weights -> scalar Adam; embedding and
    (untied) head -> their own Adam groups."""
    named = list(model.blocks.named_parameters())
    ctrl = lambda n: any(p in n for p in CONTROL_PATTERNS)     # noqa: E731
    out = {"matrix": [p for n, p in named if p.ndim == 2 and not ctrl(n)],
           "scalar": [p for n, p in named if p.ndim < 2 or ctrl(n)], "embed": [model.tok_emb.weight],
           "head": [] if model.lm_head is None else [model.lm_head.weight]}
    if model.skip_weights.numel():
        out["scalar"].append(model.skip_weights)
    return out


def build_optimizers(model: GPT, cfg: GolfConfig) -> list[torch.optim.Optimizer]:
    from .optim.muon import Muon
    g = split_parameters(model)
    adam = lambda ps, lr: torch.optim.Adam([{"params": ps, "lr": lr, "base_lr": lr}], betas=(cfg.beta1, cfg.beta2),   # noqa: E731
                                           eps=cfg.adam_eps)
    opts: list[torch.optim.Optimizer] = [adam(g["embed"], cfg.tied_embed_lr if cfg.tie_embeddings else cfg.embed_lr)]
    if g["head"]:
        opts.append(adam(g["head"], cfg.head_lr))
    muon = Muon(g["matrix"], lr=cfg.matrix_lr, momentum=cfg.muon_momentum, ns_steps=cfg.muon_backend_steps,
                weight_decay=0.0, adamw_lr=cfg.scalar_lr)
    for grp in muon.param_groups:
        grp["base_lr"] = cfg.matrix_lr
    opts += [muon, adam(g["scalar"], cfg.scalar_lr)]
    return opts


def lr_multiplier(cfg: GolfConfig, step: int, elapsed_ms: float) -> float:
    """1 until the warm-down, then linear to 0: by iteration count without a wall-clock cap, otherwise
    by the time that ``warmdown_iters`` steps at the observed pace would take before the cap."""
    if cfg.warmdown_iters <= 0:
        return 1.0
    if cfg.max_wallclock_seconds <= 0:
        start = max(cfg.iterations - cfg.warmdown_iters, 0)
        return max((cfg.iterations - step) / max(cfg.warmdown_iters, 1), 0.0) if start <= step < cfg.iterations else 1.0
    cap = 1000.0 * cfg.max_wallclock_seconds
    window = cfg.warmdown_iters * (elapsed_ms / max(step, 1))
    left = max(cap - elapsed_ms, 0.0)
    return left / max(window, 1e-9) if left <= window else 1.0


def muon_momentum_at(cfg: GolfConfig, step: int) -> float:
    f = min(step / cfg.muon_momentum_warmup_steps, 1.0) if cfg.muon_momentum_warmup_steps > 0 else 1.0
    return (1 - f) * cfg.muon_momentum_warmup_start + f * cfg.muon_momentum


# ---------------------------------------------------------------------------
# int8 export
# ---------------------------------------------------------------------------
def quantize_float_tensor(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Matrices: one scale per row from a high quantile of |w| (clip, then round to [-127, 127]);
    everything else: one scale per tensor."""
    t32 = t.float()
    if t32.ndim == 2:
        clip = torch.quantile(t32.abs(), INT8_CLIP_Q, dim=1) if t32.numel() else torch.empty(t32.shape[0])
        scale = (clip / 127.0).clamp_min(1.0 / 127.0)
        q = torch.clamp(torch.round(t32.clamp(-clip[:, None], clip[:, None]) / scale[:, None]), -127, 127)
        return q.to(torch.int8).contiguous(), scale.to(torch.float16).contiguous()
    clip = float(torch.quantile(t32.abs().flatten(), INT8_CLIP_Q)) if t32.numel() else 0.0
    scale = torch.tensor(clip / 127.0 if clip > 0 else 1.0, dtype=torch.float32)
    return torch.clamp(torch.round(t32.clamp(-clip, clip) / scale), -127, 127).to(torch.int8).contiguous(), scale


def quantize_state_dict_int8(sd: dict[str, torch.Tensor]) -> tuple[dict, dict]:
    """Large float tensors -> int8 + scales; small ones and control tensors stay float (fp16 storage, fp32 for
    control tensors); non-float tensors pass through."""
    q, scales, dtypes, passthrough, pdt, qmeta = {}, {}, {}, {}, {}, {}
    stats = {"param_count": 0, "num_tensors": 0, "baseline_tensor_bytes": 0, "int8_payload_bytes": 0}
    nbytes = lambda t: t.numel() * t.element_size()      # noqa: E731
    for name, t in sd.items():
        t = t.detach().cpu().contiguous()
        stats["param_count"] += t.numel()
        stats["num_tensors"] += 1
        stats["baseline_tensor_bytes"] += nbytes(t)
        if not t.is_floating_point():
            passthrough[name] = t
            stats["int8_payload_bytes"] += nbytes(t)
        elif t.numel() <= INT8_KEEP_FLOAT_MAX_NUMEL:
            if any(p in name for p in CONTROL_PATTERNS):
                kept = t.float()
            else:
                pdt[name] = str(t.dtype).removeprefix("torch.")
                kept = t.to(torch.float16)
            passthrough[name] = kept.contiguous()
            stats["int8_payload_bytes"] += nbytes(kept)
        else:
            qi, sc = quantize_float_tensor(t)
            if sc.ndim:
                qmeta[name] = {"scheme": "per_row", "axis": 0}
            q[name], scales[name], dtypes[name] = qi, sc, str(t.dtype).removeprefix("torch.")
            stats["int8_payload_bytes"] += nbytes(qi) + nbytes(sc)
    obj = {"__quant_format__": "int8_clean_per_row_v1", "quantized": q, "scales": scales, "dtypes": dtypes,
           "passthrough": passthrough}
    if qmeta:
        obj["qmeta"] = qmeta
    if pdt:
        obj["passthrough_orig_dtypes"] = pdt
    return obj, stats


def dequantize_state_dict_int8(obj: dict) -> dict[str, torch.Tensor]:
    out = {}
    for name, qi in obj["quantized"].items():
        dt, sc = getattr(torch, obj["dtypes"][name]), obj["scales"][name]
        w = qi.float() * (sc.float().view(qi.shape[0], *([1] * (qi.ndim - 1))) if sc.ndim else float(sc))
        out[name] = w.to(dt).contiguous()
    for name, t in obj["passthrough"].items():
        orig = obj.get("passthrough_orig_dtypes", {}).get(name)
        out[name] = t.detach().cpu().to(getattr(torch, orig)).contiguous() if orig else t.detach().cpu().contiguous()
    return out


def export_int8_zlib(model: nn.Module) -> tuple[bytes, dict]:
    obj, stats = quantize_state_dict_int8(model.state_dict())
    buf = io.BytesIO()
    torch.save(obj, buf)
    raw = buf.getvalue()
    stats["raw_torch_bytes"] = len(raw)
    return zlib.compress(raw, level=9), stats


def load_int8_zlib(model: nn.Module, blob: bytes) -> None:
    obj = torch.load(io.BytesIO(zlib.decompress(blob)), map_location="cpu")
    model.load_state_dict(dequantize_state_dict_int8(obj), strict=True)


# ---------------------------------------------------------------------------
# evaluation and training
# ---------------------------------------------------------------------------
def _all_reduce(t: torch.Tensor, op: str = "sum") -> torch.Tensor:
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.MAX)
    return t


@torch.no_grad()
def eval_val(cfg: GolfConfig, model: GPT, rank: int, world_size: int, device: torch.device, val_tokens: torch.Tensor,
             luts, *, autocast: bool = True) -> tuple[float, float]:
    """Mean CE over the validation split (sequences striped over ranks) and bits per byte with the
    tokenizer's byte tables: a leading-space piece counts one more byte unless it follows a boundary token."""
    base_bytes, lead_space, boundary = luts
    T = cfg.train_seq_len
    per = max(cfg.val_batch_size // (world_size * T), 1)
    n_seq = (val_tokens.numel() - 1) // T
    lo, hi = n_seq * rank // world_size, n_seq * (rank + 1) // world_size
    acc = torch.zeros(3, dtype=torch.float64, device=device)
    model.eval()
    for s in range(lo, hi, per):
        e = min(s + per, hi)
        loc = val_tokens[s * T: e * T + 1].to(device=device, dtype=torch.int64)
        x, y = loc[:-1].reshape(-1, T), loc[1:].reshape(-1, T)
        with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=autocast and device.type == "cuda"):
            loss = model(x, y)
        n = float(y.numel())
        bytes_ = base_bytes[y.reshape(-1)].to(torch.int16)
        bytes_ += (lead_space[y.reshape(-1)] & ~boundary[x.reshape(-1)]).to(torch.int16)
        acc += torch.stack([loss.double() * n, torch.tensor(n, dtype=torch.float64, device=device), bytes_.double().sum()])
    _all_reduce(acc)
    model.train()
    val_loss = float(acc[0] / acc[1])
    return val_loss, val_loss / math.log(2.0) * float(acc[1] / acc[2])


def train(cfg: GolfConfig, *, device: Optional[torch.device] = None, rank: int = 0, world_size: int = 1,
          log: Callable[[str], None] = print, luts=None, out_dir: Optional[Path] = None) -> dict:
    """The contest protocol end to end: rolled-back warm-up, capped training with the wall-clock warm-down,
    periodic validation, raw and int8+zlib export, round-trip validation.  Returns the final numbers."""
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if world_size <= 0 or 8 % world_size:
        raise ValueError(f"WORLD_SIZE={world_size} must divide 8 so that gradient accumulation is integral")
    accum = 8 // world_size
    torch.manual_seed(cfg.seed)
    np.random.seed(cfg.seed)
    if luts is None:
        import sentencepiece as spm
        from .sp_eval import build_sentencepiece_luts
        sp = spm.SentencePieceProcessor(model_file=cfg.tokenizer_path)
        if int(sp.vocab_size()) != cfg.vocab_size:
            raise ValueError(f"VOCAB_SIZE={cfg.vocab_size} does not match tokenizer vocab_size={int(sp.vocab_size())}")
        luts = build_sentencepiece_luts(sp, cfg.vocab_size, device)
    val_tokens = load_validation_tokens(cfg.val_files, cfg.train_seq_len)
    model = GPT(cfg).to(device)
    if device.type == "cuda":
        model = model.bfloat16()
        for m in model.modules():
            if isinstance(m, CastedLinear):
                m.float()
        for n, p in model.named_parameters():
            if p.ndim < 2 or any(c in n for c in CONTROL_PATTERNS):
                p.data = p.data.float()
    opts = build_optimizers(model, cfg)
    muon = next(o for o in opts if type(o).__name__ == "Muon")
    params = [p for p in model.parameters()]
    log(f"model_params:{sum(p.numel() for p in params)}")
    log(f"world_size:{world_size} grad_accum_steps:{accum}")

    def one_step(loader: DistributedTokenLoader, scale: float, step: int) -> torch.Tensor:
        for o in opts:
            o.zero_grad(set_to_none=True)
        tot = torch.zeros((), device=device)
        for _ in range(accum):
            x, y = loader.next_batch(cfg.train_batch_tokens, cfg.train_seq_len, accum)
            with torch.autocast(device_type=device.type, dtype=torch.bfloat16, enabled=device.type == "cuda"):
                loss = model(x, y)
            tot += loss.detach()
            (loss / accum).backward()
        if world_size > 1:
            flat = torch.cat([p.grad.reshape(-1).float() for p in params if p.grad is not None])
            _all_reduce(flat).div_(world_size)
            off = 0
            for p in params:
                if p.grad is not None:
                    p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
                    off += p.numel()
        for grp in muon.param_groups:
            grp["momentum"] = muon_momentum_at(cfg, step)
        for o in opts:
            for grp in o.param_groups:
                grp["lr"] = grp["base_lr"] * scale
        if cfg.grad_clip_norm > 0:
            torch.nn.utils.clip_grad_norm_(params, cfg.grad_clip_norm)
        for o in opts:
            o.step()
        return tot / accum

    sync = torch.cuda.synchronize if device.type == "cuda" else (lambda: None)
    if cfg.warmup_steps > 0:
        import copy
        snap_m = {k: v.detach().cpu().clone() for k, v in model.state_dict().items()}
        snap_o = [copy.deepcopy(o.state_dict()) for o in opts]
        warm = DistributedTokenLoader(cfg.train_files, rank, world_size, device)
        for w in range(cfg.warmup_steps):
            one_step(warm, 1.0, 0)
            log(f"warmup_step:{w + 1}/{cfg.warmup_steps}")
        model.load_state_dict(snap_m, strict=True)
        for o, s in zip(opts, snap_o):
            o.load_state_dict(s)
    loader = DistributedTokenLoader(cfg.train_files, rank, world_size, device)
    cap = 1000.0 * cfg.max_wallclock_seconds if cfg.max_wallclock_seconds > 0 else None
    train_ms, stop_after, step = 0.0, None, 0
    val_loss = val_bpb = float("nan")
    sync()
    t0 = time.perf_counter()
    while True:
        last = step == cfg.iterations or (stop_after is not None and step >= stop_after)
        if last or (cfg.val_loss_every > 0 and step % cfg.val_loss_every == 0):
            sync()
            train_ms += 1000.0 * (time.perf_counter() - t0)
            val_loss, val_bpb = eval_val(cfg, model, rank, world_size, device, val_tokens, luts)
            log(f"step:{step}/{cfg.iterations} val_loss:{val_loss:.4f} val_bpb:{val_bpb:.4f} "
                f"train_time:{train_ms:.0f}ms step_avg:{train_ms / max(step, 1):.2f}ms")
            sync()
            t0 = time.perf_counter()
        if last:
            if stop_after is not None and step < cfg.iterations:
                log(f"stopping_early: wallclock_cap train_time:{train_ms:.0f}ms step:{step}/{cfg.iterations}")
            break
        elapsed = train_ms + 1000.0 * (time.perf_counter() - t0)
        loss = one_step(loader, lr_multiplier(cfg, step, elapsed), step)
        step += 1
        approx = train_ms + 1000.0 * (time.perf_counter() - t0)
        if cfg.train_log_every > 0 and (step <= 10 or step % cfg.train_log_every == 0 or stop_after is not None):
            log(f"step:{step}/{cfg.iterations} train_loss:{float(loss):.4f} train_time:{approx:.0f}ms "
                f"step_avg:{approx / step:.2f}ms")
        hit = cap is not None and approx >= cap
        if world_size > 1 and cap is not None:
            hit = bool(_all_reduce(torch.tensor(int(hit), device=device), "max").item())
        if stop_after is None and hit:
            stop_after = step
    blob, stats = export_int8_zlib(model)
    out = {"steps": step, "val_loss": val_loss, "val_bpb": val_bpb, "train_time_ms": train_ms,
           "int8_zlib_bytes": len(blob), **stats}
    if out_dir is not None and rank == 0:
        Path(out_dir).mkdir(parents=True, exist_ok=True)
        torch.save(model.state_dict(), Path(out_dir) / "final_model.pt")
        (Path(out_dir) / "final_model.int8.ptz").write_bytes(blob)
    log(f"Serialized model int8+zlib: {len(blob)} bytes (payload:{stats['int8_payload_bytes']} "
        f"raw_torch:{stats['raw_torch_bytes']} payload_ratio:{stats['baseline_tensor_bytes'] / max(stats['int8_payload_bytes'], 1):.2f}x)")
    load_int8_zlib(model, blob)
    q_loss, q_bpb = eval_val(cfg, model, rank, world_size, device, val_tokens, luts)
    log(f"final_int8_zlib_roundtrip val_loss:{q_loss:.4f} val_bpb:{q_bpb:.4f}")
    log(f"final_int8_zlib_roundtrip_exact val_loss:{q_loss:.8f} val_bpb:{q_bpb:.8f}")
    out.update(roundtrip_val_loss=q_loss, roundtrip_val_bpb=q_bpb)
    return out


def main() -> int:
    import torch.distributed as dist
    cfg = GolfConfig.from_env()
    rank, ws, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if ws > 1:
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        dist.init_process_group(backend="nccl" if dev.type == "cuda" else "gloo")
    log = (lambda s: print(s, flush=True)) if rank == 0 else (lambda s: None)
    try:
        train(cfg, device=dev, rank=rank, world_size=ws, log=log, out_dir=Path("."))
    finally:
        if ws > 1:
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
