"""Fixed-stride learned tokenizer (cf. src/chaoscontrol/tokenizer.py:13-112):
byte embedding -> causal strided convolution -> straight-through vector
quantisation -> transposed-convolution decoder whose byte cross-entropy keeps
the codebook from collapsing."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .models.routing import vector_quantize

__all__ = ["FixedStrideTokenizer"]


class FixedStrideTokenizer(nn.Module):
    """``token_seq = byte_seq // stride`` (for byte_seq divisible by stride);
    ``window`` defaults to two strides of overlap."""

    def __init__(self, byte_dim: int = 64, token_dim: int = 128, codebook_size: int = 1024, stride: int = 4,
                 window: int | None = None, beta: float = 0.25) -> None:
        super().__init__()
        self.stride = stride
        self.window = stride * 2 if window is None else window
        self.beta = beta
        self.codebook_size = codebook_size
        self.byte_embed = nn.Embedding(256, byte_dim)
        self.downsample = nn.Conv1d(byte_dim, token_dim, kernel_size=self.window, stride=stride)
        self.codebook = nn.Parameter(torch.empty(codebook_size, token_dim).uniform_(-1.0 / codebook_size,
                                                                                    1.0 / codebook_size))
        self.decoder = nn.ConvTranspose1d(token_dim, 256, kernel_size=stride * 2, stride=stride)

    def forward(self, byte_ids: torch.Tensor) -> dict:
        """``byte_ids`` ``(batch, byte_seq)`` in [0, 255] -> ``token_embeds``
        ``(batch, token_seq, token_dim)``, ``token_ids``, ``commit_loss``,
        ``recon_loss`` and a reference to ``codebook``."""
        n_bytes = byte_ids.shape[1]
        x = F.pad(self.byte_embed(byte_ids).transpose(1, 2), (self.window - 1, 0))     # left pad: causal
        x = self.downsample(x).transpose(1, 2)
        token_embeds, token_ids, commit = vector_quantize(x, self.codebook, beta=self.beta)
        logits = self.decoder(token_embeds.transpose(1, 2)).transpose(1, 2)[:, :n_bytes]
        recon = F.cross_entropy(logits.reshape(-1, 256), byte_ids[:, : logits.shape[1]].reshape(-1))
        return {"token_embeds": token_embeds, "token_ids": token_ids, "commit_loss": commit,
                "recon_loss": recon, "codebook": self.codebook}
