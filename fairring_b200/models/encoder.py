"""RoBERTa-style bidirectional transformer encoder with a masked-LM head: the
1.3B workload (24 layers, d_model 2048, 32 heads, FFN 8192, vocab 50265, seq
512) used to exercise the backend with ranks grouped as 4 machines x 2 GPUs.
Post-LayerNorm blocks as in BERT/RoBERTa, learned positions, tied decoder.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class EncoderConfig:
    n_layer: int = 24
    d_model: int = 2048
    n_head: int = 32
    d_ff: int = 8192
    vocab: int = 50265
    seq_len: int = 512
    mask_prob: float = 0.15

    @staticmethod
    def roberta_1p3b() -> "EncoderConfig":
        return EncoderConfig()

    @staticmethod
    def tiny() -> "EncoderConfig":
        return EncoderConfig(n_layer=2, d_model=128, n_head=4, d_ff=512, vocab=1000, seq_len=32)


class EncoderLayer(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.n_head = cfg.n_head
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln1 = nn.LayerNorm(cfg.d_model)
        self.fc1 = nn.Linear(cfg.d_model, cfg.d_ff)
        self.fc2 = nn.Linear(cfg.d_ff, cfg.d_model)
        self.ln2 = nn.LayerNorm(cfg.d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.n_head, d // self.n_head).unbind(2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        x = self.ln1(x + self.proj(a.transpose(1, 2).reshape(b, s, d)))
        return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))


class EncoderMLM(nn.Module):
    def __init__(self, cfg: EncoderConfig):
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab, cfg.d_model)
        self.pos = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.ln_emb = nn.LayerNorm(cfg.d_model)
        self.layers = nn.ModuleList(EncoderLayer(cfg) for _ in range(cfg.n_layer))
        self.head_dense = nn.Linear(cfg.d_model, cfg.d_model)
        self.head_ln = nn.LayerNorm(cfg.d_model)
        self.head_bias = nn.Parameter(torch.zeros(cfg.vocab))
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, nn.Linear):
                nn.init.zeros_(m.bias)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor | None = None):
        """``labels``: target ids at masked positions, -100 elsewhere."""
        b, s = tokens.shape
        x = self.ln_emb(self.tok(tokens) + self.pos(torch.arange(s, device=tokens.device)))
        for layer in self.layers:
            x = layer(x)
        if labels is None:
            h = self.head_ln(F.gelu(self.head_dense(x)))
            return F.linear(h, self.tok.weight, self.head_bias)
        # Only masked positions go through the vocabulary projection.
        sel = labels.reshape(-1) != -100
        h = x.reshape(b * s, -1)[sel]
        h = self.head_ln(F.gelu(self.head_dense(h)))
        logits = F.linear(h, self.tok.weight, self.head_bias)
        return F.cross_entropy(logits.float(), labels.reshape(-1)[sel])


def mask_tokens(tokens: torch.Tensor, cfg: EncoderConfig, generator: torch.Generator, mask_id: int = 0):
    """15% of the positions are replaced by the mask id; labels keep the originals there."""
    pick = torch.rand(tokens.shape, generator=generator) < cfg.mask_prob
    labels = torch.where(pick, tokens, torch.full_like(tokens, -100))
    return torch.where(pick, torch.full_like(tokens, mask_id), tokens), labels
