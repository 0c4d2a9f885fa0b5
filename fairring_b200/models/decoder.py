"""Decoder-only transformer language model (the data-parallel training workload
the reference's end-to-end benchmark is quoted on, README.md:66-70: a 1.37B
parameter Transformer).  Pre-LayerNorm blocks, learned positions, GELU MLP,
causal attention through ``scaled_dot_product_attention``, tied input/output
embedding.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class DecoderConfig:
    n_layer: int = 26
    d_model: int = 2048
    n_head: int = 16
    d_ff: int = 8192
    vocab: int = 51200
    seq_len: int = 1024
    fused_norm: bool = True  # one-kernel LayerNorm on the GPU (fairring_b200.ops.FusedLayerNorm)
    fused_loss: bool = True  # two-kernel cross-entropy on the GPU (fairring_b200.ops.fused_cross_entropy)
    fused_residual: bool = True  # residual add inside the next LayerNorm's kernels (fairring_b200.ops.add_layer_norm)

    @staticmethod
    def flagship() -> "DecoderConfig":
        """26 layers, d_model 2048, 16 heads, FFN 8192, vocab 51200, seq 1024."""
        return DecoderConfig()

    @staticmethod
    def tiny() -> "DecoderConfig":
        return DecoderConfig(n_layer=2, d_model=128, n_head=4, d_ff=512, vocab=1024, seq_len=64)


def _layer_norm(cfg: DecoderConfig) -> nn.LayerNorm:
    if cfg.fused_norm:
        from ..ops import FusedLayerNorm  # same parameters and state dict as nn.LayerNorm

        return FusedLayerNorm(cfg.d_model)
    return nn.LayerNorm(cfg.d_model)


class Block(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.n_head = cfg.n_head
        self.ln1 = _layer_norm(cfg)
        self.qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln2 = _layer_norm(cfg)
        self.fc1 = nn.Linear(cfg.d_model, cfg.d_ff)
        self.fc2 = nn.Linear(cfg.d_ff, cfg.d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, s, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, self.n_head, d // self.n_head).unbind(2)
        a = F.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True
        )
        x = x + self.proj(a.transpose(1, 2).reshape(b, s, d))
        x = x + self.fc2(F.gelu(self.fc1(self.ln2(x)), approximate="tanh"))
        return x

    def forward_pending(self, x: torch.Tensor, pending: torch.Tensor | None):
        """The same block with every residual add moved into the LayerNorm that
        follows it: takes the stream and the output of the block before that is
        still to be added to it, returns the stream and this block's own
        pending output."""
        from ..ops import add_layer_norm

        b, s, d = x.shape
        x, h = add_layer_norm(self.ln1, x, pending)
        q, k, v = self.qkv(h).view(b, s, 3, self.n_head, d // self.n_head).unbind(2)
        a = F.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True
        )
        x, h = add_layer_norm(self.ln2, x, self.proj(a.transpose(1, 2).reshape(b, s, d)))
        return x, self.fc2(F.gelu(self.fc1(h), approximate="tanh"))


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.tok = nn.Embedding(cfg.vocab, cfg.d_model)
        self.pos = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = _layer_norm(cfg)
        self.apply(self._init)
        for blk in self.blocks:  # scaled init of the residual projections
            nn.init.normal_(blk.proj.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))
            nn.init.normal_(blk.fc2.weight, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, std=0.02)
            nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, std=0.02)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None):
        b, s = tokens.shape
        pos = torch.arange(s, device=tokens.device)
        x = self.tok(tokens) + self.pos(pos)
        if self.cfg.fused_residual and self.cfg.fused_norm and x.is_cuda and x.dtype == torch.float32:
            from ..ops import add_layer_norm

            pending = None
            for blk in self.blocks:
                x, pending = blk.forward_pending(x, pending)
            _, x = add_layer_norm(self.ln_f, x, pending)
        else:
            for blk in self.blocks:
                x = blk(x)
            x = self.ln_f(x)
        logits = F.linear(x, self.tok.weight)  # tied output embedding
        if targets is None:
            return logits
        if self.cfg.fused_loss and logits.is_cuda:
            from ..ops import fused_cross_entropy  # the logits are consumed: nothing else reads them

            return fused_cross_entropy(logits.view(b * s, -1), targets.reshape(-1))
        return F.cross_entropy(logits.view(b * s, -1).float(), targets.reshape(-1))
