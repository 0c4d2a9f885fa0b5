"""The benchmark's decoder-only language model assembled from stock
``torch.nn`` layers only (``nn.TransformerEncoderLayer`` with a causal mask,
``nn.Embedding``, ``nn.LayerNorm``): 26 layers, d_model 2048, 16 heads, FFN
8192 GELU, learned positions, tied output embedding.

This file imports nothing but PyTorch, so the benchmark arm that runs the
reference backend can build its workload without loading any code of this
repository's package.  The reference ships no model of its own; its end-to-end
figure is quoted on a 1.37B-parameter Transformer (README.md:66-70 of the
reference).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class StockDecoderLM(nn.Module):
    def __init__(self, n_layer: int = 26, d_model: int = 2048, n_head: int = 16, d_ff: int = 8192,
                 vocab: int = 51200, seq_len: int = 1024):
        super().__init__()
        self.n_layer, self.d_model, self.n_head, self.d_ff = n_layer, d_model, n_head, d_ff
        self.vocab, self.seq_len = vocab, seq_len
        self.tok = nn.Embedding(vocab, d_model)
        self.pos = nn.Embedding(seq_len, d_model)
        self.blocks = nn.ModuleList(
            nn.TransformerEncoderLayer(d_model, n_head, d_ff, dropout=0.0, activation="gelu",
                                       batch_first=True, norm_first=True)
            for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d_model)
        for m in self.modules():
            if isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, std=0.02)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None):
        b, s = tokens.shape
        x = self.tok(tokens) + self.pos(torch.arange(s, device=tokens.device))
        mask = nn.Transformer.generate_square_subsequent_mask(s, device=tokens.device)
        for blk in self.blocks:
            x = blk(x, src_mask=mask, is_causal=True)
        logits = F.linear(self.ln_f(x), self.tok.weight)
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(b * s, -1).float(), targets.reshape(-1))


def tiny() -> StockDecoderLM:
    return StockDecoderLM(n_layer=2, d_model=128, n_head=4, d_ff=512, vocab=1024, seq_len=64)
