"""GPT-2-style decoder-only transformer.

The embedding table and the output head are stored with their row count rounded up to a multiple of 64
(50 257 -> 50 304): the head's three GEMMs then run on the aligned tensor-core kernels instead of a legacy
unaligned path that is about 9x slower on B200.  The loss is ``ops.nn.linear_cross_entropy``."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.nn import CastCache, LayerNorm, Linear, _bf16_training, linear_cross_entropy, linear_gelu, split_linear


@dataclass
class GPTConfig:
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_ff: int = 0  # 0 -> 4 * d_model
    vocab_size: int = 50257
    seq_len: int = 1024
    init_std: float = 0.02
    tie_embeddings: bool = True
    vocab_multiple: int = 64  # embedding / head rows are rounded up to this; the extra rows stay zero


def padded_vocab(vocab_size: int, multiple: int) -> int:
    return -(-vocab_size // max(multiple, 1)) * max(multiple, 1)


class Block(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        d, ff = cfg.d_model, cfg.d_ff or 4 * cfg.d_model
        self.n_head = cfg.n_head
        self.ln1 = LayerNorm(d)
        self.qkv = Linear(d, 3 * d)
        self.proj = Linear(d, d)
        self.ln2 = LayerNorm(d)
        self.fc = Linear(d, ff)
        self.out = Linear(ff, d)

    def forward(self, x, pending=None):
        """``x``: residual stream; ``pending``: output of the previous block's MLP, not yet added to it.  Returns the
        stream after this block's attention and this block's MLP output (to be added by whoever normalises next), so
        that every residual add runs inside a LayerNorm kernel."""
        B, T, D = x.shape
        # One packed [3D, D] parameter (the shape the matrix optimizers see), three projections: each of q, k, v
        # is then dense in [B, T, H, hd] order, so neither the attention output nor the three gradients coming
        # back from the attention kernel need a strided copy / concatenation (about 0.3 ms per layer otherwise).
        # One autograd node for the three: input gradient accumulated inside the GEMMs, packed weight gradient.
        if pending is None:
            h = self.ln1(x)
        else:
            x, h = self.ln1(x, pending)
        q, k, v = (
            t.view(B, T, self.n_head, D // self.n_head).transpose(1, 2)
            for t in split_linear(h, self.qkv.weight, self.qkv.bias, 3, self.qkv.w16, self.qkv.b16)
        )
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x, h = self.ln2(x, self.proj(a.transpose(1, 2).reshape(B, T, D)))
        return x, self.out(linear_gelu(h, self.fc.weight, self.fc.bias, self.fc.w16, self.fc.b16))


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        rows = padded_vocab(cfg.vocab_size, cfg.vocab_multiple)
        self.wte = nn.Embedding(rows, cfg.d_model)
        self.wpe = nn.Embedding(cfg.seq_len, cfg.d_model)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = LayerNorm(cfg.d_model)
        self.head = nn.Linear(cfg.d_model, rows, bias=False)
        if cfg.tie_embeddings:
            self.head.weight = self.wte.weight
        self.apply(self._init)
        self._casts = CastCache(self)
        with torch.no_grad():  # padding rows: never indexed, zero probability, zero gradient
            self.wte.weight[cfg.vocab_size :].zero_()
            self.head.weight[cfg.vocab_size :].zero_()

    def _init(self, m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, self.cfg.init_std)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets=None):
        B, T = idx.shape
        self._casts.refresh(_bf16_training(self.wte.weight))
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        pending = None
        for blk in self.blocks:
            x, pending = blk(x, pending)
        x, h = self.ln_f(x, pending)
        if targets is None:
            return self.head(h)[..., : self.cfg.vocab_size]
        return linear_cross_entropy(h, self.head.weight, targets, self.cfg.vocab_size)


def gpt2_small(**kw):
    return GPT(GPTConfig(n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024, **kw))


def gpt_350m(**kw):
    return GPT(GPTConfig(n_layer=24, n_head=16, d_model=1024, vocab_size=50257, seq_len=1024, **kw))
