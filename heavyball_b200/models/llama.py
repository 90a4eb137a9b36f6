"""Llama-style decoder-only transformer: RMSNorm, rotary embeddings, SwiGLU MLP, grouped KV heads."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.nn import linear_cross_entropy


@dataclass
class LlamaConfig:
    n_layer: int = 24
    n_head: int = 16
    n_kv_head: int = 16
    d_model: int = 2048
    d_ff: int = 5504
    vocab_size: int = 32000
    seq_len: int = 2048
    rope_theta: float = 10000.0
    init_std: float = 0.02
    norm_eps: float = 1e-5


class RMSNorm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.eps)  # one fused kernel each way


def _rope(x, cos, sin):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class Layer(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        d, hd = cfg.d_model, cfg.d_model // cfg.n_head
        self.n_head, self.n_kv, self.hd = cfg.n_head, cfg.n_kv_head, hd
        self.norm1 = RMSNorm(d, cfg.norm_eps)
        self.wq = nn.Linear(d, cfg.n_head * hd, bias=False)
        self.wk = nn.Linear(d, cfg.n_kv_head * hd, bias=False)
        self.wv = nn.Linear(d, cfg.n_kv_head * hd, bias=False)
        self.wo = nn.Linear(cfg.n_head * hd, d, bias=False)
        self.norm2 = RMSNorm(d, cfg.norm_eps)
        self.w_gate = nn.Linear(d, cfg.d_ff, bias=False)
        self.w_up = nn.Linear(d, cfg.d_ff, bias=False)
        self.w_down = nn.Linear(cfg.d_ff, d, bias=False)

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        h = self.norm1(x)
        q = self.wq(h).view(B, T, self.n_head, self.hd).transpose(1, 2)
        k = self.wk(h).view(B, T, self.n_kv, self.hd).transpose(1, 2)
        v = self.wv(h).view(B, T, self.n_kv, self.hd).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.n_kv != self.n_head)
        x = x + self.wo(a.transpose(1, 2).reshape(B, T, -1))
        h = self.norm2(x)
        return x + self.w_down(F.silu(self.w_gate(h)) * self.w_up(h))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(Layer(cfg) for _ in range(cfg.n_layer))
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, cfg.init_std)

    def _angles(self, T, device, dtype):
        hd = self.cfg.d_model // self.cfg.n_head
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(T, device=device, dtype=torch.float32), inv)
        return ang.cos().to(dtype), ang.sin().to(dtype)

    def forward(self, idx, targets=None):
        x = self.embed(idx)
        cos, sin = self._angles(idx.shape[1], idx.device, x.dtype)
        for layer in self.layers:
            x = layer(x, cos, sin)
        h = self.norm(x)
        if targets is None:
            return self.head(h)
        return linear_cross_entropy(h, self.head.weight, targets)


def llama_1p3b(**kw):
    return Llama(LlamaConfig(n_layer=24, n_head=16, n_kv_head=16, d_model=2048, d_ff=5504, vocab_size=32000,
                             seq_len=2048, rope_theta=10000.0, **kw))  # fmt: skip


def llama3_8b(**kw):
    return Llama(LlamaConfig(n_layer=32, n_head=32, n_kv_head=8, d_model=4096, d_ff=14336, vocab_size=128256,
                             seq_len=4096, rope_theta=500000.0, **kw))  # fmt: skip
