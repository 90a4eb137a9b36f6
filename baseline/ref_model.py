"""Plain-PyTorch decoders used by the reference arm of ``bench.py`` (and by its "plain model" measurement of this
package's optimizers).

Deliberately independent of the ``heavyball_b200`` package so that the reference arm touches none of
its code: standard ``torch.nn`` modules only.

``RefGPT``: LayerNorm, learned positions, fused QKV, GELU(tanh) MLP, tied embeddings; weights N(0, 0.02), biases
zero.  ``vocab_rows`` is the row count of the embedding table / output head; rounding the 50 257-token vocabulary up
to 50 304 rows (a multiple of 64, as nanoGPT-style code does) keeps the head's three GEMMs on the aligned tensor-core
kernels.  Both benchmark arms use the same row count, so both optimizers see identical parameter shapes.

``RefLlama``: RMSNorm, rotary embeddings, SwiGLU MLP, grouped KV heads, untied head.
"""

import torch
import torch.nn as nn
import torch.nn.functional as F


class _Block(nn.Module):
    def __init__(self, d, heads, ff):
        super().__init__()
        self.heads = heads
        self.ln1, self.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.fc, self.out = nn.Linear(d, ff), nn.Linear(ff, d)

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, D))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class RefGPT(nn.Module):
    def __init__(self, n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024, vocab_rows=None):
        super().__init__()
        rows = vocab_size if vocab_rows is None else vocab_rows
        self.vocab_size = vocab_size
        self.wte, self.wpe = nn.Embedding(rows, d_model), nn.Embedding(seq_len, d_model)
        self.blocks = nn.ModuleList(_Block(d_model, n_head, 4 * d_model) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, rows, bias=False)
        self.head.weight = self.wte.weight
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, 0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, idx, targets):
        x = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        logits = self.head(self.ln_f(x))
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))


class _RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def _rope(x, cos, sin):
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)


class _LlamaLayer(nn.Module):
    def __init__(self, d, heads, kv_heads, ff):
        super().__init__()
        hd = d // heads
        self.heads, self.kv, self.hd = heads, kv_heads, hd
        self.norm1, self.norm2 = _RMSNorm(d), _RMSNorm(d)
        self.wq = nn.Linear(d, heads * hd, bias=False)
        self.wk = nn.Linear(d, kv_heads * hd, bias=False)
        self.wv = nn.Linear(d, kv_heads * hd, bias=False)
        self.wo = nn.Linear(heads * hd, d, bias=False)
        self.w_gate = nn.Linear(d, ff, bias=False)
        self.w_up = nn.Linear(d, ff, bias=False)
        self.w_down = nn.Linear(ff, d, bias=False)

    def forward(self, x, cos, sin):
        B, T, _ = x.shape
        h = self.norm1(x)
        q = self.wq(h).view(B, T, self.heads, self.hd).transpose(1, 2)
        k = self.wk(h).view(B, T, self.kv, self.hd).transpose(1, 2)
        v = self.wv(h).view(B, T, self.kv, self.hd).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv != self.heads)
        x = x + self.wo(a.transpose(1, 2).reshape(B, T, -1))
        h = self.norm2(x)
        return x + self.w_down(F.silu(self.w_gate(h)) * self.w_up(h))


class RefLlama(nn.Module):
    def __init__(self, n_layer=24, n_head=16, n_kv_head=16, d_model=2048, d_ff=5504, vocab_size=32000, seq_len=2048,
                 rope_theta=10000.0):  # fmt: skip
        super().__init__()
        self.hd, self.theta = d_model // n_head, rope_theta
        self.embed = nn.Embedding(vocab_size, d_model)
        self.layers = nn.ModuleList(_LlamaLayer(d_model, n_head, n_kv_head, d_ff) for _ in range(n_layer))
        self.norm = _RMSNorm(d_model)
        self.head = nn.Linear(d_model, vocab_size, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, 0.0, 0.02)

    def forward(self, idx, targets):
        x = self.embed(idx)
        T = idx.shape[1]
        inv = 1.0 / (self.theta ** (torch.arange(0, self.hd, 2, device=idx.device, dtype=torch.float32) / self.hd))
        ang = torch.outer(torch.arange(T, device=idx.device, dtype=torch.float32), inv)
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        for layer in self.layers:
            x = layer(x, cos, sin)
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.float().view(-1, logits.size(-1)), targets.reshape(-1))


def split(model):
    """``(matrices, rest)``: 2-D weights inside the transformer blocks / layers, and everything else."""
    mats, rest = [], []
    for name, p in model.named_parameters():
        in_block = name.startswith("blocks.") or name.startswith("layers.") or ".blocks." in name or ".layers." in name
        (mats if (p.ndim >= 2 and in_block) else rest).append(p)
    return mats, rest
