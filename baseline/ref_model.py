"""Plain-PyTorch GPT-2-shaped decoder used by the reference arm of ``bench.py``.

Deliberately independent of the ``heavyball_b200`` package so that the reference arm touches none of
its code: standard ``torch.nn`` modules only.  Architecture: LayerNorm, learned positions, fused QKV,
GELU(tanh) MLP, tied embeddings; weights N(0, 0.02), biases zero.
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
    def __init__(self, n_layer=12, n_head=12, d_model=768, vocab_size=50257, seq_len=1024):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab_size, d_model), nn.Embedding(seq_len, d_model)
        self.blocks = nn.ModuleList(_Block(d_model, n_head, 4 * d_model) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(d_model)
        self.head = nn.Linear(d_model, vocab_size, bias=False)
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


def split(model):
    mats, rest = [], []
    for name, p in model.named_parameters():
        (mats if (p.ndim >= 2 and name.startswith("blocks.")) else rest).append(p)
    return mats, rest
