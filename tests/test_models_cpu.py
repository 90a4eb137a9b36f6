"""Model families on the CPU (the framework-op fallbacks of every model-side kernel): shapes, padded vocabulary,
loss against the plain PyTorch formulation, grouped-query Llama, parameter grouping, a few optimizer steps."""

import math

import pytest
import torch
import torch.nn.functional as F

import heavyball_b200 as hb
from heavyball_b200.models import GPT, GPTConfig, Llama, LlamaConfig, split_param_groups
from heavyball_b200.models.gpt import padded_vocab
from heavyball_b200.ops.nn import add_layer_norm, layer_norm, linear, linear_cross_entropy, linear_gelu


def test_padded_vocab():
    assert padded_vocab(50257, 64) == 50304 and padded_vocab(50304, 64) == 50304 and padded_vocab(7, 1) == 7


def test_gpt_logits_and_loss_agree_with_plain_formulation():
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=2, n_head=2, d_model=64, vocab_size=1001, seq_len=32))
    assert model.wte.weight.shape == (1024, 64) and model.head.weight is model.wte.weight
    assert torch.count_nonzero(model.wte.weight[1001:]) == 0
    x = torch.randint(0, 1001, (3, 32))
    y = torch.randint(0, 1001, (3, 32))
    logits = model(x)
    assert logits.shape == (3, 32, 1001)
    loss = model(x, y)
    assert torch.allclose(loss, F.cross_entropy(logits.reshape(-1, 1001), y.reshape(-1)), atol=1e-5)
    assert abs(loss.item() - math.log(1001)) < 0.3
    loss.backward()
    assert torch.count_nonzero(model.wte.weight.grad[1001:]) == 0  # padding rows never move
    assert all(p.grad is not None for p in model.parameters())


def test_fallback_ops_are_the_framework_ops():
    torch.manual_seed(0)
    x, r = torch.randn(4, 10, 128), torch.randn(4, 10, 128)
    w, b = torch.rand(128) + 0.5, torch.randn(128)
    assert torch.equal(layer_norm(x, w, b, 1e-5), F.layer_norm(x, (128,), w, b, 1e-5))
    s, y = add_layer_norm(x, r, w, b, 1e-5)
    assert torch.equal(s, x + r) and torch.equal(y, F.layer_norm(x + r, (128,), w, b, 1e-5))
    s0, y0 = add_layer_norm(x, None, w, b, 1e-5)
    assert s0 is x and torch.equal(y0, F.layer_norm(x, (128,), w, b, 1e-5))
    lw, lb = torch.randn(32, 128), torch.randn(32)
    assert torch.equal(linear(x, lw, lb), F.linear(x, lw, lb))
    assert torch.equal(linear_gelu(x, lw, lb), F.gelu(F.linear(x, lw, lb), approximate="tanh"))
    t = torch.randint(0, 30, (4, 10))
    t[0, 0] = -100
    ref = F.cross_entropy(F.linear(x, lw)[..., :30].reshape(-1, 30), t.reshape(-1), ignore_index=-100)
    assert torch.allclose(linear_cross_entropy(x, lw, t, 30), ref, atol=1e-6)


@pytest.mark.parametrize("n_kv", [4, 2, 1])
def test_llama_with_grouped_kv_heads_trains(n_kv):
    torch.manual_seed(0)
    cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=n_kv, d_model=64, d_ff=128, vocab_size=256, seq_len=16)
    model = Llama(cfg)
    assert model.layers[0].wk.weight.shape == (n_kv * 16, 64)
    x = torch.randint(0, 256, (2, 16))
    assert model(x).shape == (2, 16, 256)
    mats, rest = split_param_groups(model)
    assert all(p.ndim == 2 for p in mats) and len(mats) == 2 * 7
    assert any(p is model.embed.weight for p in rest) and any(p is model.head.weight for p in rest)
    opt = hb.SplitOpt([{"params": mats, "optimizer": hb.Muon, "lr": 0.02}, {"params": rest, "optimizer": hb.AdamW, "lr": 3e-3}])
    losses = []
    for _ in range(8):
        loss = model(x, x)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    assert losses[-1] < losses[0] and all(math.isfinite(v) for v in losses)


def test_gpt_causality():
    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=1, n_head=2, d_model=32, vocab_size=50, seq_len=8)).eval()
    a = torch.randint(0, 50, (1, 8))
    b = a.clone()
    b[0, -1] = (b[0, -1] + 1) % 50
    la, lb = model(a), model(b)
    assert torch.allclose(la[:, :-1], lb[:, :-1], atol=1e-6) and not torch.allclose(la[:, -1], lb[:, -1])


def test_split_linear_node_matches_autograd_of_the_packed_projection():
    """The single autograd node behind the packed q / k / v projection, driven directly (on CPU the public entry
    point takes the plain path): gradients equal those of one ``F.linear`` on the same bf16 operands."""
    from heavyball_b200.ops.nn import _SplitLinearFn, split_linear

    torch.manual_seed(0)
    x = torch.randn(4, 10, 32).to(torch.bfloat16).requires_grad_()
    w = torch.randn(96, 32, requires_grad=True)
    b = torch.randn(96, requires_grad=True)
    w16, b16 = w.detach().to(torch.bfloat16), b.detach().to(torch.bfloat16)
    outs = _SplitLinearFn.apply(x, w, b, w16, b16, 3)
    dys = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, dys)
    x2, w2, b2 = x.detach().float().requires_grad_(), w16.float().requires_grad_(), b16.float().requires_grad_()
    F.linear(x2, w2, b2).backward(torch.cat(dys, -1).float())
    assert w.grad.dtype == torch.float32 and b.grad.dtype == torch.float32 and x.grad.dtype == torch.bfloat16
    assert torch.allclose(w.grad, w2.grad, atol=0.1, rtol=2e-2)
    assert torch.allclose(b.grad, b2.grad, atol=1e-4)
    assert torch.allclose(x.grad.float(), x2.grad, atol=0.2, rtol=2e-2)
    plain = split_linear(x.detach().float(), w.detach(), b.detach(), 3)
    assert torch.allclose(torch.cat(plain, -1), F.linear(x.detach().float(), w.detach(), b.detach()), atol=1e-5)
    with pytest.raises(ValueError):
        split_linear(x.detach().float(), w.detach(), b.detach(), 5)
