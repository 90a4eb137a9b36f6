"""Model-side kernels against fp32 PyTorch definitions of the same op."""

import pytest
import torch
import torch.nn.functional as F

from heavyball_b200 import ops
from heavyball_b200.ops.nn import linear_cross_entropy

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,vocab,padded", [(64, 1000, 1024), (33, 50257, 50304), (7, 8, 8), (5, 509, 512)])
def test_cross_entropy_kernel_matches_fp32_definition(rows, vocab, padded):
    torch.manual_seed(0)
    logits = (torch.randn(rows, padded, device="cuda") * 3).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    targets[rows // 2] = -100
    ref_in = logits[:, :vocab].float().requires_grad_()
    ref = F.cross_entropy(ref_in, targets, reduction="none", ignore_index=-100)
    n_valid = (targets != -100).sum()
    (ref.sum() / n_valid).backward()

    scale = (1.0 / n_valid.float()).reshape(1)
    work = logits.clone()
    losses = ops.load().cross_entropy_(work, targets, scale, vocab, -100)
    assert torch.allclose(losses, ref, atol=2e-5, rtol=1e-5)
    assert losses[rows // 2] == 0
    grad = work.float()
    assert (grad[:, vocab:] == 0).all() and (grad[rows // 2] == 0).all()
    # bf16 storage of the gradient: relative error 2^-9 per element
    assert torch.allclose(grad[:, :vocab], ref_in.grad, atol=1e-7, rtol=1e-2)


def test_linear_cross_entropy_gradients_match_autograd_of_plain_ops():
    torch.manual_seed(1)
    d, vocab, rows_w = 96, 1001, 1024
    h = torch.randn(4, 20, d, device="cuda", requires_grad=True)
    w = (torch.randn(rows_w, d, device="cuda") * 0.05).requires_grad_()
    targets = torch.randint(0, vocab, (4, 20), device="cuda")
    loss = linear_cross_entropy(h, w, targets, vocab)
    loss.backward()

    h2 = h.detach().clone().requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    logits = (h2.to(torch.bfloat16) @ w2.to(torch.bfloat16).mT)[..., :vocab]
    ref = F.cross_entropy(logits.float().reshape(-1, vocab), targets.reshape(-1))
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-4
    assert torch.allclose(h.grad, h2.grad, atol=2e-4, rtol=5e-2)
    assert torch.allclose(w.grad, w2.grad, atol=2e-4, rtol=5e-2)
    assert (w.grad[vocab:] == 0).all()


def test_gpt_pads_its_vocabulary_and_trains():
    from heavyball_b200.models import GPT, GPTConfig

    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=2, n_head=2, d_model=64, vocab_size=1001, seq_len=32)).cuda()
    assert model.wte.weight.shape[0] == 1024
    x = torch.randint(0, 1001, (4, 32), device="cuda")
    y = torch.randint(0, 1001, (4, 32), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = model(x, y)
        assert model(x).shape == (4, 32, 1001)
    loss.backward()
    assert torch.isfinite(loss) and abs(loss.item() - 6.9) < 0.3
    assert (model.wte.weight.grad[1001:] == 0).all()


@pytest.mark.parametrize("shape", [(16, 1024, 768), (3, 5, 128), (1, 1, 1024), (2000, 384)])
@pytest.mark.parametrize("bf16", [False, True])
def test_layer_norm_kernels_match_fp32_definition(shape, bf16):
    from heavyball_b200.ops.nn import layer_norm

    torch.manual_seed(0)
    d = shape[-1]
    x = (torch.randn(*shape, device="cuda") * 2 + 0.5).requires_grad_()
    w = (torch.rand(d, device="cuda") + 0.5).requires_grad_()
    b = torch.randn(d, device="cuda").requires_grad_()
    dy = torch.randn(*shape, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf16):
        y = layer_norm(x, w, b, 1e-5)
    assert y.dtype == (torch.bfloat16 if bf16 else torch.float32)
    y.backward(dy.to(y.dtype))

    x2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, w, b))
    ref = F.layer_norm(x2, (d,), w2, b2, 1e-5)
    ref.backward(dy.to(y.dtype).float())
    tol = dict(atol=2e-2, rtol=2e-2) if bf16 else dict(atol=2e-5, rtol=1e-5)
    assert torch.allclose(y.float(), ref, **tol)
    assert torch.allclose(x.grad, x2.grad, atol=1e-4, rtol=1e-4)
    rows = x.numel() // d
    assert torch.allclose(w.grad, w2.grad, atol=1e-5 * rows**0.5 + 1e-4, rtol=1e-4)
    assert torch.allclose(b.grad, b2.grad, atol=1e-5 * rows**0.5 + 1e-4, rtol=1e-4)


def test_layer_norm_module_keeps_state_dict_and_falls_back():
    from heavyball_b200.ops.nn import LayerNorm

    ln = LayerNorm(100).cuda()  # row length not a multiple of 128: framework path
    assert set(ln.state_dict()) == {"weight", "bias"}
    x = torch.randn(4, 100, device="cuda")
    assert torch.allclose(ln(x), F.layer_norm(x, (100,), ln.weight, ln.bias, ln.eps))


@pytest.mark.parametrize("rows,cols", [(16384, 768), (1000, 3072), (7, 8), (33, 200)])
def test_column_sum_kernel_matches_fp32_sum(rows, cols):
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    got = ops.load().colsum_bf16(x)
    ref = x.double().sum(0)
    assert got.dtype == torch.float32 and got.shape == (cols,)
    assert torch.allclose(got.double(), ref, atol=1e-3 * rows**0.5, rtol=1e-5)


@pytest.mark.parametrize("n", [1, 3, 4])
def test_batched_column_sums_match_fp32_sum(n):
    torch.manual_seed(0)
    xs = [torch.randn(1000, 264, device="cuda").to(torch.bfloat16) for _ in range(n)]
    out = ops.load().colsum_bf16_batch(xs)
    ops.check_status()
    assert out.shape == (n * 264,) and out.dtype == torch.float32
    ref = torch.cat([x.float().sum(0) for x in xs])
    assert torch.allclose(out, ref, atol=2e-3, rtol=1e-5)


def test_linear_under_autocast_matches_framework_linear():
    from heavyball_b200.ops.nn import linear

    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device="cuda", requires_grad=True)
    w = (torch.randn(384, 256, device="cuda") * 0.05).requires_grad_()
    b = torch.randn(384, device="cuda").requires_grad_()
    dy = torch.randn(4, 96, 384, device="cuda")
    x2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, w, b))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = linear(x, w, b)
        y2 = F.linear(x2, w2, b2)
    assert y.dtype == torch.bfloat16 and torch.equal(y, y2)
    y.backward(dy.to(y.dtype))
    y2.backward(dy.to(y.dtype))
    assert x.grad.dtype == torch.float32 and w.grad.dtype == torch.float32 and b.grad.dtype == torch.float32
    assert torch.allclose(x.grad, x2.grad, atol=1e-2, rtol=1e-2)
    assert torch.allclose(w.grad, w2.grad, atol=5e-2, rtol=1e-2)
    # the kernel sums in fp32 and rounds once; the framework path rounds the bf16 result of its own fp32 sum
    assert torch.allclose(b.grad, b2.grad, atol=0.15, rtol=1e-2)
    exact = dy.to(torch.bfloat16).double().sum((0, 1))
    assert (b.grad.double() - exact).abs().max() <= (b2.grad.double() - exact).abs().max() + 0.1
    # outside autocast nothing changes
    assert torch.equal(linear(x.detach(), w.detach(), b.detach()), F.linear(x.detach(), w.detach(), b.detach()))


def test_split_linear_matches_fp32_definition_of_the_packed_projection():
    from heavyball_b200.ops.nn import split_linear

    torch.manual_seed(0)
    d, n = 256, 3
    x = torch.randn(4, 96, d, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(n * d, d, device="cuda") * 0.05).requires_grad_()
    b = torch.randn(n * d, device="cuda").requires_grad_()
    dys = [torch.randn(4, 96, d, device="cuda").to(torch.bfloat16) for _ in range(n)]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        outs = split_linear(x, w, b, n)
    assert len(outs) == n and all(o.is_contiguous() and o.dtype == torch.bfloat16 for o in outs)
    torch.autograd.backward(outs, dys)
    assert w.grad.dtype == torch.float32 and w.grad.shape == w.shape and b.grad.shape == b.shape

    # fp32 definition on the same bf16-rounded operands
    x2 = x.detach().float().requires_grad_()
    w2 = w.detach().to(torch.bfloat16).float().requires_grad_()
    b2 = b.detach().to(torch.bfloat16).float().requires_grad_()
    ref = F.linear(x2, w2, b2)
    ref.backward(torch.cat(dys, -1).float())
    for o, r in zip(outs, ref.split(d, -1)):
        assert torch.allclose(o.float(), r, atol=2e-2, rtol=1e-2)
    assert torch.allclose(w.grad, w2.grad, atol=1e-3, rtol=1e-4)  # fp32 straight out of the GEMM
    assert torch.allclose(b.grad, b2.grad, atol=1e-3, rtol=1e-4)
    assert torch.allclose(x.grad.float(), x2.grad, atol=3e-2, rtol=2e-2)  # bf16 accumulation across the three GEMMs

    # one output unused: its rows of the packed gradients are zero
    w.grad = b.grad = x.grad = None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        outs = split_linear(x, w, b, n)
    (outs[0].float() * dys[0].float()).sum().backward()
    assert torch.allclose(w.grad[:d], w2.grad[:d], atol=1e-3, rtol=1e-4)
    assert (w.grad[d:] == 0).all() and (b.grad[d:] == 0).all()
    # outside autocast: plain slices
    plain = split_linear(x.detach().float(), w.detach(), b.detach(), n)
    assert torch.allclose(torch.cat(plain, -1), F.linear(x.detach().float(), w.detach(), b.detach()), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("rows,cols", [(16384, 3072), (1000, 3072), (37, 8), (5, 264), (1, 512)])
def test_gelu_kernels_match_fp32_definition(rows, cols):
    torch.manual_seed(0)
    u = (torch.randn(rows, cols, device="cuda") * 3).to(torch.bfloat16)
    u[0, :8] = torch.tensor([0.0, -0.0, 30.0, -30.0, 200.0, -200.0, 1e-3, -1e-3], device="cuda").to(torch.bfloat16)
    dy = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    ext = ops.load()
    y = ext.gelu_fwd(u)
    du, db = ext.gelu_bwd(dy, u)
    ops.check_status()

    # float64 definition: the fp32 one loses 1 + tanh(z) to cancellation for u below about -4 (errors of 1e-6 in
    # the slope), which the kernel's logistic form does not
    uf = u.double().requires_grad_()
    ref = F.gelu(uf, approximate="tanh")
    ref.backward(dy.double())
    assert y.dtype == torch.bfloat16 and du.dtype == torch.bfloat16 and db.dtype == torch.float32
    # one rounding to bf16 (at most 2^-8 relative) on top of fp32 arithmetic
    assert torch.allclose(y.double(), ref.detach(), atol=2e-6, rtol=2.0**-7)
    assert torch.allclose(du.double(), uf.grad, atol=2e-6, rtol=2.0**-7)
    # fp32 sums of the unrounded products: the slope (of order 1, with a zero crossing near u = -0.75) carries an
    # absolute error of a few fp32 ulps, so the bound scales with sum |dy|
    bound = 5e-6 * dy.double().abs().sum(0) + 1e-7
    assert ((db.double() - uf.grad.sum(0)).abs() <= bound).all()


def test_linear_gelu_matches_the_two_framework_calls():
    from heavyball_b200.ops.nn import linear_gelu

    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device="cuda").to(torch.bfloat16).requires_grad_()
    w = (torch.randn(1024, 256, device="cuda") * 0.05).requires_grad_()
    b = torch.randn(1024, device="cuda").requires_grad_()
    dy = torch.randn(4, 96, 1024, device="cuda").to(torch.bfloat16)
    x2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, w, b))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = linear_gelu(x, w, b)
        y2 = F.gelu(F.linear(x2, w2, b2), approximate="tanh")
    assert y.dtype == torch.bfloat16 and torch.allclose(y.float(), y2.float(), atol=1e-6, rtol=2.0**-7)
    y.backward(dy)
    y2.backward(dy)
    assert w.grad.dtype == torch.float32 and b.grad.dtype == torch.float32
    assert torch.allclose(x.grad.float(), x2.grad.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(w.grad, w2.grad, atol=5e-2, rtol=1e-2)
    assert torch.allclose(b.grad, b2.grad, atol=0.15, rtol=1e-2)
    # outside autocast: the framework calls
    xd, wd, bd = x.detach().float(), w.detach(), b.detach()
    assert torch.equal(linear_gelu(xd, wd, bd), F.gelu(F.linear(xd, wd, bd), approximate="tanh"))


def test_cast_cache_follows_parameter_updates_made_by_the_kernels():
    """The optimizer kernels write parameters through raw pointers (no autograd version bump): the bf16 copies
    must still be current in the next forward pass."""
    import heavyball_b200 as hb
    from heavyball_b200.models import GPT, GPTConfig

    torch.manual_seed(0)
    model = GPT(GPTConfig(n_layer=1, n_head=2, d_model=128, vocab_size=512, seq_len=16)).cuda()
    opt = hb.AdamW(model.parameters(), lr=1e-2)
    x = torch.randint(0, 512, (2, 16), device="cuda")
    for _ in range(2):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(x, x)
        fc = model.blocks[0].fc
        assert fc.w16 is not None and torch.equal(fc.w16, fc.weight.detach().to(torch.bfloat16))
        assert torch.equal(fc.b16, fc.bias.detach().to(torch.bfloat16))
        before = fc.weight.detach().clone()
        loss.backward()
        opt.step()
        opt.zero_grad()
        assert not torch.equal(before, fc.weight.detach())
    assert not any("16" in k for k in model.state_dict())
    model(x)  # outside autocast the copies are dropped and F.linear runs
    assert model.blocks[0].fc.w16 is None


def test_graphed_forward_backward_matches_eager_launches():
    import copy

    from heavyball_b200.models import GPT, GPTConfig, graph_forward_backward

    torch.manual_seed(0)
    eager = GPT(GPTConfig(n_layer=2, n_head=2, d_model=128, vocab_size=1001, seq_len=32)).cuda()
    graphed = copy.deepcopy(eager)
    xs = [torch.randint(0, 1001, (4, 33), device="cuda") for _ in range(3)]
    graph_forward_backward(graphed, (xs[0][:, :-1], xs[0][:, 1:]))
    for x in xs:
        losses = []
        for model in (eager, graphed):
            model.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16, cache_enabled=False):
                loss = model(x[:, :-1], x[:, 1:])
            loss.backward()
            losses.append(loss.detach().float())
        assert torch.allclose(losses[0], losses[1], atol=1e-5)
        for (name, p), q in zip(eager.named_parameters(), graphed.parameters()):
            assert p.grad is not None and q.grad is not None, name
            assert torch.allclose(p.grad, q.grad, atol=1e-4, rtol=1e-3), name
        with torch.no_grad():  # move both models the same way, through raw parameter writes as an optimizer would
            for p, q in zip(eager.parameters(), graphed.parameters()):
                p.sub_(0.1 * p.grad)
                q.sub_(0.1 * q.grad)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("d", [384, 768, 1024])
def test_add_layer_norm_matches_separate_add_and_norm(bf16, d):
    from heavyball_b200.ops.nn import add_layer_norm

    torch.manual_seed(0)
    shape = (8, 96, d)
    x = torch.randn(*shape, device="cuda").requires_grad_()
    res = torch.randn(*shape, device="cuda").to(torch.bfloat16 if bf16 else torch.float32).requires_grad_()
    w = (torch.rand(d, device="cuda") + 0.5).requires_grad_()
    b = torch.randn(d, device="cuda").requires_grad_()
    ds, dy = torch.randn(*shape, device="cuda"), torch.randn(*shape, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=bf16):
        s, y = add_layer_norm(x, res, w, b, 1e-5)
    assert s.dtype == torch.float32 and y.dtype == (torch.bfloat16 if bf16 else torch.float32)
    torch.autograd.backward([s, y], [ds, dy.to(y.dtype)])

    x2, r2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, res, w, b))
    s2 = x2 + r2.float()
    y2 = F.layer_norm(s2, (d,), w2, b2, 1e-5)
    torch.autograd.backward([s2, y2], [ds, dy.to(y.dtype).float()])
    assert torch.allclose(s, s2, atol=1e-6)
    assert torch.allclose(y.float(), y2, **(dict(atol=2e-2, rtol=2e-2) if bf16 else dict(atol=2e-5, rtol=1e-5)))
    assert torch.allclose(x.grad, x2.grad, atol=1e-4, rtol=1e-4)
    assert res.grad.dtype == res.dtype
    if bf16:  # written by the backward kernel from the same fp32 values as dx
        assert torch.equal(res.grad, x.grad.to(torch.bfloat16))
    assert torch.allclose(res.grad.float(), r2.grad.float(), atol=3e-2 if bf16 else 1e-4, rtol=2e-2 if bf16 else 1e-4)
    assert torch.allclose(w.grad, w2.grad, atol=2e-3, rtol=1e-4) and torch.allclose(b.grad, b2.grad, atol=2e-3, rtol=1e-4)
    # only the sum used downstream: the gradient passes straight through
    x3 = x.detach().clone().requires_grad_()
    s3, _ = add_layer_norm(x3, res.detach(), w.detach(), b.detach(), 1e-5)
    s3.backward(ds)
    assert torch.equal(x3.grad, ds)
