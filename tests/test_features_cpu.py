"""Feature tests on the CPU: error-compensated (ECC) state and parameters through whole optimizers,
Hessian-vector-product modes of the PSGD family, parameter EMA, per-group overrides.
Modelled on the reference's ``test/test_ecc.py``, ``test/test_ema.py``, ``test/test_closure.py`` and the
Newton-PSGD cases of ``test/test_toy_training.py``."""

import copy

import pytest
import torch

import heavyball_b200 as hb


def _problem(seed=0, n=24):
    torch.manual_seed(seed)
    w = torch.nn.Parameter(torch.randn(n, n) * 0.3)
    target = torch.randn(n, n)
    return w, target


def _loss(w, target):
    return ((w @ w.mT) - target).square().mean()


def _run(opt, w, target, steps):
    for _ in range(steps):
        _loss(w, target).backward()
        opt.step()
        opt.zero_grad()
    return w.detach().float().clone()


def _views(opt):
    for per_param in opt.state.values():
        for key, view in per_param.items():
            if isinstance(view, dict):
                yield view


@pytest.mark.parametrize("mode,narrow,corr", [("bf16+8", torch.bfloat16, torch.int8), ("bf16+16", torch.bfloat16, torch.int16),
                                              ("fp16+8", torch.float16, torch.int8)])  # fmt: skip
def test_ecc_state_is_narrow_plus_correction_and_tracks_fp32(mode, narrow, corr):
    w0, target = _problem()
    ref = _run(hb.AdamW([w0], lr=1e-2), w0, target, 30)
    w1, _ = _problem()
    opt = hb.AdamW([w1], lr=1e-2, ecc=mode)
    got = _run(opt, w1, target, 30)
    seen = 0
    for view in _views(opt):
        for key, value in view.items():
            if key.endswith("::ecc"):
                assert value.dtype == corr
                assert view[key[: -len("::ecc")]].dtype == narrow
                seen += 1
    assert seen >= 2  # both Adam moments carry a correction tensor
    assert (got - ref).abs().max() < 2e-3 * ref.abs().max().clamp(min=1.0)

    saved = copy.deepcopy(opt.state_dict())
    w2, _ = _problem()
    clone = hb.AdamW([w2], lr=1e-2, ecc=mode)
    clone.load_state_dict(saved)
    for view in _views(clone):
        for key, value in view.items():
            if key.endswith("::ecc"):
                assert value.dtype == corr and view[key[: -len("::ecc")]].dtype == narrow


def test_param_ecc_keeps_bf16_parameters_close_to_the_fp32_trajectory():
    w0, target = _problem()
    ref = _run(hb.AdamW([w0], lr=3e-3), w0, target, 60)
    w1, _ = _problem()
    opt = hb.AdamW([w1], lr=3e-3, param_ecc="bf16+8")
    assert w1.dtype == torch.bfloat16  # cast at construction
    got = _run(opt, w1, target, 60)
    w2, _ = _problem()
    w2.data = w2.data.bfloat16()
    plain = _run(hb.AdamW([w2], lr=3e-3), w2, target, 60)
    assert any(any(k.endswith("::ecc") for k in view) for view in _views(opt))
    # the correction term buys accuracy over plain bf16 parameters
    assert (got - ref).abs().mean() < (plain - ref).abs().mean()


@pytest.mark.parametrize("finite_differences", [False, True])
def test_newton_psgd_uses_hessian_vector_products(finite_differences):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(6, 6) * 0.5)
    target = torch.randn(6, 6)
    opt = hb.PSGDKron([w], lr=5e-2, preconditioner_update_probability=1.0)
    opt.hessian_approx = True
    opt.finite_differences = finite_differences
    opt.hvp_interval = 2
    calls = []

    def closure():
        calls.append(1)
        loss = _loss(w, target)
        loss.backward(create_graph=not finite_differences)
        return loss

    first = float(_loss(w, target))
    for _ in range(12):
        opt.step(closure)
        opt.zero_grad()
    assert float(_loss(w, target)) < first
    # finite differences evaluate the closure twice on the steps that take a Hessian-vector product
    assert len(calls) > 12 if finite_differences else len(calls) == 12


def test_hessian_approx_needs_a_closure():
    w, target = _problem(n=4)
    opt = hb.PSGDKron([w], lr=1e-2)
    opt.hessian_approx = True
    _loss(w, target).backward()
    with pytest.raises((ValueError, RuntimeError)):
        opt.step()


def test_parameter_ema_follows_and_swaps():
    w, target = _problem(n=8)
    opt = hb.AdamW([w], lr=1e-2)
    opt.ema_decay = 0.5
    for _ in range(5):
        _loss(w, target).backward()
        opt.step()
        opt.zero_grad()
        opt.ema_update()
    live = w.detach().clone()
    opt.copy_emas_to_params()
    averaged = w.detach().clone()
    assert not torch.equal(live, averaged)
    assert (averaged - live).abs().max() < (live.abs().max() + 1)  # an average of recent iterates, not garbage
    opt.copy_params_to_emas()
    opt.copy_emas_to_params()
    assert torch.equal(w.detach(), averaged)


def test_per_group_options_override_defaults():
    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(8, 8))
    b = torch.nn.Parameter(torch.randn(8, 8))
    opt = hb.AdamW([{"params": [a], "lr": 0.0}, {"params": [b], "ecc": "bf16+8"}], lr=1e-2)
    a0, b0 = a.detach().clone(), b.detach().clone()
    for p in (a, b):
        p.grad = torch.ones_like(p)
    opt.step()
    assert torch.equal(a.detach(), a0) and not torch.equal(b.detach(), b0)
    ecc_owners = [p for p, per in opt.state.items() if any(k.endswith("::ecc") for v in per.values() if isinstance(v, dict) for k in v)]
    assert len(ecc_owners) == 1 and ecc_owners[0] is b


def test_segmented_reduction_call_sites_fall_back_on_cpu():
    """OrthoGrad's projection and the Kron factor balance take their PyTorch definitions where the segmented
    reduction kernels do not apply."""
    import torch

    from heavyball_b200.utils import core, first_order, psgd

    torch.manual_seed(0)
    assert core._segmented_dot([torch.randn(3)], [torch.randn(3)]) is None
    assert core._segmented_absmax_rows([torch.randn(3, 3)]) is None
    w, g = [torch.randn(8, 4)], [torch.randn(8, 4)]
    out = [g[0].clone()]
    first_order.orthogonalize_grad_to_param(w, out, 1e-30, graft=False)
    ref = g[0] - ((w[0] * g[0]).sum() / ((w[0] * w[0]).sum() + 1e-30)) * w[0]
    assert torch.allclose(out[0], ref, atol=1e-6)
    assert abs((out[0] * w[0]).sum().item()) < 1e-4

    q = [torch.randn(2, 5, 5) * 4.0, torch.randn(2, 5) * 0.1]
    before = [torch.einsum("bij,bk->bijk", q[0], q[1]).clone()]
    psgd.psgd_balance_Q(q)
    assert torch.allclose(q[0].abs().amax((1, 2)), q[1].abs().amax(1), rtol=1e-5)  # common max-abs per slot
    assert torch.allclose(torch.einsum("bij,bk->bijk", q[0], q[1]), before[0], rtol=1e-4, atol=1e-6)  # product unchanged


@pytest.mark.parametrize("name", ["AdamW", "LaProp", "Muon", "SOAP", "PSGDKron", "SFAdamW"])
def test_stepping_from_backward_hooks_follows_the_explicit_loop(name):
    """``hook_optimizer_into_model`` steps every parameter as soon as its gradient is complete; the loss curve is the
    one of an explicit ``step()`` / ``zero_grad()`` loop (per-parameter optimizers see the same gradients)."""
    import heavyball_b200 as hb
    from heavyball_b200 import utils

    cls = getattr(hb, name)
    curves = []
    for hooked in (False, True):
        torch.manual_seed(0x2131290)
        model = torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh(), torch.nn.Linear(16, 16))
        kwargs = dict(lr=1e-3, weight_decay=1e-4, warmup_steps=4)
        if hooked:
            utils.hook_optimizer_into_model(model, cls, **kwargs)
        else:
            opt = cls(model.parameters(), **kwargs)
        data = torch.Generator().manual_seed(7)
        losses = []
        for _ in range(12):
            loss = model(torch.randn(64, 16, generator=data)).square().mean()
            loss.backward()
            if not hooked:
                opt.step()
                opt.zero_grad()
            losses.append(float(loss.detach()))
        curves.append(losses)
    for a, b in zip(*curves):
        assert abs(a - b) <= 0.05 * abs(a) + 1e-6
    assert curves[1][-1] < curves[1][0]
