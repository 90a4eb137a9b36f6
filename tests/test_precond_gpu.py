"""Second-order optimizers on the GPU: the batched QR of the eigenbasis refresh against Householder QR,
and SOAP trajectories with either of them."""

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import utils
from heavyball_b200.utils.orthogonal import _panel_cholesky_qr

pytestmark = pytest.mark.gpu


def _spd_power_iterate(n, batch, decades, noise, seed=0):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    basis = torch.linalg.qr(torch.randn(batch, n, n, device="cuda", dtype=torch.float64, generator=gen)).Q
    gg = (basis * torch.logspace(0, -decades, n, device="cuda", dtype=torch.float64)) @ basis.mT
    q_old = torch.linalg.qr(basis + noise * torch.randn(batch, n, n, device="cuda", dtype=torch.float64, generator=gen)).Q
    return (gg @ q_old).float()


@pytest.mark.parametrize("decades,noise", [(2, 1e-2), (10, 1e-3), (20, 1.0)])
def test_panel_qr_is_orthonormal_and_matches_householder(decades, noise):
    power = _spd_power_iterate(512, 4, decades, noise)
    q = _panel_cholesky_qr(power)
    assert q is not None
    eye = torch.eye(512, device="cuda")
    assert (q.mT @ q - eye).abs().max().item() < 1e-5
    if decades == 2:
        ref = torch.linalg.qr(power.double()).Q
        assert ((q.double() * ref).sum(-2).abs() - 1).abs().max().item() < 1e-4


def _train(fast, steps=6):
    torch.manual_seed(0)
    utils.fast_qr = fast
    try:
        ws = [torch.nn.Parameter(torch.randn(128, 96, device="cuda") * 0.1) for _ in range(3)]
        target = [torch.randn_like(w) for w in ws]
        opt = hb.SOAP(ws, lr=1e-2, precondition_frequency=2, warmup_steps=0)
        for _ in range(steps):
            loss = sum(((w @ w.mT @ t - t) ** 2).mean() for w, t in zip(ws, target))
            loss.backward()
            opt.step()
            opt.zero_grad()
        return [w.detach().clone() for w in ws]
    finally:
        utils.fast_qr = True


def test_soap_trajectory_does_not_depend_on_qr_flavour():
    """Column signs of the eigenbasis cancel in the update, so both QR routes give the same parameters."""
    a, b = _train(True), _train(False)
    for x, y in zip(a, b):
        assert torch.isfinite(x).all()
        assert (x - y).abs().max().item() < 2e-3 * y.abs().max().item()
