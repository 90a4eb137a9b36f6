"""CPU unit tests of the numerical primitives against closed-form PyTorch math.

Invariants follow the reference's CPU tier (``test/test_utils_cpu.py``, ``test/test_stochastic_utils_cpu.py``,
``test/test_utils_property.py``, ``test/test_ecc.py:66-82``, ``test/test_psgd_precond_init_stability.py``).
"""

import math

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import utils


def test_stochastic_round_is_unbiased():
    torch.manual_seed(0)
    x = torch.full((200_000,), 1.0 + 2.0**-10)  # sits 1/8 of the way between two bf16 neighbours
    r = utils.stochastic_round_(x).float()
    assert set(r.unique().tolist()) <= {1.0, 1.0 + 2.0**-7}
    assert abs(r.mean().item() - x[0].item()) < 2e-5


def test_stochastic_accumulation_beats_nearest_rounding():
    torch.manual_seed(0)
    acc_sr = torch.zeros(4096, dtype=torch.bfloat16)
    acc_rne = torch.zeros(4096, dtype=torch.bfloat16)
    inc = torch.full((4096,), 1e-3)
    for _ in range(2048):
        utils.stochastic_add_([acc_sr], [inc])
        acc_rne.add_(inc.bfloat16())
    exact = 2048 * 1e-3
    assert abs(acc_sr.float().mean().item() - exact) < 0.02 * exact
    assert abs(acc_rne.float().mean().item() - exact) > 0.2 * exact  # nearest rounding stalls


def test_dither_steps_setting_is_read_at_call_time():
    torch.manual_seed(0)
    x = torch.full((100_000,), 1.5 + 2.0**-9)  # away from a binade edge
    old = utils.dither_steps
    try:
        utils.dither_steps = 2
        r = utils.stochastic_round_(x).float()
    finally:
        utils.dither_steps = old
    assert abs(r.mean().item() - x[0].item()) < 5e-5


@pytest.mark.parametrize("mode", ["bf16+8", "bf16+16", "fp16+8", "fp16+16"])
def test_ecc_round_trip_error_bound(mode):
    torch.manual_seed(0)
    cfg = hb.chainable.ECCConfig(mode)
    x = torch.randn(50_000) * torch.logspace(-6, 3, 50_000)
    if cfg.primary_dtype == torch.float16:
        x = x.clamp(-6e4, 6e4)
    narrow = torch.zeros_like(x, dtype=cfg.primary_dtype)
    corr = torch.zeros_like(x, dtype=cfg.corr_dtype)
    st = utils._ULPState(corr, cfg.smax)
    st.encode(x, narrow)
    back = st.decode(narrow)
    ulp = torch.exp2(utils._log_ulp(narrow).float())
    # residual resolution is ulp / (2 smax); stochastic floor adds at most one unit
    assert ((back - x).abs() <= ulp / (2 * cfg.smax) * 1.01 + 1e-45).all()
    plain = (narrow.float() - x).abs().mean()
    assert (back - x).abs().mean() < plain / 20


def test_ecc_encode_is_unbiased():
    torch.manual_seed(0)
    cfg = hb.chainable.ECCConfig("bf16+8")
    x = torch.full((100_000,), 0.1234567)
    narrow = torch.zeros_like(x, dtype=torch.bfloat16)
    corr = torch.zeros_like(x, dtype=torch.int8)
    st = utils._ULPState(corr, cfg.smax)
    st.encode(x, narrow)
    assert abs(st.decode(narrow).mean().item() - 0.1234567) < 1e-7


def test_promote_and_copy_stochastic_dispatch():
    x = torch.randn(8, dtype=torch.bfloat16)
    assert utils.promote(x).dtype == torch.float32
    assert utils.promote(torch.bfloat16) == torch.float32
    assert utils.promote(torch.float64) == torch.float64
    tgt = torch.zeros(8)
    utils.copy_stochastic_(tgt, torch.arange(8.0))
    assert torch.equal(tgt, torch.arange(8.0))


@pytest.mark.parametrize("backend", ["eps_add", "eps_clamp", "atan2", "nan_to_0"])
def test_division_backends(backend):
    x, y = torch.tensor([1.0, -2.0, 0.0, 3.0]), torch.tensor([2.0, 0.5, 0.0, 1e-20])
    out = x.clone()
    utils.stochastic_divide_with_eps_(out, y, 1e-6, backend=backend)
    assert torch.isfinite(out).all()
    if backend == "eps_clamp":
        torch.testing.assert_close(out, x / y.clamp(min=1e-6))
    if backend == "nan_to_0":
        assert out[2] == 0
    with pytest.raises(ValueError):
        utils.stochastic_divide_with_eps_(x.clone(), y, backend="nope")


def test_beta_debias_makes_ema_unbiased():
    beta, vals = 0.9, [3.0, 3.0, 3.0, 3.0]
    ema = 0.0
    for t, v in enumerate(vals, 1):
        b = utils.beta_debias(beta, t)
        ema = ema * b + v * (1 - b)
        assert abs(ema - 3.0) < 1e-12


def test_clip_bounds():
    torch.manual_seed(0)
    xs = [torch.randn(64) * 10, torch.randn(8, 8) * 1e-3]
    out = utils.l2_clip_([x.clone() for x in xs], 1.0)
    assert out[0].norm() <= 1 + 1e-5 and torch.allclose(out[1], xs[1])
    out = utils.rmsnorm_clip_([x.clone() for x in xs], 0.5)
    assert out[0].square().mean().sqrt() <= 0.5 + 1e-5
    both = utils.global_l2norm_clip([x.clone() for x in xs], 2.0)
    assert math.sqrt(sum(x.square().sum().item() for x in both)) <= 2 + 1e-4
    tr = utils.trust_region_clip_([torch.tensor([-100.0, -0.01, 0.0, 0.01, 100.0])])[0]
    assert tr.abs().max() <= 2 and tr[2] == 0 and abs(tr[3] - 0.01) < 1e-3
    for fn in (utils.mu_law_compress, utils.a_law_compress, utils.softsign_compress):
        y = fn([torch.linspace(-3, 3, 13)])[0]
        assert (y[1:] >= y[:-1]).all() and y[6] == 0


def test_caution_mask_and_scale():
    g = torch.tensor([1.0, -1.0, 1.0, -1.0])
    u = torch.tensor([2.0, 2.0, -2.0, -2.0])
    out = utils.caution(g, u)
    torch.testing.assert_close(out, torch.tensor([4.0, 0.0, 0.0, -4.0]))  # 2 of 4 kept -> x2


def test_cautious_weight_decay_closed_form():
    p = torch.nn.Parameter(torch.tensor([1.0, -1.0, 1.0, -1.0]))
    u = torch.tensor([0.5, 0.5, -0.5, -0.5])
    utils.update_param_([p.data], [u], lr=0.1, decay=0.2, cautious_decay=True)
    want = torch.tensor([1.0 * (1 - 0.02) - 0.05, -1.0 - 0.05, 1.0 + 0.05, -1.0 * (1 - 0.02) + 0.05])
    torch.testing.assert_close(p.data, want)


def test_triu_line_round_trip():
    torch.manual_seed(0)
    q = [torch.randn(2, 5, 5).triu(), torch.randn(2, 7)]
    packed = utils.triu_to_line(q)
    assert packed[0][0] == (2, 5, 5) and packed[0][1].shape == (2, 15) and packed[1][0] is None
    back = utils.line_to_triu(packed)
    assert torch.equal(back[0], q[0]) and torch.equal(back[1], q[1])


def test_psgd_should_update_is_a_deterministic_accumulator():
    group = {}
    fired = [utils.psgd_should_update(group, 0.25) for _ in range(12)]
    assert sum(fired) == 3 and fired[3] and fired[7] and fired[11]
    sched = utils.precond_update_prob_schedule(flat_start=3, decay=0.5, min_prob=0.1)
    assert [sched(n) for n in (1, 3, 4, 5, 20)] == [1.0, 1.0, 0.5, 0.25, 0.1]


def test_dim_merger_and_merge_group():
    g = torch.zeros(128, 64, 3, 3)
    assert utils.dim_merger(g, 1024).shape == (128, 576)
    assert utils.dim_merger(g, 100).shape == (128, 64, 9)
    parts = utils.dim_merger(torch.zeros(4, 10, 6), 4, split=True)
    assert isinstance(parts, list) and sum(p.numel() for p in parts) == 240
    group = {"merge_dims": True, "max_precond_dim": 1024, "split": False}
    (v,) = utils.merge_group(group, torch.zeros(8, 4, 4))
    assert v.numel() == 128


def test_log_space_init_scale_is_stable():
    for mag in (1e-30, 1e-10, 1.0, 1e10):
        g = torch.full((1, 16), mag)
        s = utils.precond_init_scale(None, None, None, g, None, None, scale_max=float("inf"))
        want = max(mag, 1e-12) ** -0.25  # (mean |g|^4)^(-1/8), then the default power 0.5; |g| is floored at 1e-12
        assert math.isclose(s, want, rel_tol=1e-4), (mag, s, want)
    with pytest.raises(utils.PrecondInitError):
        utils.precond_init_scale(None, None, None, torch.zeros(1, 4), None, None)


def test_max_eigenvalue_and_singular_value_estimates():
    torch.manual_seed(0)
    a = torch.randn(3, 24, 24)
    spd = a @ a.mT + torch.eye(24)
    est = utils.max_eigenvalue_spd(spd, power_iter=16)
    exact = torch.linalg.eigvalsh(spd)[..., -1]
    assert ((est - exact).abs() / exact < 0.05).all()
    sv = utils.max_singular_value(a, power_iter=24)
    assert ((sv - torch.linalg.svdvals(a)[..., 0]).abs() / sv < 0.1).all()


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    g = torch.randn(16, 64)
    o = utils.zeropower_via_newtonschulz5(g)
    sv = torch.linalg.svdvals(o.float())
    assert sv.min() > 0.5 and sv.max() < 1.3
    tall = utils.inplace_orthogonal_(torch.randn(64, 16), scale_mode="scale")
    assert abs(torch.linalg.svdvals(tall).median().item() - 2.0) < 0.5  # max(1, 64/16) ** 0.5


def test_sam_step_and_hooks():
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.ones(4))
    p.grad = torch.full((4,), 2.0)
    (old,) = utils.sam_step([p], 0.1)
    assert torch.equal(old, torch.ones(4)) and torch.allclose(p.data, torch.full((4,), 1.2)) and p.grad.abs().sum() == 0

    model = torch.nn.Linear(3, 2)
    before = model.weight.detach().clone()
    opts = utils.hook_optimizer_into_model(model, hb.AdamW, lr=1e-2)
    model(torch.randn(5, 3)).sum().backward()
    assert len(opts) == 2 and not torch.equal(before, model.weight) and model.weight.grad is None

    model = torch.nn.Linear(3, 2)
    before = model.weight.detach().clone()
    utils.fused_hook(model.parameters(), hb.AdamW, lr=1e-2)
    model(torch.randn(5, 3)).sum().backward()
    assert not torch.equal(before, model.weight)


def test_panel_cholesky_qr_matches_householder_up_to_column_signs():
    """The batched QR used for eigenbasis refreshes on the GPU: orthonormal to rounding level and the
    same subspace sequence as Householder QR, also for a spectrum spanning 12 decades."""
    from heavyball_b200.utils.orthogonal import _panel_cholesky_qr

    torch.manual_seed(0)
    n = 160
    basis = torch.linalg.qr(torch.randn(3, n, n, dtype=torch.float64)).Q
    eye = torch.eye(n)
    for decades, noise in ((2, 1e-2), (12, 1e-3), (12, 1.0)):
        gg = (basis * torch.logspace(0, -decades, n, dtype=torch.float64)) @ basis.mT
        q_old = torch.linalg.qr(basis + noise * torch.randn(3, n, n, dtype=torch.float64)).Q
        power = (gg @ q_old).float()
        q = _panel_cholesky_qr(power)
        assert q is not None and q.shape == power.shape
        assert (q.mT @ q - eye).abs().max() < 5e-6
        if decades == 2:
            ref = torch.linalg.qr(power.double()).Q
            assert ((q.double() * ref).sum(-2).abs() - 1).abs().max() < 1e-4
    assert _panel_cholesky_qr(torch.zeros(2, 64, 64)) is None


# ---------------------------------------------------------------------------------------- overflow-safe roots (PSGD initial scale)


def _log_mean_pow(x64, power):
    """log(mean(|x|^power)) in fp64 through the log-sum-exp form (the direct power overflows for the cases below)."""
    logs = x64.abs().clamp(min=1e-300).log() * power
    return torch.logsumexp(logs, 0) - math.log(x64.numel())


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-2), (torch.float32, 1e-5), (torch.float64, 1e-10)])
def test_stable_exp_matches_exp_on_both_sides_of_zero(dtype, tol):
    x = torch.linspace(-10, 10, 41, dtype=torch.float64)
    got = utils.stable_exp(x.to(dtype)).double()
    want = x.to(dtype).double().exp()
    assert torch.allclose(got, want, rtol=tol, atol=0)


@pytest.mark.parametrize("scale", [1e-3, 1.0, 1e3])
@pytest.mark.parametrize("power", [1, 3, 7, 15])
@pytest.mark.parametrize("numel", [1, 4, 512])
def test_roots_of_power_means_do_not_overflow(numel, power, scale):
    """``mean_root`` = mean(|x|^p)^(-1/2p), ``divided_root`` = the ratio of two such roots (inverted): evaluated through
    logarithms, so 1e3^15 (far beyond fp32) is no problem."""
    gen = torch.Generator().manual_seed(numel * 31 + power)
    x = (torch.rand(numel, generator=gen) + 0.1) * scale
    y = (torch.rand(numel, generator=gen) + 0.1) * scale * 3
    x64, y64 = x.double(), y.double()
    lse = utils._lse_mean(x, power, 1e-30)
    assert torch.isfinite(lse).all()
    assert abs(float(lse) - float(_log_mean_pow(x64, power)) / power / 2) < 1e-4 * max(1.0, abs(float(lse)))
    root = utils.mean_root(x, power)
    want_root = math.exp(-float(_log_mean_pow(x64, power)) / power / 2)
    assert math.isfinite(float(root)) and abs(float(root) - want_root) < 1e-4 * want_root
    ratio = utils.divided_root(x, y, power, power)
    want_ratio = math.exp(float(_log_mean_pow(x64, power)) / power / 2 - float(_log_mean_pow(y64, power)) / power / 2)
    assert math.isfinite(float(ratio)) and abs(float(ratio) - want_ratio) < 1e-4 * want_ratio


# ---------------------------------------------------------------------------------------- spectral estimators


def _with_spectrum(rows, cols, decades, dtype=torch.float32, seed=0, rank=None):
    """``U diag(s) V^T`` with singular values spread log-uniformly over ``decades`` decades below 1 (``rank``: only that
    many are non-zero)."""
    gen = torch.Generator().manual_seed(seed)
    r = min(rows, cols)
    u = torch.linalg.qr(torch.randn(rows, r, generator=gen, dtype=torch.float64)).Q
    v = torch.linalg.qr(torch.randn(cols, r, generator=gen, dtype=torch.float64)).Q
    s = torch.logspace(0, -decades, r, dtype=torch.float64)
    if rank is not None:
        s[rank:] = 0
    return ((u * s) @ v.T).to(dtype)


@pytest.mark.parametrize("shape,decades,dtype,iters,rtol", [
    ((128, 128), 10, torch.float64, 20, 0.01),
    ((32, 32), 4, torch.float64, 8, 0.03),
    ((128, 96), 1, torch.float32, 20, 0.03),
    ((32, 48), 4, torch.float32, 8, 0.03),
    ((4, 4), 8, torch.float32, 8, 0.03),
    ((32, 32), 1, torch.bfloat16, 8, 0.1),
])  # fmt: skip
def test_largest_singular_value_by_power_iteration(shape, decades, dtype, iters, rtol):
    a = _with_spectrum(*shape, decades, dtype)
    want = float(torch.linalg.svdvals(a.double()).max())
    got = float(utils.max_singular_value(a, power_iter=iters))
    assert abs(got - want) <= rtol * want + 1e-6


@pytest.mark.parametrize("n", [32, 128, 512])
def test_largest_singular_value_of_rank_deficient_and_ill_conditioned_matrices(n):
    low_rank = _with_spectrum(n, n, 1, rank=max(1, n // 8))
    want = float(torch.linalg.svdvals(low_rank.double()).max())
    got = float(utils.max_singular_value(low_rank, power_iter=16))
    assert 0.92 * want <= got <= 1.01 * want  # a lower bound that closes slowly when the leading values are clustered
    idx = torch.arange(1, n + 1, dtype=torch.float64)
    hilbert = (1.0 / (idx[:, None] + idx[None, :] - 1)).float()  # condition number beyond any float format
    want = float(torch.linalg.svdvals(hilbert.double()).max())
    assert abs(float(utils.max_singular_value(hilbert, power_iter=16)) - want) <= 0.03 * want
    assert float(utils.max_singular_value(torch.zeros(n, n))) == 0.0


@pytest.mark.parametrize("n,decades,dtype,rtol", [(32, 0, torch.float64, 0.01), (32, 1, torch.float64, 0.1), (4, 4, torch.float64, 0.1),
                                                  (32, 0, torch.float32, 0.01), (64, 1, torch.float32, 0.5)])  # fmt: skip
def test_smallest_eigenvalue_of_a_symmetric_psd_matrix(n, decades, dtype, rtol):
    gen = torch.Generator().manual_seed(n)
    u = torch.linalg.qr(torch.randn(n, n, generator=gen, dtype=torch.float64)).Q
    a = ((u * torch.logspace(0, -decades, n, dtype=torch.float64)) @ u.T).to(dtype)
    want = float(torch.linalg.eigvalsh(a.double()).min())
    got = float(utils.min_singular_value(a, power_iter=20))
    assert abs(got - want) <= rtol * want + 1e-5
