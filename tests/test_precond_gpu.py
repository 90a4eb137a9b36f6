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


def test_recursive_triangular_solve_matches_library():
    """PSGD's ``V Q^-1``: recursion over column blocks with tensor-core products against cuBLAS TRSM."""
    from heavyball_b200.utils.psgd import _solve_right_upper

    torch.manual_seed(0)
    for d, rows in ((1024, 512), (640, 300), (100, 64)):
        q = torch.randn(4, d, d, device="cuda").triu() * 0.05 + torch.eye(d, device="cuda") * 2
        b = torch.randn(4, rows, d, device="cuda")
        got = _solve_right_upper(q, b)
        ref = torch.linalg.solve_triangular(q.double(), b.double(), upper=True, left=False)
        lib = torch.linalg.solve_triangular(q, b, upper=True, left=False)
        err = (got.double() - ref).abs().max().item()
        lib_err = (lib.double() - ref).abs().max().item()
        assert err < max(20 * lib_err, 1e-4), (d, err, lib_err)
    hb.ops.check_status()


def test_psgd_kron_steps_with_tensor_core_products_match_library_products():
    def run(flag):
        utils.tensor_core_matmul = flag
        try:
            torch.manual_seed(0)
            ws = [torch.nn.Parameter(torch.randn(256, 192, device="cuda") * 0.1) for _ in range(2)]
            opt = hb.PSGDKron(ws, lr=1e-3, preconditioner_update_probability=1.0)
            for _ in range(4):
                torch.manual_seed(1)
                loss = sum((w @ w.mT).square().mean() for w in ws)
                loss.backward()
                opt.step()
                opt.zero_grad()
            return [w.detach().clone() for w in ws]
        finally:
            utils.tensor_core_matmul = True

    a, b = run(True), run(False)
    for x, y in zip(a, b):
        assert torch.isfinite(x).all()
        assert (x - y).abs().max().item() < 1e-3 * y.abs().max().item()


@pytest.mark.parametrize("n,k,m,p", [(1024, 1024, 512, 32), (1000, 300, 7, 32), (130, 64, 64, 32), (4096, 256, 224, 20)])
def test_tall_skinny_products_match_matmul(n, k, m, p):
    ext = hb.ops.load()
    torch.manual_seed(0)
    base = torch.randn(3, n, k, device="cuda")
    w = torch.randn(3, n, p, device="cuda")
    parts = ext.tall_t_mul(base, m, w)
    ref = base[..., :m].double().mT @ w.double()
    assert parts.shape[1:] == (3, m, p)
    assert torch.allclose(parts.sum(0).double(), ref, atol=1e-3, rtol=1e-4)


def test_cholesky_qr2_fast_path_and_its_failure_flag():
    """Well-conditioned refresh inputs take two rounds of Cholesky QR (matrix products only); badly conditioned ones are
    flagged on the device, and ``_qr_basis`` then climbs to the variants with shifted rounds in front (or, past those,
    to the panel-wise method)."""
    from heavyball_b200.utils import orthogonal
    from heavyball_b200.utils.orthogonal import _cholesky_qr2, _qr_basis

    eye = torch.eye(512, device="cuda")
    easy = _spd_power_iterate(512, 4, 2, 1e-2)
    q, bad = _cholesky_qr2(easy)
    assert int(bad.sum()) == 0
    assert (q.mT @ q - eye).abs().max().item() < 3e-5
    ref = torch.linalg.qr(easy.double()).Q
    assert ((q.double() * ref).sum(-2).abs() - 1).abs().max().item() < 1e-4
    hard = _spd_power_iterate(512, 4, 20, 1.0)
    _, bad = _cholesky_qr2(hard)
    assert int(bad.sum()) > 0
    before = dict(orthogonal.qr_stats)
    q = _qr_basis(hard)
    assert (q.mT @ q - eye).abs().max().item() < 1e-4
    assert orthogonal.qr_stats["cholesky_qr2"] == before["cholesky_qr2"]  # the plain variant was refused ...
    assert sum(orthogonal.qr_stats.values()) == sum(before.values()) + 1  # ... and exactly one other route produced it
    for _ in range(3):  # replayed from its graph from the second call on
        q = _qr_basis(easy)
    assert (q.mT @ q - eye).abs().max().item() < 3e-5


@pytest.mark.parametrize("decades,shifted", [(2, 0), (5, 1), (7, 3)])
def test_shifted_cholesky_qr_reaches_worse_conditioning(decades, shifted):
    """Every variant returns the Householder factor's Q (up to column signs) while the input is within its reach."""
    from heavyball_b200.utils.orthogonal import _cholesky_qr2

    torch.manual_seed(decades)
    n = 512
    u = torch.linalg.qr(torch.randn(2, n, n, device="cuda", dtype=torch.float64)).Q
    v = torch.linalg.qr(torch.randn(2, n, n, device="cuda", dtype=torch.float64)).Q
    a = (u * torch.logspace(0, -decades, n, device="cuda", dtype=torch.float64)) @ v.mT
    q, bad = _cholesky_qr2(a.float(), shifted)
    assert int(bad.sum()) == 0
    assert (q.mT @ q - torch.eye(n, device="cuda")).abs().max().item() < 1e-4
    if decades <= 5:  # beyond that the trailing columns of the fp32 input are rounding noise in any method
        ref = torch.linalg.qr(a).Q
        assert ((q.double() * ref).sum(-2).abs() - 1).abs().max().item() < 1e-2


@pytest.mark.parametrize("n", [128, 300, 1024])
def test_blocked_cholesky_with_the_leaf_kernel(n):
    """128-wide leaves are factored and inverted by one kernel for the whole batch; the inverses serve every solve of
    the recursion.  A matrix that is not positive definite is counted, the others are unaffected."""
    from heavyball_b200.utils.orthogonal import _chol_upper_blocked, _leaf_inverse_buffer

    torch.manual_seed(n)
    B = 3
    x = torch.randn(B, n, 2 * n, device="cuda", dtype=torch.float64)
    g64 = x @ x.mT / (2 * n) + 0.1 * torch.eye(n, device="cuda", dtype=torch.float64)
    g = g64.float()
    g[1, n // 2, n // 2] = -1.0  # breaks matrix 1 only
    ref = torch.linalg.cholesky(g64, upper=True)
    work, r = g.clone(), torch.zeros_like(g)
    bad = torch.zeros(B, dtype=torch.int32, device="cuda")
    inv = _leaf_inverse_buffer(work)
    assert inv is not None
    _chol_upper_blocked(work, r, bad, 0, n, inv)
    torch.cuda.synchronize()
    assert bad.tolist()[0] == 0 and bad.tolist()[2] == 0 and bad.tolist()[1] > 0
    for b in (0, 2):
        assert float((r[b].double() - ref[b]).abs().max()) < 2e-4 * float(ref[b].abs().max())
        assert float(r[b].tril(-1).abs().max()) == 0
        for blk in range((n + 127) // 128):
            lo, hi = blk * 128, min(n, blk * 128 + 128)
            want = torch.linalg.inv(r[b, lo:hi, lo:hi].double())
            got = inv[b, blk, : hi - lo, : hi - lo].double()
            assert float((got - want).abs().max()) < 1e-3 * float(want.abs().max())


@pytest.mark.parametrize("n,r", [(5000, 7), (300_000, 23), (1_000_003, 32)])
def test_skinny_gram_of_very_tall_matrices(n, r):
    """``A^T B`` over millions of rows (the low-rank preconditioner's flattened parameter vector) on the long-dimension
    product kernel, cut into enough slices to fill the machine."""
    from heavyball_b200.utils.psgd import _skinny_gram

    g = torch.Generator(device="cuda").manual_seed(n)
    a = torch.randn(n, r, device="cuda", generator=g)
    b = torch.randn(n, r, device="cuda", generator=g)
    got = _skinny_gram(a, b)
    want = a.double().T @ b.double()
    assert got.shape == (r, r)
    assert float((got.double() - want).abs().max()) < 1e-5 * float((a.double().abs().T @ b.double().abs()).max())
