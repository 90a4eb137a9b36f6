"""Split-tf32 GEMM epilogues and the staged SOAP / PSGD programs on a B200, against fp64 / PyTorch definitions."""

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import lowering, ops

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 128, 256], ids=["tile-auto", "tile-128", "tile-256"])
def tile(request):
    """Runs a GEMM-level test with the tile size chosen by problem size and with each tile size forced."""
    ext = ops.load()
    ext.set_tf32_gemm_tile(request.param)
    yield request.param
    ext.set_tf32_gemm_tile(0)


def _rand(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, device="cuda", generator=g)


def _unsplit(s, K):
    """Dense value of a split operand: hi + lo of the first K columns."""
    kp = s.shape[-1] // 2
    return (s[..., :K].double() + s[..., kp : kp + K].double())


def _tol(a, b):
    return 3e-5 * float((a.abs() @ b.abs().transpose(-1, -2)).max())


@pytest.mark.parametrize("B,M,N,K", [(2, 256, 128, 384), (3, 200, 136, 160), (1, 129, 300, 130)])
def test_split_and_plain_product(B, M, N, K, tile):
    a, b = _rand(B, M, K, seed=1), _rand(B, N, K, seed=2)
    a_s, a_t = ops.tf32_split(a, True, True)
    assert torch.allclose(_unsplit(a_s, K), a.double(), atol=1e-6)
    assert torch.allclose(_unsplit(a_t, M), a.double().transpose(1, 2), atol=1e-6)
    kpK, kpM = a_s.shape[-1] // 2, a_t.shape[-1] // 2
    assert float(a_s[..., K:kpK].abs().max() if kpK > K else 0) == 0 and float(a_t[..., M:kpM].abs().max() if kpM > M else 0) == 0
    b_s, _ = ops.tf32_split(b, True, False)
    want = a.double() @ b.double().transpose(1, 2)
    out = torch.empty(B, M, N, device="cuda")
    ops.tf32_gemm(a_s, b_s, K, out=out, alpha=0.5)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((out.double() - 0.5 * want).abs().max()) < _tol(a.double(), b.double())


@pytest.mark.parametrize("B,M,N,K", [(2, 256, 128, 256), (2, 200, 136, 160)])
def test_split_outputs_feed_the_next_product(B, M, N, K, tile):
    a, b = _rand(B, M, K, seed=3), _rand(B, N, K, seed=4)
    a_s, _ = ops.tf32_split(a, True, False)
    b_s, _ = ops.tf32_split(b, True, False)
    want = a.double() @ b.double().transpose(1, 2)
    tol = _tol(a.double(), b.double())
    rows = ops.tf32_gemm(a_s, b_s, K, split_out=ops.SPLIT_ROWS)
    cols = ops.tf32_gemm(a_s, b_s, K, split_out=ops.SPLIT_COLS)
    torch.cuda.synchronize()
    assert rows.shape == (B, M, 2 * ((N + 31) // 32 * 32)) and cols.shape == (B, N, 2 * ((M + 31) // 32 * 32))
    assert float((_unsplit(rows, N) - want).abs().max()) < tol
    assert float((_unsplit(cols, M) - want.transpose(1, 2)).abs().max()) < tol
    kpN, kpM = rows.shape[-1] // 2, cols.shape[-1] // 2
    if kpN > N:
        assert float(rows[..., N:kpN].abs().max()) == 0 and float(rows[..., kpN + N :].abs().max()) == 0
    if kpM > M:
        assert float(cols[..., M:kpM].abs().max()) == 0 and float(cols[..., kpM + M :].abs().max()) == 0
    # chain: (A B^T) C^T through the split output, no intermediate split pass
    c = _rand(B, 144, N, seed=5)
    c_s, _ = ops.tf32_split(c, True, False)
    out = torch.empty(B, M, 144, device="cuda")
    ops.tf32_gemm(rows, c_s, N, out=out)
    torch.cuda.synchronize()
    ops.check_status()
    want2 = want @ c.double().transpose(1, 2)
    assert float((out.double() - want2).abs().max()) < 3e-5 * float((want.abs() @ c.double().abs().transpose(1, 2)).max())


@pytest.mark.parametrize("B,M,K", [(2, 256, 128), (2, 136, 200), (3, 520, 96), (1, 1024, 160)])
def test_lerp_epilogue_on_a_symmetric_product(B, M, K, tile):
    """``GG <- lerp(GG, X X^T)`` with one buffer as both operands: only the tiles on or above the diagonal are computed,
    each is stored mirrored as well (tiles on the diagonal are computed whole, in two summation orders)."""
    x = _rand(B, M, K, seed=6)
    x_s, _ = ops.tf32_split(x, True, False)
    gg = _rand(B, M, M, seed=7)
    gg = (gg + gg.transpose(1, 2)) / 2
    want = gg.double() + (x.double() @ x.double().transpose(1, 2) - gg.double()) * 0.25
    ops.tf32_gemm(x_s, x_s, K, mode=ops.EPI_LERP, w=0.25, out=gg)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((gg.double() - want).abs().max()) < _tol(x.double(), x.double())
    assert float((gg - gg.transpose(1, 2)).abs().max()) < 1e-5 * float(gg.abs().max())  # diagonal tiles: two summation orders


def test_lerp_epilogue_with_distinct_operands_updates_every_tile(tile):
    B, M, K = 2, 264, 128
    a, b = _rand(B, M, K, seed=12), _rand(B, M, K, seed=13)
    a_s, _ = ops.tf32_split(a, True, False)
    b_s, _ = ops.tf32_split(b, True, False)
    c = _rand(B, M, M, seed=14)
    want = c.double() + (a.double() @ b.double().transpose(1, 2) - c.double()) * 0.5
    ops.tf32_gemm(a_s, b_s, K, mode=ops.EPI_LERP, w=0.5, out=c)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((c.double() - want).abs().max()) < _tol(a.double(), b.double())


@pytest.mark.parametrize("B,M,K,pad", [(2, 384, 256, 0), (2, 200, 136, 8)])
def test_symmetric_store(B, M, K, pad, tile):
    x = _rand(B, M, K, seed=15)
    x_s, _ = ops.tf32_split(x, True, False)
    buf = torch.full((B, M, M + pad), 7.0, device="cuda")
    out = buf[:, :, :M]
    ops.tf32_gemm(x_s, x_s, K, out=out, alpha=2.0)
    torch.cuda.synchronize()
    ops.check_status()
    want = 2.0 * (x.double() @ x.double().transpose(1, 2))
    assert float((out.double() - want).abs().max()) < 2 * _tol(x.double(), x.double())
    assert float((out - out.transpose(1, 2)).abs().max()) < 1e-5 * float(out.abs().max())
    if pad:
        assert float((buf[:, :, M:] - 7.0).abs().max()) == 0


@pytest.mark.parametrize("B,n", [(2, 384), (3, 200), (1, 1024), (2, 520)])
def test_product_of_two_upper_triangular_matrices(B, n, tile):
    """Only the K range where both factors are non-zero is walked; the part below the diagonal is exact zeros."""
    a, b = _rand(B, n, n, seed=16).triu(), _rand(B, n, n, seed=17).triu()
    got = ops.matmul3(a, b, upper_upper=True)
    torch.cuda.synchronize()
    ops.check_status()
    want = a.double() @ b.double()
    assert float((got.double() - want).abs().max()) < 3e-5 * float((a.double().abs() @ b.double().abs()).max())
    assert float(got.tril(-1).abs().max()) == 0


@pytest.mark.parametrize("mode", ["adam", "laprop"])
@pytest.mark.parametrize("B,M,N,K", [(2, 256, 128, 256), (2, 200, 138, 160)])
def test_moment_epilogues(mode, B, M, N, K, tile):
    a, b = _rand(B, M, K, seed=8), _rand(B, N, K, seed=9)
    a_s, _ = ops.tf32_split(a, True, False)
    b_s, _ = ops.tf32_split(b, True, False)
    m, v = _rand(B, M, N, seed=10) * 0.1, _rand(B, M, N, seed=11).abs()
    m64, v64 = m.double(), v.double()
    x = a.double() @ b.double().transpose(1, 2)
    b1, b2, eps = 0.9, 0.95, 1e-8
    v64 = v64 * b2 + x * x * (1 - b2)
    d = v64.sqrt().clamp(min=eps)
    if mode == "adam":
        m64 = m64 * b1 + x * (1 - b1)
        want = m64 / d
    else:
        m64 = m64 * b1 + (x / d) * (1 - b1)
        want = m64
    out = torch.empty(B, M, N, device="cuda")
    s = ops.tf32_gemm(a_s, b_s, K, mode=ops.EPI_ADAM if mode == "adam" else ops.EPI_LAPROP, b1=b1, b2c=b2, eps=eps, m=m, v=v,
                      out=out, split_out=ops.SPLIT_ROWS)  # fmt: skip
    torch.cuda.synchronize()
    ops.check_status()
    tol = 1e-3
    assert float((m.double() - m64).abs().max()) < tol * float(m64.abs().max())
    assert float((v.double() - v64).abs().max()) < tol * float(v64.abs().max())
    assert float((out.double() - want).abs().max()) < tol * float(want.abs().max())
    assert float((_unsplit(s, N) - out.double()).abs().max()) < 1e-6 * float(want.abs().max()) + 1e-6


def _train(name, kwargs, lowered, shapes, steps=6):
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(*s, device="cuda") * 0.1) for s in shapes]
    before = lowering.enabled
    lowering.enabled = lowered
    try:
        torch.manual_seed(1)
        opt = getattr(hb, name)(params, **kwargs)
        g = torch.Generator(device="cuda").manual_seed(5)
        for _ in range(steps):
            for p in params:
                p.grad = torch.randn(p.shape, device="cuda", generator=g) * 0.1
            opt.step()
        torch.cuda.synchronize()
        ops.check_status()
        return [p.detach().clone() for p in params], opt
    finally:
        lowering.enabled = before


# (no few-row matrix for SOAP: statistics that gain only a few ranks per step leave the refreshed eigenbasis to rounding
# noise in both paths)
PROGRAM_SHAPES = [(256, 384), (256, 384), (384, 128), (512,), (130, 200), (64, 32), (1, 256)]
SOAP_SHAPES = PROGRAM_SHAPES[:-1]
PROGRAM_CASES = [
    ("SOAP", dict(lr=1e-2, precondition_frequency=100, max_precond_dim=512)),  # no refresh: moments and statistics only
    ("SOAP", dict(lr=1e-2, precondition_frequency=3, max_precond_dim=300, caution=True)),
    ("SOLP", dict(lr=1e-2, precondition_frequency=100, max_precond_dim=512)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=1.0)),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=0.5, max_size_triangular=300, ecc="bf16+8")),
    ("PSGDKron", dict(lr=1e-2, preconditioner_update_probability=1.0, update_clipping=None, caution=True)),
]


@pytest.mark.parametrize("name,kwargs", PROGRAM_CASES, ids=[f"{n}-{i}" for i, (n, _) in enumerate(PROGRAM_CASES)])
def test_staged_program_follows_the_pytorch_path(name, kwargs):
    """Same chain with and without lowering.  Exact agreement is not expected (different product kernels, and for PSGD
    the random probe of the fit is drawn per bucket in both paths but the fit is chaotic), so the bound is relative to
    the distance travelled."""
    shapes = SOAP_SHAPES if name.startswith("SO") else PROGRAM_SHAPES
    start, _ = _train(name, kwargs, True, shapes, steps=0)
    want, _ = _train(name, kwargs, False, shapes)
    got, opt = _train(name, kwargs, True, shapes)
    prog = lowering._program(opt)
    assert prog is not None and any(k[0] == "bucket" for k in prog.workspace)
    loose = name == "PSGDKron" or kwargs.get("precondition_frequency", 100) < 100
    for s, w, g in zip(start, want, got):
        moved = float((w - s).abs().max())
        assert torch.isfinite(g).all() and moved > 0
        assert float((g - w).abs().max()) <= (0.25 if loose else 0.02) * moved, (name, tuple(s.shape))


def test_psgd_diagonal_factor_statistics_on_the_gpu():
    """A dimension above ``max_size_triangular`` gets a diagonal factor; its statistics are a diagonal, not a matrix."""
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(640, 256, device="cuda") * 0.1)
    opt = hb.PSGDKron([p], lr=1e-3, max_size_triangular=512, preconditioner_update_probability=1.0)
    for _ in range(3):
        p.grad = torch.randn_like(p) * 0.1
        opt.step()
    assert torch.isfinite(p).all()
    q = opt.state[p][0][opt._find_val_name("Q")]
    assert q[0][0] is None and q[0][1].shape == (1, 640)  # packed form: diagonal factor for the 640 side


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,n", [(3, 5), (2, 128), (1, 1000), (4, 257)])
def test_packed_triangle_kernels_match_index_arithmetic(B, n, dtype):
    from heavyball_b200.utils import psgd

    q = _rand(B, n, n, seed=21).to(dtype)
    rows, cols = torch.triu_indices(n, n, device="cuda")
    (shape, line), = psgd.triu_to_line([q])
    assert shape == (B, n, n) and torch.equal(line, q[:, rows, cols])
    (dense,) = psgd.line_to_triu([(shape, line)])
    assert torch.equal(dense, q.triu())


@pytest.mark.parametrize("n", [128, 200, 1024])
def test_block_inverse_triangular_solve(n):
    """``X q = b`` through the inverses of the 128-wide diagonal blocks against the library's triangular solve."""
    from heavyball_b200.utils.psgd import _solve_right_upper

    g = torch.Generator(device="cuda").manual_seed(n)
    q = torch.randn(3, n, n, device="cuda", generator=g).triu() * 0.05
    q.diagonal(dim1=-2, dim2=-1).add_(1.0)
    b = torch.randn(3, 260, n, device="cuda", generator=g)
    want = torch.linalg.solve_triangular(q.double(), b.double(), upper=True, left=False)
    got = _solve_right_upper(q, b)
    torch.cuda.synchronize()
    ops.check_status()
    assert float((got.double() - want).abs().max()) < 1e-4 * float(want.abs().max())


def test_captured_fit_matches_eager():
    """Preconditioner fits replayed from CUDA graphs give the trajectory of the same fits run eagerly."""
    from heavyball_b200 import matrix_stage

    shapes = [(256, 384), (256, 384), (384, 128)]
    for name, kwargs in (PROGRAM_CASES[3], PROGRAM_CASES[5]):
        matrix_stage.use_graphs = False
        try:
            want, _ = _train(name, kwargs, True, shapes, steps=8)
        finally:
            matrix_stage.use_graphs = True
        got, opt = _train(name, kwargs, True, shapes, steps=8)
        regions = [v for k, v in lowering._program(opt).workspace.items() if k[0] == "bucket"]
        assert any(b.fit_region.graph is not None for b in regions), name
        for w, g in zip(want, got):  # the fit's random probe comes from the generator in both modes: same trajectory
            assert torch.isfinite(g).all()
            assert float((g - w).abs().max()) <= 0.05 * float(w.abs().max())


@pytest.mark.parametrize("B,M,N,K", [(2, 200, 136, 160), (1, 264, 264, 128)])
def test_sentinels_around_gemm_outputs_survive_every_epilogue(B, M, N, K, tile):
    """Outputs (plain, lerp, add, mirrored, moments) are views with padding rows and columns full of a sentinel value:
    no epilogue writes outside ``[M, N]``; split outputs are checked through their zero padding."""
    sentinel = -7.0
    a, b = _rand(B, M, K, seed=31), _rand(B, N, K, seed=32)
    a_s, _ = ops.tf32_split(a, True, False)
    b_s, _ = ops.tf32_split(b, True, False)

    def padded(rows, cols):
        buf = torch.full((B, rows + 3, cols + 12), sentinel, device="cuda")
        return buf, buf[:, 1 : rows + 1, 4 : cols + 4]

    def intact(buf, rows, cols):
        probe = buf.clone()
        probe[:, 1 : rows + 1, 4 : cols + 4] = sentinel
        return bool((probe == sentinel).all())

    want = a.double() @ b.double().transpose(1, 2)
    tol = _tol(a.double(), b.double())
    for mode, kwargs in (("store", {}), ("lerp", dict(mode=ops.EPI_LERP, w=0.5)), ("add", dict(mode=ops.EPI_ADD, alpha=-1.0))):
        buf, view = padded(M, N)
        view.zero_()
        ops.tf32_gemm(a_s, b_s, K, out=view, **kwargs)
        torch.cuda.synchronize()
        assert intact(buf, M, N), mode
        scale = {"store": 1.0, "lerp": 0.5, "add": -1.0}[mode]
        assert float((view.double() - scale * want).abs().max()) < tol, mode
    if M == N:  # one buffer as both operands: upper tiles plus mirrored stores
        buf, view = padded(M, M)
        view.zero_()
        ops.tf32_gemm(a_s, a_s, K, mode=ops.EPI_ADD, alpha=1.0, out=view)
        torch.cuda.synchronize()
        assert intact(buf, M, M)
        assert float((view.double() - a.double() @ a.double().transpose(1, 2)).abs().max()) < _tol(a.double(), a.double())
    m, v = torch.zeros(B, M, N, device="cuda"), torch.zeros(B, M, N, device="cuda")
    guard_m = torch.full((B * M * N + 64,), sentinel, device="cuda")
    m = guard_m[32 : 32 + B * M * N].view(B, M, N).zero_()
    s = ops.tf32_gemm(a_s, b_s, K, mode=ops.EPI_ADAM, b1=0.9, b2c=0.99, eps=1e-8, m=m, v=v, split_out=ops.SPLIT_COLS)
    torch.cuda.synchronize()
    ops.check_status()
    assert bool((guard_m[:32] == sentinel).all()) and bool((guard_m[32 + B * M * N :] == sentinel).all())
    kp = s.shape[-1] // 2
    assert s.shape == (B, N, 2 * kp) and (kp == M or float(s[..., M:kp].abs().max()) == 0)
