"""GPU numerics tests for the sm_100a kernels.  Each kernel is compared with a plain PyTorch fp32
restatement of the same operation (the definitions in ``heavyball_b200.utils`` with lowering off)."""

import copy

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import lowering, ops, utils

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _params(shapes, dtype=torch.float32, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(*s, device=DEV, generator=g, dtype=torch.float32).to(dtype)) for s in shapes]


def _run(cls, kwargs, shapes, steps, lowered, pdtype=torch.float32, gdtype=None, seed=0):
    torch.manual_seed(seed)
    params = _params(shapes, pdtype, seed)
    opt = cls(params, **kwargs)
    gen = torch.Generator(device=DEV).manual_seed(seed + 1)
    old = lowering.enabled
    lowering.enabled = lowered
    try:
        for _ in range(steps):
            for p in params:
                g = torch.randn(p.shape, device=DEV, generator=gen, dtype=torch.float32) * 0.1
                p.grad = g.to(gdtype or p.dtype)
            opt.step()
    finally:
        lowering.enabled = old
    return params, opt


SHAPES = [(257,), (64, 33), (3, 5, 7), (8193,), (128, 256), (1,)]

FIRST_ORDER = [
    (hb.AdamW, {"lr": 1e-2, "weight_decay": 0.1}),
    (hb.AdamW, {"lr": 1e-2, "caution": True}),
    (hb.AdamW, {"lr": 1e-2, "mars": True, "cautious_weight_decay": True, "weight_decay": 0.1}),
    (hb.AdamW, {"lr": 1e-2, "palm": True, "warmup_steps": 3}),
    (hb.LaProp, {"lr": 1e-2}),
    (hb.ADOPT, {"lr": 1e-2}),
    (hb.AdEMAMix, {"lr": 1e-2, "alpha_warmup": 10, "beta3_warmup": 10}),
    (hb.RMSprop, {"lr": 1e-2}),
    (hb.UnscaledAdamW, {"lr": 1e-2}),
    (hb.SGD, {"lr": 1e-2, "caution": True}),
    (hb.AdamC, {"lr": 1e-2, "max_lr": 2e-2, "weight_decay": 0.1}),
    (hb.NAdam, {"lr": 1e-2}),
    (hb.NAdam, {"lr": 1e-2, "weight_decay": 0.1, "decoupled_weight_decay": True, "caution": True}),
    (hb.SFAdamW, {"lr": 1e-2, "weight_decay": 0.1, "warmup_steps": 2}),
    (hb.AdamW, {"lr": 1e-2, "gradient_clipping": "l2_clip_"}),
    (hb.AdamW, {"lr": 1e-2, "gradient_clipping": "rmsnorm_clip_", "caution": True}),
    (hb.LaProp, {"lr": 1e-2, "gradient_clipping": "global_l2norm_clip"}),
    (hb.AdamW, {"lr": 1e-2, "gradient_clipping": "global_rmsnorm_clip"}),
]


NORMED = [
    (hb.SignLaProp, {"lr": 1e-2}),
    (hb.SignLaProp, {"lr": 1e-2, "weight_decay": 0.1, "cautious_weight_decay": True}),
    (hb.OrthoLaProp, {"lr": 1e-2}),
    (hb.OrthoLaProp, {"lr": 1e-2, "caution": True, "weight_decay": 0.1}),
    (hb.LaPropOrtho, {"lr": 1e-2, "weight_decay": 0.1}),
    (hb.MSAMLaProp, {"lr": 1e-2}),
    (hb.MSAMLaProp, {"lr": 1e-2, "weight_decay": 0.1, "cautious_weight_decay": True, "sam_step_size": 0.05}),
    (hb.HyperBallAdamW, {"lr": 1e-2}),
    (hb.HyperBallAdamW, {"lr": 1e-2, "weight_decay": 0.1}),
]


@pytest.mark.parametrize("cls,kw", NORMED, ids=lambda x: getattr(x, "__name__", str(x))[:40])
def test_sign_and_orthograd_chains_are_lowered(cls, kw):
    """Chains whose update depends on a per-tensor norm or projection: the sums come from the rule's own launch or from
    one segmented reduction, the rescaling happens on load in the launch that writes the parameters."""
    shapes = [(257,), (64, 33), (3, 5, 7), (8193,), (128, 256), (16,)]
    ref, _ = _run(cls, kw, shapes, 6, lowered=False)
    before = ops.launch_counter.count
    got, opt = _run(cls, kw, shapes, 6, lowered=True)
    prog = lowering._program(opt)
    subs = [sub for _, sub in prog.routes] if prog.kind == "route" else [prog]
    assert any(sub.pre_project or sub.after is not None for sub in subs)
    assert ops.launch_counter.count - before <= 6 * 6  # the PyTorch definitions never touch the counter; a step is <= 6 launches
    assert ops.launch_counter.count - before >= 5 * 2  # the first step creates state through the PyTorch definitions
    for a, b in zip(ref, got):
        torch.testing.assert_close(b.data, a.data, rtol=1e-4, atol=1e-5)


def test_orthograd_with_a_scalar_parameter_takes_the_pytorch_definition():
    ref, _ = _run(hb.OrthoLaProp, {"lr": 1e-2}, [(1,), (64, 33)], 4, lowered=False)
    got, _ = _run(hb.OrthoLaProp, {"lr": 1e-2}, [(1,), (64, 33)], 4, lowered=True)
    for a, b in zip(ref, got):
        torch.testing.assert_close(b.data, a.data, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("cls,kw", FIRST_ORDER, ids=lambda x: getattr(x, "__name__", str(x))[:40])
def test_fused_chain_matches_pytorch_fp32(cls, kw):
    ref, _ = _run(cls, kw, SHAPES, 6, lowered=False)
    got, opt = _run(cls, kw, SHAPES, 6, lowered=True)
    assert lowering._program(opt) is not None
    for a, b in zip(ref, got):
        torch.testing.assert_close(b.data, a.data, rtol=2e-5, atol=2e-6)


def test_routed_chain_is_lowered_per_branch():
    """MuonAdamW: matrices through momentum + Newton-Schulz, the rest through Adam, each branch as its own program."""
    kw = {"lr": 1e-2, "weight_decay": 0.01}
    shapes = [(257,), (64, 96), (128, 256), (128, 256), (8,)]
    ref, _ = _run(hb.MuonAdamW, kw, shapes, 5, lowered=False)
    got, opt = _run(hb.MuonAdamW, kw, shapes, 5, lowered=True)
    prog = lowering._program(opt)
    assert prog is not None and prog.kind == "route" and [r[1].kind for r in prog.routes] == ["orthogonal", "elementwise"]
    for a, b in zip(ref, got):
        if a.ndim >= 2:  # stochastic rounding inside the iteration differs between the two implementations
            assert (a.data - b.data).abs().max().item() < 5e-2 * 5 * 1e-2 + 1e-4
        else:
            torch.testing.assert_close(b.data, a.data, rtol=2e-5, atol=2e-6)


def test_fused_chain_state_matches():
    _, o1 = _run(hb.AdamW, {"lr": 1e-2}, SHAPES, 5, lowered=False)
    _, o2 = _run(hb.AdamW, {"lr": 1e-2}, SHAPES, 5, lowered=True)
    s1, s2 = o1.state_dict()["state"], o2.state_dict()["state"]
    for k in s1:
        for name, v in s1[k][0].items():
            if isinstance(v, torch.Tensor) and v.is_floating_point():
                torch.testing.assert_close(s2[k][0][name], v, rtol=2e-5, atol=1e-7)
            elif name == "is_initialized":
                assert s2[k][0][name] == v


@pytest.mark.parametrize("kw", [{"storage_dtype": "bfloat16"}, {"ecc": "bf16+8"}, {"ecc": "bf16+16"}, {"ecc": "fp16+8"},
                                {"ecc": "bf16+8", "param_ecc": "bf16+8"}], ids=str)
def test_fused_chain_low_precision_storage(kw):
    """Stochastic rounding / ECC encode use different random streams than PyTorch, so compare
    statistically: results must agree to well within the storage format's noise."""
    ref, _ = _run(hb.AdamW, {"lr": 1e-2}, SHAPES, 8, lowered=False)  # fp32 everything
    low_ref, _ = _run(hb.AdamW, {"lr": 1e-2, **kw}, SHAPES, 8, lowered=False)
    got, opt = _run(hb.AdamW, {"lr": 1e-2, **kw}, SHAPES, 8, lowered=True)
    for r, a, b in zip(ref, low_ref, got):
        err_ref = (a.data.float() - r.data).abs().mean().item()
        err_got = (b.data.float() - r.data).abs().mean().item()
        assert err_got <= 2.0 * err_ref + 1e-4, (kw, err_got, err_ref)
    if "ecc" in kw and "param_ecc" not in kw:  # (bf16 parameters get bf16 gradients here, a different input)
        # the decoded state must track the fp32 state closely (ULP / (2 smax) resolution)
        _, o32 = _run(hb.AdamW, {"lr": 1e-2}, SHAPES, 8, lowered=True)
        key = "update_by_adam_exp_avg_0"
        for p32, pl in zip(o32.param_groups[0]["params"], opt.param_groups[0]["params"]):
            st = opt.state[pl][0]
            cfgecc = hb.chainable.ECCConfig(kw["ecc"])
            dec = utils._ULPState(st[key + "::ecc"], cfgecc.smax).decode(st[key])
            want = o32.state[p32][0][key]
            # one encode resolves ulp / (2 smax); after eight noisy re-encodes of a decaying EMA the
            # RMS error must still sit far below what the 16-bit primary alone could resolve (~ulp / 4)
            ulp_rel = 2.0 ** (-7 if "bf16" in kw["ecc"] else -10)
            rms_err = (dec - want).square().mean().sqrt().item()
            rms_val = want.square().mean().sqrt().item()
            assert rms_err <= 0.02 * ulp_rel * rms_val + 1e-9, (kw, rms_err, rms_val)


def test_bf16_params_stochastic_rounding_is_unbiased():
    shapes = [(4096,)]
    acc = torch.zeros(4096, device=DEV)
    base = None
    n = 24
    for seed in range(n):
        torch.manual_seed(seed)
        p = torch.nn.Parameter(torch.full((4096,), 1.0, device=DEV, dtype=torch.bfloat16))
        opt = hb.SGD([p], lr=1e-3, beta=0.0)
        for i in range(2):
            p.grad = torch.full_like(p, 0.37)
            opt.step()
        acc += p.data.float()
    mean = (acc / n).mean().item()
    # exact: 1 - 2 * 1e-3 * 0.37 (first step runs in PyTorch, second in the kernel); bf16 spacing near 1 is 2^-7
    assert abs(mean - (1 - 2 * 1e-3 * 0.37)) < 2e-4, mean


# ----------------------------------------------------------------------------------------- Newton–Schulz


def _ns_reference(G, coeffs, eps=1e-7):
    x = G.float() / G.float().norm(dim=(-2, -1), keepdim=True).clamp(min=eps)
    tall = G.shape[-2] > G.shape[-1]
    if tall:
        x = x.mT
    for a, b, c in coeffs:
        s = x @ x.mT
        eye = torch.eye(s.shape[-1], device=G.device)
        x = (a * eye + b * s + c * (s @ s)) @ x
    return x.mT if tall else x


@pytest.mark.parametrize("shape", [(128, 128), (768, 3072), (3072, 768), (200, 136), (96, 1000), (768, 768)], ids=str)
@pytest.mark.parametrize("batch", [1, 3])
def test_newton_schulz_kernel_vs_fp32(shape, batch):
    torch.manual_seed(0)
    mats = [torch.randn(*shape, device=DEV) for _ in range(batch)]
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS, out_scale=1.0)
    torch.cuda.synchronize()
    ops.check_status()
    for m, o in zip(mats, out):
        want = _ns_reference(m, utils.NS5_COEFFS)
        rel = ((o - want).norm() / want.norm()).item()
        assert rel < 4e-2, (shape, rel)  # bf16 operands through 15 chained GEMMs
        sv, sv_want = torch.linalg.svdvals(o.float()), torch.linalg.svdvals(want)
        assert sv.max().item() < 1.3, sv.max().item()
        # wide matrices are well conditioned and must come out near-orthogonal; square Gaussian ones keep
        # a tail of tiny singular values after five steps, in the kernel exactly as in fp32
        assert abs(sv.median().item() - sv_want.median().item()) < 0.05


@pytest.mark.parametrize("tile,m,n", [(128, 256, 384), (256, 256, 384), (256, 520, 712), (256, 1024, 1280)])
def test_ns_gemm_modes_vs_matmul(tile, m, n):
    """The three products of one polynomial step, with the 128x128-tile kernel and with the 256x256-tile one (forced:
    by default it is only chosen for large problems), ragged sizes included."""
    ext = ops.load()
    ext.set_ns_gemm_tile(tile)
    try:
        _ns_gemm_modes(ext, 2, m, n)
    finally:
        ext.set_ns_gemm_tile(0)


def _ns_gemm_modes(ext, B, m, n):
    torch.manual_seed(1)
    x = (torch.randn(B, m, n, device=DEV) / n**0.5).bfloat16()
    xt = x.mT.contiguous()
    S = torch.empty(B, m, m, device=DEV, dtype=torch.bfloat16)
    Y = torch.empty_like(S)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ext.ns_gemm(x, n, m * n, x, n, m * n, m, m, n, B, ops.MODE_GRAM, True, S, m, m * m, S, m, m * m,
                None, 0, 0, False, 1.0, None, 0, 0, 0.0, 0.0, 0.0, status)
    want_S = x.float() @ x.float().mT
    torch.testing.assert_close(S.float(), want_S, rtol=2e-2, atol=2e-2)
    a, b, c = 3.0, -4.0, 2.0
    ext.ns_gemm(S, m, m * m, S, m, m * m, m, m, m, B, ops.MODE_POLY, True, Y, m, m * m, Y, m, m * m,
                None, 0, 0, False, 1.0, S, m, m * m, a, b, c, status)
    Sf = S.float()
    want_Y = c * (Sf @ Sf) + b * Sf + a * torch.eye(m, device=DEV)
    torch.testing.assert_close(Y.float(), want_Y, rtol=3e-2, atol=3e-2)
    nx, nxt = torch.empty_like(x), torch.empty_like(xt)
    F = torch.empty(B, m, n, device=DEV)
    ext.ns_gemm(Y, m, m * m, xt, m, n * m, m, n, m, B, ops.MODE_APPLY, False, nx, n, m * n, nxt, m, n * m,
                F, n, m * n, False, 0.5, None, 0, 0, 0.0, 0.0, 0.0, status)
    want_X = Y.float() @ x.float()
    torch.testing.assert_close(nx.float(), want_X, rtol=3e-2, atol=3e-2)
    assert torch.equal(nxt, nx.mT.contiguous())
    torch.testing.assert_close(F, nx.float() * 0.5, rtol=0, atol=0)
    assert int(status.item()) == 0


@pytest.mark.parametrize("table", ["polar_express", "legacy"])
def test_other_coefficient_tables_through_the_kernel(table):
    """The 10-step Polar-Express table (8 triples) and the fixed legacy triple run through the same GEMM chain."""
    from heavyball_b200.utils import orthogonal as O

    torch.manual_seed(0)
    coeffs = [O.ABC_LIST_STABLE[min(i, len(O.ABC_LIST_STABLE) - 1)] for i in range(10)] if table == "polar_express" \
        else [O.LEGACY_COEFFS] * 5
    mats = [torch.randn(256, 640, device=DEV) for _ in range(2)]
    out = ops.newton_schulz_batched(mats, coeffs, out_scale=1.0)
    torch.cuda.synchronize()
    ops.check_status()
    for m, o in zip(mats, out):
        want = _ns_reference(m, coeffs)
        assert ((o - want).norm() / want.norm()).item() < 6e-2
        if table == "polar_express":  # ten steps reach the polar factor: singular values at 1
            sv = torch.linalg.svdvals(o.float())
            assert 0.9 < sv.min().item() and sv.max().item() < 1.1


@pytest.mark.parametrize("shape,batch", [((1024, 4096), 2), ((2048, 2048), 3), ((256, 512), 160)], ids=str)
def test_newton_schulz_large_and_many(shape, batch):
    """A 4096-wide operand, square 2048 matrices (the 256x256-tile kernel by default) and a batch of more than one
    wave of tiles."""
    torch.manual_seed(0)
    mats = [torch.randn(*shape, device=DEV) for _ in range(batch)]
    out = ops.newton_schulz_batched(mats, utils.NS5_COEFFS, out_scale=1.0)
    torch.cuda.synchronize()
    ops.check_status()
    for i in (0, batch - 1):
        want = _ns_reference(mats[i], utils.NS5_COEFFS)
        assert ((out[i] - want).norm() / want.norm()).item() < 4e-2, shape


def test_muon_lowered_matches_pytorch():
    shapes = [(256, 512), (512, 256), (256, 512), (64,), (128, 128)]
    ref, _ = _run(hb.Muon, {"lr": 0.02, "weight_decay": 0.01}, shapes, 4, lowered=False)
    got, opt = _run(hb.Muon, {"lr": 0.02, "weight_decay": 0.01}, shapes, 4, lowered=True)
    ops.check_status()
    assert lowering._program(opt).kind == "orthogonal"
    for a, b in zip(ref, got):
        d0 = 4 * 0.02 * (max(1, a.shape[0] / a.shape[-1]) ** 0.5 if a.ndim > 1 else 1)
        # both paths orthogonalise with bf16 operands and different rounding noise
        assert ((a.data - b.data).norm() / (a.data.numel() ** 0.5)).item() < 0.05 * d0


def test_graft_smoke():
    import __graft_entry__ as entry

    entry.smoke()


@pytest.mark.parametrize("shape", [(1, 128, 128, 128), (3, 256, 384, 512), (2, 200, 130, 150), (1, 1024, 1024, 1024)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_split_tf32_matmul_is_close_to_fp32(shape, ta, tb):
    """3-term tf32 product on tcgen05: error about 2^-18 of |a||b| (set by the tensor core's accumulator rounding,
    not by the operand split), against 2^-11 for a single tf32 pass."""
    batch, m, n, k = shape
    torch.manual_seed(0)
    a = torch.randn(batch, *((k, m) if ta else (m, k)), device="cuda")
    b = torch.randn(batch, *((n, k) if tb else (k, n)), device="cuda")
    a = a * torch.logspace(-3, 3, a.shape[-1], device="cuda")  # wide dynamic range along one axis
    got = ops.matmul3(a, b, ta, tb, alpha=0.5)
    ops.check_status()
    a64, b64 = a.double(), b.double()
    ref = 0.5 * ((a64.mT if ta else a64) @ (b64.mT if tb else b64))
    bound = 0.5 * ((a64.mT if ta else a64).abs() @ (b64.mT if tb else b64).abs())
    err = ((got.double() - ref).abs() / bound).max().item()
    assert got.shape == ref.shape and got.dtype == torch.float32
    assert err < 8e-6, err


def test_peer_wait_gives_up_after_its_budget_and_reports_the_missing_rank():
    """A flag that nothing sets: the wait returns after its clock budget with the absent rank in the status
    word, and the context keeps working."""
    import time

    ext = ops.load()
    flags = torch.zeros(2 * ext.MAX_WORLD, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags[0] = 1  # rank 0 has arrived at epoch 1, rank 1 never does
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ext.peer_wait(flags, 0, 2, 1, 0.2, status)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert status.item() == 2 + 1
    assert 0.1 < waited < 2.0
    status.zero_()
    flags[1] = 1
    ext.peer_wait(flags, 0, 2, 1, 0.2, status)
    assert status.item() == 0
    assert torch.ones(4, device="cuda").sum().item() == 4.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_segmented_dot_and_absmax_match_fp32_definitions(dtype):
    torch.manual_seed(0)
    sizes = [(1,), (7,), (1024, 1024), (33, 65), (70001,), (3, 5, 7)]
    xs = [torch.randn(*s, device="cuda").to(dtype) for s in sizes]
    ys = [torch.randn(*s, device="cuda").to(dtype) for s in sizes]
    # starts that are not 16-byte aligned: the scalar load path
    xs[3] = torch.randn(33 * 65 + 1, device="cuda").to(dtype)[1:].view(33, 65)
    ys[3] = torch.randn(33 * 65 + 1, device="cuda").to(dtype)[1:].view(33, 65)
    dots = ops.dot(xs, ys)
    peaks = ops.absmax(xs)
    ops.check_status()
    assert dots.dtype == torch.float32 and dots.shape == (len(xs),)
    for i, (x, y) in enumerate(zip(xs, ys)):
        ref = (x.double() * y.double()).sum()
        scale = (x.double() * y.double()).abs().sum()
        assert abs(dots[i].item() - ref.item()) <= 1e-5 * scale.item() + 1e-12
        assert peaks[i].item() == x.float().abs().max().item()  # a maximum is exact
    bad = [x.clone() for x in xs]
    bad[2][5, 7] = float("nan")
    out = ops.absmax(bad)
    assert torch.isnan(out[2]) and not torch.isnan(out[[0, 1, 3, 4, 5]]).any()


def test_orthograd_and_kron_balance_use_the_segmented_reductions():
    """Both call sites against their plain PyTorch definitions (the path they take on CPU)."""
    from heavyball_b200.utils import first_order, psgd

    torch.manual_seed(0)
    ws = [torch.randn(64, 32, device="cuda"), torch.randn(1000, device="cuda")]
    gs = [torch.randn_like(w) for w in ws]
    got = [g.clone() for g in gs]
    before = ops.launch_counter.count
    first_order.orthogonalize_grad_to_param(ws, got, 1e-30, graft=False)
    assert ops.launch_counter.count > before
    for w, g, o in zip(ws, gs, got):
        ref = g - ((w * g).sum() / ((w * w).sum() + 1e-30)) * w
        assert torch.allclose(o, ref, atol=1e-5, rtol=1e-5)
        assert abs((o * w).sum().item()) < 2e-2  # orthogonal to the weight

    qs = [torch.randn(4, 48, 48, device="cuda").triu() * 3.0, torch.randn(4, 16, device="cuda") * 0.1]
    ref = [q.clone().cpu() for q in qs]
    psgd.psgd_balance_Q(qs)
    psgd.psgd_balance_Q(ref)
    for q, r in zip(qs, ref):
        assert torch.allclose(q.cpu(), r, atol=1e-6, rtol=1e-5)


def test_scion_matrices_of_one_shape_share_a_batched_iteration():
    """The spectral LMO of Scion: same-shape matrices go through one batched Newton-Schulz chain; the result is the
    per-tensor one up to the rounding noise of the bf16 iteration."""
    from heavyball_b200.utils import orthogonal

    gen = torch.Generator(device=DEV).manual_seed(3)
    mats = [torch.randn(192, 320, device=DEV, generator=gen) for _ in range(3)] + [torch.randn(64, 64, device=DEV, generator=gen)]
    vec = torch.randn(300, device=DEV, generator=gen)
    want = [orthogonal._scion_matrix_direction(m.clone(), False) * 0.5 for m in mats]
    want_vec = orthogonal._scion_bias_rms_direction(vec.clone()) * 0.5
    work = [m.clone() for m in mats] + [vec.clone()]
    before = ops.launch_counter.count
    orthogonal.scion_auto_lmo_(work, 0.5)
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_counter.count > before
    for got, ref in zip(work[:-1], want):
        assert float((got - ref).norm() / ref.norm()) < 0.05
        s = torch.linalg.svdvals(got.double())
        unit = 0.5 * (got.shape[0] / got.shape[1]) ** 0.5  # five steps leave the smallest singular values of a square matrix short
        assert float(s.max()) < 1.3 * unit and 0.7 * unit < float(s.median()) < 1.3 * unit
    torch.testing.assert_close(work[-1], want_vec)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shift", [0, 1])
def test_canary_words_around_every_buffer_survive_the_fused_chain(dtype, shift):
    """Every tensor of a launch is carved out of one arena with sentinel words before and after it (sizes 1 .. 8193,
    16-byte aligned and - with ``shift`` - deliberately misaligned starts, which take the scalar path): after Adam
    steps with caution (two launches, scratch and mask counters included) no sentinel has changed and the parameters
    match the PyTorch arithmetic."""
    sizes = [1, 7, 63, 64, 65, 4099, 8191, 8192, 8193]
    gap, sentinel = 32, -12288.0  # exactly representable in bf16
    gen = torch.Generator(device=DEV).manual_seed(11 + shift)

    def arena(fill):
        total = sum(n + gap for n in sizes) + gap + 8
        buf = torch.full((total,), sentinel, device=DEV, dtype=torch.float32 if fill == "f32" else dtype)
        views, mask, off = [], torch.ones(total, dtype=torch.bool, device=DEV), gap + shift
        for n in sizes:
            off = (off + 3) // 4 * 4 + shift
            views.append(buf[off : off + n])
            mask[off : off + n] = False
            off += n + gap
        return buf, views, mask

    bufs = {name: arena("f32" if name in ("u",) else "x") for name in ("p", "g", "m", "v", "u")}
    p, g, m, v, u = (bufs[k][1] for k in ("p", "g", "m", "v", "u"))
    for t in p:
        t.copy_(torch.randn(t.shape, device=DEV, generator=gen))
    for t in m + v + u:
        t.zero_()
    ref_p = [t.float().clone() for t in p]
    ref_m, ref_v = [torch.zeros_like(t) for t in ref_p], [torch.zeros_like(t) for t in ref_p]
    lr, b1, b2, eps = 1e-2, 0.9, 0.99, 1e-8
    for step in range(1, 4):
        for t in g:
            t.copy_(torch.randn(t.shape, device=DEV, generator=gen) * 0.1)
        d1, d2 = 1 - (1 - b1) / (1 - b1**step), 1 - (1 - b2) / (1 - b2**step)
        masked = torch.zeros(len(sizes), dtype=torch.int32, device=DEV)
        common = dict(algo=ops.ADAM, n_state=2, b1=d1, b2=d2, eps=eps, dt_g=ops.dtype_code(g[0]), dt_s=ops.dtype_code(m[0]),
                      dt_p=ops.dtype_code(p[0]))  # fmt: skip
        ops.fused_chain(g=g, u=u, s0=m, s1=v, masked=masked, count_caution=1, out_mode=ops.OUT_UPDATE, dt_u=ops.F32, seed=step,
                        **common)  # fmt: skip
        ops.fused_chain(p=p, u=u, masked=masked, algo=ops.IDENTITY, u_is_input=1, caution_apply=1, out_mode=ops.OUT_PARAM,
                        dt_u=ops.F32, dt_p=common["dt_p"], dt_g=ops.NONE, dt_s=ops.NONE, lr=lr, wd=0.0, seed=step + 100)  # fmt: skip
        if dtype == torch.float32:
            for i in range(len(sizes)):
                g32 = g[i].float()
                ref_m[i] = ref_m[i] * (1 - (1 - d1)) + g32 * (1 - d1)
                ref_v[i] = ref_v[i] * (1 - (1 - d2)) + g32 * g32 * (1 - d2)
                upd = ref_m[i] / ref_v[i].sqrt().clamp(min=eps)
                keep = ~(g32.signbit() ^ upd.signbit())
                upd = upd * keep * (upd.numel() / max(1, int(keep.sum())))
                ref_p[i] = ref_p[i] - lr * upd
    torch.cuda.synchronize()
    for name, (buf, _, mask) in bufs.items():
        assert bool((buf[mask].float() == sentinel).all()), name
    if dtype == torch.float32:
        for got, want in zip(p, ref_p):
            torch.testing.assert_close(got, want, rtol=2e-5, atol=2e-6)
    else:
        assert all(torch.isfinite(t.float()).all() for t in p)
