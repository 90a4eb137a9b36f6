"""CPU tests of the transform engine, the optimizer runtime and the public-class features.

Invariants follow the reference's CPU tier (``test/test_chainable_cpu.py``, ``test/test_cpu_features.py``,
``test/test_optimizer_cpu_smoke.py``, ``test/test_toy_training.py``, ``test/test_no_grad.py``,
``test/test_nd_param.py``, ``test/test_ema.py``, ``test/test_closure.py``).
"""

import copy
import io
import pickle
import warnings

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import chainable as C
from heavyball_b200 import utils

ALL = [n for n in hb.__all__ if n not in ("capture_param_shapes", "SplitOpt", "SAMWrapper")]


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))


def _steps(model, opt, n=3, seed=1):
    torch.manual_seed(seed)
    x = torch.randn(8, 6)
    for _ in range(n):
        model(x).square().mean().backward()
        opt.step()
        opt.zero_grad()


# ------------------------------------------------------------------------------------------ numbering / tags

EXPECTED_KEYS = {
    "SGD": {"heavyball_momentum_momentum_0"},
    "AdamW": {"update_by_adam_exp_avg_0", "update_by_adam_exp_avg_sq_0"},
    "NAdam": {"update_by_nadam_exp_avg_0", "update_by_nadam_exp_avg_sq_0", "update_by_nadam_mu_product_1"},
    "Muon": {"nesterov_ema_momentum_2"},
    "MuonLaProp": {"scale_by_laprop_exp_avg_2", "scale_by_laprop_exp_avg_sq_2"},
    "SFAdamW": {"scale_by_exp_avg_sq_exp_avg_sq_2", "update_by_schedule_free_z_0"},
    "MSAMLaProp": {"scale_by_exp_avg_sq_exp_avg_sq_4", "update_by_msam_z_1", "update_by_msam_exp_avg_2"},
    "SOAP": {"scale_by_soap_exp_avg_2", "scale_by_soap_exp_avg_sq_2", "scale_by_soap_Q_3", "scale_by_soap_GG_3"},
    "PSGDKron": {
        "exp_avg_exp_avg_6", "scale_by_psgd_Q_4", "scale_by_psgd_Q_cache_4", "scale_by_psgd_running_lower_bound_4",
        "scale_by_psgd_step_4",
    },
    "LATHER": {
        "scale_by_lather_exp_avg_4", "scale_by_lather_exp_avg_sq_4", "scale_by_lather_Q_5", "scale_by_lather_Q_basis_5",
        "scale_by_lather_running_lower_bound_5", "scale_by_lather_step_5",
    },
    "PSGDLRA": {"exp_avg_exp_avg_5", "scale_by_psgd_lra_U_3", "scale_by_psgd_lra_V_3", "scale_by_psgd_lra_d_3"},
}  # fmt: skip


@pytest.mark.parametrize("name", sorted(EXPECTED_KEYS))
def test_state_key_names(name):
    m = _model()
    opt = getattr(hb, name)(m.parameters())
    _steps(m, opt)
    keys = {k for st in opt.state_dict()["state"].values() for v in st.values() for k in v}
    keys -= {"is_initialized", "step"}
    keys = {k for k in keys if not k.startswith("_")}
    assert keys == EXPECTED_KEYS[name]


def test_flags_shift_indices():
    m = _model()
    opt = hb.AdamW(m.parameters(), mars=True)
    _steps(m, opt)
    keys = {k for st in opt.state_dict()["state"].values() for v in st.values() for k in v}
    assert {"mars_mars_old_grad_2", "update_by_adam_exp_avg_0"} <= keys
    opt = hb.Muon(_model().parameters(), mars=True)
    assert opt._find_val_name("mars_old_grad") == "mars_mars_old_grad_4"
    assert opt._find_val_name("momentum") == "nesterov_ema_momentum_2"


NEEDS_GATHER = {
    "SGD": False, "AdamW": False, "NAdam": False, "AdEMAMix": False, "UnscaledAdamW": False, "AdamC": False,
    "RMSprop": False, "SFAdamW": False, "ADOPT": False, "LaProp": False, "SUDSAdamW": True, "Scion": True,
    "HyperBallAdamW": True, "MuonAdamW": True, "MSAMLaProp": True, "Muon": True, "MuonLaProp": True, "SOAP": True,
    "KLShampoo": True, "SignLaProp": True, "OrthoLaProp": True, "LaPropOrtho": True, "PSGDKron": True, "LATHER": True,
    "PSGDPRO": True, "QSGD": True, "PSGDLRA": True,
}  # fmt: skip


@pytest.mark.parametrize("name", sorted(NEEDS_GATHER))
def test_needs_gather_table(name):
    kw = {"rank": 2} if name == "PSGDLRA" else {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = getattr(hb, name)(_model().parameters(), **kw)
    assert opt._needs_gather is NEEDS_GATHER[name]


def test_set_indices_retain_and_offset():
    fns = C.set_indices((C.scale_by_adam, C.sign), retain=False)
    assert fns[1].transform_idx == 0 and fns[0].transform_idx == 2
    again = C.set_indices(fns, retain=True)
    assert [f.transform_idx for f in again] == [2, 0]
    more = C.set_indices((*again, C.exp_avg), retain=True)
    assert more[2].transform_idx == 4
    with pytest.raises(ValueError):
        C.set_indices(fns, retain=True, offset=3)


# ------------------------------------------------------------------------------------------ engine behaviour


def test_chain_skip_and_final_update():
    p = [torch.nn.Parameter(torch.ones(4))]
    g = [torch.full((4,), 2.0)]
    group = {"lr": 0.1, "weight_decay": 0.0, "caution": False, "step": 1}
    with torch.no_grad():
        C.chain([{}], group, g, p, C.identity)
        assert torch.allclose(p[0].data, torch.full((4,), 0.8))
        C.chain([{}], group, g, p, lambda *a: C._SKIP)
    assert torch.allclose(p[0].data, torch.full((4,), 0.8))


def test_parallel_merges_branches_and_route_splits_by_predicate():
    fns = C.set_indices(
        [C.Parallel([[C.identity], [C.sign]], lambda outs: [(a + b) / 2 for a, b in zip(*outs)])], retain=False
    )
    u = [torch.tensor([2.0, -4.0])]
    (out,) = fns[0]([{}], {"lr": 1}, u, u, u)
    want = (u[0] + u[0].sign() * (u[0].norm() / (2**0.5))) / 2
    torch.testing.assert_close(out, want)

    r = C.Route((lambda p: p.ndim >= 2, C.sign), default=None)
    (r,) = C.set_indices([r], retain=False)
    ps = [torch.zeros(2, 2), torch.zeros(3)]
    us = [torch.tensor([[1.0, -1.0], [2.0, 0.5]]), torch.tensor([3.0, -3.0, 1.0])]
    out = r([{}, {}], {}, us, us, ps)
    assert torch.equal(out[1], us[1]) and (out[0].abs() - out[0].abs()[0, 0]).abs().max() < 1e-6

    bad = C.Route((lambda p: p.ndim >= 2, C.apply_update), default=C.identity)
    (bad,) = C.set_indices([bad], retain=False)
    with pytest.raises(ValueError):
        bad([{}, {}], {"lr": 0.1, "weight_decay": 0, "caution": False}, us, us, [p.clone() for p in ps])


def test_user_defined_transform_with_guards_and_fns_reassignment():
    @C.zero_guard("count")
    @C.no_state
    def count_calls(group, update, grad, param, count):
        for c in count:
            c += 1
        return update

    m = _model()
    opt = hb.SGD(m.parameters(), lr=1e-2)
    opt.fns = (*opt.fns, count_calls)
    _steps(m, opt, 3)
    key = opt._find_val_name("count")
    assert key == "count_calls_count_2"  # existing indices are retained, the new transform is numbered after them
    assert all(bool((st[0][key] == 3).all()) for st in opt.state.values())


def test_no_grad_means_no_state_and_partial_grads_are_fine():
    m = _model()
    opt = hb.AdamW(m.parameters())
    opt.step()
    assert opt.state_size() == 0
    m[0].weight.grad = torch.ones_like(m[0].weight)
    opt.step()
    assert opt.state_size() == 2 * m[0].weight.numel() * 4 + 8  # two fp32 moments + the int64 step counter
    assert m[0].weight.grad is None  # consumed


def test_consume_grad_false_keeps_gradients():
    m = _model()
    opt = hb.AdamW(m.parameters(), consume_grad=False)
    m(torch.randn(2, 6)).sum().backward()
    opt.step()
    assert m[0].weight.grad is not None


def test_sgd_exact_arithmetic_and_warmup():
    p = torch.nn.Parameter(torch.tensor([1.0, 2.0]))
    opt = hb.SGD([p], lr=0.1, beta=0.5, weight_decay=0.1, warmup_steps=1)
    want, mom = p.data.clone(), torch.zeros(2)
    for step in (1, 2, 3):
        g = torch.tensor([0.5, -1.0]) * step
        p.grad = g.clone()
        opt.step()
        lr = 0.1 * step / max(step, 2)
        mom = mom * 0.5 + g
        want = want * (1 - 0.1 * lr) - lr * mom
        torch.testing.assert_close(p.data, want)
    assert opt.param_groups[0]["lr"] == 0.1 and opt.param_groups[0]["step"] is None


def test_kwarg_validation_and_renames():
    with pytest.raises(TypeError, match="unknown keyword"):
        hb.AdamW(_model().parameters(), not_a_kwarg=1)
    with pytest.raises(TypeError, match="Removed in HeavyBall 3.0"):
        hb.AdamW(_model().parameters(), stochastic_schedule=True)
    with pytest.warns(FutureWarning):
        opt = hb.AdamW(_model().parameters(), foreach=False)
    assert opt.param_groups[0]["multi_tensor"] is False
    with pytest.raises(ValueError):
        hb.AdEMAMix(_model().parameters(), betas=(0.9, 0.99))
    with pytest.raises(ValueError, match="Unknown function"):
        hb.AdamW(_model().parameters(), gradient_clipping="no_such_clip")


def test_subclass_overrides_defaults_and_string_clipping():
    class Clipped(hb.AdamW):
        gradient_clipping = "l2_clip_"
        palm = True

    opt = Clipped(_model().parameters())
    names = [getattr(f, "__name__", "") for f in opt.fns]
    assert names[0].startswith("apply_l2_clip__to_2") and "palm_beta2" in names
    # update clipping disables the fused update_by_* form
    opt = hb.AdamW(_model().parameters(), update_clipping=utils.trust_region_clip_)
    assert any(getattr(f, "fn_name", "") == "scale_by_adam" for f in opt.fns)


@pytest.mark.parametrize("name", ["SFAdamW", "MSAMLaProp"])
def test_train_eval_switch_is_idempotent(name):
    m = _model()
    opt = getattr(hb, name)(m.parameters(), lr=1e-2)
    _steps(m, opt, 4)
    train_w = m[0].weight.detach().clone()
    opt.eval()
    eval_w = m[0].weight.detach().clone()
    opt.eval()
    assert torch.equal(eval_w, m[0].weight)
    assert not torch.equal(train_w, eval_w)
    opt.train()
    opt.train()
    torch.testing.assert_close(m[0].weight.detach(), train_w, rtol=1e-5, atol=1e-6)


def test_closure_and_ema():
    m = _model()
    opt = hb.AdamW(m.parameters(), lr=1e-2)
    opt.use_ema = True
    x = torch.randn(4, 6)

    def closure():
        loss = m(x).square().mean()
        loss.backward()
        return loss

    l0 = opt.step(closure)
    l1 = opt.step(closure)
    assert l1 < l0
    before = m[0].weight.detach().clone()
    opt.copy_emas_to_params()
    assert not torch.equal(before, m[0].weight)
    opt.copy_params_to_emas()
    assert torch.equal(before, m[0].weight)


def test_split_opt_and_sam_wrapper():
    m = _model()
    mats = [p for p in m.parameters() if p.ndim >= 2]
    vecs = [p for p in m.parameters() if p.ndim < 2]
    opt = hb.SplitOpt([{"params": mats, "optimizer": hb.Muon, "lr": 0.02}, {"params": vecs, "optimizer": hb.AdamW}])
    _steps(m, opt)
    sd = opt.state_dict()
    assert set(sd) == {"optimizers"} and len(sd["optimizers"]) == 2
    opt.load_state_dict(copy.deepcopy(sd))
    with pytest.raises(ValueError):
        hb.SplitOpt([{"params": [], "optimizer": hb.AdamW}])

    m = _model()
    sam = hb.SAMWrapper(m.parameters(), hb.AdamW(m.parameters(), lr=1e-2), ball=0.05)
    x = torch.randn(4, 6)

    def closure():
        loss = m(x).square().mean()
        loss.backward()
        return loss

    l0 = float(sam.step(closure))
    for _ in range(5):
        l = float(sam.step(closure))
    assert l < l0
    with pytest.raises(ValueError):
        sam.step()
    assert set(sam.state_dict()) == {"wrapped", "ball"}


@pytest.mark.parametrize("shape", [(7,), (1, 5), (3, 1, 4), (2, 3, 1, 1, 2), ()])
@pytest.mark.parametrize("name", ["AdamW", "Muon", "SOAP", "PSGDKron"])
def test_nd_parameters(name, shape):
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(shape) if shape else torch.randn(()))
    if name in ("SOAP", "PSGDKron") and p.ndim == 0:
        pytest.skip("scalar parameters are not supported by the Kronecker-factored methods")
    opt = getattr(hb, name)([p], lr=1e-2)
    start = p.detach().clone()
    for _ in range(3):
        p.grad = torch.randn_like(p)
        opt.step()
    assert torch.isfinite(p).all() and not torch.equal(start, p.detach())


# ------------------------------------------------------------------------------------------ checkpoints


@pytest.mark.parametrize("name", ["AdamW", "SOAP", "PSGDKron", "SFAdamW"])
def test_state_dict_is_weights_only_loadable_and_resumes_exactly(name):
    m = _model().double()
    kw = {"lr": 1e-2, "storage_dtype": "float64"}  # fp64 parameters need fp64 state in the Kronecker methods
    if name == "PSGDKron":
        kw["q_dtype"] = "float64"
    opt = getattr(hb, name)(m.parameters(), **kw)
    x = torch.randn(8, 6, dtype=torch.float64)

    def run(model, optimizer, n):
        for i in range(n):
            torch.manual_seed(100 + i)
            model(x).square().mean().backward()
            optimizer.step()
            optimizer.zero_grad()

    run(m, opt, 4)
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    sd = torch.load(buf, weights_only=True)
    m2 = copy.deepcopy(m)
    opt2 = getattr(hb, name)(m2.parameters(), **kw)
    opt2.load_state_dict(sd)
    torch.manual_seed(5)
    run(m, opt, 3)
    torch.manual_seed(5)
    run(m2, opt2, 3)
    for a, b in zip(m.parameters(), m2.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-7, atol=1e-10)


def test_precond_schedule_pickle_is_reference_compatible_and_restricted():
    from heavyball_b200.utils import pickle_compat

    sched = utils.precond_update_prob_schedule(min_prob=0.05)
    data = pickle_compat.dumps(sched)
    assert b"heavyball.utils" in data and b"heavyball_b200" not in data
    back = pickle_compat.loads(data)
    assert back(5000) == sched(5000) and back.keywords["min_prob"] == 0.05
    assert pickle_compat.loads(pickle_compat.dumps(0.5)) == 0.5
    assert pickle_compat.loads(pickle_compat.dumps(None)) is None
    # what the reference itself would have written for its default PSGD schedule
    ref_bytes = (
        b"\x80\x04\x95\xac\x00\x00\x00\x00\x00\x00\x00\x8c\tfunctools\x94\x8c\x07partial\x94\x93\x94\x8c\x0fheavyball.utils"
        b"\x94\x8c#_inner_precond_update_prob_schedule\x94\x93\x94\x85\x94R\x94(h\x05)}\x94(\x8c\x08max_prob\x94G?\xf0\x00"
        b"\x00\x00\x00\x00\x00\x8c\x08min_prob\x94G?\x9e\xb8Q\xeb\x85\x1e\xb8\x8c\x05decay\x94G?\xef\xf7\xce\xd9\x16\x87+"
        b"\x8c\nflat_start\x94M\xe8\x03uNt\x94b."
    )
    assert pickle_compat.loads(ref_bytes)(1) == 1.0
    evil = pickle.dumps(print)
    with pytest.raises(pickle.UnpicklingError):
        pickle_compat.loads(evil)
