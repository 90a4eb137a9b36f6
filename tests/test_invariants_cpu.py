"""Behavioural invariants every optimizer has to keep, checked on CPU (fp64 where exactness is the point).

Modelled on the reference's ``test/test_foreach.py:41`` (multi-tensor == per-tensor), ``test/test_save_restore.py:51-88``
(a reloaded optimizer continues exactly, also with merged / split dimensions), ``test/test_nd_param.py:25`` (1-D to
5-D parameters with size-1 dims), ``test/test_ecc.py:452-616`` (error-corrected state survives every load order) and
``test/test_migrate_cli.py:640-738`` (every former class name migrates end to end).
"""

import copy
import inspect

import pytest
import torch

import heavyball_b200 as hb
from heavyball_b200 import migrate

# one class per distinct chain shape
REPRESENTATIVE = ["AdamW", "NAdam", "LaProp", "ADOPT", "AdEMAMix", "RMSprop", "SGD", "SFAdamW", "Muon", "MuonAdamW",
                  "SOAP", "KLShampoo", "PSGDKron", "PSGDPRO", "LATHER", "SignLaProp", "OrthoLaProp", "Scion"]  # fmt: skip


def _kwargs(name, **extra):
    kw = {"lr": 1e-2}
    if "max_lr" in inspect.signature(getattr(hb, name).__init__).parameters:
        kw["max_lr"] = 1e-2
    if name == "SFAdamW":
        kw["warmup_steps"] = 1
    kw.update(extra)
    return kw


def _fp64(name, **extra):
    """Keyword arguments for a run in double precision: state (and PSGD factors) stored in fp64 too."""
    accepted = inspect.signature(getattr(hb, name).__init__).parameters
    wide = {k: "float64" for k in ("storage_dtype", "q_dtype") if k in accepted}
    return _kwargs(name, **wide, **extra)


def _net(dtype, seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(6, 12), torch.nn.Tanh(), torch.nn.Linear(12, 12), torch.nn.Tanh(),
                               torch.nn.Linear(12, 3)).to(dtype)  # fmt: skip


def _train(model, opt, steps, dtype, data_seed=1):
    g = torch.Generator().manual_seed(data_seed)
    x, y = torch.randn(32, 6, generator=g).to(dtype), torch.randn(32, 3, generator=g).to(dtype)
    losses = []
    for _ in range(steps):
        def closure():
            loss = torch.nn.functional.mse_loss(model(x), y)
            loss.backward()
            return loss
        losses.append(float(opt.step(closure)))
        opt.zero_grad()
    return losses


# ------------------------------------------------------------------ multi-tensor == per-tensor
_PER_TENSOR_RNG = {"Muon", "MuonAdamW", "PSGDKron", "PSGDPRO", "LATHER", "Scion"}  # random draws depend on the batching


@pytest.mark.parametrize("name", REPRESENTATIVE)
def test_multi_tensor_matches_per_tensor(name):
    results = []
    for multi in (True, False):
        model = _net(torch.float64)
        torch.manual_seed(3)
        opt = getattr(hb, name)(model.parameters(), **_fp64(name, multi_tensor=multi))
        results.append((_train(model, opt, 5, torch.float64), [p.detach().clone() for p in model.parameters()]))
    (la, pa), (lb, pb) = results
    if name in _PER_TENSOR_RNG:
        assert abs(la[-1] - lb[-1]) <= 0.2 * abs(la[0]) + 1e-6
    else:
        for a, b in zip(pa, pb):  # batched and per-tensor products sum in a different order
            torch.testing.assert_close(a, b, rtol=1e-7, atol=1e-10)


# ------------------------------------------------------------------ exact resume
RESUME = [(n, {}) for n in REPRESENTATIVE if n not in ("Scion",)] + [
    ("SOAP", {"merge_dims": True, "max_precond_dim": 16}),
    ("SOAP", {"merge_dims": True, "split": True, "max_precond_dim": 8}),
    ("PSGDKron", {"merge_dims": True, "max_size_triangular": 8}),
    ("AdamW", {"mars": True, "caution": True, "palm": True}),
]


@pytest.mark.parametrize("name,extra", RESUME, ids=[f"{n}-{i}" for i, (n, _) in enumerate(RESUME)])
def test_reloaded_optimizer_continues_exactly_in_fp64(name, extra):
    def build():
        model = _net(torch.float64)
        torch.manual_seed(3)
        return model, getattr(hb, name)(model.parameters(), **_fp64(name, **extra))

    model, opt = build()
    _train(model, opt, 4, torch.float64)
    saved_model, saved_opt = copy.deepcopy(model.state_dict()), copy.deepcopy(opt.state_dict())
    rng = torch.get_rng_state()
    straight = _train(model, opt, 3, torch.float64, data_seed=2)
    model2, opt2 = build()
    model2.load_state_dict(saved_model)
    opt2.load_state_dict(saved_opt)
    torch.set_rng_state(rng)
    resumed = _train(model2, opt2, 3, torch.float64, data_seed=2)
    # schedule-free keeps its running weight sum as an fp32 scalar in the checkpoint (the interchange format)
    tol = 1e-6 if name == "SFAdamW" else 1e-9
    assert resumed == pytest.approx(straight, rel=tol, abs=1e-12)
    for a, b in zip(model.parameters(), model2.parameters()):
        torch.testing.assert_close(a, b, rtol=tol, atol=tol * 1e-2)


# ------------------------------------------------------------------ parameter ranks
ND_SHAPES = [(7,), (1,), (4, 3), (1, 5), (5, 1), (2, 3, 4), (2, 1, 3, 2), (2, 2, 1, 2, 3)]


@pytest.mark.parametrize("name", REPRESENTATIVE)
def test_parameters_of_any_rank_are_stepped(name):
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(s) * 0.5 + 0.1) for s in ND_SHAPES]
    opt = getattr(hb, name)(params, **_kwargs(name))
    before = [p.detach().clone() for p in params]
    for _ in range(3):
        for p in params:
            p.grad = torch.randn_like(p) * 0.1 + 0.05
        opt.step()
    for s, b, p in zip(ND_SHAPES, before, params):
        assert p.shape == torch.Size(s) and torch.isfinite(p).all(), (name, s)
        if name == "OrthoLaProp" and s == (1,):
            continue  # a one-element gradient is parallel to its weight: nothing is left after the projection
        assert not torch.equal(b, p.detach()), (name, s)


def test_no_gradient_means_no_state():
    params = [torch.nn.Parameter(torch.randn(3, 3)) for _ in range(2)]
    opt = hb.AdamW(params, lr=1e-2)
    opt.step()
    assert opt.state_size() == 0


# ------------------------------------------------------------------ error-corrected state across load orders
def _ecc_opt(params, **kw):
    return hb.AdamW(params, lr=1e-2, ecc="bf16+8", **kw)


def _step(opt, params, n=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    for _ in range(n):
        for p in params:
            p.grad = torch.randn(p.shape, generator=g).to(p.dtype) * 0.1
        opt.step()


def _ecc_layout_ok(opt, params, param_ecc):
    for p in params:
        st = opt.state[p][0]
        for k, v in st.items():
            if not isinstance(v, torch.Tensor) or k in ("step",):
                continue
            if k.endswith("::ecc"):
                assert v.dtype == torch.int8, (k, v.dtype)
            elif k + "::ecc" in st:
                assert v.dtype == torch.bfloat16, (k, v.dtype)
        if param_ecc:
            assert p.dtype == torch.bfloat16 and st["param::ecc"].dtype == torch.int8


@pytest.mark.parametrize("param_ecc", [False, True])
@pytest.mark.parametrize("order", ["optimizer_first", "model_first", "empty_state", "stripped_residuals"])
def test_ecc_state_survives_every_load_order(param_ecc, order):
    torch.manual_seed(0)
    extra = {"param_ecc": "bf16+8"} if param_ecc else {}
    src = [torch.nn.Parameter(torch.randn(8, 4)), torch.nn.Parameter(torch.randn(5))]
    opt = _ecc_opt(src, **extra)
    if order != "empty_state":
        _step(opt, src)
    sd = copy.deepcopy(opt.state_dict())
    weights = [p.detach().clone() for p in src]
    if order == "stripped_residuals":  # a checkpoint written without the parameter residuals must be re-hydrated
        for per_view in sd["state"].values():
            for st in per_view.values():
                st.pop("param::ecc", None)

    dst = [torch.nn.Parameter(torch.randn(8, 4)), torch.nn.Parameter(torch.randn(5))]
    if order == "model_first":
        with torch.no_grad():
            for d, w in zip(dst, weights):
                d.data = w.clone()
        new = _ecc_opt(dst, **extra)
        new.load_state_dict(sd)
    else:
        new = _ecc_opt(dst, **extra)
        new.load_state_dict(sd)
        with torch.no_grad():
            for d, w in zip(dst, weights):
                d.data.copy_(w)
    _step(new, dst, seed=1)
    _ecc_layout_ok(new, dst, param_ecc)
    assert all(torch.isfinite(p.float()).all() for p in dst)
    if order not in ("empty_state", "stripped_residuals") and not param_ecc:
        _step(opt, src, seed=1)  # the original continues to (nearly) the same point: residual rounding is random
        for a, b in zip(src, dst):
            assert (a.float() - b.float()).abs().max() < 5e-3


# ------------------------------------------------------------------ every former class name migrates end to end
def _flat_v1(opt_cls, params):
    """A 1.x-style checkpoint of ``opt_cls``: run the current class for a step, then flatten its nested state
    (``state[p][view][key_idx]`` -> ``state[p][key]``) and rename the group keys back."""
    opt = opt_cls(params, **({"lr": 1e-3, "max_lr": 1e-2} if "max_lr" in inspect.signature(opt_cls.__init__).parameters else {"lr": 1e-3}))
    for p in params:
        p.grad = torch.ones_like(p) * 0.1
    opt.step()
    sd = opt.state_dict()
    flat = {}
    for idx, per_view in sd["state"].items():
        entry = {}
        for key, value in per_view[0].items():
            base = key.rsplit("_", 1)[0] if key.rsplit("_", 1)[-1].isdigit() else key
            entry[base] = value
        flat[idx] = entry
    groups = []
    for g in sd["param_groups"]:
        g = dict(g)
        g["foreach"] = g.pop("multi_tensor", True)
        g["stochastic_schedule"] = False
        groups.append(g)
    return {"state": flat, "param_groups": groups}


_MIGRATABLE = sorted(old for old, new in migrate._CLASS_RENAMES.items()
                     if new in ("AdamW", "LaProp", "ADOPT", "RMSprop", "SGD", "Muon", "AdEMAMix", "SFAdamW", "NAdam"))  # fmt: skip


@pytest.mark.parametrize("old_name", _MIGRATABLE)
def test_former_class_names_migrate_end_to_end(old_name, tmp_path):
    new_cls = getattr(hb, migrate._CLASS_RENAMES[old_name])
    params = [torch.nn.Parameter(torch.randn(4, 3)), torch.nn.Parameter(torch.randn(3))]
    path = tmp_path / "old.pt"
    torch.save({"optimizer": _flat_v1(new_cls, params)}, path)
    out = tmp_path / "new.pt"
    assert migrate.main([str(path), f"heavyball.{old_name}", "--state-key", "optimizer", "-o", str(out)]) == 0
    sd = torch.load(out, weights_only=False)["optimizer"]
    assert migrate._detect_version(sd) == 3
    fresh = [torch.nn.Parameter(p.detach().clone()) for p in params]
    kw = {"lr": 1e-3, "max_lr": 1e-2} if "max_lr" in inspect.signature(new_cls.__init__).parameters else {"lr": 1e-3}
    opt = new_cls(fresh, **kw)
    opt.load_state_dict(sd)
    for p in fresh:
        p.grad = torch.ones_like(p) * 0.1
    opt.step()
    assert all(torch.isfinite(p).all() for p in fresh)
