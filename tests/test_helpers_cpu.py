"""Hyper-parameter search helpers: numeric utilities, design space, HEBO quality on standard test functions,
the natural-gradient strategy, and the Optuna adapters driven through a stand-in for Optuna's API.
Modelled on the reference's ``test/test_helpers_cpu.py``."""

import math

import numpy as np
import pandas as pd
import pytest
import torch

from heavyball_b200 import helpers
from heavyball_b200.helpers import HEBO, DesignSpace, FastINGO

import fake_optuna as fo


def test_bound_to_torch_and_nextafter():
    arr = np.array([[0.0, 1.0], [2.0, 5.0], [-1.0, 3.0]])
    t = helpers.bound_to_torch(arr.tobytes(), arr.shape, "cpu")
    assert t.shape == (2, 3) and torch.equal(t, torch.from_numpy(arr.T.copy()))
    assert helpers.nextafter(0.5, 1.0) == np.nextafter(0.5, 1.0)
    assert helpers.nextafter(1, 0) == np.nextafter(1, 0)


def test_manual_seed_restores_generator_state():
    torch.manual_seed(7)
    expected = torch.rand(3)
    torch.manual_seed(7)
    with helpers.manual_seed(123):
        inside = torch.rand(3)
    assert torch.equal(torch.rand(3), expected)
    with helpers.manual_seed(123):
        assert torch.equal(torch.rand(3), inside)


def test_design_space_round_trip_and_reparse():
    space = DesignSpace().parse([
        {"name": "lr", "type": "pow", "lb": 1e-4, "ub": 1.0},
        {"name": "n", "type": "int", "lb": 1, "ub": 9},
        {"name": "w", "type": "pow_int", "lb": 8, "ub": 512},
    ])  # fmt: skip
    df = pd.DataFrame({"lr": [1e-3, 0.5], "n": [3, 9], "w": [16, 256]})
    x = space.transform(df)
    assert torch.allclose(x[:, 0], torch.tensor([math.log(1e-3), math.log(0.5)]), atol=1e-6)
    back = space.inverse_transform(x)
    assert np.allclose(back["lr"], df["lr"]) and list(back["n"]) == [3, 9] and list(back["w"]) == [16, 256]
    assert space.opt_lb()[0].item() == pytest.approx(math.log(1e-4))
    space.parse([{"name": "z", "type": "num", "lb": 0, "ub": 1}])
    assert space.para_names == ["z"] and list(space.paras) == ["z"]


def test_gp_interpolates_smooth_function():
    torch.manual_seed(0)
    x = torch.rand(40, 2) * 2 - 1
    f = lambda p: torch.sin(3 * p[:, 0]) + p[:, 1] ** 2  # noqa: E731
    model = helpers._Surrogate(num_epochs=150, lr=0.05)
    model.fit(x, f(x))
    q = torch.rand(200, 2) * 1.6 - 0.8
    mu, var = model.predict(q)
    assert (mu - f(q)).abs().mean() < 0.1
    assert (var > 0).all()
    mu_train, var_train = model.predict(x)
    assert var_train.mean() < var.mean() + 1e-3 and (mu_train - f(x)).abs().max() < 0.15


def _run_hebo(cfg, objective, n_iter, seed=42):
    opt = HEBO(DesignSpace().parse(cfg), scramble_seed=seed)
    for _ in range(n_iter):
        s = opt.suggest(1)
        opt.observe(s, np.array([[objective(s)]]))
    return opt


def _branin(x1, x2):
    b, c, t = 5.1 / (4 * math.pi**2), 5 / math.pi, 1 / (8 * math.pi)
    return (x2 - b * x1**2 + c * x1 - 6) ** 2 + 10 * (1 - t) * math.cos(x1) + 10


def test_hebo_quality_sphere_branin_mixed():
    box = lambda lo, hi: [{"name": "x1", "type": "num", "lb": lo[0], "ub": hi[0]}, {"name": "x2", "type": "num", "lb": lo[1], "ub": hi[1]}]  # noqa: E731
    sphere = _run_hebo(box((-5, -5), (5, 5)), lambda s: s["x1"].iloc[0] ** 2 + s["x2"].iloc[0] ** 2, 15)
    assert sphere.best_y < 2.0  # random search over 15 points: median about 4
    branin = _run_hebo(box((-5, 0), (10, 15)), lambda s: _branin(s["x1"].iloc[0], s["x2"].iloc[0]), 20)
    assert branin.best_y < 4.0  # optimum 0.398; random search over 20 points: median about 6

    def mixed(s):
        return (math.log10(s["lr"].iloc[0]) + 0.5) ** 2 + 100 * (s["wd"].iloc[0] - 0.09) ** 2 + (s["layers"].iloc[0] - 7) ** 2

    cfg = [{"name": "lr", "type": "pow", "lb": 1e-5, "ub": 1.0}, {"name": "wd", "type": "num", "lb": 0.0, "ub": 0.1},
           {"name": "layers", "type": "int", "lb": 1, "ub": 8}]  # fmt: skip
    opt = _run_hebo(cfg, mixed, 25)
    assert opt.best_y < 2.0
    assert isinstance(opt.best_x["layers"].iloc[0], (int, np.integer))


def test_hebo_discrete_space_visits_every_value_and_skips_nonfinite():
    opt = HEBO(DesignSpace().parse([{"name": "k", "type": "int", "lb": 0, "ub": 3}]), scramble_seed=0)
    seen = set()
    for _ in range(12):
        s = opt.suggest(1)
        k = int(s["k"].iloc[0])
        seen.add(k)
        opt.observe(s, np.array([[float("nan") if len(seen) == 1 and len(opt.X) == 0 else (k - 2) ** 2]]))
    assert seen == {0, 1, 2, 3}
    assert np.isfinite(opt.y).all() and opt.best_y == 0


def test_fast_ingo_moves_toward_minimum():
    opt = FastINGO(np.array([2.0, -3.0, 1.0]), np.ones(3), -5 * np.ones(3), 5 * np.ones(3), seed=0, device="cpu")
    start = float((opt._mean**2).sum())
    for _ in range(300):
        x = opt.ask()
        assert (x >= -5).all() and (x <= 5).all()
        opt.tell(float((x**2).sum()))
    assert opt.generation == 300
    assert float((opt._mean**2).sum()) < 0.8 * start
    assert opt.population_size % 2 == 0


def test_adapters_need_optuna_when_it_is_missing():
    try:
        import optuna  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="optuna"):
            helpers.HEBOSampler
        with pytest.raises(AttributeError):
            helpers.no_such_name


# ------------------------------------------------------------------ adapters against the Optuna stand-in


@pytest.fixture(scope="module")
def bound():
    return fo.install()


SPACE = {"x": fo.FloatDistribution(-5, 5), "y": fo.FloatDistribution(-5, 5)}


def test_untransform_handles_steps_logs_and_ints(bound):
    u = bound._untransform_numerical_param_torch
    assert u(torch.tensor(0.26), fo.FloatDistribution(0, 1, step=0.25), False).item() == pytest.approx(0.25)
    assert u(torch.tensor(math.log(200.0), dtype=torch.float64), fo.FloatDistribution(1, 100, log=True), True).item() < 100.0
    out = u(torch.tensor(6.6), fo.IntDistribution(1, 9, step=2), True)
    assert out.dtype == torch.int64 and out.item() == 7
    assert u(torch.tensor(math.log(40.0)), fo.IntDistribution(1, 32, log=True), True).item() == 32
    tr = bound.SearchSpaceTransform({"a": fo.FloatDistribution(1e-3, 1, log=True), "n": fo.IntDistribution(1, 4)}, transform_0_1=True)
    assert tr.bounds.tolist() == [[0.0, 1.0], [0.0, 1.0]]
    assert tr.untransform(torch.tensor([0.0, 1.0])) == {"a": pytest.approx(1e-3), "n": 4}
    assert tr.untransform(tr.transform({"a": 0.1, "n": 2})) == {"a": pytest.approx(0.1), "n": 2}
    with pytest.raises(ValueError):
        bound.SearchSpaceTransform({"c": fo.CategoricalDistribution(["p", "q"])})


def test_samplers_reject_unknown_keywords(bound):
    with pytest.raises(TypeError):
        bound.BoTorchSampler(SPACE, consider_running_trials=True)
    with pytest.raises(TypeError):
        bound.HEBOSampler(SPACE, constant_liar=True)
    with pytest.raises(TypeError):
        bound.ImplicitNaturalGradientSampler(SPACE, warn_independent_sampling=False)
    with pytest.raises(TypeError):
        bound.AutoSampler(search_space=SPACE, constraints_func=lambda *_: None)
    with pytest.raises(ValueError):
        bound.AutoSampler()


def test_hebo_sampler_beats_random_on_sphere(bound):
    sphere = lambda p: p["x"] ** 2 + p["y"] ** 2  # noqa: E731
    best = fo.Study(bound.HEBOSampler(SPACE, seed=1), SPACE).run(sphere, 18)
    assert best < 1.5
    grid = {"x": fo.FloatDistribution(-4, 4, step=0.5), "n": fo.IntDistribution(1, 64, log=True)}
    study = fo.Study(bound.HEBOSampler(grid, seed=0), grid, direction=fo.StudyDirection.MAXIMIZE)
    study.run(lambda p: -(p["x"] - 1.5) ** 2 - (math.log2(p["n"]) - 3) ** 2, 14)
    for t in study.trials:
        assert (t.params["x"] * 2) == round(t.params["x"] * 2) and 1 <= t.params["n"] <= 64
    assert max(t.value for t in study.trials) > -3.0


def test_botorch_sampler_with_custom_and_builtin_candidates(bound):
    calls = []

    def centre(train_x, train_obj, train_con, bounds, pending):
        calls.append((train_x.shape, train_obj.shape, bounds.shape))
        return torch.full((1, train_x.shape[1]), 0.5, dtype=train_x.dtype)

    study = fo.Study(bound.BoTorchSampler(SPACE, candidates_func=centre, n_startup_trials=2, seed=0), SPACE)
    study.run(lambda p: p["x"] ** 2 + p["y"] ** 2, 4)
    assert calls and calls[0][2] == (2, 2) and calls[-1][0] == (3, 2)
    assert study.trials[-1].params == {"x": pytest.approx(0.0), "y": pytest.approx(0.0)}
    best = fo.Study(bound.BoTorchSampler(SPACE, n_startup_trials=4, seed=0), SPACE).run(lambda p: p["x"] ** 2 + p["y"] ** 2, 14)
    assert best < 2.0


def test_ingo_sampler_tags_generations(bound):
    sampler = bound.ImplicitNaturalGradientSampler(SPACE, seed=3)
    study = fo.Study(sampler, SPACE)
    study.run(lambda p: (p["x"] - 1) ** 2 + (p["y"] + 2) ** 2, 30)
    tags = [t.system_attrs.get("ingo") for t in study.trials[1:]]
    assert tags == sorted(tags) and tags[-1] >= 20
    assert sampler.infer_relative_search_space(study, None).keys() == SPACE.keys()
    one = {"x": fo.FloatDistribution(-1, 1)}
    assert bound.ImplicitNaturalGradientSampler(one).sample_relative(fo.Study(None, one), None, one) == {}


def test_auto_sampler_switches_on_schedule_and_pickles(bound):
    import pickle

    made = []

    def first(study, seed, trials, space):
        made.append(("first", len(trials)))
        return fo.RandomSampler(seed)

    def second(study, seed, trials, space):
        made.append(("second", len(trials)))
        return bound.init_hebo(study, seed, trials, space)

    auto = bound.AutoSampler(samplers=[(5, second), (0, first)], search_space=SPACE, seed=0)
    study = fo.Study(auto, SPACE)
    study.run(lambda p: p["x"] ** 2 + p["y"] ** 2, 9)
    assert made == [("first", 1), ("second", 5)]
    names = [t.system_attrs["auto:sampler"] for t in study.trials]
    assert names[0] == names[4] == "RandomSampler" and names[6] == "HEBOSampler"
    clone = pickle.loads(pickle.dumps(bound.AutoSampler(samplers=[(0, bound.init_random)], seed=1)))
    assert isinstance(clone._sampler, fo.RandomSampler)
    with pytest.raises(ValueError):
        auto.after_trial(study, study.trials[0], fo.TrialState.RUNNING, None)
