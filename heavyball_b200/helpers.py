"""Hyper-parameter search helpers: a compact HEBO-style Bayesian optimiser, an implicit-natural-gradient
evolution strategy, and (when ``optuna`` is installed) sampler adapters for both plus a scheduled
``AutoSampler``.

Capability parity: ``heavyball/helpers.py:1-1111`` of the reference.  Differences by design:

* the Gaussian process is written here in plain PyTorch (exact GP, constant mean, scaled ARD Matern-5/2
  kernel, Gaussian noise with a lower bound and a log-normal prior) instead of depending on ``gpytorch``;
* the search-space transform used by the adapters is written here instead of importing Optuna's private
  ``_SearchSpaceTransform``;
* the core classes (``DesignSpace``, ``HEBO``, ``FastINGO``) import without Optuna.  The adapter classes
  (``SimpleAPIBaseSampler``, ``BoTorchSampler``, ``HEBOSampler``, ``ImplicitNaturalGradientSampler``,
  ``AutoSampler``) subclass ``optuna.samplers.BaseSampler`` and exist only when ``optuna`` imports;
  asking for one without it raises ``ImportError`` naming the missing package.

This module is not imported by ``heavyball_b200/__init__.py``.
"""

from __future__ import annotations

import copy
import functools
import math
import threading
from contextlib import contextmanager
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
from torch import Tensor
from torch.quasirandom import SobolEngine

_MAXINT32 = (1 << 31) - 1
_SAMPLER_KEY = "auto:sampler"


@contextmanager
def manual_seed(seed: Optional[int] = None):
    """Seeds ``torch.random`` inside the block and restores the previous generator state afterwards."""
    if seed is None:
        yield
        return
    saved = torch.random.get_rng_state()
    torch.random.manual_seed(seed)
    try:
        yield
    finally:
        torch.random.set_rng_state(saved)


@functools.cache
def bound_to_torch(bound: bytes, shape: tuple, device: str) -> Tensor:
    """``(n, 2)`` float64 bounds given as raw bytes -> ``(2, n)`` tensor (row 0 lower, row 1 upper)."""
    arr = np.frombuffer(bound, dtype=np.float64).reshape(shape)
    return torch.from_numpy(arr.T.copy()).to(torch.device(device))


@functools.cache
def nextafter(x: float, y: float) -> Union[float, int]:
    return np.nextafter(x, y)


def _use_cuda() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


# ------------------------------------------------------------------------------------ design space


class _Param:
    """One numeric search dimension.  ``ptype``: ``num`` (float), ``int``, ``pow`` (log-scaled float),
    ``pow_int`` (log-scaled integer)."""

    __slots__ = ("name", "ptype", "lb", "ub")

    def __init__(self, name, ptype, lb, ub):
        if ptype not in ("num", "int", "pow", "pow_int"):
            raise ValueError(f"unknown parameter type {ptype!r}")
        self.name, self.ptype, self.lb, self.ub = name, ptype, float(lb), float(ub)

    is_log = property(lambda self: self.ptype in ("pow", "pow_int"))
    is_int = property(lambda self: self.ptype in ("int", "pow_int"))
    is_discrete_after_transform = property(lambda self: self.ptype == "int")
    opt_lb = property(lambda self: math.log(self.lb) if self.is_log else self.lb)
    opt_ub = property(lambda self: math.log(self.ub) if self.is_log else self.ub)

    def transform(self, x):
        return np.log(x) if self.is_log else x

    def inverse(self, x):
        v = np.exp(x) if self.is_log else x
        return np.round(v).astype(int) if self.is_int else v


class DesignSpace:
    """Ordered set of ``_Param``; maps data frames of raw values to optimiser coordinates and back."""

    def __init__(self):
        self.paras: Dict[str, _Param] = {}
        self.para_names: List[str] = []

    def parse(self, configs):
        self.paras = {c["name"]: _Param(c["name"], c["type"], c["lb"], c["ub"]) for c in configs}
        self.para_names = [c["name"] for c in configs]
        return self

    @property
    def num_paras(self):
        return len(self.para_names)

    def opt_lb(self, device="cpu"):
        return torch.tensor([self.paras[n].opt_lb for n in self.para_names], device=device)

    def opt_ub(self, device="cpu"):
        return torch.tensor([self.paras[n].opt_ub for n in self.para_names], device=device)

    def transform(self, df, device="cpu"):
        cols = [self.paras[n].transform(df[n].values.astype(float)) for n in self.para_names]
        data = np.column_stack(cols) if cols else np.zeros((len(df), 0))
        return torch.as_tensor(data, dtype=torch.float32, device=device)

    def inverse_transform(self, x):
        import pandas as pd

        x = x.detach().cpu().numpy() if isinstance(x, Tensor) else np.asarray(x)
        return pd.DataFrame({n: self.paras[n].inverse(x[:, i]) for i, n in enumerate(self.para_names)})


# ------------------------------------------------------------------------------------ Gaussian process


def _softplus_inv(v: float) -> float:
    return math.log(math.expm1(v))


class _MaternGP(torch.nn.Module):
    """Exact GP regression: constant mean, ``s * Matern52(|x - x'| / l)`` with one length scale per input
    dimension, homoscedastic noise ``>= noise_lb`` with a ``LogNormal(log 0.01, 0.5)`` prior."""

    def __init__(self, dims: int, noise_lb: float, noise_init: float):
        super().__init__()
        self.noise_lb = noise_lb
        self.raw_length = torch.nn.Parameter(torch.zeros(dims))
        self.raw_scale = torch.nn.Parameter(torch.zeros(()))
        self.raw_noise = torch.nn.Parameter(torch.full((), _softplus_inv(max(noise_init - noise_lb, 1e-6))))
        self.mean = torch.nn.Parameter(torch.zeros(()))

    @property
    def noise(self):
        return torch.nn.functional.softplus(self.raw_noise) + self.noise_lb

    def kernel(self, a: Tensor, b: Tensor) -> Tensor:
        length = torch.nn.functional.softplus(self.raw_length)
        d = torch.cdist(a / length, b / length).clamp_min(1e-15)
        r = math.sqrt(5.0) * d
        return torch.nn.functional.softplus(self.raw_scale) * (1.0 + r + r.square() / 3.0) * torch.exp(-r)

    def _factor(self, x: Tensor, jitter: float = 0.0) -> Tensor:
        k = self.kernel(x, x)
        k = k + (self.noise + jitter) * torch.eye(x.shape[0], dtype=x.dtype, device=x.device)
        return torch.linalg.cholesky(k)

    def neg_log_marginal(self, x: Tensor, y: Tensor) -> Tensor:
        chol = self._factor(x)
        resid = (y - self.mean).unsqueeze(-1)
        alpha = torch.cholesky_solve(resid, chol)
        n = x.shape[0]
        mll = -0.5 * (resid * alpha).sum() - chol.diagonal().log().sum() - 0.5 * n * math.log(2 * math.pi)
        log_noise = self.noise.log()
        prior = -log_noise - 0.5 * ((log_noise - math.log(0.01)) / 0.5) ** 2 - math.log(0.5 * math.sqrt(2 * math.pi))
        return -(mll + prior) / n

    @torch.no_grad()
    def posterior(self, x: Tensor, y: Tensor, query: Tensor, jitter: float = 1e-3):
        chol = self._factor(x, jitter)
        cross = self.kernel(x, query)
        alpha = torch.cholesky_solve((y - self.mean).unsqueeze(-1), chol)
        mu = self.mean + (cross.mT @ alpha).squeeze(-1)
        half = torch.linalg.solve_triangular(chol, cross, upper=False)
        var = torch.nn.functional.softplus(self.raw_scale) - half.square().sum(0)
        return mu, var


class _Surrogate:
    """Input scaling to ``[-1, 1]``, target standardisation, ``num_epochs`` Adam steps on the marginal
    likelihood.  Parity: ``heavyball/helpers.py:442-489``."""

    def __init__(self, num_epochs: int = 100, lr: float = 0.01, noise_lb: float = 8e-4):
        self.num_epochs, self.lr, self.noise_lb = num_epochs, lr, noise_lb

    def _scale_x(self, X):
        return 2 * (X - self._x_min) / (self._x_max - self._x_min).clamp(min=1e-8) - 1

    def fit(self, X: Tensor, y: Tensor):
        self._x_min, self._x_max = X.min(0).values, X.max(0).values
        self._y_mu, self._y_std = y.mean(), y.std(correction=0).clamp(min=1e-8)
        self._xs = self._scale_x(X)
        self._ys = ((y - self._y_mu) / self._y_std).reshape(-1)
        self.gp = _MaternGP(X.shape[1], self.noise_lb, max(1e-2, self.noise_lb)).to(X.device)
        opt = torch.optim.Adam(self.gp.parameters(), lr=self.lr)
        with torch.enable_grad():
            for _ in range(self.num_epochs):
                try:
                    opt.zero_grad()
                    self.gp.neg_log_marginal(self._xs, self._ys).backward()
                    opt.step()
                except RuntimeError:  # Cholesky of an indefinite kernel matrix: keep the last good parameters
                    break

    @torch.no_grad()
    def predict(self, X: Tensor):
        mu, var = self.gp.posterior(self._xs, self._ys, self._scale_x(X))
        return mu * self._y_std + self._y_mu, (var * self._y_std**2).clamp(min=1e-8)


# ------------------------------------------------------------------------------------ HEBO


class HEBO:
    """Minimal heteroscedastic-evolutionary-BO loop for minimisation: scrambled-Sobol start-up points,
    then a GP on power-transformed targets and the lower confidence bound ``mu - kappa * sigma`` ranked over
    a fresh Sobol candidate set; points already evaluated are skipped.  Parity: ``heavyball/helpers.py:492-597``."""

    def __init__(self, space: DesignSpace, scramble_seed=None, rand_sample=None, device="cpu"):
        import pandas as pd

        self.space = space
        self.device = torch.device(device)
        self.X = pd.DataFrame(columns=space.para_names)
        self.y = np.zeros((0, 1))
        self.rand_sample = (1 + space.num_paras) if rand_sample is None else rand_sample
        self._seed = scramble_seed
        self.sobol = SobolEngine(space.num_paras, scramble=True, seed=scramble_seed)

    def _round_discrete(self, pts: Tensor) -> Tensor:
        for i, name in enumerate(self.space.para_names):
            if self.space.paras[name].is_discrete_after_transform:
                pts[:, i] = pts[:, i].round()
        return pts

    def _quasi_sample(self, n):
        lb, ub = self.space.opt_lb(), self.space.opt_ub()
        return self.space.inverse_transform(self._round_discrete(self.sobol.draw(n) * (ub - lb) + lb))

    def _transform_y(self) -> Tensor:
        from sklearn.preprocessing import power_transform

        scaled = self.y / max(self.y.std(), 1e-8)
        try:
            if self.y.min() <= 0:
                out = power_transform(scaled, method="yeo-johnson")
            else:
                out = power_transform(scaled, method="box-cox")
                if out.std() < 0.5:
                    out = power_transform(scaled, method="yeo-johnson")
            if out.std() < 0.5 or not np.isfinite(out).all():
                raise ValueError("degenerate power transform")
        except (RuntimeError, ValueError):
            out = self.y
        return torch.as_tensor(out, dtype=torch.float32, device=self.device)

    def suggest(self, n_suggestions: int = 1):
        if self.X.shape[0] < self.rand_sample:
            return self._quasi_sample(n_suggestions)
        try:
            return self._suggest_bo(n_suggestions)
        except (RuntimeError, ValueError):
            return self._quasi_sample(n_suggestions)

    def _suggest_bo(self, n_suggestions):
        import pandas as pd

        dev = self.device
        X = self.space.transform(self.X, device=dev)
        model = _Surrogate()
        model.fit(X, self._transform_y())

        dim, n_obs = X.shape[1], max(1, self.X.shape[0])
        kappa = math.sqrt(2.0 * math.log(n_obs * dim)) if n_obs * dim > 1 else 0.0
        lb, ub = self.space.opt_lb(dev).float(), self.space.opt_ub(dev).float()
        n_cand = max(2000, 200 * dim)
        seed = None if self._seed is None else self._seed + n_obs
        cands = SobolEngine(dim, scramble=True, seed=seed).draw(n_cand).to(dev)
        cands = self._round_discrete(lb + (ub - lb) * cands)

        mu, var = model.predict(cands)
        ranked = (mu - kappa * var.sqrt()).argsort().cpu().numpy()
        cands_np = cands.cpu().numpy()
        seen = {tuple(row) for row in X.cpu().numpy()}
        chosen = []
        for idx in ranked:
            key = tuple(cands_np[idx])
            if key in seen:
                continue
            seen.add(key)
            chosen.append(idx)
            if len(chosen) >= n_suggestions:
                break
        result = self.space.inverse_transform(cands_np[chosen])
        while len(result) < n_suggestions:
            result = pd.concat([result, self._quasi_sample(n_suggestions - len(result))], ignore_index=True)
        return result.head(n_suggestions)

    def observe(self, X, y):
        import pandas as pd

        y = np.asarray(y, dtype=float)
        ok = np.isfinite(y.reshape(-1))
        fresh = X[ok]
        self.X = fresh.reset_index(drop=True) if len(self.X) == 0 else pd.concat([self.X, fresh], ignore_index=True)
        self.y = np.vstack([self.y, y[ok].reshape(-1, 1)])

    @property
    def best_x(self):
        return self.X.iloc[[self.y.ravel().argmin()]]

    @property
    def best_y(self):
        return self.y.min()


# ------------------------------------------------------------------------------------ implicit natural gradient


class FastINGO:
    """Implicit natural-gradient optimiser over a diagonal Gaussian (mean, inverse variance): ``ask`` draws
    one clamped sample, ``tell`` feeds its objective value (minimised).  Every ``tell`` recomputes the
    distribution from the last ``last_n`` samples: scores are log-objectives standardised with
    exponentially decaying weights, each sample proposes a target (mean, inverse variance) one step
    ``loco_step_size`` along its score-weighted gradient, and the new distribution is the decayed average of
    those targets.  Parity: ``heavyball/helpers.py:725-826``."""

    def __init__(self, mean, inv_sigma, lower, upper, seed: Optional[int] = None, population_size: Optional[int] = None,
                 last_n: int = 4096, loco_step_size: float = 0.1, device: Optional[str] = None,
                 batchnorm_decay: float = 0.99, score_decay: float = 0.99):  # fmt: skip
        device = _use_cuda() if device is None else device
        dim = len(mean)
        if population_size is None:
            population_size = 2 * ((4 + int(math.floor(3 * math.log(dim)))) // 2)
        as_t = lambda a: torch.as_tensor(np.asarray(a, dtype=np.float64)).to(device)  # noqa: E731
        self._mean, self._sigma, self._lower, self._upper = as_t(mean), as_t(inv_sigma), as_t(lower), as_t(upper)
        self.generator = torch.Generator(device=device)
        self.generator.manual_seed(0x123123 if seed is None else seed)
        self.last_n, self.loco_step_size = last_n, loco_step_size
        self.batchnorm_decay, self.score_decay = batchnorm_decay, score_decay
        self._population_size, self.device = population_size, device
        self._ys = self._means = self._z = self._stds = None
        self._g = 0

    dim = property(lambda self: self._mean.shape[0])
    generation = property(lambda self: self._g)
    population_size = property(lambda self: self._population_size)

    def _push(self, name: str, row) -> None:
        if isinstance(row, np.ndarray):
            row = torch.from_numpy(row).to(self.device)
        elif not isinstance(row, Tensor):
            row = torch.as_tensor(float(row), dtype=self._mean.dtype, device=self._mean.device).view(1)
        prev = getattr(self, name)
        setattr(self, name, row if prev is None else torch.cat((prev, row), dim=0)[-self.last_n :])

    @torch.no_grad()
    def ask(self) -> np.ndarray:
        z = torch.randn(self.dim, generator=self.generator, device=self.device, dtype=torch.float64)
        self._push("_z", z[None])
        self._push("_means", self._mean[None])
        self._push("_stds", self._sigma[None])
        x = z / self._sigma.clamp(min=1e-8).sqrt() + self._mean
        return x.clamp(min=self._lower, max=self._upper).cpu().numpy()

    @torch.no_grad()
    def tell(self, y: float) -> None:
        self._g += 1
        self._push("_ys", y)
        ys = self._ys
        if ys.numel() <= 2:
            return
        lo, hi = ys.min(), ys.max()
        if torch.isclose(hi, lo, rtol=0.0, atol=1e-12):
            return
        if lo <= 0:
            ys = ys + (1e-8 - lo)
        ys = ys.clamp_min(1e-8).log()

        age = -torch.arange(ys.size(0), device=ys.device, dtype=ys.dtype)  # same (oldest-first) weighting as the reference

        def decayed(rate):
            w = rate**age
            return w / w.sum().clamp(min=1e-8)

        w = decayed(self.batchnorm_decay)
        mu = w @ ys
        sd = (w @ ys.square() - mu.square()).clamp(min=1e-8).sqrt()
        score = ((ys - mu) / sd).view(-1, 1)

        z, mean0, prec0 = self._z, self._means, self._stds
        target_mean = mean0 - self.loco_step_size * score * (z / prec0.clamp(min=1e-8).sqrt())
        target_prec = prec0 + self.loco_step_size * score * z.square() * prec0
        w = decayed(self.score_decay)
        self._mean, self._sigma = w @ target_mean, w @ target_prec


# ------------------------------------------------------------------------------------ Optuna adapters

_ADAPTER_NAMES = (
    "SimpleAPIBaseSampler", "BoTorchSampler", "HEBOSampler", "ImplicitNaturalGradientSampler", "AutoSampler",
    "ThreadLocalSampler", "init_cmaes", "init_hebo", "init_botorch", "init_nsgaii", "init_random", "init_ingo",
    "_untransform_numerical_param_torch", "_convert_to_hebo_design_space", "SearchSpaceTransform", "untransform",
)  # fmt: skip


def _reject_unknown(kwargs, where):
    if kwargs:
        raise TypeError(f"{where} got unexpected keyword arguments: {sorted(kwargs)}")


def _logei_over_sobol(train_x: Tensor, train_y: Tensor, bounds: Tensor, n_candidates: int = 4096, seed=None) -> Tensor:
    """Default candidate generator of ``BoTorchSampler`` when no ``candidates_func`` is given: fits the GP of
    this module to ``(train_x, train_y)`` (maximisation) and returns the Sobol candidate with the largest
    log expected improvement."""
    dim = train_x.shape[1]
    model = _Surrogate()
    model.fit(train_x.float(), train_y.reshape(-1).float())
    cands = SobolEngine(dim, scramble=True, seed=seed).draw(n_candidates).to(train_x.device)
    cands = bounds[0].float() + (bounds[1] - bounds[0]).float() * cands
    mu, var = model.predict(cands)
    sd = var.sqrt()
    z = (mu - train_y.max()) / sd
    normal = torch.distributions.Normal(0.0, 1.0)
    ei = sd * (z * normal.cdf(z) + normal.log_prob(z).exp())
    return cands[ei.clamp_min(1e-38).log().argmax()].to(train_x.dtype)


def _build_optuna_adapters(optuna) -> Dict[str, Any]:
    from optuna.distributions import BaseDistribution, CategoricalDistribution, FloatDistribution, IntDistribution
    from optuna.samplers import BaseSampler, CmaEsSampler, RandomSampler
    from optuna.study import StudyDirection
    from optuna.trial import TrialState

    def _untransform_numerical_param_torch(trans_param, distribution, transform_log: bool) -> Tensor:
        """Optimiser coordinate -> parameter value inside the distribution's support (log undone, grid
        snapped, open upper end kept strictly below ``high``)."""
        d = distribution
        just_below_high = lambda: nextafter(d.high, d.high - 1)  # noqa: E731
        if isinstance(d, FloatDistribution):
            if d.log:
                value = trans_param.exp() if transform_log else trans_param
                return value if d.single() else value.clamp(max=just_below_high())
            if d.step is not None:
                return (((trans_param - d.low) / d.step).round() * d.step + d.low).clamp(min=d.low, max=d.high)
            return trans_param if d.single() else trans_param.clamp(max=just_below_high())
        if not isinstance(d, IntDistribution):
            raise ValueError(f"Unexpected distribution type: {type(d)}")
        if d.log:
            value = trans_param.exp().round() if transform_log else trans_param
        else:
            value = ((trans_param - d.low) / d.step).round() * d.step + d.low
        return value.clamp(min=d.low, max=d.high).to(torch.int64)

    class SearchSpaceTransform:
        """Numeric search space <-> box in optimiser coordinates.  Log-distributed parameters are searched in
        log space; integer / stepped parameters get half a step of slack on either side so that rounding
        gives every value equal mass.  ``transform_0_1`` rescales the box to the unit cube."""

        def __init__(self, search_space, transform_log: bool = True, transform_step: bool = True, transform_0_1: bool = False):
            self._search_space = dict(search_space)
            self._transform_log, self._transform_0_1 = transform_log, transform_0_1
            rows = []
            for name, d in self._search_space.items():
                if isinstance(d, CategoricalDistribution):
                    raise ValueError("We don't support categorical parameters.")
                half = 0.5 * d.step if (transform_step and getattr(d, "step", None) is not None and not d.log) else 0.0
                if isinstance(d, IntDistribution) and d.log and transform_step:
                    lo, hi = d.low - 0.5, d.high + 0.5
                else:
                    lo, hi = d.low - half, d.high + half
                if d.log and transform_log:
                    lo, hi = math.log(lo), math.log(hi)
                rows.append((lo, hi))
            self._raw_bounds = np.asarray(rows, dtype=np.float64).reshape(-1, 2)
            self.column_to_encoded_columns = [np.array([i]) for i in range(len(rows))]

        @property
        def bounds(self) -> np.ndarray:
            if self._transform_0_1:
                return np.tile(np.array([[0.0, 1.0]]), (len(self._raw_bounds), 1))
            return self._raw_bounds

        def transform(self, params: Dict[str, Any]) -> np.ndarray:
            out = np.empty(len(self._search_space), dtype=np.float64)
            for i, (name, d) in enumerate(self._search_space.items()):
                v = float(params[name])
                out[i] = math.log(v) if (d.log and self._transform_log) else v
            if self._transform_0_1:
                lo, hi = self._raw_bounds[:, 0], self._raw_bounds[:, 1]
                out = (out - lo) / np.where(hi > lo, hi - lo, 1.0)
            return out

        @torch.no_grad()
        def untransform(self, trans_params) -> Dict[str, Any]:
            t = torch.as_tensor(np.asarray(trans_params) if not isinstance(trans_params, Tensor) else trans_params)
            assert t.shape == (self._raw_bounds.shape[0],)
            if self._transform_0_1:
                lo = torch.as_tensor(self._raw_bounds[:, 0]).to(t)
                hi = torch.as_tensor(self._raw_bounds[:, 1]).to(t)
                t = lo + t * (hi - lo)
            return {
                name: _untransform_numerical_param_torch(t[i], d, self._transform_log).item()
                for i, (name, d) in enumerate(self._search_space.items())
            }

    def untransform(transform: SearchSpaceTransform, trans_params) -> Dict[str, Any]:
        return transform.untransform(trans_params)

    class SimpleAPIBaseSampler(BaseSampler):
        """Sampler over a search space fixed at construction; ``suggest_all(trial)`` asks for every parameter."""

        def __init__(self, search_space: Optional[Dict[str, BaseDistribution]] = None):
            self.search_space = {} if search_space is None else dict(search_space)

        def suggest_all(self, trial):
            return {name: trial._suggest(name, dist) for name, dist in self.search_space.items()}

    class BoTorchSampler(SimpleAPIBaseSampler):
        """GP-based sampler: random start-up trials, then ``candidates_func(train_x, train_obj, train_con,
        bounds, pending_x)`` proposes the next point in the unit cube (objectives are passed as
        to-be-maximised).  Without a ``candidates_func`` the log-EI-over-Sobol generator of this module is
        used (single objective, no constraints).  Parity: ``heavyball/helpers.py:177-361``."""

        def __init__(self, search_space=None, *, candidates_func: Optional[Callable] = None, constraints_func=None,
                     n_startup_trials: int = 10, independent_sampler=None, seed: Optional[int] = None,
                     device: Optional[str] = None, **kwargs):  # fmt: skip
            _reject_unknown(kwargs, "BoTorchSampler")
            super().__init__(search_space)
            self._candidates_func, self._constraints_func = candidates_func, constraints_func
            self._n_startup_trials, self._seed = n_startup_trials, seed
            self._independent_sampler = independent_sampler or RandomSampler(seed=seed)
            self._device = torch.device(device or "cpu")
            self._cache: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}

        def infer_relative_search_space(self, study, trial):
            return self.search_space

        def _observations(self, study, trans):
            xs, ys = [], []
            signs = np.array([-1.0 if d == StudyDirection.MINIMIZE else 1.0 for d in study.directions])
            for t in study.get_trials(deepcopy=False, states=(TrialState.COMPLETE,)):
                tid = t._trial_id
                if tid not in self._cache:
                    if any(name not in t.params for name in self.search_space):
                        continue
                    self._cache[tid] = (trans.transform(t.params), np.asarray(t.values, dtype=np.float64))
                x, v = self._cache[tid]
                xs.append(x)
                ys.append(signs * v)
            return xs, ys

        def sample_relative(self, study, trial, search_space):
            if not search_space:
                return {}
            trans = SearchSpaceTransform(search_space, transform_0_1=True)
            xs, ys = self._observations(study, trans)
            if len(xs) < self._n_startup_trials:
                return {}
            train_x = torch.as_tensor(np.stack(xs), dtype=torch.float64, device=self._device)
            train_y = torch.as_tensor(np.stack(ys), dtype=torch.float64, device=self._device)
            bounds = bound_to_torch(trans.bounds.astype(np.float64).tobytes(), trans.bounds.shape, str(self._device))
            with manual_seed(self._seed):
                if self._candidates_func is not None:
                    cand = self._candidates_func(train_x, train_y, None, bounds, None)
                else:
                    if train_y.shape[1] != 1 or self._constraints_func is not None:
                        raise ValueError("the built-in candidate generator handles one unconstrained objective; pass candidates_func")
                    cand = _logei_over_sobol(train_x, train_y[:, 0], bounds, seed=self._seed)
                if self._seed is not None:
                    self._seed += 1
            cand = cand.reshape(-1, train_x.shape[1])[0] if cand.dim() > 1 else cand
            return trans.untransform(cand.detach().cpu())

        def sample_independent(self, study, trial, param_name, param_distribution):
            return self._independent_sampler.sample_independent(study, trial, param_name, param_distribution)

        def reseed_rng(self) -> None:
            self._independent_sampler.reseed_rng()
            if self._seed is not None:
                self._seed = int(np.random.RandomState().randint(_MAXINT32))

        def before_trial(self, study, trial) -> None:
            self._independent_sampler.before_trial(study, trial)

        def after_trial(self, study, trial, state, values) -> None:
            if self._constraints_func is not None:
                study._storage.set_trial_system_attr(trial._trial_id, "constraints", tuple(self._constraints_func(trial)))
            self._independent_sampler.after_trial(study, trial, state, values)

    def _convert_to_hebo_design_space(search_space) -> DesignSpace:
        if not search_space:
            raise ValueError("Empty search space.")
        configs = []
        for name, d in search_space.items():
            if not isinstance(d, (FloatDistribution, IntDistribution)):
                raise NotImplementedError(f"Unsupported distribution: {d}")
            if not d.log and d.step is not None:  # grid: searched as the integer index of the grid point
                n = int(round((d.high - d.low) / d.step + 1))
                configs.append({"name": name, "type": "int", "lb": 0, "ub": n - 1})
            elif d.log:
                configs.append({"name": name, "type": "pow_int" if isinstance(d, IntDistribution) else "pow", "lb": d.low, "ub": d.high})
            else:
                configs.append({"name": name, "type": "num", "lb": d.low, "ub": d.high})
        return DesignSpace().parse(configs)

    def _is_grid(d) -> bool:
        return isinstance(d, (IntDistribution, FloatDistribution)) and not d.log and d.step is not None

    class HEBOSampler(SimpleAPIBaseSampler):
        """Feeds finished trials to a ``HEBO`` instance and samples its next suggestion.  Parity:
        ``heavyball/helpers.py:627-722``."""

        def __init__(self, search_space, *, seed: Optional[int] = None, independent_sampler=None, **kwargs):
            _reject_unknown(kwargs, "HEBOSampler")
            super().__init__(search_space)
            self._seed = seed
            self._hebo = HEBO(_convert_to_hebo_design_space(self.search_space), scramble_seed=seed)
            self._independent_sampler = independent_sampler or RandomSampler(seed=seed)
            self._seen: set = set()

        def _observe_trial(self, study, trial, values) -> None:
            import pandas as pd

            sign = 1.0 if study.direction == StudyDirection.MINIMIZE else -1.0
            value = np.array([[sign * values[0]]], dtype=float)
            row = pd.DataFrame([trial.params])
            for name, d in trial.distributions.items():
                if _is_grid(d):
                    row[name] = (row[name] - d.low) / d.step
            self._hebo.observe(row, value)

        def _ingest_existing(self, study) -> None:
            for t in study.get_trials(deepcopy=False, states=(TrialState.COMPLETE,)):
                if t._trial_id not in self._seen and t.values is not None:
                    self._observe_trial(study, t, t.values)
                    self._seen.add(t._trial_id)

        def infer_relative_search_space(self, study, trial):
            return self.search_space

        def sample_relative(self, study, trial, search_space):
            self._ingest_existing(study)
            out = {}
            for name, col in self._hebo.suggest().items():
                if name not in search_space:
                    continue
                d, v = search_space[name], col.iloc[0]
                out[name] = d.low + v * d.step if _is_grid(d) else v
            return out

        def sample_independent(self, study, trial, param_name, param_distribution):
            return self._independent_sampler.sample_independent(study, trial, param_name, param_distribution)

        def after_trial(self, study, trial, state, values) -> None:
            if values is not None and trial._trial_id not in self._seen:
                self._observe_trial(study, trial, values)
                self._seen.add(trial._trial_id)

    class ImplicitNaturalGradientSampler(BaseSampler):
        """Drives ``FastINGO`` from a study: every sampled trial is tagged with the optimiser's generation
        counter; finished trials of the current generation are fed back before the next draw.  Categorical
        and single-valued parameters are left to the independent sampler.  Parity:
        ``heavyball/helpers.py:829-975``."""

        def __init__(self, search_space, x0: Optional[Dict[str, Any]] = None, sigma0: Optional[float] = None,
                     n_startup_trials: int = 1, independent_sampler=None, seed: Optional[int] = None,
                     population_size: Optional[int] = None, **kwargs):  # fmt: skip
            _reject_unknown(kwargs, "ImplicitNaturalGradientSampler")
            self.search_space = dict(search_space)
            self._x0, self._sigma0 = x0, sigma0
            self._independent_sampler = independent_sampler or RandomSampler(seed=seed)
            self._n_startup_trials, self._seed, self._population_size = n_startup_trials, seed, population_size
            self._optimizer: Optional[FastINGO] = None
            self._param_queue: List[Dict[str, Any]] = []

        def reseed_rng(self) -> None:
            self._independent_sampler.reseed_rng()
            if self._optimizer is not None:
                self._optimizer.generator.seed()

        def infer_relative_search_space(self, study, trial):
            return {
                name: d
                for name, d in self.search_space.items()
                if not d.single() and isinstance(d, (FloatDistribution, IntDistribution))
            }

        def _init_optimizer(self, trans, population_size=None) -> FastINGO:
            lower, upper = trans.bounds[:, 0], trans.bounds[:, 1]
            mean = lower + (upper - lower) / 2 if self._x0 is None else trans.transform(self._x0)
            sigma0 = float(np.min((upper - lower) / 6)) if self._sigma0 is None else self._sigma0
            return FastINGO(mean=mean, inv_sigma=np.full(len(lower), 1.0 / sigma0), lower=lower, upper=upper,
                            seed=self._seed, population_size=population_size)  # fmt: skip

        def sample_relative(self, study, trial, search_space):
            self._raise_error_if_multi_objective(study)
            if len(search_space) <= 1:
                return {}
            done = study.get_trials(deepcopy=False, states=[TrialState.COMPLETE])
            if len(done) < self._n_startup_trials:
                return {}
            trans = SearchSpaceTransform(search_space)
            if self._optimizer is None or self._optimizer.dim != len(trans.bounds):
                self._optimizer = self._init_optimizer(trans, self._population_size)
                self._param_queue.clear()
            generation = self._optimizer.generation
            for t in done:
                if t.system_attrs.get("ingo", -1) == generation:
                    self._optimizer.tell(-t.value if study.direction == StudyDirection.MAXIMIZE else t.value)
            study._storage.set_trial_system_attr(trial._trial_id, "ingo", self._optimizer.generation)
            return trans.untransform(self._optimizer.ask())

        def sample_independent(self, study, trial, param_name, param_distribution):
            self._raise_error_if_multi_objective(study)
            return self._independent_sampler.sample_independent(study, trial, param_name, param_distribution)

        def after_trial(self, study, trial, state, values) -> None:
            self._independent_sampler.after_trial(study, trial, state, values)

    class ThreadLocalSampler(threading.local):
        sampler = None

    def init_cmaes(study, seed, trials, search_space):
        ordered = sorted(copy.deepcopy(trials), key=lambda t: t.datetime_complete)
        return CmaEsSampler(seed=seed, source_trials=ordered, lr_adapt=True)

    def init_hebo(study, seed, trials, search_space):
        sampler = HEBOSampler(search_space=search_space, seed=seed)
        for t in trials:
            sampler.after_trial(study, t, TrialState.COMPLETE, t.values)
        return sampler

    def init_botorch(study, seed, trials, search_space):
        return BoTorchSampler(search_space=search_space, seed=seed, device=_use_cuda())

    def init_nsgaii(study, seed, trials, search_space):
        """NSGA-II seeded with the finished trials when ``optunahub`` provides that sampler, Optuna's own
        NSGA-II otherwise."""
        try:
            import optunahub

            return optunahub.load_module("samplers/nsgaii_with_initial_trials").NSGAIIwITSampler(seed=seed)
        except Exception:  # package or registry not reachable
            return optuna.samplers.NSGAIISampler(seed=seed)

    def init_random(study, seed, trials, search_space):
        return RandomSampler(seed=seed)

    def init_ingo(study, seed, trials, search_space):
        return ImplicitNaturalGradientSampler(search_space=search_space, seed=seed)

    class AutoSampler(BaseSampler):
        """Switches samplers by the number of completed trials: ``samplers`` is ``[(threshold, factory)]``
        with ``factory(study, seed, completed_trials, search_space)``; default HEBO from the start and
        NSGA-II from 100 trials on.  One sampler instance per thread.  Parity: ``heavyball/helpers.py:1016-1111``."""

        def __init__(self, samplers: Optional[Iterable[Tuple[int, Callable]]] = None, search_space=None, *,
                     seed: Optional[int] = None, **kwargs):  # fmt: skip
            _reject_unknown(kwargs, "AutoSampler")
            if samplers is None:
                if search_space is None:
                    raise ValueError("AutoSampler requires a search_space when using the default sampler schedule.")
                samplers = ((0, init_hebo), (100, init_nsgaii))
            schedule = sorted(samplers, key=lambda item: item[0])
            self.sampler_indices = np.array([item[0] for item in schedule], dtype=np.int32)
            self.samplers = [item[1] for item in schedule]
            self.search_space = {} if search_space is None else dict(search_space)
            self._rng = np.random.RandomState(seed)
            self._random_sampler = RandomSampler(seed=seed)
            self._thread_local_sampler = ThreadLocalSampler()
            self._completed_trials, self._current_index = 0, -1

        def __getstate__(self):
            state = self.__dict__.copy()
            del state["_thread_local_sampler"]
            return state

        def __setstate__(self, state) -> None:
            self.__dict__.update(state)
            self._thread_local_sampler = ThreadLocalSampler()

        @property
        def _sampler(self):
            if self._thread_local_sampler.sampler is None:
                self._thread_local_sampler.sampler = RandomSampler(seed=int(self._rng.randint(_MAXINT32)))
            return self._thread_local_sampler.sampler

        @_sampler.setter
        def _sampler(self, sampler) -> None:
            self._thread_local_sampler.sampler = sampler

        def reseed_rng(self) -> None:
            self._rng.seed()
            self._sampler.reseed_rng()

        def _update_sampler(self, study) -> None:
            if len(study.directions) > 1:
                raise ValueError("Multi-objective optimization is not supported.")
            if isinstance(self._sampler, CmaEsSampler):
                return
            done = study._get_trials(deepcopy=False, states=(TrialState.COMPLETE,), use_cache=True)
            self._completed_trials = max(self._completed_trials, len(done))
            index = int((self._completed_trials >= self.sampler_indices).sum()) - 1
            if index < 0 or index == self._current_index:
                return
            self._current_index = index
            self._sampler = self.samplers[index](study, int(self._rng.randint(_MAXINT32)), done, self.search_space)

        def infer_relative_search_space(self, study, trial):
            return self._sampler.infer_relative_search_space(study, trial)

        def sample_relative(self, study, trial, search_space):
            return self._sampler.sample_relative(study, trial, search_space or self.search_space)

        def sample_independent(self, study, trial, param_name, param_distribution):
            return self._random_sampler.sample_independent(study, trial, param_name, param_distribution)

        def before_trial(self, study, trial) -> None:
            # the switch happens here so that before_trial, sample_relative and after_trial of one trial all
            # see the same sampler
            if len(study._get_trials(deepcopy=False, states=(TrialState.COMPLETE,), use_cache=True)) != 0:
                self._update_sampler(study)
            study._storage.set_trial_system_attr(trial._trial_id, _SAMPLER_KEY, type(self._sampler).__name__)
            self._sampler.before_trial(study, trial)

        def after_trial(self, study, trial, state, values) -> None:
            if state not in (TrialState.COMPLETE, TrialState.FAIL, TrialState.PRUNED):
                raise ValueError(f"Unsupported trial state: {state}.")
            self._sampler.after_trial(study, trial, state, values)

    scope = locals()
    exported = {name: scope[name] for name in _ADAPTER_NAMES}
    for name, obj in exported.items():  # picklable: found again as module attributes
        obj.__qualname__, obj.__module__ = name, __name__
    return exported


try:
    import optuna as _optuna
except ImportError:
    _optuna = None

    def __getattr__(name):
        if name in _ADAPTER_NAMES:
            raise ImportError(f"heavyball_b200.helpers.{name} needs the 'optuna' package, which is not installed")
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
else:
    globals().update(_build_optuna_adapters(_optuna))
