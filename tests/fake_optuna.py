"""A stand-in for the small part of Optuna's public API that ``heavyball_b200.helpers`` uses, so that the
sampler adapters can be exercised where Optuna is not installed.  ``install()`` registers it in
``sys.modules`` under Optuna's module names and returns a loader for a private copy of the helpers module
bound to it."""

import enum
import importlib.util
import os
import sys
import types

import numpy as np


class BaseDistribution:
    def single(self):
        return self.low == self.high


class FloatDistribution(BaseDistribution):
    def __init__(self, low, high, log=False, step=None):
        self.low, self.high, self.log, self.step = float(low), float(high), log, step


class IntDistribution(BaseDistribution):
    def __init__(self, low, high, log=False, step=1):
        self.low, self.high, self.log, self.step = int(low), int(high), log, step


class CategoricalDistribution(BaseDistribution):
    def __init__(self, choices):
        self.choices = tuple(choices)

    def single(self):
        return len(self.choices) == 1


class StudyDirection(enum.Enum):
    MINIMIZE = 1
    MAXIMIZE = 2


class TrialState(enum.Enum):
    RUNNING = 0
    COMPLETE = 1
    PRUNED = 2
    FAIL = 3


class BaseSampler:
    def infer_relative_search_space(self, study, trial):
        return {}

    def sample_relative(self, study, trial, search_space):
        return {}

    def before_trial(self, study, trial):
        pass

    def after_trial(self, study, trial, state, values):
        pass

    def reseed_rng(self):
        pass

    def _raise_error_if_multi_objective(self, study):
        if len(study.directions) > 1:
            raise ValueError("multi-objective studies are not supported")


class RandomSampler(BaseSampler):
    def __init__(self, seed=None):
        self._rng = np.random.RandomState(seed)

    def reseed_rng(self):
        self._rng.seed()

    def sample_independent(self, study, trial, name, d):
        if isinstance(d, CategoricalDistribution):
            return d.choices[self._rng.randint(len(d.choices))]
        if d.log:
            v = float(np.exp(self._rng.uniform(np.log(d.low), np.log(d.high))))
        else:
            v = float(self._rng.uniform(d.low, d.high))
        if isinstance(d, IntDistribution):
            return int(min(max(round(v), d.low), d.high))
        if d.step is not None:
            v = d.low + round((v - d.low) / d.step) * d.step
        return v


class CmaEsSampler(RandomSampler):
    def __init__(self, seed=None, source_trials=None, lr_adapt=False):
        super().__init__(seed)
        self.source_trials = source_trials


class NSGAIISampler(RandomSampler):
    pass


class FrozenTrial:
    def __init__(self, trial_id, distributions):
        self._trial_id, self.distributions = trial_id, dict(distributions)
        self.params, self.values, self.system_attrs = {}, None, {}
        self.state, self.datetime_complete = TrialState.RUNNING, trial_id

    @property
    def value(self):
        return None if self.values is None else self.values[0]


class _Storage:
    def __init__(self, study):
        self._study = study

    def set_trial_system_attr(self, trial_id, key, value):
        self._study.trials[trial_id].system_attrs[key] = value


class Study:
    """Sequential ask / evaluate / tell loop over a fixed search space."""

    def __init__(self, sampler, search_space, direction=StudyDirection.MINIMIZE):
        self.sampler, self.search_space = sampler, dict(search_space)
        self.direction, self.directions = direction, [direction]
        self.trials, self._storage = [], _Storage(self)

    def get_trials(self, deepcopy=True, states=None):
        return [t for t in self.trials if states is None or t.state in tuple(states)]

    def _get_trials(self, deepcopy=True, states=None, use_cache=False):
        return self.get_trials(deepcopy, states)

    def run(self, objective, n_trials):
        for _ in range(n_trials):
            trial = FrozenTrial(len(self.trials), self.search_space)
            self.trials.append(trial)
            self.sampler.before_trial(self, trial)
            space = self.sampler.infer_relative_search_space(self, trial)
            trial.params.update(self.sampler.sample_relative(self, trial, space))
            for name, d in self.search_space.items():
                if name not in trial.params:
                    trial.params[name] = self.sampler.sample_independent(self, trial, name, d)
            trial.values = [float(objective(trial.params))]
            trial.state = TrialState.COMPLETE
            self.sampler.after_trial(self, trial, TrialState.COMPLETE, trial.values)
        return min(t.value for t in self.trials) if self.direction == StudyDirection.MINIMIZE else max(t.value for t in self.trials)


def install():
    """Registers the stand-in and returns the helpers module loaded against it (a private copy: the regular
    ``heavyball_b200.helpers`` import is left as it is)."""
    top = types.ModuleType("optuna")
    parts = {
        "distributions": dict(BaseDistribution=BaseDistribution, FloatDistribution=FloatDistribution,
                              IntDistribution=IntDistribution, CategoricalDistribution=CategoricalDistribution),
        "samplers": dict(BaseSampler=BaseSampler, RandomSampler=RandomSampler, CmaEsSampler=CmaEsSampler,
                         NSGAIISampler=NSGAIISampler),
        "study": dict(StudyDirection=StudyDirection, Study=Study),
        "trial": dict(TrialState=TrialState, FrozenTrial=FrozenTrial),
    }  # fmt: skip
    saved = {k: sys.modules.get(k) for k in ["optuna"] + [f"optuna.{p}" for p in parts]}
    sys.modules["optuna"] = top
    for name, members in parts.items():
        mod = types.ModuleType(f"optuna.{name}")
        mod.__dict__.update(members)
        setattr(top, name, mod)
        sys.modules[f"optuna.{name}"] = mod
    try:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "heavyball_b200", "helpers.py")
        spec = importlib.util.spec_from_file_location("heavyball_b200_helpers_with_fake_optuna", path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = module  # stays registered so that its classes pickle
        spec.loader.exec_module(module)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    return module
