"""Optimizer runtime shared by every class.

Three small collaborators do the work, ``StatefulOptimizer`` wires them to ``torch.optim.Optimizer``:

* :class:`ViewIndex` - which tensors a parameter is stepped as.  ``merge_dims`` / ``split`` can turn one parameter
  into several views; optimizer state is addressed per view, ``optimizer.state[param][view_index]``, and a view is
  found again from its storage address.
* :class:`Scratch` - values that live for one step only and travel beside a tensor through the chain (the probe vector
  and Hessian-vector product of a curvature step, a memory format to restore).
* :class:`CurvatureProbe` - Hessian-vector products for preconditioners fitted on curvature: exact (double backward)
  or by finite differences, with a one-way fallback from the first to the second when autograd cannot differentiate
  the model twice.

What the checkpoint format dictates is kept as is: the ``"heavyball"`` block of ``state_dict()`` with its key names
(``heavyball/utils.py:1527-1549`` in the reference), the instance attributes that constructors accept as keyword
arguments (``heavyball/utils.py:1497-1512``), and the public method names optimizers and user code call
(``state_``, ``split_p_and_g_in_group``, ``ema_update`` ..., ``heavyball/utils.py:1479-1834``).  The backward-hook
helpers mirror ``heavyball/utils.py:3807-3838``, the shape capture ``heavyball/utils.py:500-504``.
"""

from __future__ import annotations

import contextlib
import functools
import inspect
import re
from typing import Callable, Dict, Iterator, List, Optional, Tuple, Union

import torch
from torch import Tensor

from . import pickle_compat
from .core import beta_debias, promote, stochastic_add_, stochastic_add_divide_, warn_once
from .psgd import psgd_should_update
from .soap import merge_group

use_default = object()


class ExactHVPFailed(ValueError):
    """The exact Hessian-vector product could not be formed (no second derivative for some parameter, or autograd
    refused the double backward)."""


def _tensor_key(x: Tensor):
    return x.data_ptr(), x.numel(), x.dtype, x.device


def capture_param_shapes(params):
    """Record parameter shapes before a sharding wrapper flattens them; pass the result as
    ``orig_shapes=`` to any optimizer."""
    source = params.parameters() if hasattr(params, "parameters") else params
    return {id(p): tuple(p.shape) for p in source}


# ---------------------------------------------------------------------------------------- per-step scratch


class Scratch:
    """Per-step side values keyed by tensor identity, kept under ``group["_tmp"]`` (underscore keys never reach a
    checkpoint).  An entry remembers its tensor so that clean-up can act on it."""

    KEY = "_tmp"

    @classmethod
    def put(cls, group: dict, tensor: Tensor, **values):
        if not values:
            return
        table = group.setdefault(cls.KEY, {})
        entry = table.get(id(tensor))
        if entry is None:
            entry = table[id(tensor)] = {"tensor": tensor}
        entry.update(values)

    @classmethod
    def peek(cls, group: dict, tensor: Tensor) -> Optional[dict]:
        table = group.get(cls.KEY)
        return table.get(id(tensor)) if table else None

    @classmethod
    def take(cls, group: dict, tensor: Tensor, *names):
        entry = cls.peek(group, tensor)
        values = [None] * len(names) if entry is None else [entry.pop(n, None) for n in names]
        if entry is not None and set(entry) == {"tensor"}:
            del group[cls.KEY][id(tensor)]
        return values[0] if len(names) == 1 else tuple(values)

    @classmethod
    def drain(cls, group: dict) -> List[dict]:
        table = group.pop(cls.KEY, None)
        return list(table.values()) if table else []


# function-style access used throughout the transform library
def set_temporary(group: dict, tensor: Tensor, **kwargs):
    Scratch.put(group, tensor, **kwargs)


def get_temporary(group: dict, tensor: Tensor):
    return Scratch.peek(group, tensor)


def take_temporary(group: dict, tensor: Tensor, *keys):
    return Scratch.take(group, tensor, *keys)


# ---------------------------------------------------------------------------------------- views


class ViewIndex:
    """Bookkeeping of the tensors each parameter is stepped as.

    ``forward[param]`` is the list of views of that parameter (one entry unless dimension merging / splitting cuts it
    up); ``backward[address key]`` names ``(param, view_index)`` for a view.  Both dictionaries are also what
    ``optimizer.mapping`` / ``optimizer.mapping_inverse`` expose."""

    def __init__(self):
        self.forward: Dict[Tensor, List[Tensor]] = {}
        self.backward: Dict[tuple, Tuple[Tensor, int]] = {}
        self._plain: Dict[int, int] = {}  # id(param) -> storage address it was registered with as its own only view

    def register(self, param: Tensor, views) -> None:
        self._plain.pop(id(param), None)
        self.forward[param] = views
        for index, view in enumerate(views):
            self.backward[_tensor_key(view)] = (param, index)

    def register_plain(self, param: Tensor) -> None:
        """``register(param, (param,))`` for the per-step path of unmerged groups: nothing to do while the parameter
        still lives at the address it was registered with (``forward`` keeps the parameter alive, so its ``id`` cannot
        have been handed to another tensor)."""
        address = param.data_ptr()
        if self._plain.get(id(param)) == address:
            return
        self.register(param, (param,))
        self._plain[id(param)] = address

    def is_plain(self, tensor: Tensor) -> bool:
        views = self.forward.get(tensor)
        return views is not None and len(views) == 1 and views[0] is tensor

    def ensure(self, groups) -> None:
        for group in groups:
            for param in group["params"]:
                if param not in self.forward:
                    self.register(param, merge_group(group, param))

    def locate(self, tensor: Tensor) -> Optional[Tuple[Tensor, int]]:
        return self.backward.get(_tensor_key(tensor))


# ---------------------------------------------------------------------------------------- Hessian-vector products


@contextlib.contextmanager
def patch_backward():
    """While active, every ``Tensor.backward`` / ``torch.autograd.backward`` call builds a differentiable graph
    (``create_graph=True``), so the gradients a user closure produces can be differentiated once more."""
    originals = {}

    def forcing(original):
        signature = inspect.signature(original)

        @functools.wraps(original)
        def call(*args, **kwargs):
            bound = signature.bind(*args, **kwargs)
            bound.arguments["create_graph"] = True
            return original(*bound.args, **bound.kwargs)

        return call

    for owner in (torch.Tensor, torch.autograd):
        originals[owner] = owner.backward
        owner.backward = forcing(owner.backward)
    try:
        yield
    finally:
        for owner, original in originals.items():
            owner.backward = original


class CurvatureProbe:
    """Produces, for every parameter with a gradient, a random probe ``v`` and the product ``H v`` and leaves them in
    the step scratch (``vector`` / ``hessian_vector``) next to the gradient, for preconditioners that fit on
    ``(v, H v)`` pairs.  Two ways: one extra differentiation of the gradients (exact), or a second closure evaluation
    at ``p + sqrt(eps) v`` (finite differences)."""

    # autograd's wording when a kernel has no second derivative / when a compiled region cannot be differentiated twice
    NO_DOUBLE_BACKWARD = re.compile(r"the derivative for .* is not implemented\. Double backwards .* To run double backwards")
    COMPILED_REGION = re.compile(r"compile.*does not currently support double backward")
    HINT = (
        "You can accelerate startup by globally enabling finite_differences first "
        "(via opt.finite_differences=True or by subclassing it)\nOriginal Error: "
    )

    def __init__(self, optimizer):
        self.opt = optimizer

    def _raw_pairs(self) -> Iterator[Tuple[dict, Tensor, Tensor]]:
        for group in self.opt.param_groups:
            for p, g in self.opt.split_p_and_g_in_group(group, skip_none=True, raw=True):
                yield group, p, g

    def finite_differences(self, closure):
        with torch.enable_grad():
            loss = closure()
        h = torch.finfo(torch.float32).eps ** 0.5
        base = []
        for group, p, g in self._raw_pairs():
            v = torch.randn_like(p)
            base.append(g)
            Scratch.put(group, p, vector=v, orig=p.data.clone())
            stochastic_add_(p.data, v, h)
        with torch.enable_grad():
            closure()
        for (group, p, shifted), g0 in zip(list(self._raw_pairs()), base):
            # (g(p + h v) - g(p)) / h, formed in place; the parameter comes back from its saved copy, not by subtraction
            stochastic_add_divide_(shifted, g0, -1, h)
            Scratch.put(group, p, grad=g0, hessian_vector=shifted)
            p.data.copy_(Scratch.take(group, p, "orig"))
        return loss

    def exact(self, closure):
        with torch.enable_grad(), patch_backward():
            loss = closure()
        found = list(self._raw_pairs())
        if not found:
            raise ValueError("No parameter has gradients")
        groups, params, grads = zip(*found)
        probes = [torch.randn_like(p) for p in params]
        try:
            with torch.enable_grad():
                products = torch.autograd.grad(grads, params, probes, create_graph=False, retain_graph=False, allow_unused=True)
        except RuntimeError as err:
            raise ExactHVPFailed(str(err.args))
        flat = []
        for group, p, g, v, hv in zip(groups, params, grads, probes, products):
            Scratch.put(group, p, grad=g.detach(), vector=v.detach(), hessian_vector=None if hv is None else hv.detach())
            if hv is None:
                flat.append(list(p.shape))
        if flat:
            raise ExactHVPFailed(f"Parameters with the following shapes have no 2nd order derivative: {flat}")
        return loss

    def _explains(self, err, pattern) -> bool:
        return any(isinstance(a, str) and pattern.match(a) for a in err.args)

    def run(self, closure):
        """Exact product unless finite differences are configured or were fallen back to; a failure of the exact route
        that is a known autograd limitation switches the optimizer to finite differences for good (with one warning)."""
        opt = self.opt
        if opt.finite_differences or opt._fallback_enabled:
            return self.finite_differences(closure)
        try:
            return self.exact(closure)
        except NotImplementedError as err:
            if not (opt.fallback_to_finite_differences and self._explains(err, self.NO_DOUBLE_BACKWARD)):
                raise
            warn_once(
                "CUDNN doesn't support double-backward for some models (including RNNs). "
                f"Falling back to finite_differences.\n{self.HINT}{err}"
            )
        except ExactHVPFailed as err:
            if not opt.fallback_to_finite_differences:
                raise
            warn_once(f"Exact HVP calculation failed.\n{self.HINT}{err}")
        except RuntimeError as err:
            if not (opt.fallback_to_finite_differences and self._explains(err, self.COMPILED_REGION)):
                raise
            warn_once(
                "torch.compile does not support double-backward. Disabling it may be beneficial, depending on "
                f"the model.\n{self.HINT}{err}"
            )
        opt._fallback_enabled = True
        return self.finite_differences(closure)


# ---------------------------------------------------------------------------------------- the optimizer base class


def _encode_schedule(value):
    return pickle_compat.dumps(value)


def _decode_schedule(blob):
    return pickle_compat.loads(blob)


class StatefulOptimizer(torch.optim.Optimizer):
    """Base of every optimizer here: per-view state, gradient hand-off to the chain, closures and curvature probes,
    a parameter EMA, and the metadata block of the checkpoint.

    ``finite_differences`` trades memory for compute when Hessian-vector products are needed (the alternative is an
    exact double-backward product); both have unsupported corner cases."""

    ema_decay: float = 0.001
    compile_step: bool = False
    hessian_approx: bool = False
    precond_schedule: Union[Callable, float, None] = None
    finite_differences: bool = False
    fallback_to_finite_differences: bool = True
    _fallback_enabled: bool = False
    hvp_interval: int = 1
    consume_grad: bool = True

    # constructor keyword arguments that configure the instance instead of the param groups
    _INSTANCE_ATTRS = (
        "compile_step",
        "finite_differences",
        "fallback_to_finite_differences",
        "hvp_interval",
        "hessian_approx",
        "consume_grad",
    )
    # checkpoint block: key -> (attribute, encoder, decoder); the key set and spelling are the interchange format
    _CHECKPOINT_FIELDS = {
        "inner_group": ("inner_group", None, None),
        "use_ema": ("use_ema", None, None),
        "ema_decay": ("ema_decay", None, None),
        "compile_step": ("compile_step", None, None),
        "hessian_approx": ("hessian_approx", None, None),
        "precond_schedule": ("precond_schedule", _encode_schedule, _decode_schedule),
        "fallback_to_finite_differences": ("fallback_to_finite_differences", None, None),
        "_fallback_enabled": ("_fallback_enabled", None, None),
        "hvp_interval": ("hvp_interval", None, None),
    }
    _REMOVED_STATS = frozenset({"stochastic_schedule", "precond_rng"})  # written by older releases, ignored on load

    def __init__(self, params, defaults, use_ema: bool = False):
        for name in self._INSTANCE_ATTRS:
            value = defaults.pop(name, use_default)
            if value is not use_default:
                setattr(self, name, value)
        if self.hessian_approx and self.compile_step:
            raise ValueError("Hessian approximation can't be used with compile_step.")
        defaults.setdefault("multi_tensor", True)
        self.views = ViewIndex()
        self.probe = CurvatureProbe(self)
        super().__init__(params, defaults)
        self.use_ema = use_ema
        self.inner_group = {}
        self._is_preconditioning = None
        self.register_state_dict_post_hook(StatefulOptimizer._store_stats)
        self.register_load_state_dict_pre_hook(StatefulOptimizer._load_stats)

    # ------------------------------------------------------------------ checkpoint metadata
    def _store_stats(self, state_dict):
        block = {}
        for key, (attr, encode, _) in self._CHECKPOINT_FIELDS.items():
            value = getattr(self, attr)
            block[key] = value if encode is None else encode(value)
        state_dict["heavyball"] = block

    def _load_stats(self, state_dict):
        for key, value in state_dict.get("heavyball", {}).items():
            if key in self._REMOVED_STATS:
                continue
            attr, _, decode = self._CHECKPOINT_FIELDS.get(key, (key, None, None))
            if decode is not None:
                try:
                    value = decode(value)
                except Exception as err:  # noqa: BLE001 - a schedule that may not be loaded must not lose the checkpoint
                    warn_once(f"checkpoint's {key} was not loaded, keeping the optimizer's own: {err}")
                    continue
            setattr(self, attr, value)

    # ------------------------------------------------------------------ state addressing
    @property
    def mapping(self):
        return self.views.forward

    @property
    def mapping_inverse(self):
        return self.views.backward

    def get_groups(self, group):
        return [group]

    def _register_views(self, p, views):
        self.views.register(p, views)

    def _init_mapping(self, group: Optional[dict] = None):
        self.views.ensure(self.param_groups if group is None else [group])

    def state_(self, arg: Tensor, fail: bool = True):
        """State dictionary of a view (found by its storage address)."""
        if self.views.is_plain(arg):  # a parameter that is its own only view: no address arithmetic needed
            return self.state.setdefault(arg, {}).setdefault(0, {})
        where = self.views.locate(arg)
        if where is None:
            self.views.ensure(self.param_groups)
            where = self.views.locate(arg)
        if where is None:
            if fail:
                raise KeyError("Tensor has no tracked state.")
            return {}
        param, index = where
        return self.state.setdefault(param, {}).setdefault(index, {})

    def state_size(self) -> int:
        """Bytes held by optimizer state, every tensor counted once."""
        counted, stack, total = set(), [self.state], 0
        while stack:
            node = stack.pop()
            if isinstance(node, Tensor):
                if id(node) not in counted:
                    counted.add(id(node))
                    total += node.numel() * node.element_size()
            elif isinstance(node, dict):
                stack.extend(node.values())
            elif isinstance(node, (list, tuple, set)):
                stack.extend(node)
        return total

    # ------------------------------------------------------------------ gradient hand-off
    _CHANNELS_LAST = (torch.channels_last, torch.channels_last_3d)

    def _take_grad(self, p):
        grad = getattr(p, "grad", None)
        if grad is not None and self.consume_grad:
            p.grad = None  # the chain owns it from here; it is freed as soon as the step is through with it
        return grad

    def _make_dense(self, group, p):
        """Dimension merging reshapes the parameter, which needs a row-major layout: channels-last parameters are made
        contiguous for the step and get their format back in the clean-up."""
        if not group.get("merge_dims", False) or p.data.is_contiguous():
            return
        for fmt in self._CHANNELS_LAST:
            if p.data.is_contiguous(memory_format=fmt):
                Scratch.put(group, p, restore_memory_format=fmt)
                break
        p.data = p.data.contiguous()

    def split_p_and_g_in_group(self, group: dict, skip_none: bool = True, should_promote: bool = True, raw: bool = False):
        """Yields ``(parameter view, gradient view)`` pairs of a group.  ``raw`` yields whole parameters with their
        gradients untouched (no views, no promotion); otherwise a curvature step's stored gradient takes precedence
        over ``p.grad`` and its probe / product are re-attached to the views they belong to."""
        plain = not raw and not group.get("merge_dims", False)
        for p in group["params"]:
            if raw:
                grad = self._take_grad(p)
                if grad is not None or not skip_none:
                    yield p, grad
                continue
            if plain and not group.get(Scratch.KEY):
                # the common case, kept short because it runs for every parameter of every step: one view per
                # parameter (the parameter itself) and nothing stored for the group by a curvature step
                grad = self._take_grad(p)
                if grad is None and skip_none:
                    continue
                self.views.register_plain(p)
                if grad is not None:
                    grad = (promote(grad) if should_promote else grad).detach()
                yield p, grad
                continue
            stored = Scratch.take(group, p, "grad", "vector", "hessian_vector")
            live = self._take_grad(p)
            grad = stored[0] if stored[0] is not None else live
            if grad is None and skip_none:
                continue
            self._make_dense(group, p)
            views = merge_group(group, p)
            self.views.register(p, views)
            columns = [merge_group(group, t) if t is not None else [None] * len(views) for t in (grad, *stored[1:])]
            for view, g, v, hv in zip(views, *columns):
                if should_promote:
                    g, v, hv = (None if t is None else promote(t) for t in (g, v, hv))
                g, v, hv = (None if t is None else t.detach() for t in (g, v, hv))
                if v is not None or hv is not None:
                    Scratch.put(group, view, vector=v, hessian_vector=hv)
                yield view, g

    # ------------------------------------------------------------------ parameter EMA
    def _ema_entries(self):
        for group in self.param_groups:
            for p in group["params"]:
                yield group, p, self.state_(p)

    def ema_update(self):
        """``ema <- lerp(ema, p, w)`` with the debiased weight of the group's EMA step count."""
        with torch.no_grad():
            ticked = set()
            for group, p, st in self._ema_entries():
                if id(group) not in ticked:
                    ticked.add(id(group))
                    group["ema_step"] = group.get("ema_step", -1) + 1
                ema = st.get("param_ema")
                if ema is None:
                    ema = st["param_ema"] = torch.zeros_like(p.data, memory_format=torch.preserve_format)
                ema.lerp_(p.data, beta_debias(1 - self.ema_decay, group["ema_step"] + 1))

    def _exchange_with_ema(self):
        with torch.no_grad():
            for _, p, st in self._ema_entries():
                ema = st.get("param_ema")
                if ema is not None:
                    keep = p.data.clone()
                    p.data.copy_(ema)
                    ema.copy_(keep)

    def copy_emas_to_params(self):
        self._exchange_with_ema()

    def copy_params_to_emas(self):
        self._exchange_with_ema()

    # ------------------------------------------------------------------ closures and curvature steps
    def _finite_differences_hvp(self, closure):
        return self.probe.finite_differences(closure)

    def _double_backward_hvp(self, closure):
        return self.probe.exact(closure)

    def _handle_closure(self, closure):
        """Evaluates the closure.  On preconditioner steps of a ``hessian_approx`` optimizer (every ``hvp_interval``-th
        closure call skips it) the evaluation also produces the probe / Hessian-vector pairs."""
        curvature_step = bool(self.hessian_approx and self._is_preconditioning)
        if closure is None:
            if curvature_step:
                raise ValueError("Hessian approximation requires a closure.")
            return None
        calls = self.inner_group.get("total_hvp_steps", 0)
        self.inner_group["total_hvp_steps"] = calls + 1
        if curvature_step and calls % self.hvp_interval != 0:
            return self.probe.run(closure)
        with torch.enable_grad():
            return closure()

    # ------------------------------------------------------------------ step
    def _cleanup_temporary_tensors(self):
        for group in self.param_groups:
            for entry in Scratch.drain(group):
                fmt = entry.get("restore_memory_format")
                if fmt is None:
                    continue
                t = entry["tensor"]
                self.views.backward.pop(_tensor_key(t), None)
                t.data = t.data.to(memory_format=fmt)
                self.views.backward[_tensor_key(t)] = (t, 0)

    def _step(self, group):
        raise NotImplementedError

    def _decide_preconditioning(self) -> bool:
        if self.precond_schedule is None:
            return False
        return psgd_should_update(self.inner_group, self.precond_schedule)

    def step(self, closure: Optional[Callable] = None):
        self._is_preconditioning = self._decide_preconditioning()
        loss = self._handle_closure(closure)
        if self.use_ema:
            self.ema_update()
        try:
            with torch.no_grad():
                for group in self.param_groups:
                    group.setdefault("param_count", sum(p.numel() for p in group["params"]))
                    group["is_preconditioning"] = self._is_preconditioning
                    self._step(group)
        finally:
            self._cleanup_temporary_tensors()
        return loss


# ---------------------------------------------------------------------------------------- backward hooks


def hook_optimizer_into_model(model, optimizer, *args, **kwargs):
    """One optimizer instance per parameter, stepped from the parameter's post-accumulate-grad hook
    (the update overlaps with the rest of the backward pass and the gradient is freed at once)."""
    owners = {p: optimizer([p], *args, **kwargs) for p in model.parameters()}

    def step_owner(p: Tensor):
        owners[p].step()
        owners[p].zero_grad()

    for p in owners:
        p.register_post_accumulate_grad_hook(step_owner)
    return owners


def fused_hook(parameters, optimizer, *args, **kwargs):
    """A single optimizer stepped from the gradient hooks; its public ``step`` becomes a warning."""
    parameters = list(parameters)
    opt = optimizer(parameters, *args, **kwargs)
    inner_step = opt.step

    def step_all(_p: Tensor):
        inner_step()
        opt.zero_grad()

    for p in parameters:
        p.register_post_accumulate_grad_hook(step_all)
    opt.step = functools.partial(warn_once, msg="You're trying to call `step` on a fused optimizer. This will not do anything.")
    return opt
