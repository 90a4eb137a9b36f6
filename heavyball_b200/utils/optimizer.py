"""Optimizer runtime shared by every class: per-view state addressing, gradient hand-off, closure /
Hessian-vector-product handling, parameter EMA, checkpoint metadata and backward-hook stepping.

Behavioural parity targets: ``heavyball/utils.py:1479-1834`` (``StatefulOptimizer``),
``heavyball/utils.py:1414-1465`` (backward patching, per-step temporaries),
``heavyball/utils.py:3807-3838`` (hook helpers), ``heavyball/utils.py:500-504`` (shape capture).

State is addressed by *view*: ``merge_dims`` / ``split`` can turn one parameter into several tensors,
each owning ``optimizer.state[param][view_index]``.
"""

from __future__ import annotations

import contextlib
import functools
import inspect
import itertools
import re
from typing import Callable, Optional, Union

import torch
from torch import Tensor
from torch.utils._pytree import tree_map

from . import pickle_compat
from .core import beta_debias, detach, promote_detach, stochastic_add_, stochastic_add_divide_, warn_once
from .psgd import psgd_should_update
from .soap import merge_group

use_default = object()

_cudnn_double_backward_pattern = re.compile(
    r"the derivative for .* is not implemented\. Double backwards .* To run double backwards"
)
_torch_compile_double_backward_pattern = re.compile(r"compile.*does not currently support double backward")
_fd_error = (
    "You can accelerate startup by globally enabling finite_differences first "
    "(via opt.finite_differences=True or by subclassing it)\nOriginal Error: "
)


class ExactHVPFailed(ValueError):
    pass


def _tensor_key(x: Tensor):
    return x.data_ptr(), x.numel(), x.dtype, x.device


@contextlib.contextmanager
def patch_backward():
    """Forces ``create_graph=True`` on every ``backward`` issued inside the block so that the
    gradients can be differentiated again for an exact Hessian-vector product."""

    def wrap(owner):
        original = owner.backward
        sig = inspect.signature(original)

        @functools.wraps(original)
        def patched(*args, **kwargs):
            bound = sig.bind(*args)
            bound.apply_defaults()
            call = dict(bound.arguments)
            call.update(kwargs)
            call["create_graph"] = True
            return original(**call)

        owner.backward = patched
        return original

    saved = [(owner, wrap(owner)) for owner in (torch.Tensor, torch.autograd)]
    try:
        yield
    finally:
        for owner, original in saved:
            owner.backward = original


# per-step scratch attached to a param group under "_tmp": {id(tensor): {"tensor": t, ...}}
def set_temporary(group: dict, tensor: Tensor, **kwargs):
    if kwargs:
        group.setdefault("_tmp", {}).setdefault(id(tensor), {"tensor": tensor}).update(kwargs)


def get_temporary(group: dict, tensor: Tensor):
    tmp = group.get("_tmp")
    return None if tmp is None else tmp.get(id(tensor))


def take_temporary(group: dict, tensor: Tensor, *keys):
    slot = get_temporary(group, tensor)
    if slot is None:
        return None if len(keys) == 1 else (None,) * len(keys)
    out = tuple(slot.pop(k, None) for k in keys)
    if len(slot) == 1:
        group["_tmp"].pop(id(tensor), None)
    return out[0] if len(keys) == 1 else out


def capture_param_shapes(params):
    """Record parameter shapes before a sharding wrapper flattens them; pass the result as
    ``orig_shapes=`` to any optimizer."""
    if hasattr(params, "parameters"):
        params = params.parameters()
    return {id(p): tuple(p.shape) for p in params}


class StatefulOptimizer(torch.optim.Optimizer):
    """``finite_differences`` trades memory for compute when Hessian-vector products are needed
    (the alternative is an exact double-backward product); both have unsupported corner cases."""

    ema_decay: float = 0.001
    compile_step: bool = False
    hessian_approx: bool = False
    precond_schedule: Union[Callable, float, None] = None
    finite_differences: bool = False
    fallback_to_finite_differences: bool = True
    _fallback_enabled: bool = False
    hvp_interval: int = 1
    consume_grad: bool = True

    _INSTANCE_ATTRS = (
        "compile_step",
        "finite_differences",
        "fallback_to_finite_differences",
        "hvp_interval",
        "hessian_approx",
        "consume_grad",
    )
    _REMOVED_STATS = frozenset({"stochastic_schedule", "precond_rng"})

    def __init__(self, params, defaults, use_ema: bool = False):
        for attr in self._INSTANCE_ATTRS:
            if attr in defaults:
                val = defaults.pop(attr)
                if val is not use_default:
                    setattr(self, attr, val)
        defaults.setdefault("multi_tensor", True)
        super().__init__(params, defaults)
        self.use_ema = use_ema
        self.mapping = {}
        self.mapping_inverse = {}
        self.inner_group = {}
        self._is_preconditioning = None
        if self.hessian_approx and self.compile_step:
            raise ValueError("Hessian approximation can't be used with compile_step.")
        self.register_state_dict_post_hook(StatefulOptimizer._store_stats)
        self.register_load_state_dict_pre_hook(StatefulOptimizer._load_stats)

    # ------------------------------------------------------------------ checkpoint metadata
    def _store_stats(self, state_dict):
        state_dict["heavyball"] = {
            "inner_group": self.inner_group,
            "use_ema": self.use_ema,
            "ema_decay": self.ema_decay,
            "compile_step": self.compile_step,
            "hessian_approx": self.hessian_approx,
            "precond_schedule": pickle_compat.dumps(self.precond_schedule),
            "fallback_to_finite_differences": self.fallback_to_finite_differences,
            "_fallback_enabled": self._fallback_enabled,
            "hvp_interval": self.hvp_interval,
        }

    def _load_stats(self, state_dict):
        for k, v in state_dict.get("heavyball", {}).items():
            if k in self._REMOVED_STATS:
                continue
            if k == "precond_schedule":
                try:
                    v = pickle_compat.loads(v)
                except Exception as err:  # noqa: BLE001 - a schedule that may not be loaded must not lose the checkpoint
                    warn_once(f"checkpoint's precond_schedule was not loaded, keeping the optimizer's own: {err}")
                    continue
            setattr(self, k, v)

    # ------------------------------------------------------------------ state addressing
    def get_groups(self, group):
        return [group]

    def _register_views(self, p, views):
        self.mapping[p] = views
        for i, v in enumerate(views):
            self.mapping_inverse[_tensor_key(v)] = (p, i)

    def _init_mapping(self, group: Optional[dict] = None):
        for g in self.param_groups if group is None else [group]:
            for p in g["params"]:
                if p not in self.mapping:
                    self._register_views(p, merge_group(g, p))

    def state_(self, arg: Tensor, fail: bool = True):
        key = _tensor_key(arg)
        hit = self.mapping_inverse.get(key)
        if hit is None:
            self._init_mapping()
            hit = self.mapping_inverse.get(key)
        if hit is None:
            if not fail:
                return {}
            raise KeyError("Tensor has no tracked state.")
        owner, index = hit
        return self.state.setdefault(owner, {}).setdefault(index, {})

    def state_size(self) -> int:
        seen, total = set(), 0

        def visit(x):
            nonlocal total
            if isinstance(x, Tensor) and id(x) not in seen:
                seen.add(id(x))
                total += x.numel() * x.element_size()

        for st in self.state.values():
            tree_map(visit, st)
        return total

    # ------------------------------------------------------------------ gradient hand-off
    def split_p_and_g_in_group(self, group: dict, skip_none: bool = True, should_promote: bool = True, raw: bool = False):
        """Yields ``(param_view, grad_view)`` pairs.  Gradients are *taken* from the parameters
        (``p.grad = None``) when ``consume_grad`` is set, which frees them as soon as the chain has
        finished with them."""
        tmp = group.get("_tmp")
        for p in group["params"]:
            if raw:
                grad = getattr(p, "grad", None)
                if grad is None and skip_none:
                    continue
                if self.consume_grad:
                    p.grad = None
                yield p, grad
                continue

            slot = None if tmp is None else tmp.get(id(p))
            grad = None if slot is None else slot.pop("grad", None)
            if grad is None:
                grad = getattr(p, "grad", None)
            if grad is None and skip_none:
                continue
            if self.consume_grad:
                p.grad = None

            if group.get("merge_dims", False) and not p.data.is_contiguous():
                for fmt in (torch.channels_last, torch.channels_last_3d):
                    if p.data.is_contiguous(memory_format=fmt):
                        set_temporary(group, p, restore_memory_format=fmt)
                        break
                p.data = p.data.contiguous()

            views = merge_group(group, p)
            self._register_views(p, views)

            vector = hessian_vector = None
            if slot is not None:
                vector = slot.pop("vector", None)
                hessian_vector = slot.pop("hessian_vector", None)
                if len(slot) == 1:
                    tmp.pop(id(p), None)
            n = len(views)
            gs = itertools.repeat(None, n) if grad is None else merge_group(group, grad)
            vs = itertools.repeat(None, n) if vector is None else merge_group(group, vector)
            hvs = itertools.repeat(None, n) if hessian_vector is None else merge_group(group, hessian_vector)
            for pv, g, v, hv in zip(views, gs, vs, hvs):
                g, v, hv = (promote_detach(t, should_promote) for t in (g, v, hv))
                if v is not None or hv is not None:
                    set_temporary(group, pv, vector=v, hessian_vector=hv)
                yield pv, g

    # ------------------------------------------------------------------ parameter EMA
    def _ema_pairs(self):
        for group in self.param_groups:
            for p in group["params"]:
                yield group, p, self.state_(p)

    def ema_update(self):
        with torch.no_grad():
            for group in self.param_groups:
                if not group["params"]:
                    continue
                k = group["ema_step"] = group.get("ema_step", -1) + 1
                w = beta_debias(1 - self.ema_decay, k + 1)
                for p in group["params"]:
                    st = self.state_(p)
                    if "param_ema" not in st:
                        st["param_ema"] = torch.zeros_like(p.data, memory_format=torch.preserve_format)
                    st["param_ema"].lerp_(p.data, w)

    def _swap_with_ema(self):
        with torch.no_grad():
            for _, p, st in self._ema_pairs():
                if "param_ema" in st:
                    held = p.data.clone()
                    p.data.copy_(st["param_ema"])
                    st["param_ema"].copy_(held)

    def copy_emas_to_params(self):
        self._swap_with_ema()

    def copy_params_to_emas(self):
        self._swap_with_ema()

    # ------------------------------------------------------------------ closures and HVPs
    def _finite_differences_hvp(self, closure):
        with torch.enable_grad():
            loss = closure()
        scale = torch.finfo(torch.float32).eps ** 0.5
        grads = []
        for group in self.param_groups:
            for p, g in self.split_p_and_g_in_group(group, skip_none=True, raw=True):
                grads.append(g)
                vector = torch.randn_like(p)
                set_temporary(group, p, vector=vector, orig=p.data.clone())
                stochastic_add_(p.data, vector, scale)
        with torch.enable_grad():
            closure()
        # parameters are restored from the saved copy rather than by subtracting the probe again
        for group in self.param_groups:
            for p, g in self.split_p_and_g_in_group(group, skip_none=True, raw=True):
                grad = grads.pop(0)
                set_temporary(group, p, grad=grad, hessian_vector=g)
                stochastic_add_divide_(g, grad, -1, scale)
                p.data.copy_(take_temporary(group, p, "orig"))
        return loss

    def _double_backward_hvp(self, closure):
        with torch.enable_grad(), patch_backward():
            loss = closure()
        params, grads, groups = [], [], []
        for group in self.param_groups:
            for p, g in self.split_p_and_g_in_group(group, skip_none=True, raw=True):
                params.append(p)
                grads.append(g)
                groups.append(group)
        if not params:
            raise ValueError("No parameter has gradients")
        vs = [torch.randn_like(p) for p in params]
        with torch.enable_grad():
            try:
                hvs = torch.autograd.grad(grads, params, vs, create_graph=False, retain_graph=False, allow_unused=True)
            except RuntimeError as e:
                raise ExactHVPFailed(str(e.args))
        unused = []
        for group, p, g, v, hv in zip(groups, params, grads, vs, hvs):
            set_temporary(group, p, grad=detach(g), vector=detach(v), hessian_vector=detach(hv))
            if hv is None:
                unused.append(list(p.shape))
        if unused:
            raise ExactHVPFailed(f"Parameters with the following shapes have no 2nd order derivative: {unused}")
        return loss

    def _handle_closure(self, closure):
        want_hvp = self.hessian_approx and self._is_preconditioning
        if closure is None:
            if want_hvp:
                raise ValueError("Hessian approximation requires a closure.")
            return None
        n = self.inner_group["total_hvp_steps"] = self.inner_group.get("total_hvp_steps", 0) + 1
        if not want_hvp or (n - 1) % self.hvp_interval == 0:
            with torch.enable_grad():
                return closure()
        if self.finite_differences or self._fallback_enabled:
            return self._finite_differences_hvp(closure)
        try:
            return self._double_backward_hvp(closure)
        except NotImplementedError as e:
            if not self.fallback_to_finite_differences:
                raise
            if not any(isinstance(a, str) and _cudnn_double_backward_pattern.match(a) for a in e.args):
                raise
            warn_once(
                "CUDNN doesn't support double-backward for some models (including RNNs). "
                f"Falling back to finite_differences.\n{_fd_error}{e}"
            )
        except RuntimeError as e:
            if not self.fallback_to_finite_differences:
                raise
            if not any(isinstance(a, str) and _torch_compile_double_backward_pattern.match(a) for a in e.args):
                raise
            warn_once(
                "torch.compile does not support double-backward. Disabling it may be beneficial, depending on "
                f"the model.\n{_fd_error}{e}"
            )
        except ExactHVPFailed as e:
            if not self.fallback_to_finite_differences:
                raise
            warn_once(f"Exact HVP calculation failed.\n{_fd_error}{e}")
        self._fallback_enabled = True
        return self._handle_closure(closure)

    # ------------------------------------------------------------------ step
    def _cleanup_temporary_tensors(self):
        for group in self.param_groups:
            tmp = group.pop("_tmp", None)
            if tmp is None:
                continue
            for slot in tmp.values():
                fmt = slot.get("restore_memory_format")
                if fmt is None:
                    continue
                t = slot["tensor"]
                self.mapping_inverse.pop(_tensor_key(t), None)
                t.data = t.data.to(memory_format=fmt)
                self.mapping_inverse[_tensor_key(t)] = (t, 0)

    def _step(self, group):
        raise NotImplementedError

    def step(self, closure: Optional[Callable] = None):
        if self.precond_schedule is None:
            self._is_preconditioning = False
        else:
            self._is_preconditioning = psgd_should_update(self.inner_group, self.precond_schedule)
        loss = self._handle_closure(closure)
        if self.use_ema:
            self.ema_update()
        with torch.no_grad():
            try:
                for group in self.param_groups:
                    if "param_count" not in group:
                        group["param_count"] = sum(p.numel() for p in group["params"])
                    group["is_preconditioning"] = self._is_preconditioning
                    self._step(group)
            finally:
                self._cleanup_temporary_tensors()
        return loss


# ---------------------------------------------------------------------------------------- backward hooks


def hook_optimizer_into_model(model, optimizer, *args, **kwargs):
    """One optimizer instance per parameter, stepped from the parameter's post-accumulate-grad hook
    (the update overlaps with the rest of the backward pass and the gradient is freed at once)."""
    per_param = {}

    def on_grad(p: Tensor):
        o = per_param[p]
        o.step()
        o.zero_grad()

    for p in model.parameters():
        per_param[p] = optimizer([p], *args, **kwargs)
        p.register_post_accumulate_grad_hook(on_grad)
    return per_param


def fused_hook(parameters, optimizer, *args, **kwargs):
    """A single optimizer stepped from the gradient hooks; its public ``step`` becomes a warning."""
    parameters = list(parameters)
    o = optimizer(parameters, *args, **kwargs)
    real_step = o.step
    o.step = functools.partial(
        warn_once, msg="You're trying to call `step` on a fused optimizer. This will not do anything."
    )

    def on_grad(p: Tensor):
        real_step()
        o.zero_grad()

    for p in parameters:
        p.register_post_accumulate_grad_hook(on_grad)
    return o
